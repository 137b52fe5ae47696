"""CUDA-graph drivers for the policy forward, with the capture/replay protocol of the reference.

Counterparts of ``python/cuda_graphs.py`` (``copy_static`` :22-32, ``_Graphed`` :35-68) and
``python/rollout_graph.py`` (``GraphedRollout`` :45-104).  Everything the forward launches goes to
the stream that is current when it is called and lives in buffers owned by the policy (the packed
weight arena, one workspace per batch size), so a capture records plain kernel launches with
fixed addresses:

* weights are repacked IN PLACE (``NotePolicy.refresh_fp16_caches``), so a live graph sees new
  weights on its next replay;
* the sampling counter lives in a device tensor that the captured ``rng_state[1] += 1`` advances,
  so every replay draws fresh actions;
* a workspace that a capture used is never released by the policy (``NotePolicy._workspace``).

``StandInEnv`` plays the part of the CUDA environment in tests and tick benchmarks: it keeps the
observation, reward and done buffers the real ``CudaVecEnv`` preallocates and rewrites them in
place with the library's stand-in step kernel.
"""
from __future__ import annotations

import torch

from . import _native as nat
from . import policy as _policy

GRAPH_WARMUP = 3   # eager iterations before a capture (allocator, lazily loaded kernels)


def copy_static(static: torch.Tensor, value: torch.Tensor, non_blocking: bool = False) -> None:
    """Copy ``value`` into a fixed input buffer of a graph, refusing what ``copy_`` would silently
    fix up: another shape would broadcast and another dtype would cast, and either would corrupt
    every later replay (python/cuda_graphs.py:22-32)."""
    if value.shape != static.shape or value.dtype != static.dtype:
        raise RuntimeError(f"static input expects {tuple(static.shape)} {static.dtype}, "
                           f"got {tuple(value.shape)} {value.dtype}")
    static.copy_(value, non_blocking=non_blocking)


class Graphed:
    """Base of a graphed computation: subclasses copy their inputs into static buffers with
    ``_copy_static`` and call ``_run()``, which runs ``_compute()`` eagerly on a side stream for
    ``GRAPH_WARMUP`` calls, captures it on the next call, and replays the graph from then on.
    ``_out`` holds the outputs (the same storages on every replay once captured)."""

    def __init__(self):
        self.graph = None
        self._out = None
        self._calls = 0
        self._side = torch.cuda.Stream()

    def _compute(self):
        raise NotImplementedError

    def _copy_static(self, static, value, non_blocking=False):
        copy_static(static, value, non_blocking=non_blocking)

    def _run(self):
        if self.graph is not None:
            self.graph.replay()
            return self._out
        if self._calls < GRAPH_WARMUP:
            cur = torch.cuda.current_stream()
            self._side.wait_stream(cur)
            with torch.cuda.stream(self._side):
                self._out = self._compute()
            cur.wait_stream(self._side)
            self._calls += 1
            return self._out
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):        # records the launches, does not run them
            self._out = self._compute()
        self.graph.replay()
        return self._out


class GraphedForward(Graphed):
    """``policy.forward_stacked`` behind a static obs buffer: ``g(obs) -> (logits, value)``, the
    outputs being static tensors that the next call overwrites (the graphed argmax forward of the
    reference's ScoreSaber bench, python/bench_scoresaber.py:130-150)."""

    def __init__(self, policy, n_envs: int, obs_dtype=torch.float32):
        super().__init__()
        dev = next(policy.parameters()).device
        self.policy = policy
        self.obs = torch.zeros(n_envs, _policy.OBS_DIM, dtype=obs_dtype, device=dev)
        policy.flatten_fp16()

    def _compute(self):
        with torch.no_grad():
            return self.policy.forward_stacked(self.obs)

    def __call__(self, obs):
        self._copy_static(self.obs, obs, non_blocking=True)
        return self._run()


class GraphedRollout:
    """Policy forward + action sampling + environment step as ONE graph, replayed once per tick
    (python/rollout_graph.py:45-104).

    ``venv`` needs the CUDA environment's surface: ``_obs`` (n_envs, 630) static observation
    tensor that ``step(action)`` rewrites in place, and optionally ``_reward`` / ``_done``.  With
    ``buffers`` (a dict of per-tick row tensors ``b_act``, ``b_logp``, ``b_val``, ``b_obs`` and the
    scalars ``ret_sig``, ``ret_mu``) the tick runs ``policy.rollout_step`` so that the trainer's
    buffer rows are written by the same kernels; the rows are static too, the caller copies them
    into slot t of its buffers.
    """

    def __init__(self, policy, venv, warmup: int = GRAPH_WARMUP, buffers: dict | None = None):
        if not venv._obs.is_cuda:
            raise RuntimeError("GraphedRollout needs the CUDA environment")
        self.policy, self.venv = policy, venv
        self.buffers = dict(buffers or {})
        self._version = None
        # the stream mode the graph is captured under is baked into its kernels
        self.captured_fp16 = bool(getattr(policy, "fp16", False))
        self.refresh()                      # the arena must exist, and stay put, before the capture
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(warmup):
                self._tick()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        gen = getattr(venv, "_gen", None)
        if gen is not None:                 # an environment that draws from a torch generator while stepping
            self.graph.register_generator_state(gen)
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self.action, self.logp, self.value = self._tick()

    def _tick(self):
        if self.buffers:
            a, logp, _, v = self.policy.rollout_step(self.venv._obs, need_entropy=False, **self.buffers)
        else:
            a, logp, _, v = self.policy.get_action_and_value(self.venv._obs, need_entropy=False)
        self.venv.step(a)
        return a, logp, v

    def refresh(self) -> None:
        """Repack the weight arena in place, once per weights version; call after every optimizer
        step and before the next replay.  Raises if ``policy.fp16`` no longer is what the graph was
        captured with (python/rollout_graph.py:76-97)."""
        live = bool(getattr(self.policy, "fp16", False))
        if live != self.captured_fp16:
            raise RuntimeError(f"GraphedRollout was captured with policy.fp16={self.captured_fp16} but the "
                               f"policy is now fp16={live}; recapture or restore the flag")
        if self._version != _policy._weights_version:
            self.policy.refresh_fp16_caches()
            self._version = _policy._weights_version

    def step(self):
        """One tick: replay, return the static outputs (copy what you keep before the next one)."""
        self.graph.replay()
        v = self.venv
        return self.action, self.logp, self.value, getattr(v, "_reward", None), getattr(v, "_done", None)


class StandInEnv:
    """Environment stand-in with the CUDA env's buffer contract (``_obs``, ``_reward``, ``_done``
    preallocated, rewritten in place by ``step``); the dynamics are the library's hash-based
    stand-in kernel, not a simulation."""

    def __init__(self, n_envs: int, device="cuda", seed: int = 0):
        dev = torch.device(device)
        g = torch.Generator().manual_seed(seed)
        self.n_envs = n_envs
        self._state = torch.randint(0, 2 ** 31 - 1, (n_envs,), generator=g, dtype=torch.int64).to(torch.int32).to(dev)
        obs = torch.randn(n_envs, _policy.OBS_DIM, generator=g).clamp_(-5, 5)
        obs[:, _policy.OFF_NOTE_MASK:_policy.OFF_NOTE_MASK + _policy.N_NOTE_SLOTS] = 1.0
        self._obs = obs.to(dev)
        self._reward = torch.zeros(n_envs, dtype=torch.float32, device=dev)
        self._done = torch.zeros(n_envs, dtype=torch.uint8, device=dev)

    def step(self, action: torch.Tensor):
        if action.dtype is not torch.int64 or tuple(action.shape) != (self.n_envs, _policy.N_ACTION_HEADS):
            raise ValueError(f"action must be int64 ({self.n_envs}, {_policy.N_ACTION_HEADS})")
        with torch.cuda.device(self._obs.device):
            nat.check(nat.lib.bsrl_standin_env_step(
                action.data_ptr(), self.n_envs, self._state.data_ptr(), self._obs.data_ptr(),
                self._reward.data_ptr(), self._done.data_ptr(), torch.cuda.current_stream().cuda_stream))
        return self._obs, self._reward, self._done
