"""``NotePolicy`` with the reference's surface, running the forward on the sm_100a kernels.

Mirrors the part of the reference's ``python/policy.py`` that callers of the policy-forward
path touch (``train_batch.py`` rollout and PPO recompute, ``rollout_graph.py``,
``cuda_graphs.py`` style graph drivers, the forward benches):

* constructor keywords and checks           -- ``NotePolicy.__init__``, python/policy.py:795-850
* parameter names / ``state_dict`` layout    -- python/policy.py:940-1067 (a reference checkpoint's
  ``state_dict`` loads with ``load_state_dict`` unchanged)
* ``forward_stacked`` / ``forward`` / ``get_action_and_value`` -- python/policy.py:1179-1196,
  :1463-1516
* ``flatten_fp16`` / ``refresh_fp16_caches`` and the module-level ``bump_weights_version`` --
  python/policy.py:1405-1461, python/fp16_linear.py:241-246: here they repack the fp32 masters
  into the packed fp16 arena IN PLACE, so storages captured in a CUDA graph stay valid.

The fp32 parameters are the masters (trainable by any optimizer); the forward itself is
inference-only (no autograd graph is built).  There is no torch or CPU fallback: a CPU tensor,
or a missing ``libbsrl.so``, raises.
"""
from __future__ import annotations

import ctypes as C
import math

import torch
import torch.nn as nn

from . import _native as nat

OBS_DIM = 630
N_NOTE_SLOTS = 24
NOTE_FEAT = 18
OFF_NOTES = 102
OFF_NOTE_MASK = OFF_NOTES + N_NOTE_SLOTS * NOTE_FEAT
SABER_FEAT, TORSO_FEAT, LEG_FEAT = 47, 29, 32
NOTE_GEO_FEAT = 22
N_ACTION_HEADS = 29
MASK_BIAS = 16384.0
MASKED_LOGIT = -1e9
TRUNK_ARCHS = ("simba", "simbav2")
ACCUM_MODES = ("off", "fwd", "all")
FFN_MODES = ("off", "on", "up16", "up16dn16")

_weights_version = 0


def bump_weights_version() -> None:
    """Tell every policy that the fp32 masters changed (call after ``optimizer.step()``); the
    next forward, or ``refresh_fp16_caches()``, repacks the fp16 arena in place.
    Same role as ``fp16_linear.bump_weights_version`` (python/fp16_linear.py:241-246)."""
    global _weights_version
    _weights_version += 1


def _mlp(sizes):
    layers = []
    for i in range(len(sizes) - 1):
        layers.append(nn.Linear(sizes[i], sizes[i + 1]))
        if i < len(sizes) - 2:
            layers.append(nn.ReLU())
    return nn.Sequential(*layers)


class _Block(nn.Module):
    """Parameter holder of one pre-LN block (names as python/policy.py:498-507)."""

    def __init__(self, d: int, ffn_mult: int, value_residual: bool = False):
        super().__init__()
        self.ln_attn = nn.LayerNorm(d)
        self.q_proj = nn.Linear(d, d)
        self.k_proj = nn.Linear(d, d)
        self.v_proj = nn.Linear(d, d)
        self.out_proj = nn.Linear(d, d)
        self.ln_ffn = nn.LayerNorm(d)
        self.ffn = _mlp([d, ffn_mult * d, d])
        if value_residual:      # registered last, only when on (python/policy.py:512-520)
            self.vres_a = nn.Parameter(torch.ones(1))
            self.vres_b = nn.Parameter(torch.zeros(1))


_ACT_DTYPES = {torch.uint8: nat.U8, torch.int32: nat.I32, torch.int64: nat.I64}


class _RecomputeFn(torch.autograd.Function):
    """The policy forward as ONE autograd node: ``bsrl_forward_train`` going forward (the rollout's own
    kernels, so log-probs match the rollout bit for bit, plus a save buffer), ``bsrl_backward`` coming
    back.  Stands in for the chain of autograd.Functions of the reference's fp16 stream
    (python/fp16_linear.py:461-767, :931-1064, :1197-1251; python/fused_ln.py:58-107)."""

    @staticmethod
    def forward(ctx, policy, obs, action, *params):
        B, dev = obs.shape[0], obs.device
        cfg = policy._cfg
        f32 = dict(dtype=torch.float32, device=dev)
        logits = torch.empty(B, N_ACTION_HEADS, policy.k_max, **f32)
        logprob, entropy, value = torch.empty(B, **f32), torch.empty(B, **f32), torch.empty(B, **f32)
        ent_h = torch.empty(B, N_ACTION_HEADS, **f32)
        vlogits = torch.empty(B, policy.value_bins, **f32)
        n_save = nat.lib.bsrl_train_save_bytes(C.byref(cfg), B)
        if n_save < 0:
            raise nat.BsrlError(int(n_save), nat.last_error())
        save = torch.empty(max(n_save, 256), dtype=torch.uint8, device=dev)
        ws = policy._workspace(B, dev)
        with torch.cuda.device(dev):
            nat.check(nat.lib.bsrl_forward_train(
                C.byref(cfg), policy._arena.data_ptr(), obs.data_ptr(), policy._obs_dtype(obs), B,
                action.data_ptr(), _ACT_DTYPES[action.dtype], logits.data_ptr(), logprob.data_ptr(),
                entropy.data_ptr(), ent_h.data_ptr(), value.data_ptr(), vlogits.data_ptr(), save.data_ptr(),
                save.numel(), ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream))
        ctx.policy, ctx.save, ctx.action, ctx.B = policy, save, action, B
        ctx.needs = [p.requires_grad for p in params]
        ctx.mark_non_differentiable(ent_h)
        return logits, logprob, entropy, value, vlogits, ent_h

    @staticmethod
    def backward(ctx, g_logits, g_logprob, g_entropy, g_value, g_vlogits, _g_ent_h):
        policy, B = ctx.policy, ctx.B
        cfg, dev = policy._cfg, ctx.save.device
        n = len(policy._param_table)
        offs = (C.c_int64 * n)()
        total = nat.lib.bsrl_grad_floats(C.byref(cfg), offs, n)
        if total < 0:
            raise nat.BsrlError(int(total), nat.last_error())
        flat = torch.empty(total, dtype=torch.float32, device=dev)
        n_ws = nat.lib.bsrl_backward_workspace_bytes(C.byref(cfg), B)
        ws = torch.empty(max(n_ws, 256), dtype=torch.uint8, device=dev)
        scale = float(policy.grad_scale)

        def up(g):
            return None if g is None else g.contiguous().float()
        ups = [up(g) for g in (g_logprob, g_entropy, g_value, g_vlogits, g_logits)]
        ptr = lambda t: t.data_ptr() if t is not None else None
        with torch.cuda.device(dev):
            nat.check(nat.lib.bsrl_backward(
                C.byref(cfg), policy._arena.data_ptr(), B, ctx.action.data_ptr(), _ACT_DTYPES[ctx.action.dtype],
                ctx.save.data_ptr(), ctx.save.numel(), ptr(ups[0]), ptr(ups[1]), ptr(ups[2]), ptr(ups[3]), ptr(ups[4]),
                scale, flat.data_ptr(), total, ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream))
        flat.mul_(1.0 / scale)
        grads = []
        for i, (_, rows, cols) in enumerate(policy._param_table):
            if not ctx.needs[i]:
                grads.append(None)
                continue
            grads.append(flat[offs[i]: offs[i] + rows * cols])
        ctx.save = None
        return (None, None, None, *grads)


class NotePolicy(nn.Module):
    def __init__(self, embed: int = 128, trunk_dim: int = 256, encoder: str = "transformer",
                 n_blocks: int = 3, n_heads: int = 4, n_gears: int = 3, ffn_mult: int = 4,
                 note_geo: bool = False, value_bins: int = 101, value_vmax: float = 6.0,
                 value_sigma: float = 0.75, trunk_hidden: int | None = None, z_asinh: float = 8.0,
                 game: str = "standard", fp16_accum: str = "off", fused_ffn: str = "off",
                 emb_ln: bool = False, value_residual: bool = False, final_ln: bool = False,
                 trunk_arch: str = "simba", head_gears: tuple | list | None = None):
        super().__init__()
        if trunk_arch not in TRUNK_ARCHS:
            raise ValueError(f"trunk_arch must be one of {TRUNK_ARCHS}, got {trunk_arch!r}")
        if game not in ("standard", "flux"):
            raise ValueError(f"game must be 'standard' or 'flux', got {game!r}")
        if not float(z_asinh) > 0:
            raise ValueError(f"z_asinh must be > 0 (metres), got {z_asinh}")
        if fp16_accum not in ACCUM_MODES:
            raise ValueError(f"fp16_accum must be one of {ACCUM_MODES}, got {fp16_accum!r}")
        if fused_ffn not in FFN_MODES:
            raise ValueError(f"fused_ffn must be one of {FFN_MODES}, got {fused_ffn!r}")
        assert encoder == "transformer", f"unknown encoder: {encoder}"
        assert n_gears in (3, 5, 7), f"n_gears must be 3/5/7, got {n_gears}"
        assert value_bins > 1, f"value_bins must be > 1, got {value_bins}"
        # fp16_accum ("fwd" / "all") is a PERMISSION in the reference: it lets cuBLAS accumulate its fp16 GEMMs in
        # fp16 where that is faster (python/fp16_linear.py:84-131).  The tensor cores used here accumulate fp16
        # products in fp32 at full rate, so the mode is accepted, recorded in `arch` like the reference does, and
        # changes nothing: results stay at least as close to the fp32 forward as the reference's own.
        if head_gears is None:
            head_gears = (n_gears,) * N_ACTION_HEADS
        head_gears = tuple(int(k) for k in head_gears)
        assert len(head_gears) == N_ACTION_HEADS and all(3 <= k <= 7 for k in head_gears), (
            f"head_gears must be {N_ACTION_HEADS} counts in [3, 7], got {head_gears}")
        self.encoder, self.embed, self.n_heads, self.n_gears = encoder, embed, n_heads, n_gears
        self.head_sizes = head_gears
        self.k_max = max(head_gears)
        H = int(trunk_hidden) if trunk_hidden else trunk_dim
        self.arch = {"embed": embed, "trunk_dim": trunk_dim, "n_blocks": n_blocks, "n_heads": n_heads,
                     "n_gears": n_gears, "obs_dim": OBS_DIM, "ffn_mult": ffn_mult,
                     "critic": "adapool_v1", "n_action_heads": N_ACTION_HEADS, "body_token": True,
                     "body_tokens": 3, "note_geo": bool(note_geo), "note_geo_norm": True,
                     "blade_geo": 1, "z_asinh": float(z_asinh), "trunk_arch": trunk_arch,
                     "trunk_hidden": H, "value_bins": int(value_bins),
                     "value_vmax": float(value_vmax), "value_sigma": float(value_sigma),
                     "game": game, "fp16_accum": fp16_accum, "fused_ffn": fused_ffn,
                     "emb_ln": bool(emb_ln), "value_residual": bool(value_residual), "final_ln": bool(final_ln)}
        if head_gears != (n_gears,) * N_ACTION_HEADS:
            self.arch["head_gears"] = list(head_gears)
        self.value_bins = int(value_bins)
        self.value_sigma_bins = float(value_sigma)
        centers = torch.linspace(-float(value_vmax), float(value_vmax), self.value_bins)
        self.register_buffer("value_centers", centers, persistent=False)
        self.value_sigma = float(value_sigma) * float(centers[1] - centers[0])
        self.note_geo, self.z_asinh, self.game = bool(note_geo), float(z_asinh), game
        self.body_tokens, self.n_lead = 3, 5
        # fp32 masters, created in the reference's order so a seeded init draws the same stream
        self.note_mlp = _mlp([NOTE_FEAT + (NOTE_GEO_FEAT if note_geo else 0), embed, embed])
        self.saber_mlp = _mlp([SABER_FEAT + 2, embed, embed])
        self.torso_mlp = _mlp([TORSO_FEAT, embed, embed])
        self.leg_mlp = _mlp([LEG_FEAT + 2, embed, embed])
        self.emb_ln = nn.LayerNorm(embed) if emb_ln else None          # --emb-ln (python/policy.py:962)
        self.value_residual = bool(value_residual)
        self.blocks = nn.ModuleList(_Block(embed, ffn_mult, self.value_residual and i > 0) for i in range(n_blocks))
        self.final_ln = nn.LayerNorm(embed) if final_ln else None      # --final-ln (python/policy.py:969)
        self.trunk_arch = trunk_arch
        if trunk_arch == "simba":
            self.trunk_proj = nn.Linear(self.n_lead * embed, trunk_dim)
            self.trunk_ln1 = nn.LayerNorm(trunk_dim)
            self.trunk_fc1 = nn.Linear(trunk_dim, H)
            self.trunk_fc2 = nn.Linear(H, trunk_dim)
            self.trunk_ln2 = nn.LayerNorm(trunk_dim)
        else:
            # SimBaV2 (python/policy.py:1003-1021): orthogonal, row-normalised matrices with frozen zero
            # biases, per-feature scalers; same creation order, so a seeded init matches the reference's
            self.trunk_in = nn.Linear(self.n_lead * embed, trunk_dim)
            self.trunk_w1 = nn.Linear(trunk_dim, H)
            self.trunk_w2 = nn.Linear(H, trunk_dim)
            for lin in (self.trunk_in, self.trunk_w1, self.trunk_w2):
                nn.init.orthogonal_(lin.weight)
                nn.init.zeros_(lin.bias)
                lin.bias.requires_grad_(False)
            self.trunk_s_in = nn.Parameter(torch.full((trunk_dim,), math.sqrt(2.0 / trunk_dim)))
            self.trunk_s_1 = nn.Parameter(torch.full((H,), math.sqrt(2.0 / H)))
            self.trunk_alpha = nn.Parameter(torch.full((trunk_dim,), 1.0 / math.sqrt(trunk_dim)))
            self.project_trunk_weights()
        self.heads = nn.ModuleList(nn.Linear(trunk_dim, n) for n in self.head_sizes)
        self.critic_ln = nn.LayerNorm(embed)
        self.critic_q = nn.Linear(embed, embed)
        self.critic_k = nn.Linear(embed, embed)
        self.critic_v = nn.Linear(embed, embed)
        self.critic_out = nn.Linear(embed, embed)
        self.critic_mlp = _mlp([embed + trunk_dim, trunk_dim, trunk_dim, self.value_bins])
        # runtime state (plain attributes, not in state_dict)
        self.fp16 = True            # the stream is always fp16 operands / fp32 accumulate here
        self.fp16_accum = fp16_accum
        self.fused_ffn = fused_ffn
        self.upgraded_from = None
        self._diag_stash = False
        self._diag_h = None
        self._ent_h = None
        self._value_logits = None
        self.keep_value_logits = False   # set True to have forwards fill _value_logits
        # loss scale of the backward's fp16 activation gradients (gradients come back unscaled); raise it if
        # tiny upstream gradients underflow, lower it if large ones overflow
        self.grad_scale = 4096.0
        self._cfg = nat.make_config(embed, n_heads, n_blocks, ffn_mult, trunk_dim, H, self.value_bins,
                                    note_geo, head_gears, float(z_asinh), float(value_vmax),
                                    float(self.blocks[0].ln_attn.eps), emb_ln=emb_ln, final_ln=final_ln,
                                    game_flux=(game == "flux"), value_residual=value_residual,
                                    trunk_v2=(trunk_arch == "simbav2"))
        nat.check(nat.lib.bsrl_config_validate(C.byref(self._cfg)))
        self._param_table = nat.param_table(self._cfg)
        self._arena = None
        self._arena_version = None
        self._workspaces = {}
        self._rng_state = None

    # ------------------------------------------------------------------ weights
    def _pack(self, force: bool = False) -> None:
        dev = self.critic_q.weight.device
        if dev.type != "cuda":
            raise RuntimeError("NotePolicy runs on a CUDA device only (no CPU path): call .cuda() first")
        key = (_weights_version, dev)
        if not force and self._arena is not None and self._arena_version == key:
            return
        n_bytes = nat.lib.bsrl_weights_bytes(C.byref(self._cfg))
        if self._arena is None or self._arena.device != dev:
            self._arena = torch.empty(n_bytes, dtype=torch.uint8, device=dev)
        sd = dict(self.named_parameters())
        ptrs = (C.c_void_p * len(self._param_table))()
        keep = []
        for i, (name, rows, cols) in enumerate(self._param_table):
            p = sd[name].detach()
            assert p.dtype is torch.float32 and p.numel() == rows * cols, name
            p = p.contiguous()
            keep.append(p)
            ptrs[i] = p.data_ptr()
        with torch.cuda.device(dev):
            nat.check(nat.lib.bsrl_pack_weights(C.byref(self._cfg), ptrs, len(keep),
                                                self._arena.data_ptr(), n_bytes,
                                                torch.cuda.current_stream().cuda_stream))
        self._arena_version = key

    def flatten_fp16(self) -> None:
        """Build the packed fp16 arena now (call once before CUDA-graph capture)."""
        self._pack(force=True)

    def refresh_fp16_caches(self, check: bool = False) -> None:
        """Repack the arena in place from the current fp32 masters (after optimizer steps;
        a captured graph keeps reading the same storage).  ``check=True`` also runs
        ``check_device()`` (a device synchronisation) first."""
        if check:
            self.check_device()
        self._pack(force=True)

    _MAX_IDLE_WORKSPACES = 2    # workspaces of batch sizes no captured graph uses, kept for reuse

    def _workspace(self, B: int, dev):
        """The forward's intermediates for a batch of B on ``dev``.

        A CUDA graph captured around a forward holds this buffer's raw address, so a workspace
        that was used while a stream was capturing is kept for the module's lifetime: a later
        call with another batch size (the PPO recompute on minibatches, after the rollout graph
        was captured at n_envs) gets a workspace of its own instead of replacing it.  Other
        workspaces are kept for reuse, the least recently used dropped beyond a small limit."""
        key = (B, dev)
        capturing = torch.cuda.is_current_stream_capturing()
        ent = self._workspaces.pop(key, None)
        if ent is None:
            n = nat.lib.bsrl_workspace_bytes(C.byref(self._cfg), B)
            if n < 0:
                raise nat.BsrlError(int(n), nat.last_error())
            ent = [torch.empty(max(n, 256), dtype=torch.uint8, device=dev), False]
        ent[1] = ent[1] or capturing
        self._workspaces[key] = ent                 # most recently used last
        if not capturing:
            # kernels of an earlier call may still be reading a workspace on another stream when the
            # allocator hands its memory out again: tie the buffer to every stream that uses it
            ent[0].record_stream(torch.cuda.current_stream(dev))
            idle = [k for k, (_, pinned) in self._workspaces.items() if not pinned and k != key]
            for k in idle[:max(0, len(idle) - (self._MAX_IDLE_WORKSPACES - 1))]:
                del self._workspaces[k]
        return ent[0]

    def check_device(self) -> None:
        """Raise if a bounded wait inside one of the kernels ran out since the last check.

        The kernels never spin without a limit: a wait that runs out makes the kernel set a status
        word and return, and that launch's outputs are garbage.  This synchronises the device, reads
        and clears the word (``bsrl_device_status``) and raises ``BsrlError`` (status -7) if it was
        set.  Call it where the host synchronises anyway -- the end of a rollout, before an update
        consumes the rollout's outputs; ``refresh_fp16_caches`` does."""
        dev = self.critic_q.weight.device
        if dev.type != "cuda":
            return
        with torch.cuda.device(dev):
            nat.check(nat.lib.bsrl_device_status())

    def _stash_diag(self, B: int, dev) -> None:
        """``_diag_stash`` of the reference (python/policy.py:1068-1073, :1309-1310): keep the trunk
        output h (B, trunk_dim) of the forward that just ran, copied out of the workspace."""
        off, rows, cols, ld, dt = (C.c_int64(), C.c_int64(), C.c_int64(), C.c_int64(), C.c_int32())
        nat.check(nat.lib.bsrl_workspace_region(C.byref(self._cfg), B, b"trunk_h", C.byref(off), C.byref(rows),
                                                C.byref(cols), C.byref(ld), C.byref(dt)))
        ws = self._workspaces[(B, dev)][0]
        flat = ws[off.value: off.value + (rows.value - 1) * ld.value * 2 + cols.value * 2].view(torch.float16)
        self._diag_h = torch.as_strided(flat, (rows.value, cols.value), (ld.value, 1)).clone()

    @staticmethod
    def _obs_dtype(obs):
        if obs.dtype is torch.float32:
            return nat.F32
        if obs.dtype is torch.float16:
            return nat.F16
        raise TypeError(f"obs must be float32 or float16, got {obs.dtype}")

    def _check_obs(self, obs):
        if not obs.is_cuda:
            raise RuntimeError("obs must live on a CUDA device (this library has no CPU path)")
        if obs.dim() != 2 or obs.shape[1] != OBS_DIM:
            raise ValueError(f"obs must be (B, {OBS_DIM}), got {tuple(obs.shape)}")
        return obs.contiguous()

    # ------------------------------------------------------------------ forward
    def _wants_grad(self) -> bool:
        return torch.is_grad_enabled() and any(p.requires_grad for p in self.parameters())

    def _recompute(self, obs, action):
        """Grad-mode forward: one autograd node over all parameters (see ``_RecomputeFn``)."""
        obs = self._check_obs(obs)
        self._pack()
        named = dict(self.named_parameters())
        params = [named[n] for n, _, _ in self._param_table]
        shapes = [p.shape for p in params]
        flat_params = [p.reshape(-1) if p.dim() != 1 else p for p in params]   # the node hands back flat gradients
        del shapes
        return _RecomputeFn.apply(self, obs, action, *flat_params)

    def forward_stacked(self, obs: torch.Tensor):
        """obs (B, 630) -> stacked logits (B, 29, k_max) fp32 + the critic's value (B,) fp32.  In grad mode
        the outputs carry gradients to every parameter (``_value_logits`` too)."""
        if self._wants_grad():
            dummy = torch.zeros(obs.shape[0], N_ACTION_HEADS, dtype=torch.uint8, device=obs.device)
            logits, _, _, value, vl, _ = self._recompute(obs, dummy)
            self._value_logits = vl
            return logits, value
        with torch.no_grad():
            return self._forward_stacked_nograd(obs)

    def _forward_stacked_nograd(self, obs: torch.Tensor):
        obs = self._check_obs(obs)
        self._pack()
        B, dev = obs.shape[0], obs.device
        logits = torch.empty(B, N_ACTION_HEADS, self.k_max, dtype=torch.float32, device=dev)
        value = torch.empty(B, dtype=torch.float32, device=dev)
        vl = (torch.empty(B, self.value_bins, dtype=torch.float32, device=dev)
              if self.keep_value_logits else None)
        ws = self._workspace(B, dev)
        with torch.cuda.device(dev):
            nat.check(nat.lib.bsrl_forward(
                C.byref(self._cfg), self._arena.data_ptr(), obs.data_ptr(), self._obs_dtype(obs), B,
                logits.data_ptr(), value.data_ptr(), vl.data_ptr() if vl is not None else None,
                ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream))
        self._value_logits = vl
        if self._diag_stash:
            self._stash_diag(B, dev)
        return logits, value

    def forward(self, obs: torch.Tensor):
        logits, value = self.forward_stacked(obs)
        return list(logits.unbind(1)), value

    def get_action_and_value(self, obs, action=None, need_entropy=True):
        """With ``action`` given (the PPO recompute call) the log-softmax, the summed log-prob
        and the entropy come out of the fused head kernel; in grad mode they (and ``_value_logits``)
        carry gradients to every parameter, computed by the library's backward.  With ``action=None``
        the actions are drawn inside the head kernel by Gumbel-max on the log-softmax, as the reference
        does (python/policy.py:1475-1490), from a Philox stream keyed by ``self.seed_sampler(seed)``
        (default: seeded from torch's generator at first use)."""
        if action is None:
            return self._sample(obs, need_entropy)
        if self._wants_grad():
            B, dev = obs.shape[0], obs.device
            if action.dtype not in _ACT_DTYPES:
                action = action.long()
            action = action.contiguous()
            if tuple(action.shape) != (B, N_ACTION_HEADS) or action.device != dev:
                raise ValueError(f"action must be ({B}, {N_ACTION_HEADS}) on {dev}")
            _, logprob, entropy, value, vl, ent_h = self._recompute(obs, action)
            self._ent_h = ent_h if need_entropy else None
            self._value_logits = vl
            return action, logprob, (entropy if need_entropy else None), value
        with torch.no_grad():
            return self._evaluate_nograd(obs, action, need_entropy)

    def _evaluate_nograd(self, obs, action, need_entropy):
        obs = self._check_obs(obs)
        self._pack()
        B, dev = obs.shape[0], obs.device
        if action.dtype not in _ACT_DTYPES:
            action = action.long()
        action = action.contiguous()
        if tuple(action.shape) != (B, N_ACTION_HEADS) or action.device != dev:
            raise ValueError(f"action must be ({B}, {N_ACTION_HEADS}) on {dev}")
        f32 = dict(dtype=torch.float32, device=dev)
        logprob, value = torch.empty(B, **f32), torch.empty(B, **f32)
        entropy = torch.empty(B, **f32) if need_entropy else None
        ent_h = torch.empty(B, N_ACTION_HEADS, **f32) if need_entropy else None
        vl = torch.empty(B, self.value_bins, **f32) if self.keep_value_logits else None
        ws = self._workspace(B, dev)
        ptr = lambda t: t.data_ptr() if t is not None else None
        with torch.cuda.device(dev):
            nat.check(nat.lib.bsrl_forward_act(
                C.byref(self._cfg), self._arena.data_ptr(), obs.data_ptr(), self._obs_dtype(obs), B,
                action.data_ptr(), _ACT_DTYPES[action.dtype], None, logprob.data_ptr(), ptr(entropy),
                ptr(ent_h), value.data_ptr(), ptr(vl), ws.data_ptr(), ws.numel(),
                torch.cuda.current_stream().cuda_stream))
        if need_entropy:
            self._ent_h = ent_h
        self._value_logits = vl
        if self._diag_stash:
            self._stash_diag(B, dev)
        return action, logprob, entropy, value

    def seed_sampler(self, seed: int) -> None:
        """(Re)start the action-sampling stream: [seed, call counter] in a device tensor that the
        head kernel reads, so a captured CUDA graph draws fresh numbers on every replay."""
        dev = self.critic_q.weight.device
        vals = torch.tensor([seed & 0x7FFFFFFFFFFFFFFF, 0], dtype=torch.int64)
        if self._rng_state is not None and self._rng_state.device == dev:
            self._rng_state.copy_(vals)      # in place: a captured graph keeps reading this tensor
        else:
            self._rng_state = vals.to(dev)

    @torch.no_grad()
    def _sample(self, obs, need_entropy):
        obs = self._check_obs(obs)
        self._pack()
        B, dev = obs.shape[0], obs.device
        if getattr(self, "_rng_state", None) is None or self._rng_state.device != dev:
            self.seed_sampler(int(torch.randint(0, 2 ** 62, (1,)).item()))
        f32 = dict(dtype=torch.float32, device=dev)
        action = torch.empty(B, N_ACTION_HEADS, dtype=torch.int64, device=dev)
        logprob, value = torch.empty(B, **f32), torch.empty(B, **f32)
        entropy = torch.empty(B, **f32) if need_entropy else None
        ent_h = torch.empty(B, N_ACTION_HEADS, **f32) if need_entropy else None
        ws = self._workspace(B, dev)
        ptr = lambda t: t.data_ptr() if t is not None else None
        with torch.cuda.device(dev):
            nat.check(nat.lib.bsrl_forward_sample(
                C.byref(self._cfg), self._arena.data_ptr(), obs.data_ptr(), self._obs_dtype(obs), B,
                self._rng_state.data_ptr(), action.data_ptr(), None, logprob.data_ptr(), ptr(entropy),
                ptr(ent_h), value.data_ptr(), ws.data_ptr(), ws.numel(),
                torch.cuda.current_stream().cuda_stream))
            self._rng_state[1] += 1          # next call (or graph replay) draws new numbers
        if need_entropy:
            self._ent_h = ent_h
        self._value_logits = None
        return action, logprob, entropy, value

    def trunk_projected(self):
        """The Linears whose rows project_trunk_weights keeps unit-norm ([] for the SimBa trunk)."""
        return [self.trunk_in, self.trunk_w1, self.trunk_w2] if self.trunk_arch == "simbav2" else []

    @torch.no_grad()
    def project_trunk_weights(self) -> bool:
        """SimBaV2 weight projection (python/policy.py:1165-1177): every output row of W_in / W1 / W2 back onto
        the unit sphere, biases to 0, in place; the caller bumps the weights version afterwards."""
        lins = self.trunk_projected()
        for lin in lins:
            lin.weight.div_(lin.weight.norm(dim=1, keepdim=True).clamp_min(1e-12))
            lin.bias.zero_()
        return bool(lins)

    @torch.no_grad()
    def rollout_step(self, obs, b_act=None, b_logp=None, b_val=None, b_obs=None, ret_sig=None, ret_mu=None,
                     need_entropy=False):
        """One rollout tick with the trainer's per-tick buffer stores fused into the forward's kernels.

        Stands in for the loop body ``b_obs[t] = obs; a, logp, _, v = get_action_and_value(obs);
        b_act[t], b_logp[t] = a, logp; b_val[t].copy_(v).mul_(ret_sig).add_(ret_mu)`` of the reference
        trainer (python/train_batch.py:2299-2350).  Pass ROW VIEWS of the buffers: ``b_act`` (B, 29) uint8,
        ``b_logp`` (B,) f32, ``b_val`` (B,) f32, ``b_obs`` (B, 630) f16; ``ret_sig`` / ``ret_mu`` are the 0-d
        device tensors of the return normaliser (None = 1 / 0).  Any buffer may be None.  Returns
        ``(action int64, logprob, entropy | None, value)`` like ``get_action_and_value``.
        """
        obs = self._check_obs(obs)
        self._pack()
        B, dev = obs.shape[0], obs.device
        if getattr(self, "_rng_state", None) is None or self._rng_state.device != dev:
            self.seed_sampler(int(torch.randint(0, 2 ** 62, (1,)).item()))
        f32 = dict(dtype=torch.float32, device=dev)

        def row(t, shape, dtype, name):
            if t is None:
                return None
            if tuple(t.shape) != shape or t.dtype != dtype or t.device != dev or not t.is_contiguous():
                raise ValueError(f"{name} must be a contiguous {dtype} tensor of shape {shape} on {dev}")
            return t

        b_act = row(b_act, (B, N_ACTION_HEADS), torch.uint8, "b_act")
        b_val = row(b_val, (B,), torch.float32, "b_val")
        b_obs = row(b_obs, (B, OBS_DIM), torch.float16, "b_obs")
        logprob = row(b_logp, (B,), torch.float32, "b_logp")
        if logprob is None:
            logprob = torch.empty(B, **f32)
        for name, s in (("ret_sig", ret_sig), ("ret_mu", ret_mu)):
            if s is not None and (s.numel() != 1 or s.dtype != torch.float32 or s.device != dev):
                raise ValueError(f"{name} must be a one-element float32 tensor on {dev}")
        action = torch.empty(B, N_ACTION_HEADS, dtype=torch.int64, device=dev)
        value = torch.empty(B, **f32)
        entropy = torch.empty(B, **f32) if need_entropy else None
        ent_h = torch.empty(B, N_ACTION_HEADS, **f32) if need_entropy else None
        ws = self._workspace(B, dev)
        ptr = lambda t: t.data_ptr() if t is not None else None
        with torch.cuda.device(dev):
            nat.check(nat.lib.bsrl_forward_rollout(
                C.byref(self._cfg), self._arena.data_ptr(), obs.data_ptr(), self._obs_dtype(obs), B,
                self._rng_state.data_ptr(), action.data_ptr(), ptr(b_act), logprob.data_ptr(), ptr(entropy),
                ptr(ent_h), value.data_ptr(), ptr(b_val), ptr(ret_sig), ptr(ret_mu), ptr(b_obs),
                ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream))
            self._rng_state[1] += 1
        if need_entropy:
            self._ent_h = ent_h
        self._value_logits = None
        return action, logprob, entropy, value

    # ------------------------------------------------------------------ introspection
    def mac_per_env(self) -> int:
        return int(nat.lib.bsrl_mac_per_env(C.byref(self._cfg)))
