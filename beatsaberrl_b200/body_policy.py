"""``BodyObjectPolicy``: the single-body-token policy layout (one body token + n_obj object tokens) on the
library's sm_100a kernels.

The reference's tokenizer is fixed at 29 tokens (python/policy.py:174-275); this module is the front and back
end for policies laid out as ``T = 1 + n_obj`` tokens instead -- body ``Linear(body_dim, d)``, object
``Linear(obj_dim, d)``, blocks as the reference's ``Block`` (python/policy.py:483-715) with an exact-GELU FFN,
readout = the body token, ``heads = Linear(d, 29 K)``, ``value = Linear(d, 1)`` -- with the same calling surface
as ``NotePolicy``: ``forward_stacked``, ``forward``, ``get_action_and_value(obs, action)``, ``flatten_fp16`` /
``refresh_fp16_caches`` (in-place repack).  Inference only; no CPU path.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.nn as nn

from . import _native as nat
from . import policy as _policy

N_ACTION_HEADS = 29


class _GBlock(nn.Module):
    def __init__(self, d: int, ffn_mult: int):
        super().__init__()
        self.ln_attn = nn.LayerNorm(d)
        self.q_proj = nn.Linear(d, d)
        self.k_proj = nn.Linear(d, d)
        self.v_proj = nn.Linear(d, d)
        self.out_proj = nn.Linear(d, d)
        self.ln_ffn = nn.LayerNorm(d)
        self.ffn = nn.Sequential(nn.Linear(d, ffn_mult * d), nn.GELU(), nn.Linear(ffn_mult * d, d))


class BodyObjectPolicy(nn.Module):
    def __init__(self, embed: int = 128, n_heads: int = 4, n_blocks: int = 2, ffn_mult: int = 4, n_obj: int = 16,
                 n_gears: int = 5, body_dim: int = 340, obj_dim: int = 16):
        super().__init__()
        self.embed, self.n_heads, self.n_obj, self.n_gears = embed, n_heads, n_obj, n_gears
        self.k_max = n_gears
        self.body_dim, self.obj_dim = body_dim, obj_dim
        self.obs_dim = body_dim + n_obj * obj_dim + n_obj
        self.body_enc = nn.Linear(body_dim, embed)
        self.obj_enc = nn.Linear(obj_dim, embed)
        self.blocks = nn.ModuleList(_GBlock(embed, ffn_mult) for _ in range(n_blocks))
        self.heads = nn.Linear(embed, N_ACTION_HEADS * n_gears)
        self.value = nn.Linear(embed, 1)
        self._ent_h = None
        cfg = nat.GConfig()
        cfg.embed, cfg.n_heads, cfg.n_blocks, cfg.ffn_mult = embed, n_heads, n_blocks, ffn_mult
        cfg.n_obj, cfg.n_gears, cfg.body_dim, cfg.obj_dim = n_obj, n_gears, body_dim, obj_dim
        cfg.eps = float(self.blocks[0].ln_attn.eps)
        self._cfg = cfg
        nat.check(nat.lib.bsrl_g_config_validate(C.byref(cfg)))
        n = nat.lib.bsrl_g_param_count(C.byref(cfg))
        buf, r, c = C.create_string_buffer(128), C.c_int64(), C.c_int64()
        self._param_table = []
        for i in range(n):
            nat.check(nat.lib.bsrl_g_param_desc(C.byref(cfg), i, buf, 128, C.byref(r), C.byref(c)))
            self._param_table.append((buf.value.decode(), r.value, c.value))
        self._arena = None
        self._arena_version = None
        self._workspaces = {}

    # ------------------------------------------------------------------ weights
    def _pack(self, force: bool = False) -> None:
        dev = self.value.weight.device
        if dev.type != "cuda":
            raise RuntimeError("BodyObjectPolicy runs on a CUDA device only (no CPU path): call .cuda() first")
        key = (_policy._weights_version, dev)
        if not force and self._arena is not None and self._arena_version == key:
            return
        n_bytes = nat.lib.bsrl_g_weights_bytes(C.byref(self._cfg))
        if self._arena is None or self._arena.device != dev:
            self._arena = torch.empty(n_bytes, dtype=torch.uint8, device=dev)
        sd = dict(self.named_parameters())
        ptrs = (C.c_void_p * len(self._param_table))()
        keep = []
        for i, (name, rows, cols) in enumerate(self._param_table):
            p = sd[name].detach().contiguous()
            assert p.dtype is torch.float32 and p.numel() == rows * cols, name
            keep.append(p)
            ptrs[i] = p.data_ptr()
        with torch.cuda.device(dev):
            nat.check(nat.lib.bsrl_g_pack_weights(C.byref(self._cfg), ptrs, len(keep), self._arena.data_ptr(), n_bytes,
                                                  torch.cuda.current_stream().cuda_stream))
        self._arena_version = key

    def flatten_fp16(self) -> None:
        self._pack(force=True)

    def refresh_fp16_caches(self) -> None:
        self._pack(force=True)

    def _workspace(self, B: int, dev):
        key = (B, dev)
        capturing = torch.cuda.is_current_stream_capturing()
        ent = self._workspaces.pop(key, None)
        if ent is None:
            n = nat.lib.bsrl_g_workspace_bytes(C.byref(self._cfg), B)
            ent = [torch.empty(max(n, 256), dtype=torch.uint8, device=dev), False]
        ent[1] = ent[1] or capturing          # a workspace a graph capture used is never released
        self._workspaces[key] = ent
        if not capturing:
            ent[0].record_stream(torch.cuda.current_stream(dev))
            idle = [k for k, (_, pinned) in self._workspaces.items() if not pinned and k != key]
            for k in idle[:max(0, len(idle) - 1)]:
                del self._workspaces[k]
        return ent[0]

    # ------------------------------------------------------------------ forward
    def _run(self, obs, action, need_entropy, want_logits):
        if not obs.is_cuda:
            raise RuntimeError("obs must live on a CUDA device (this library has no CPU path)")
        if obs.dim() != 2 or obs.shape[1] != self.obs_dim or obs.dtype is not torch.float32:
            raise ValueError(f"obs must be float32 (B, {self.obs_dim}), got {obs.dtype} {tuple(obs.shape)}")
        obs = obs.contiguous()
        self._pack()
        B, dev = obs.shape[0], obs.device
        f32 = dict(dtype=torch.float32, device=dev)
        logits = torch.empty(B, N_ACTION_HEADS, self.n_gears, **f32) if want_logits else None
        value = torch.empty(B, **f32)
        logprob = entropy = ent_h = None
        act_ptr, act_dt = None, nat.I64
        if action is not None:
            if action.dtype not in _policy._ACT_DTYPES:
                action = action.long()
            action = action.contiguous()
            if tuple(action.shape) != (B, N_ACTION_HEADS) or action.device != dev:
                raise ValueError(f"action must be ({B}, {N_ACTION_HEADS}) on {dev}")
            act_ptr, act_dt = action.data_ptr(), _policy._ACT_DTYPES[action.dtype]
            logprob = torch.empty(B, **f32)
            if need_entropy:
                entropy, ent_h = torch.empty(B, **f32), torch.empty(B, N_ACTION_HEADS, **f32)
        ws = self._workspace(B, dev)
        ptr = lambda t: t.data_ptr() if t is not None else None
        with torch.cuda.device(dev):
            nat.check(nat.lib.bsrl_g_forward(C.byref(self._cfg), self._arena.data_ptr(), obs.data_ptr(), B, act_ptr, act_dt,
                                             ptr(logits), ptr(logprob), ptr(entropy), ptr(ent_h), value.data_ptr(),
                                             ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream))
        return logits, value, logprob, entropy, ent_h

    @torch.no_grad()
    def forward_stacked(self, obs: torch.Tensor):
        """obs (B, obs_dim) -> logits (B, 29, n_gears) fp32 + value (B,) fp32."""
        logits, value, _, _, _ = self._run(obs, None, False, True)
        return logits, value

    def forward(self, obs: torch.Tensor):
        logits, value = self.forward_stacked(obs)
        return list(logits.unbind(1)), value

    @torch.no_grad()
    def get_action_and_value(self, obs, action, need_entropy=True):
        """The recompute call: summed log-prob of the given actions, entropy and value from the fused head kernel."""
        _, value, logprob, entropy, ent_h = self._run(obs, action, need_entropy, False)
        self._ent_h = ent_h
        return action, logprob, entropy, value

    def mac_per_env(self) -> int:
        return int(nat.lib.bsrl_g_mac_per_env(C.byref(self._cfg)))
