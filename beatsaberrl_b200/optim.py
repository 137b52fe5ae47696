"""AdamW over a ``NotePolicy``'s fp32 masters whose step also refreshes the packed fp16 arena.

The reference trainer runs a fused Adam step and then ``bump_weights_version()``, after which the next
forward recasts the flat fp16 replica (python/train_batch.py:2847-2854, python/fp16_linear.py:236-246).
Here one call -- ``bsrl_adam_step_pack``, a handful of launches for the whole model -- updates the
masters in place and writes every updated value straight to its place(s) in the arena, so there is no
separate refresh pass and a captured rollout graph sees the new weights on its next replay.

Arithmetic and hyper-parameters are ``torch.optim.AdamW``'s; like the reference's ``--weight-decay``
(python/train_batch.py:276-290) the decoupled decay applies to parameters with two or more
dimensions only.  Parameters without a gradient (frozen, or owned by another optimizer such as the
reference's Muon half) are left alone and only re-scattered.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _native as nat


class PackedAdamW:
    def __init__(self, policy, lr: float = 3e-4, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, lr_scale: dict | None = None):
        """``lr_scale`` maps parameter-name prefixes to learning-rate multipliers (the reference
        trains its critic at 3x the actor's rate)."""
        self.policy = policy
        self.lr, self.betas, self.eps, self.weight_decay = float(lr), tuple(betas), float(eps), float(weight_decay)
        self.lr_scale = dict(lr_scale or {})
        self.step_count = 0
        named = dict(policy.named_parameters())
        self.names = [n for n, _, _ in policy._param_table]
        self.params = [named[n] for n in self.names]
        for p in self.params:
            if p.dtype is not torch.float32 or not p.is_contiguous():
                raise ValueError("PackedAdamW needs contiguous float32 parameters")
        self.exp_avg = [torch.zeros_like(p, memory_format=torch.preserve_format) for p in self.params]
        self.exp_avg_sq = [torch.zeros_like(p, memory_format=torch.preserve_format) for p in self.params]
        n = len(self.params)
        self._ptr = lambda ts: (C.c_void_p * n)(*[t.data_ptr() if t is not None else None for t in ts])

    def _lr_of(self, name: str) -> float:
        for prefix, mult in self.lr_scale.items():
            if name.startswith(prefix):
                return self.lr * mult
        return self.lr

    def zero_grad(self, set_to_none: bool = True) -> None:
        for p in self.params:
            if p.grad is not None:
                if set_to_none:
                    p.grad = None
                else:
                    p.grad.zero_()

    @torch.no_grad()
    def step(self, inv_scale: torch.Tensor | None = None, found_inf: torch.Tensor | None = None) -> None:
        pol = self.policy
        dev = self.params[0].device
        if dev.type != "cuda":
            raise RuntimeError("PackedAdamW runs on a CUDA device only")
        pol._pack()                           # the arena exists and its padding is zero
        self.step_count += 1
        n = len(self.params)
        grads = [p.grad.contiguous() if (p.grad is not None and p.requires_grad) else None for p in self.params]
        lr = (C.c_float * n)(*[self._lr_of(nm) for nm in self.names])
        wd = (C.c_float * n)(*[self.weight_decay if p.dim() >= 2 else 0.0 for p in self.params])
        for name, s in (("inv_scale", inv_scale), ("found_inf", found_inf)):
            if s is not None and (s.numel() != 1 or s.dtype is not torch.float32 or s.device != dev):
                raise ValueError(f"{name} must be a one-element float32 tensor on {dev}")
        with torch.cuda.device(dev):
            nat.check(nat.lib.bsrl_adam_step_pack(
                C.byref(pol._cfg), self._ptr(self.params), self._ptr(grads), self._ptr(self.exp_avg),
                self._ptr(self.exp_avg_sq), n, lr, wd, self.betas[0], self.betas[1], self.eps, self.step_count,
                inv_scale.data_ptr() if inv_scale is not None else None,
                found_inf.data_ptr() if found_inf is not None else None,
                pol._arena.data_ptr(), pol._arena.numel(), torch.cuda.current_stream().cuda_stream))
        # the arena already holds the new weights: no version bump, no repack

    def state_dict(self) -> dict:
        return {"step": self.step_count,
                "exp_avg": {n: t.clone() for n, t in zip(self.names, self.exp_avg)},
                "exp_avg_sq": {n: t.clone() for n, t in zip(self.names, self.exp_avg_sq)}}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd["step"])
        for n, m, v in zip(self.names, self.exp_avg, self.exp_avg_sq):
            m.copy_(sd["exp_avg"][n])
            v.copy_(sd["exp_avg_sq"][n])
