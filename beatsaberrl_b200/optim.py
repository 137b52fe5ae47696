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

``PackedMuon`` is that other half (python/train_batch.py:797-968): Nesterov momentum, five quintic Newton-Schulz
steps towards the nearest orthogonal matrix, an RMS-matched step scale, on the hidden 2-D matrices only.  The
small matrix products run as batched fp32 ``torch.bmm`` chains, one per matrix shape; the step itself -- masters
plus their places in the arena -- is again one call of the library (``bsrl_apply_updates_pack``).
"""
from __future__ import annotations

import ctypes as C
import math
from collections import defaultdict

import torch

from . import _native as nat


class PackedAdamW:
    def __init__(self, policy, lr: float = 3e-4, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, lr_scale: dict | None = None, exclude=()):
        """``lr_scale`` maps parameter-name prefixes to learning-rate multipliers (the reference
        trains its critic at 3x the actor's rate); ``exclude`` names parameters another optimizer owns
        (``muon_param_names``): their gradients are ignored here."""
        self.policy = policy
        self.exclude = frozenset(exclude)
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
        grads = [p.grad.contiguous() if (p.grad is not None and p.requires_grad and nm not in self.exclude) else None
                 for nm, p in zip(self.names, self.params)]
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


# Newton-Schulz coefficients, one (a, b, c) per step, applied as a x + b x^3 + c x^5 to the singular values of the
# normalised update: the published five-step schedule the reference adopted (python/train_batch.py:797-816).
MUON_NS_COEFS = ((4.0848, -6.8946, 2.9270),
                 (3.9505, -6.3029, 2.6377),
                 (3.7418, -5.5913, 2.3037),
                 (2.8769, -3.1427, 1.2046),
                 (2.8366, -3.0525, 1.2012))


def muon_param_names(policy, enc_hidden: bool = False) -> list:
    """The parameters Muon owns (python/train_batch.py:947-967): hidden 2-D matrices only.  The 29 heads, the critic's
    final value-bin layer, every bias / LayerNorm vector and the token encoders stay with Adam; with ``enc_hidden``
    the encoders' second layers move to Muon and only their input layers (``*_mlp.0``) stay."""
    enc = ("note_mlp", "saber_mlp", "torso_mlp", "leg_mlp")
    last_critic = f"critic_mlp.{len(policy.critic_mlp) - 1}.weight"
    names = []
    for n, p in policy.named_parameters():
        if p.ndim != 2 or n.startswith("heads.") or n == last_critic:
            continue
        if n.startswith(enc) and (not enc_hidden or ".0." in n):
            continue
        names.append(n)
    return names


def orthogonalize(stack: torch.Tensor, eps: float = 1e-7) -> torch.Tensor:
    """Five Newton-Schulz steps on a stack (k, m, n) of wide (m <= n) fp32 matrices: each is scaled to unit Frobenius
    norm and pushed towards the nearest orthogonal matrix; the iteration runs on the small (m, m) Gram matrix."""
    x = stack / (torch.linalg.vector_norm(stack, dim=(1, 2), keepdim=True) + eps)
    for a, b, c in MUON_NS_COEFS:
        gram = torch.bmm(x, x.transpose(1, 2))
        poly = torch.baddbmm(gram, gram, gram, beta=b, alpha=c)          # b s + c s s
        x = torch.baddbmm(x, poly, x, beta=a)                            # a x + (b s + c s s) x
    return x


class PackedMuon:
    def __init__(self, policy, names=None, lr: float = 0.02, momentum: float = 0.95, weight_decay: float = 0.0,
                 lr_scale: dict | None = None):
        """``names``: the parameters this optimizer owns (default ``muon_param_names(policy)``); pair it with
        ``PackedAdamW(policy, ..., exclude=names)`` for the rest."""
        self.policy = policy
        self.lr, self.momentum, self.weight_decay = float(lr), float(momentum), float(weight_decay)
        self.lr_scale = dict(lr_scale or {})
        named = dict(policy.named_parameters())
        self.table = [n for n, _, _ in policy._param_table]              # every parameter, the library's order
        self.all_params = [named[n] for n in self.table]
        self.names = list(names) if names is not None else muon_param_names(policy)
        for n in self.names:
            if n not in named or named[n].ndim != 2:
                raise ValueError(f"PackedMuon owns 2-D parameters only: {n}")
        self.params = [named[n] for n in self.names]
        self.bufs = [torch.zeros_like(p) for p in self.params]
        self._slot = {n: i for i, n in enumerate(self.table)}

    def _lr_of(self, name: str) -> float:
        for prefix, mult in self.lr_scale.items():
            if name.startswith(prefix):
                return self.lr * mult
        return self.lr

    def zero_grad(self, set_to_none: bool = True) -> None:
        for p in self.params:
            if p.grad is not None:
                p.grad = None if set_to_none else p.grad.zero_()

    @torch.no_grad()
    def step(self, found_inf: torch.Tensor | None = None) -> None:
        pol = self.policy
        dev = self.params[0].device
        if dev.type != "cuda":
            raise RuntimeError("PackedMuon runs on a CUDA device only")
        pol._pack()
        live = [(n, p, b) for n, p, b in zip(self.names, self.params, self.bufs) if p.grad is not None and p.requires_grad]
        updates = [None] * len(self.table)
        if live:
            grads = [p.grad for _, p, _ in live]
            bufs = [b for _, _, b in live]
            torch._foreach_mul_(bufs, self.momentum)
            torch._foreach_add_(bufs, grads)
            nesterov = torch._foreach_add(grads, bufs, alpha=self.momentum)
            by_shape = defaultdict(list)
            for i, (_, p, _) in enumerate(live):
                by_shape[(min(p.shape), max(p.shape))].append(i)
            for idx in by_shape.values():                                 # one chain of batched products per shape
                tall = [live[i][1].shape[0] > live[i][1].shape[1] for i in idx]
                stack = torch.stack([nesterov[i].t() if t else nesterov[i] for i, t in zip(idx, tall)])
                ortho = orthogonalize(stack)
                for k, (i, t) in enumerate(zip(idx, tall)):
                    name, p, _ = live[i]
                    lr = self._lr_of(name)
                    upd = (ortho[k].t() if t else ortho[k]) * (-lr * 0.2 * math.sqrt(max(p.shape)))
                    if self.weight_decay:
                        upd = upd - (lr * self.weight_decay) * p
                    updates[self._slot[name]] = upd.contiguous()
        n = len(self.table)
        ptr = lambda ts: (C.c_void_p * n)(*[t.data_ptr() if t is not None else None for t in ts])
        if found_inf is not None and (found_inf.numel() != 1 or found_inf.dtype is not torch.float32 or found_inf.device != dev):
            raise ValueError(f"found_inf must be a one-element float32 tensor on {dev}")
        with torch.cuda.device(dev):
            nat.check(nat.lib.bsrl_apply_updates_pack(
                C.byref(pol._cfg), ptr(self.all_params), ptr(updates), n,
                found_inf.data_ptr() if found_inf is not None else None,
                pol._arena.data_ptr(), pol._arena.numel(), torch.cuda.current_stream().cuda_stream))

    def state_dict(self) -> dict:
        return {"momentum": self.momentum, "bufs": {n: b.clone() for n, b in zip(self.names, self.bufs)}}

    def load_state_dict(self, sd: dict) -> None:
        if set(sd["bufs"]) != set(self.names):
            raise ValueError("muon state does not match this policy's muon parameters")
        for n, b in zip(self.names, self.bufs):
            b.copy_(sd["bufs"][n])
