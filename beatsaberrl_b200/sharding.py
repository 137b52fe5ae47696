"""Env-batch sharding across the GPUs of one box.

Environments are independent (no kernel of the forward mixes rows of different envs), so a batch
of ``total`` envs is split into contiguous ranges, one per rank, weights are replicated, and the
forward itself needs no collective.  The only exchange is the optional reduction of a few rollout
statistics the trainer prints once per update -- in the single-GPU reference these are plain
tensor reductions at its print sync (python/train_batch.py:2329, :2885-2888).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def env_range(total: int, rank: int, world: int) -> tuple[int, int]:
    """[start, stop) of the envs rank ``rank`` owns: contiguous, sizes differ by at most one,
    earlier ranks take the remainder."""
    if not (0 <= rank < world) or total < 0:
        raise ValueError(f"bad shard request total={total} rank={rank} world={world}")
    base, rem = divmod(total, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def broadcast_weights(module: torch.nn.Module, src: int = 0, group=None) -> None:
    """One-time replication of the fp32 masters from ``src`` (call before ``flatten_fp16``)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return
    for p in module.parameters():
        dist.broadcast(p.data, src=src, group=group)


def reduce_rollout_stats(ent_head: torch.Tensor, logprob: torch.Tensor, value: torch.Tensor, group=None) -> dict:
    """Global means over all ranks' envs of the per-head entropy (29,), the log-prob and the
    value, weighted by each rank's env count.  One small all-reduce (31 + 1 floats)."""
    n = torch.tensor([float(ent_head.shape[0])], dtype=torch.float64, device=ent_head.device)
    packed = torch.cat([ent_head.double().sum(0), logprob.double().sum().view(1),
                        value.double().sum().view(1), n])
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
    total = packed[-1]
    return {"ent_head_mean": (packed[:29] / total).float(), "logprob_mean": float(packed[29] / total),
            "value_mean": float(packed[30] / total), "n_envs": int(total.item())}
