"""world_size-2 gloo run of the sharding logic on the CPU (the forward itself is stood in for by
the oracle, since the product has no CPU path): shards cover the batch exactly, and the reduced
rollout statistics equal the single-process ones."""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def test_env_range_covers_batch():
    from beatsaberrl_b200.sharding import env_range
    for total in (0, 1, 7, 8, 1000, 1_048_576):
        for world in (1, 2, 3, 8):
            spans = [env_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    assert env_range(1_048_576, 3, 8) == (393216, 524288)
    with pytest.raises(ValueError):
        env_range(10, 2, 2)


def _worker(rank, world, port, total, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from helpers import golden_case, po
    from beatsaberrl_b200.sharding import broadcast_weights, env_range, reduce_rollout_stats
    cfg, sd = golden_case("tiny_plain")
    # rank 1 starts from different weights; the broadcast must overwrite them
    holder = torch.nn.ParameterDict({k.replace(".", "_"): torch.nn.Parameter(v.clone() + rank) for k, v in sd.items()})
    broadcast_weights(holder, src=0)
    sd_r = {k: holder[k.replace(".", "_")].data for k in sd}
    obs = po.make_obs(total, 5, padded=True)
    act = po.make_actions(total, cfg, 6)
    a, b = env_range(total, rank, world)
    logits, value = po.forward_stacked(sd_r, cfg, obs[a:b])
    lp, ent, ent_h = po.evaluate_actions(logits, act[a:b])
    stats = reduce_rollout_stats(ent_h, lp, value)
    torch.save(stats, os.path.join(out_dir, f"stats{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_stats_match_single_process(tmp_path):
    from helpers import golden_case, po
    total, world = 37, 2
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, total, str(tmp_path)), nprocs=world, join=True)
    cfg, sd = golden_case("tiny_plain")
    obs = po.make_obs(total, 5, padded=True)
    act = po.make_actions(total, cfg, 6)
    logits, value = po.forward_stacked(sd, cfg, obs)
    lp, ent, ent_h = po.evaluate_actions(logits, act)
    for r in range(world):
        s = torch.load(tmp_path / f"stats{r}.pt")
        assert s["n_envs"] == total
        torch.testing.assert_close(s["ent_head_mean"], ent_h.mean(0), atol=1e-5, rtol=1e-5)
        assert abs(s["logprob_mean"] - float(lp.mean())) < 1e-4
        assert abs(s["value_mean"] - float(value.mean())) < 1e-5
