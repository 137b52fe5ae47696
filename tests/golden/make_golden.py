"""Generates tests/golden/policy_golden.npz from the REFERENCE implementation.

Run in a container that has the reference checkout (default: $BSRL_REFERENCE, else a `reference` directory
beside this repository):

    python tests/golden/make_golden.py [/path/to/reference]

For each case the reference ``NotePolicy`` (python/policy.py) is built on the CPU from a seed,
run in fp32 on a stored obs batch, and its outputs are stored: stacked logits, value, the value
bin logits, and log-prob / entropy / per-head entropy for stored actions, plus a float64
checksum of every parameter so a test can prove it rebuilt the same weights from the seed.
The reference cannot travel to the GPU box; these vectors can.
"""
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
from oracle import policy_oracle as po  # noqa: E402

CASES = [
    # name, config, note_geo, head_gears, xavier, weight seed, ln_jitter, B, padded, obs seed, options
    ("tiny_plain", "tiny", False, None, False, 11, 0.0, 16, True, 21, {}),
    ("tiny_geo_mixed", "tiny", True, (5,) * 8 + (7,) + (5,) * 6 + (7,) + (5,) * 13, True, 12, 0.1, 16, True, 22, {}),
    ("cfg1", "cfg1", False, None, False, 0, 0.0, 8, False, 0, {}),
    # the A/B options that change the forward: --emb-ln, --final-ln, --game flux (note-geo variant)
    ("tiny_options", "tiny", True, None, False, 13, 0.1, 16, True, 23,
     dict(emb_ln=True, final_ln=True, game="flux")),
    # --value-residual on a 3-block model (blocks 1 and 2 mix block 0's values in; (a, b) moved off (1, 0))
    ("tiny_vres", "tiny", False, None, False, 14, 0.1, 16, True, 24, dict(value_residual=True, n_blocks=3)),
    # --trunk-arch simbav2 (orthogonal, row-normalised trunk matrices; scalers moved off their init)
    ("tiny_simbav2", "tiny", False, None, False, 15, 0.1, 16, True, 25, dict(trunk_arch="simbav2")),
]


# cases that also get parameter gradients (name -> batch of the gradient run)
GRAD_CASES = {"tiny_plain": 48, "tiny_geo_mixed": 40, "cfg1": 64, "tiny_options": 44, "tiny_vres": 36, "tiny_simbav2": 52}


def case_config(cfg_name, geo, hg, opts=None):
    cfg = po.named_config(cfg_name)
    cfg.note_geo = geo
    cfg.head_gears = hg
    for k, v in (opts or {}).items():
        setattr(cfg, k, v)
    cfg.__post_init__()
    return cfg


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("BSRL_REFERENCE", str(Path(__file__).resolve().parents[3] / "reference"))
    sys.dont_write_bytecode = True
    sys.path.insert(0, os.path.join(ref, "python"))
    import policy as rp  # the reference module

    out = {}
    for name, cfg_name, geo, hg, xav, seed, jit, B, padded, oseed, opts in CASES:
        cfg = case_config(cfg_name, geo, hg, opts)
        torch.manual_seed(seed)
        m = rp.NotePolicy(**cfg.ref_kwargs()).eval()
        if xav:
            for mod in m.modules():
                if isinstance(mod, torch.nn.Linear):
                    torch.nn.init.xavier_uniform_(mod.weight)
                    torch.nn.init.zeros_(mod.bias)
        if jit > 0:   # same LayerNorm perturbation the oracle's build_state_dict applies
            sd = po.build_state_dict(cfg, seed, xavier=xav, ln_jitter=jit)
            m.load_state_dict({k: sd[k] for k in m.state_dict()})
        obs = po.make_obs(B, oseed, padded=padded)
        act = po.make_actions(B, cfg, oseed + 1)
        with torch.no_grad():
            logits, value = m.forward_stacked(obs)
            _, lp, ent, _ = m.get_action_and_value(obs, act)
            ent_h = m._ent_h
        with torch.enable_grad():
            m.forward_stacked(obs)
            vlogits = m._value_logits.detach()
        out[f"{name}/obs"] = obs.numpy()
        out[f"{name}/actions"] = act.numpy()
        out[f"{name}/logits"] = logits.numpy()
        out[f"{name}/value"] = value.numpy()
        out[f"{name}/value_logits"] = vlogits.numpy()
        out[f"{name}/logprob"] = lp.numpy()
        out[f"{name}/entropy"] = ent.numpy()
        out[f"{name}/ent_head"] = ent_h.numpy()
        names = sorted(m.state_dict())
        out[f"{name}/param_sums"] = np.array(
            [[float(m.state_dict()[k].double().sum()), float(m.state_dict()[k].double().abs().sum())]
             for k in names])
        out[f"{name}/param_names"] = np.array(names)
    # gradients of every parameter for the PPO-recompute call, from the reference's own autograd (fp32, CPU)
    grads = {}
    for name, cfg_name, geo, hg, xav, seed, jit, B, padded, oseed, opts in CASES:
        if name not in GRAD_CASES:
            continue
        cfg = case_config(cfg_name, geo, hg, opts)
        torch.manual_seed(seed)
        m = rp.NotePolicy(**cfg.ref_kwargs()).train()
        if jit > 0:
            sd = po.build_state_dict(cfg, seed, xavier=xav, ln_jitter=jit)
            m.load_state_dict({k: sd[k] for k in m.state_dict()})
        Bg = GRAD_CASES[name]
        obs = po.make_obs(Bg, oseed + 100, padded=padded)
        act = po.make_actions(Bg, cfg, oseed + 101)
        up = po.make_upstream(Bg, cfg, oseed + 102)
        with torch.enable_grad():
            _, lp, ent, val = m.get_action_and_value(obs, act)
            loss = (up["logprob"] * lp).sum() + (up["entropy"] * ent).sum() + (up["value"] * val).sum() \
                + (up["value_logits"] * m._value_logits).sum()
            loss.backward()
        for k, prm in m.named_parameters():
            g = prm.grad if prm.grad is not None else torch.zeros_like(prm)
            # norm and four fixed random projections of every gradient (po.grad_stats): enough to pin the
            # oracle's autograd to the reference's without storing megabytes of gradients
            grads[f"{name}/stat/{k}"] = po.grad_stats(k, g).numpy()
        grads[f"{name}/loss"] = np.array([float(loss)])
    np.savez_compressed(HERE / "policy_grads_golden.npz", **grads)
    print("wrote", HERE / "policy_grads_golden.npz", sum(v.nbytes for v in grads.values()), "bytes raw")
    # lane tables straight from the reference module
    out["lanes/saber_l"] = np.array(rp._SABER_L_IDX)
    out["lanes/saber_r"] = np.array(rp._SABER_R_IDX)
    out["lanes/torso"] = np.array(rp._TORSO_IDX)
    out["lanes/leg_l"] = np.array(rp._LEG_L_IDX)
    out["lanes/leg_r"] = np.array(rp._LEG_R_IDX)
    np.savez_compressed(HERE / "policy_golden.npz", **out)
    print("wrote", HERE / "policy_golden.npz", sum(v.nbytes for v in out.values()), "bytes raw")


if __name__ == "__main__":
    main()
