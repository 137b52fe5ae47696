"""The oracle's autograd gradients of the PPO-recompute call against gradient statistics generated from
the reference's own autograd (tests/golden/make_golden.py): this pins the gradient oracle that the GPU
backward is then compared with."""
import numpy as np
import pytest
import torch

from helpers import ROOT, golden_case, po

GRAD_CASES = {"tiny_plain": (48, 21), "tiny_geo_mixed": (40, 22), "cfg1": (64, 0),           # batch, obs seed of the case
              "tiny_options": (44, 23), "tiny_vres": (36, 24), "tiny_simbav2": (52, 25)}


def oracle_grads(cfg, sd, obs, act, up):
    """Gradients of sum(up . outputs) w.r.t. every parameter, by torch autograd through the oracle in fp32."""
    sd_g = {k: v.clone().requires_grad_(True) for k, v in sd.items()}
    with torch.enable_grad():
        logits, value, keep = po.forward_stacked.__wrapped__(sd_g, cfg, obs, want=True)
        lp, ent, _ = po.evaluate_actions.__wrapped__(logits, act)
        loss = (up["logprob"] * lp).sum() + (up["entropy"] * ent).sum() + (up["value"] * value).sum() \
            + (up["value_logits"] * keep["value_logits"]).sum()
        loss.backward()
    frozen = po.frozen_params(cfg)          # no gradient in the reference (requires_grad False)
    return {k: (v.grad if v.grad is not None and k not in frozen else torch.zeros_like(v)) for k, v in sd_g.items()}, float(loss)


def grad_inputs(name):
    cfg, sd = golden_case(name)
    B, oseed = GRAD_CASES[name]
    padded = name != "cfg1"
    obs = po.make_obs(B, oseed + 100, padded=padded)
    act = po.make_actions(B, cfg, oseed + 101)
    up = po.make_upstream(B, cfg, oseed + 102)
    return cfg, sd, obs, act, up


@pytest.mark.parametrize("name", sorted(GRAD_CASES))
def test_oracle_gradients_match_the_reference(name):
    gold = np.load(ROOT / "tests" / "golden" / "policy_grads_golden.npz")
    cfg, sd, obs, act, up = grad_inputs(name)
    grads, loss = oracle_grads(cfg, sd, obs, act, up)
    assert abs(loss - float(gold[f"{name}/loss"][0])) <= 1e-5 * max(1.0, abs(loss))
    keys = [k[len(name) + 6:] for k in gold.files if k.startswith(f"{name}/stat/")]
    assert sorted(keys) == sorted(sd.keys())
    # a few gradients are zero in exact arithmetic (the key bias: a shift of every score of a row) and come
    # out as rounding noise, so the floor of the tolerance is relative to the largest gradient of the model
    top = max(float(gold[f"{name}/stat/{k}"][0]) for k in keys)
    for k in keys:
        want = torch.from_numpy(gold[f"{name}/stat/{k}"])
        got = po.grad_stats(k, grads[k])
        assert float((got - want).abs().max()) <= 2e-4 * float(want[0]) + 1e-5 * top, (k, got, want)
