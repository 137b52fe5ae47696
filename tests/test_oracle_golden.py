"""The oracle restatement against vectors generated from the reference itself."""
import numpy as np
import pytest
import torch

from helpers import GOLDEN_CASES, golden_case, po


@pytest.mark.parametrize("name", sorted(GOLDEN_CASES))
def test_seeded_weights_match_reference_checksums(golden, name):
    cfg, sd = golden_case(name)
    names = [str(n) for n in golden[f"{name}/param_names"]]
    assert names == sorted(sd)
    sums = np.array([[float(sd[k].double().sum()), float(sd[k].double().abs().sum())] for k in names])
    np.testing.assert_allclose(sums, golden[f"{name}/param_sums"], rtol=1e-9, atol=1e-9)


@pytest.mark.parametrize("name", sorted(GOLDEN_CASES))
def test_forward_matches_reference(golden, name):
    cfg, sd = golden_case(name)
    obs = torch.from_numpy(golden[f"{name}/obs"])
    logits, value, keep = po.forward_stacked(sd, cfg, obs, want=True)
    ref = torch.from_numpy(golden[f"{name}/logits"])
    assert logits.shape == ref.shape
    # CPU BLAS summation order may differ between hosts: fp32 round-off only
    torch.testing.assert_close(logits, ref, atol=2e-5, rtol=1e-5)
    torch.testing.assert_close(value, torch.from_numpy(golden[f"{name}/value"]), atol=2e-5, rtol=1e-5)
    torch.testing.assert_close(keep["value_logits"], torch.from_numpy(golden[f"{name}/value_logits"]),
                               atol=5e-5, rtol=1e-5)


@pytest.mark.parametrize("name", sorted(GOLDEN_CASES))
def test_action_tail_matches_reference(golden, name):
    cfg, sd = golden_case(name)
    logits = torch.from_numpy(golden[f"{name}/logits"])
    act = torch.from_numpy(golden[f"{name}/actions"])
    lp, ent, ent_h = po.evaluate_actions(logits, act)
    torch.testing.assert_close(lp, torch.from_numpy(golden[f"{name}/logprob"]), atol=1e-5, rtol=1e-6)
    torch.testing.assert_close(ent, torch.from_numpy(golden[f"{name}/entropy"]), atol=1e-5, rtol=1e-6)
    torch.testing.assert_close(ent_h, torch.from_numpy(golden[f"{name}/ent_head"]), atol=1e-6, rtol=1e-6)


def test_lane_tables_match_reference(golden):
    for tok in ("saber_l", "saber_r", "torso", "leg_l", "leg_r"):
        assert po.token_lanes(tok) == golden[f"lanes/{tok}"].tolist()


def test_mixed_heads_are_masked(golden):
    logits = golden["tiny_geo_mixed/logits"]
    assert logits.shape[-1] == 7
    assert (logits[:, 0, 5:] < -1e8).all() and (logits[:, 8, :] > -1e8).all()


def test_mac_counts():
    # figures of the hot-path scope table (multiply-accumulates per env-forward)
    assert po.mac_per_env(po.named_config("cfg1")) == 9_791_104
    assert po.mac_per_env(po.named_config("cfg2")) == 84_832_512
    assert po.mac_per_env(po.named_config("cfg4")) == 520_229_376


def test_masked_slots_cannot_leak():
    """Junk in dead slots must not change the output (reference test_policy.py:42-63)."""
    cfg, sd = golden_case("tiny_plain")
    obs = po.make_obs(8, 3, padded=True)
    l0, v0 = po.forward_stacked(sd, cfg, obs)
    junk = obs.clone()
    mask = obs[:, po.OFF_MASK:po.OFF_MASK + po.N_SLOTS]
    notes = junk[:, po.OFF_NOTES:po.OFF_MASK].view(8, po.N_SLOTS, po.NOTE_FEAT)
    notes += (1.0 - mask)[:, :, None] * 37.0
    l1, v1 = po.forward_stacked(sd, cfg, junk)
    torch.testing.assert_close(l0, l1, atol=1e-5, rtol=0)
    torch.testing.assert_close(v0, v1, atol=1e-5, rtol=0)
