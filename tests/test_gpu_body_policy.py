"""The single-body-token layout on the GPU (BodyObjectPolicy -> C ABI) against its oracle and the vectors
generated from the reference's Block modules; same parity gates as the reference layout."""
import pytest
import torch

from helpers import assert_parity, po
from oracle import body_policy_oracle as bo
from test_body_policy_oracle import GCASES, gcase

pytestmark = pytest.mark.gpu


def cuda_body_policy(cfg, sd):
    from beatsaberrl_b200.body_policy import BodyObjectPolicy
    m = BodyObjectPolicy(**cfg.kwargs())
    m.load_state_dict(sd)
    return m.cuda()


@pytest.mark.parametrize("name", sorted(GCASES))
def test_golden_vectors(name):
    import numpy as np
    from helpers import ROOT
    gold = np.load(ROOT / "tests" / "golden" / "body_policy_golden.npz")
    cfg, sd = gcase(name)
    m = cuda_body_policy(cfg, sd)
    obs = torch.from_numpy(gold[f"{name}/obs"]).cuda()
    logits, value = m.forward_stacked(obs)
    assert logits.shape == (obs.shape[0], 29, cfg.n_gears)
    assert_parity(logits, value, torch.from_numpy(gold[f"{name}/logits"]), torch.from_numpy(gold[f"{name}/value"]), argmax_min=0.99)
    act = torch.from_numpy(gold[f"{name}/actions"]).cuda()
    for a in (act, act.to(torch.int32), act.to(torch.uint8)):
        _, lp, ent, v2 = m.get_action_and_value(obs, a)
        torch.testing.assert_close(lp.cpu(), torch.from_numpy(gold[f"{name}/logprob"]), atol=5e-2, rtol=1e-2)
        torch.testing.assert_close(ent.cpu(), torch.from_numpy(gold[f"{name}/entropy"]), atol=5e-2, rtol=1e-2)
        assert torch.equal(v2, value)
        torch.testing.assert_close(ent, m._ent_h.sum(-1), atol=1e-4, rtol=1e-5)


@pytest.mark.parametrize("name,seed,xavier,B,padded", [
    ("cfg1", 0, False, 1024, False),       # T = 17, d = 128
    ("cfg2", 1, True, 1024, False),        # T = 33, d = 256, Xavier init seed 1: fused GELU block tail
    ("cfg2", 1, True, 768, True),          # absent objects zeroed and masked
    ("cfg4", 3, False, 128, True),         # T = 65, d = 512, head_dim 64, 7 gears: the unfused kernels
])
def test_parity_gates(name, seed, xavier, B, padded):
    cfg = bo.named_config(name)
    sd = bo.build_state_dict(cfg, seed, xavier=xavier)
    m = cuda_body_policy(cfg, sd)
    obs = bo.make_obs(B, cfg, seed + 2, padded=padded)
    ref_l, ref_v = bo.forward(sd, cfg, obs)
    logits, value = m.forward_stacked(obs.cuda())
    rep = assert_parity(logits, value, ref_l, ref_v, argmax_min=0.998 if B < 512 else 0.999)
    print(name, rep)
    act = bo.make_actions(B, cfg, 4).cuda()
    _, lp, ent, _ = m.get_action_and_value(obs.cuda(), act)
    rlp, rent, _ = po.evaluate_actions(ref_l, act.cpu())
    torch.testing.assert_close(lp.cpu(), rlp, atol=29 * 2e-2, rtol=1e-2)
    torch.testing.assert_close(ent.cpu(), rent, atol=5e-2, rtol=1e-2)


@pytest.mark.parametrize("B", [1, 3, 127, 129, 500])
def test_ragged_batches_and_batch_invariance(B):
    cfg, sd = gcase("gtiny")
    m = cuda_body_policy(cfg, sd)
    obs = bo.make_obs(500, cfg, 9, padded=True)
    full_l, full_v = m.forward_stacked(obs.cuda())
    l, v = m.forward_stacked(obs[:B].cuda())
    assert torch.equal(l, full_l[:B]) and torch.equal(v, full_v[:B])


def test_all_objects_absent_and_junk_cannot_leak():
    cfg, sd = gcase("gtiny_xavier")
    m = cuda_body_policy(cfg, sd)
    obs = bo.make_obs(64, cfg, 5)
    obs[:, -cfg.n_obj:] = 0.0                      # every object absent: the body token attends to itself only
    l0, v0 = m.forward_stacked(obs.cuda())
    assert torch.isfinite(l0).all() and torch.isfinite(v0).all()
    ref_l, ref_v = bo.forward(sd, cfg, obs)
    assert_parity(l0, v0, ref_l, ref_v, argmax_min=0.995)
    junk = obs.clone()
    junk[:, cfg.body_dim: cfg.body_dim + cfg.n_obj * cfg.obj_dim] = 33.0
    l1, v1 = m.forward_stacked(junk.cuda())
    torch.testing.assert_close(l0, l1, atol=1e-5, rtol=0)
    torch.testing.assert_close(v0, v1, atol=1e-5, rtol=0)


def test_in_place_weight_refresh():
    from beatsaberrl_b200.policy import bump_weights_version
    cfg, sd = gcase("gtiny")
    m = cuda_body_policy(cfg, sd)
    obs = bo.make_obs(32, cfg, 1).cuda()
    l0, _ = m.forward_stacked(obs)
    ptr = m._arena.data_ptr()
    with torch.no_grad():
        m.heads.weight.mul_(2.0)
        m.heads.bias.mul_(2.0)
    bump_weights_version()
    l1, _ = m.forward_stacked(obs)
    assert m._arena.data_ptr() == ptr
    torch.testing.assert_close(l1, 2 * l0, atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("B", [1, 5, 131, 700])
def test_fused_attention_path_batch_invariance_and_masking(B):
    """33 tokens, head_dim 32: the fused projection + attention kernel.  An env's result does not depend on its
    position or on the batch size (bit for bit), and absent objects' lanes cannot leak."""
    cfg = bo.named_config("cfg2")
    sd = bo.build_state_dict(cfg, 7, xavier=True)
    m = cuda_body_policy(cfg, sd)
    obs = bo.make_obs(700, cfg, 11, padded=True)
    full_l, full_v = m.forward_stacked(obs.cuda())
    l, v = m.forward_stacked(obs[:B].cuda())
    assert torch.equal(l, full_l[:B]) and torch.equal(v, full_v[:B])
    junk = obs[:B].clone()
    live = junk[:, -cfg.n_obj:]
    objs = junk[:, cfg.body_dim: cfg.body_dim + cfg.n_obj * cfg.obj_dim].view(B, cfg.n_obj, cfg.obj_dim)
    objs += (1.0 - live)[:, :, None] * 29.0
    l2, v2 = m.forward_stacked(junk.cuda())
    torch.testing.assert_close(l2, l, atol=1e-5, rtol=0)
    torch.testing.assert_close(v2, v, atol=1e-5, rtol=0)


def test_full_size_properties():
    """65,536 envs of the 33-token configuration: finite outputs, rows re-ordered -> outputs re-ordered bit for bit,
    and a sample of 512 envs spread over the batch within the gates of the oracle."""
    cfg = bo.named_config("cfg2")
    sd = bo.build_state_dict(cfg, 1, xavier=True)
    m = cuda_body_policy(cfg, sd)
    B = 65536
    obs = bo.make_obs(B, cfg, 3, padded=True).cuda()
    logits, value = m.forward_stacked(obs)
    assert torch.isfinite(logits).all() and torch.isfinite(value).all()
    perm = torch.randperm(B, device="cuda", generator=torch.Generator(device="cuda").manual_seed(0))
    l2, v2 = m.forward_stacked(obs[perm].contiguous())
    assert torch.equal(l2, logits[perm]) and torch.equal(v2, value[perm])
    idx = torch.arange(0, B, 128, device="cuda")
    ref_l, ref_v = bo.forward(sd, cfg, obs[idx].cpu())
    assert_parity(logits[idx], value[idx], ref_l, ref_v, argmax_min=0.998)
