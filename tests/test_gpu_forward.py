"""Whole-forward parity of the CUDA path (through the NotePolicy facade -> C ABI) against the
oracle and the reference-generated golden vectors."""
import pytest
import torch

from helpers import GOLDEN_CASES, assert_parity, cuda_policy, golden_case, make_cfg, po

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", sorted(GOLDEN_CASES))
def test_golden_vectors(golden, name):
    cfg, sd = golden_case(name)
    m = cuda_policy(cfg, sd)
    obs = torch.from_numpy(golden[f"{name}/obs"]).cuda()
    m.keep_value_logits = True
    logits, value = m.forward_stacked(obs)
    assert logits.shape == (obs.shape[0], 29, cfg.k_max) and logits.dtype is torch.float32
    ref_l = torch.from_numpy(golden[f"{name}/logits"])
    ref_v = torch.from_numpy(golden[f"{name}/value"])
    assert_parity(logits, value, ref_l, ref_v, argmax_min=0.99)   # few heads: one near-tie may flip
    dead = ref_l < -1e8
    assert torch.equal(logits.cpu()[dead], ref_l[dead])            # masked lanes are exactly -1e9
    torch.testing.assert_close(m._value_logits.cpu(), torch.from_numpy(golden[f"{name}/value_logits"]),
                               atol=3e-2, rtol=1e-2)
    act = torch.from_numpy(golden[f"{name}/actions"]).cuda()
    for a in (act, act.to(torch.uint8), act.long()):
        a2, lp, ent, v2 = m.get_action_and_value(obs, a)
        # 29 summed log-probs: 29 x the per-logit tolerance is the bound, observed far smaller
        torch.testing.assert_close(lp.cpu(), torch.from_numpy(golden[f"{name}/logprob"]), atol=5e-2, rtol=1e-2)
        torch.testing.assert_close(ent.cpu(), torch.from_numpy(golden[f"{name}/entropy"]), atol=5e-2, rtol=1e-2)
        torch.testing.assert_close(m._ent_h.cpu(), torch.from_numpy(golden[f"{name}/ent_head"]), atol=5e-3, rtol=1e-2)
        torch.testing.assert_close(v2, value, atol=0, rtol=0)
        torch.testing.assert_close(ent, m._ent_h.sum(-1), atol=1e-4, rtol=1e-5)


@pytest.mark.parametrize("name,geo,xavier,seed,B,padded", [
    ("cfg1", False, False, 0, 1024, False),      # the CPU-reference configuration, whole
    ("cfg2", False, True, 1, 2048, False),       # single-GPU rollout model, Xavier seed 1
    ("cfg2", False, True, 1, 16384, False),      # the same on 16,384 envs: the argmax gate on 475 K head decisions
    ("cfg2", False, True, 1, 1536, True),        # padded objects: masked attention path
    ("recipe", True, False, 5, 512, True),       # the reference's production shape (head_dim 48, geo)
    ("cfg4", False, False, 3, 256, False),       # wide policy, 7 gears
])
def test_parity_gates(name, geo, xavier, seed, B, padded):
    cfg = make_cfg(name, geo)
    sd = po.build_state_dict(cfg, seed, xavier=xavier)
    m = cuda_policy(cfg, sd)
    obs = po.make_obs(B, seed + (2 if padded else 0), padded=padded)
    ref_l, ref_v = po.forward_stacked(sd, cfg, obs)
    logits, value = m.forward_stacked(obs.cuda())
    rep = assert_parity(logits, value, ref_l, ref_v)
    print(name, rep)
    act = po.make_actions(B, cfg, 4).cuda()
    _, lp, ent, _ = m.get_action_and_value(obs.cuda(), act)
    rlp, rent, _ = po.evaluate_actions(ref_l, act.cpu())
    torch.testing.assert_close(lp.cpu(), rlp, atol=29 * 2e-2, rtol=1e-2)
    torch.testing.assert_close(ent.cpu(), rent, atol=5e-2, rtol=1e-2)


@pytest.mark.parametrize("B", [1, 3, 127, 129, 1000])
def test_ragged_batches_and_batch_invariance(B):
    cfg, sd = golden_case("tiny_geo_mixed")
    m = cuda_policy(cfg, sd)
    obs = po.make_obs(1000, 31, padded=True)
    full_l, full_v = m.forward_stacked(obs.cuda())
    l, v = m.forward_stacked(obs[:B].cuda())
    # an env's result does not depend on the batch around it (reference test_attn29.py:128-140)
    assert torch.equal(l, full_l[:B]) and torch.equal(v, full_v[:B])
    ref_l, ref_v = po.forward_stacked(sd, cfg, obs[:B])
    assert_parity(l, v, ref_l, ref_v, argmax_min=0.99 if B < 100 else 0.998)


def test_all_slots_masked_and_all_live():
    cfg, sd = golden_case("tiny_plain")
    m = cuda_policy(cfg, sd)
    obs = po.make_obs(64, 8)
    dead = obs.clone()
    dead[:, po.OFF_MASK:po.OFF_MASK + 24] = 0.0
    for o in (obs, dead):
        l, v = m.forward_stacked(o.cuda())
        assert torch.isfinite(l).all() and torch.isfinite(v).all()
        ref_l, ref_v = po.forward_stacked(sd, cfg, o)
        assert_parity(l, v, ref_l, ref_v, argmax_min=0.995)
    # junk in masked slots cannot leak (reference test_policy.py:42-63)
    junk = dead.clone()
    junk[:, po.OFF_NOTES:po.OFF_MASK] = 55.0
    l2, v2 = m.forward_stacked(junk.cuda())
    l1, v1 = m.forward_stacked(dead.cuda())
    torch.testing.assert_close(l1, l2, atol=1e-5, rtol=0)
    torch.testing.assert_close(v1, v2, atol=1e-5, rtol=0)


def test_weight_refresh_in_place_and_sampling():
    from beatsaberrl_b200.policy import bump_weights_version
    cfg, sd = golden_case("tiny_plain")
    m = cuda_policy(cfg, sd)
    obs = po.make_obs(256, 3).cuda()
    l0, _ = m.forward_stacked(obs)
    ptr = m._arena.data_ptr()
    with torch.no_grad():
        for p in m.heads.parameters():
            p.mul_(2.0)
    bump_weights_version()
    l1, _ = m.forward_stacked(obs)
    assert m._arena.data_ptr() == ptr                    # refreshed in place
    torch.testing.assert_close(l1, 2 * l0, atol=1e-2, rtol=1e-2)
    m.seed_sampler(0)
    a, lp, ent, v = m.get_action_and_value(obs)          # sampled actions
    assert a.shape == (256, 29) and a.dtype is torch.int64 and int(a.max()) < cfg.k_max
    _, lp2, ent2, _ = m.get_action_and_value(obs, a)
    torch.testing.assert_close(lp, lp2, atol=1e-4, rtol=1e-5)
    torch.testing.assert_close(ent, ent2, atol=1e-4, rtol=1e-5)


def test_cuda_graph_capture_replays():
    """The forward allocates nothing between replays and never syncs, so it can be captured the
    way the reference's graph drivers do (python/cuda_graphs.py:22-68)."""
    cfg, sd = golden_case("tiny_plain")
    m = cuda_policy(cfg, sd)
    m.flatten_fp16()
    static_obs = po.make_obs(128, 1).cuda()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):
            m.forward_stacked(static_obs)
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        gl, gv = m.forward_stacked(static_obs)
    new = po.make_obs(128, 2).cuda()
    static_obs.copy_(new)
    g.replay()
    el, ev = m.forward_stacked(new)
    assert torch.equal(gl, el) and torch.equal(gv, ev)


def test_fused_sampling_distribution_and_determinism():
    """Actions drawn inside the head kernel (Gumbel-max, Philox): same seed and counter -> same
    draw; a new counter -> a new draw; frequencies follow softmax(logits); lanes past a head's gear
    count are never drawn; the returned log-prob is the log-prob of the drawn actions."""
    cfg, sd = golden_case("tiny_geo_mixed")          # heads 8 and 15 have 7 gears, the rest 5
    m = cuda_policy(cfg, sd)
    one = po.make_obs(1, 5, padded=True)
    obs = one.repeat(20000, 1).cuda()                 # same env 20,000 times: i.i.d. draws of one distribution
    m.seed_sampler(1234)
    a1, lp1, ent1, v1 = m.get_action_and_value(obs)
    a2, lp2, _, _ = m.get_action_and_value(obs)       # counter advanced
    m.seed_sampler(1234)
    a3, lp3, _, _ = m.get_action_and_value(obs)
    assert torch.equal(a1, a3) and torch.equal(lp1, lp3)
    assert not torch.equal(a1, a2)
    assert a1.dtype is torch.int64 and a1.shape == (20000, 29)
    gears = torch.tensor(cfg.head_gears, device="cuda")
    assert bool((a1 < gears[None, :]).all()) and bool((a1 >= 0).all())
    logits, _ = m.forward_stacked(obs[:1])
    probs = torch.softmax(logits[0], -1)              # (29, k_max); masked lanes -> 0
    freq = torch.stack([(a1 == k).float().mean(0) for k in range(cfg.k_max)], -1)
    # 20,000 draws: standard error of a frequency <= 0.0036; 5 sigma
    assert float((freq - probs).abs().max()) < 0.018
    _, lp_given, ent_given, _ = m.get_action_and_value(obs, a1)
    torch.testing.assert_close(lp1, lp_given, atol=1e-5, rtol=1e-6)
    torch.testing.assert_close(ent1, ent_given, atol=1e-5, rtol=1e-6)


@pytest.mark.parametrize("name,geo,B", [("cfg1", True, 300),      # fused kernels (head_dim 32)
                                        ("recipe", True, 200),    # fused, head_dim 48
                                        ("cfg4", False, 96)])     # separate GEMM / LayerNorm / attention kernels
def test_constructor_options(name, geo, B):
    """--emb-ln, --final-ln, --value-residual and the Flux note-geo variant (python/policy.py:962, :969, :512-520, :357-360) on
    every kernel path, against the oracle (which the options golden case pins to the reference)."""
    cfg = make_cfg(name, geo, opts=dict(emb_ln=True, final_ln=True, game="flux", value_residual=True))
    sd = po.build_state_dict(cfg, 17, ln_jitter=0.1)
    m = cuda_policy(cfg, sd)
    obs = po.make_obs(B, 31, padded=True)
    ref_l, ref_v = po.forward_stacked(sd, cfg, obs)
    logits, value = m.forward_stacked(obs.cuda())
    assert_parity(logits, value, ref_l, ref_v, argmax_min=0.995)   # few heads at these batch sizes
    # the options really are in the path: switching them off changes the output
    plain = make_cfg(name, geo)
    l0, _ = cuda_policy(plain, {k: v for k, v in sd.items() if not k.startswith(("emb_ln", "final_ln")) and "vres_" not in k}).forward_stacked(obs.cuda())
    assert (l0 - logits).abs().max() > 1e-2


def test_simbav2_trunk():
    """--trunk-arch simbav2 (python/policy.py:1140-1155) at a production-like width, against the oracle
    (pinned to the reference by the golden case tiny_simbav2); the facade's seeded init equals the oracle's."""
    cfg = make_cfg("recipe", True, opts=dict(trunk_arch="simbav2"))
    sd = po.build_state_dict(cfg, 19, ln_jitter=0.1)
    m = cuda_policy(cfg, sd)
    obs = po.make_obs(400, 33, padded=True)
    ref_l, ref_v = po.forward_stacked(sd, cfg, obs)
    logits, value = m.forward_stacked(obs.cuda())
    assert_parity(logits, value, ref_l, ref_v, argmax_min=0.995)
    from beatsaberrl_b200.policy import NotePolicy
    torch.manual_seed(19)
    fresh = NotePolicy(**cfg.ref_kwargs()).state_dict()
    plain = po.build_state_dict(cfg, 19)
    for k in ("trunk_in.weight", "trunk_w2.weight", "trunk_s_1", "trunk_alpha", "heads.0.weight"):
        assert torch.equal(fresh[k], plain[k]), k


def test_rollout_step_writes_buffer_rows():
    """The fused rollout tick draws the same actions as get_action_and_value under the same seed and
    counter, and its buffer rows are what the reference's loop body stores: uint8 actions, log-prob,
    value * ret_sig + ret_mu, the fp16 obs row (python/train_batch.py:2299-2350)."""
    cfg, sd = golden_case("tiny_geo_mixed")
    m = cuda_policy(cfg, sd)
    B, T = 777, 3
    obs = po.make_obs(B, 7, padded=True).cuda()
    b_act = torch.zeros(T, B, 29, dtype=torch.uint8, device="cuda")
    b_logp = torch.zeros(T, B, device="cuda")
    b_val = torch.zeros(T + 1, B, device="cuda")
    b_obs = torch.zeros(T, B, 630, dtype=torch.float16, device="cuda")
    ret_sig = torch.tensor(2.5, device="cuda")
    ret_mu = torch.tensor(-0.75, device="cuda")
    m.seed_sampler(99)
    a_ref, lp_ref, ent_ref, v_ref = m.get_action_and_value(obs)
    m.seed_sampler(99)
    t = 1
    a, lp, ent, v = m.rollout_step(obs, b_act[t], b_logp[t], b_val[t], b_obs[t], ret_sig, ret_mu, need_entropy=True)
    assert torch.equal(a, a_ref) and torch.equal(lp, lp_ref) and torch.equal(v, v_ref) and torch.equal(ent, ent_ref)
    assert torch.equal(b_act[t].long(), a) and torch.equal(b_logp[t], lp)
    torch.testing.assert_close(b_val[t], v * 2.5 - 0.75, atol=1e-6, rtol=1e-6)
    assert torch.equal(b_obs[t], obs.half())
    # the other rows are untouched; all outputs optional
    assert not b_act[0].any() and not b_act[2].any() and not b_val[0].any() and not b_obs[2].any()
    a2, lp2, ent2, v2 = m.rollout_step(obs)
    assert ent2 is None and a2.shape == (B, 29) and not torch.equal(a2, a)
    with pytest.raises(ValueError):
        m.rollout_step(obs, b_act=b_act[t].int())


def test_full_size_properties():
    """At the padded-objects size (131,072 envs, uniform 0..24 live slots): outputs finite, an
    env's result independent of its position in the batch (rows re-ordered -> outputs re-ordered,
    bit for bit), junk in masked slots changes nothing, and a sample agrees with the oracle."""
    cfg = make_cfg("cfg2")
    sd = po.build_state_dict(cfg, 1, xavier=True)
    m = cuda_policy(cfg, sd)
    B = 131072
    obs = po.make_obs(B, 2, padded=True).cuda()
    logits, value = m.forward_stacked(obs)
    assert torch.isfinite(logits).all() and torch.isfinite(value).all()
    perm = torch.randperm(B, device="cuda", generator=torch.Generator(device="cuda").manual_seed(0))
    l2, v2 = m.forward_stacked(obs[perm].contiguous())
    assert torch.equal(l2, logits[perm]) and torch.equal(v2, value[perm])
    junk = obs.clone()
    mask = junk[:, po.OFF_MASK:po.OFF_MASK + 24]
    notes = junk[:, po.OFF_NOTES:po.OFF_MASK].view(B, 24, 18)
    notes += (1.0 - mask)[:, :, None] * 41.0
    l3, v3 = m.forward_stacked(junk)
    torch.testing.assert_close(l3, logits, atol=1e-5, rtol=0)
    torch.testing.assert_close(v3, value, atol=1e-5, rtol=0)
    idx = torch.arange(0, B, 128, device="cuda")      # 1,024 envs spread over the batch
    ref_l, ref_v = po.forward_stacked(sd, cfg, obs[idx].cpu())
    assert_parity(logits[idx], value[idx], ref_l, ref_v, argmax_min=0.998)
