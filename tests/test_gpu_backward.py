"""Backward of the PPO-recompute call on the GPU (bsrl_forward_train + bsrl_backward behind the facade's
autograd node) against the oracle's autograd in fp32 -- itself pinned to the reference's gradients by
tests/test_oracle_grads.py."""
import pytest
import torch

from helpers import cuda_policy, golden_case, make_cfg, po
from test_oracle_grads import GRAD_CASES, grad_inputs, oracle_grads

pytestmark = pytest.mark.gpu

# Relative error (L2, per parameter tensor) against fp32 autograd.  The arithmetic itself agrees to a few 1e-3
# (the single-stage tests below hold every backward kernel to that); what dominates end to end is ReLU sign
# flips: a pre-activation within fp16-operand rounding (~1e-3 relative) of zero lands on the other side of
# the ReLU than in fp32, and that unit's gradient for that row is then off by 100 %.  A fraction f of flipped
# units gives an L2 error of sqrt(f): ~1-1.5 % per ReLU layer crossed was measured, and a gradient crosses up
# to five of them.  Measured worst cases: 3 % on the actor side and 4.7 % on the critic side (two ReLUs of its
# own MLP on top) at d = 128 / 256, up to 7 % on the d = 64 models.  The reference holds its own fp16 stream
# to 2e-2 Frobenius against its fp32 path at d = 192 and otherwise judges a kernel against the unfused fp16
# path's own error (python/tests/test_fused_ffn.py:160-173, :289-307).
REL_TOL = {"tiny": 8e-2, "wide": 6e-2}
COS_MIN = {"tiny": 0.996, "wide": 0.998}


def _loss(m, obs, act, up):
    _, lp, ent, val = m.get_action_and_value(obs, act)
    return ((up["logprob"].cuda() * lp).sum() + (up["entropy"].cuda() * ent).sum() + (up["value"].cuda() * val).sum()
            + (up["value_logits"].cuda() * m._value_logits).sum())


def _check_grads(m, ref, tag, tol="tiny"):
    top = max(float(g.norm()) for g in ref.values())
    bad = []
    for k, p in m.named_parameters():
        if not p.requires_grad and p.grad is None:                 # frozen (the SimBaV2 trunk's biases, as in the reference)
            continue
        assert p.grad is not None, k
        g, r = p.grad.float().cpu(), ref[k]
        err = float((g - r).norm())
        cos = float((g * r).sum() / (g.norm() * r.norm() + 1e-30))
        if float(r.norm()) < 2e-3 * top:                          # (near-)zero gradients such as the key bias: noise only
            ok = err <= 2e-3 * top
        else:
            ok = err <= REL_TOL[tol] * float(r.norm()) and cos >= COS_MIN[tol]
        if not ok:
            bad.append((k, err, float(r.norm()), cos))
    assert not bad, (tag, bad[:8])


@pytest.mark.parametrize("name", sorted(GRAD_CASES))
def test_gradients_of_every_parameter(name):
    cfg, sd, obs, act, up = grad_inputs(name)
    ref, ref_loss = oracle_grads(cfg, sd, obs, act, up)
    m = cuda_policy(cfg, sd)
    with torch.enable_grad():
        loss = _loss(m, obs.cuda(), act.cuda(), up)
        loss.backward()
    assert abs(float(loss) - ref_loss) <= 2e-2 * max(abs(ref_loss), 1e-3)
    m.check_device()
    _check_grads(m, ref, name, "wide" if name == "cfg1" else "tiny")


def test_rollout_and_recompute_forwards_are_bitwise_identical():
    """What the rollout stored and what the update recomputes must be the same numbers, or the PPO ratio
    starts off 1 (the reference's r1 diagnostic, python/train_batch.py:2669-2741)."""
    cfg, sd = golden_case("tiny_geo_mixed")
    m = cuda_policy(cfg, sd)
    obs = po.make_obs(300, 5, padded=True).cuda()
    act = po.make_actions(300, cfg, 6).cuda()
    with torch.no_grad():
        _, lp0, ent0, v0 = m.get_action_and_value(obs, act)
        l0, _ = m.forward_stacked(obs)
    with torch.enable_grad():
        _, lp1, ent1, v1 = m.get_action_and_value(obs, act)
        assert lp1.requires_grad and v1.requires_grad and m._value_logits.requires_grad
        l1, v2 = m.forward_stacked(obs)
        assert l1.requires_grad
    assert torch.equal(lp0, lp1) and torch.equal(ent0, ent1) and torch.equal(v0, v1)
    assert torch.equal(l0, l1) and torch.equal(v0, v2)


def test_cfg2_shape_gradients_and_frozen_parameters():
    """d = 256 / 8 heads (the fused tcgen05 kernels going forward, split-K weight gradients coming back), a
    frozen parameter, and gradient accumulation over two backward calls."""
    cfg = make_cfg("cfg2")
    cfg.n_blocks = 2
    cfg.__post_init__()
    sd = po.build_state_dict(cfg, 1, xavier=True)
    B = 96
    obs, act, up = po.make_obs(B, 9, padded=True), po.make_actions(B, cfg, 10), po.make_upstream(B, cfg, 11)
    ref, _ = oracle_grads(cfg, sd, obs, act, up)
    m = cuda_policy(cfg, sd)
    m.trunk_fc1.weight.requires_grad_(False)
    with torch.enable_grad():
        _loss(m, obs.cuda(), act.cuda(), up).backward()
        assert m.trunk_fc1.weight.grad is None
        g1 = m.blocks[0].ffn[0].weight.grad.clone()
        _loss(m, obs.cuda(), act.cuda(), up).backward()
    torch.testing.assert_close(m.blocks[0].ffn[0].weight.grad, 2 * g1, rtol=1e-3, atol=1e-7)
    for p in m.parameters():
        if p.grad is not None:
            p.grad.mul_(0.5)
    m.trunk_fc1.weight.grad = ref["trunk_fc1.weight"].cuda()
    _check_grads(m, ref, "cfg2-2blocks", "wide")


def test_recipe_shape_gradients():
    """The reference's production shape (d = 192, four heads of 48, note geometry features), two blocks: the
    head_dim-48 attention backward and 192 / 384 / 768-wide weight gradients against the gradient oracle."""
    cfg = make_cfg("recipe", True)
    cfg.n_blocks = 2
    cfg.__post_init__()
    sd = po.build_state_dict(cfg, 5)
    B = 80
    obs, act, up = po.make_obs(B, 12, padded=True), po.make_actions(B, cfg, 13), po.make_upstream(B, cfg, 14)
    ref, ref_loss = oracle_grads(cfg, sd, obs, act, up)
    m = cuda_policy(cfg, sd)
    with torch.enable_grad():
        loss = _loss(m, obs.cuda(), act.cuda(), up)
        loss.backward()
    assert abs(float(loss) - ref_loss) <= 2e-2 * max(abs(ref_loss), 1e-3)
    m.check_device()
    _check_grads(m, ref, "recipe-2blocks", "wide")


def test_wide_policy_shape_gradients():
    """The wide policy's widths (d = 512, eight heads of 64, 7 gears), two blocks: the streamed fused attention and the
    projection + LayerNorm kernel going forward, head_dim-64 attention backward and 512 / 2048-wide weight gradients
    coming back, against the gradient oracle."""
    cfg = make_cfg("cfg4")
    cfg.n_blocks = 2
    cfg.__post_init__()
    sd = po.build_state_dict(cfg, 3)
    B = 72
    obs, act, up = po.make_obs(B, 15, padded=True), po.make_actions(B, cfg, 16), po.make_upstream(B, cfg, 17)
    ref, ref_loss = oracle_grads(cfg, sd, obs, act, up)
    m = cuda_policy(cfg, sd)
    with torch.enable_grad():
        loss = _loss(m, obs.cuda(), act.cuda(), up)
        loss.backward()
    assert abs(float(loss) - ref_loss) <= 2e-2 * max(abs(ref_loss), 1e-3)
    m.check_device()
    _check_grads(m, ref, "cfg4-2blocks", "wide")


# ---- single stages: every backward kernel against torch autograd on identical inputs (no ReLU sign can
# flip here, so the tolerances are those of fp16 operands with fp32 accumulation)
import ctypes as C

import torch.nn.functional as F


def _st():
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("rows,d", [(1, 64), (77, 128), (1000, 256), (130, 512)])
def test_layernorm_bwd_stage(native, rows, d):
    g = torch.Generator().manual_seed(rows + d)
    x = (torch.randn(rows, d, generator=g) * 2 + 0.3).requires_grad_(True)
    w = (1 + 0.1 * torch.randn(d, generator=g)).requires_grad_(True)
    b = (0.1 * torch.randn(d, generator=g)).requires_grad_(True)
    gy, gres = torch.randn(rows, d, generator=g), torch.randn(rows, d, generator=g)
    with torch.enable_grad():
        F.layer_norm(x, (d,), w, b, 1e-5).backward(gy)
    xd, wd, gyd, gresd = x.detach().cuda(), w.detach().cuda(), gy.cuda(), gres.cuda()
    gx, gw, gb = torch.empty(rows, d, device="cuda"), torch.zeros(d, device="cuda"), torch.zeros(d, device="cuda")
    native.check(native.lib.bsrl_layernorm_bwd(xd.data_ptr(), wd.data_ptr(), 1e-5, gyd.data_ptr(), gresd.data_ptr(), rows, d,
                                               gx.data_ptr(), gw.data_ptr(), gb.data_ptr(), _st()))
    torch.testing.assert_close(gx.cpu(), x.grad + gres, atol=2e-5, rtol=1e-4)
    torch.testing.assert_close(gw.cpu(), w.grad, atol=1e-4 * rows ** 0.5, rtol=1e-4)
    torch.testing.assert_close(gb.cpu(), b.grad, atol=1e-4 * rows ** 0.5, rtol=1e-4)


@pytest.mark.parametrize("B,d,H,q_first,n_q", [(3, 64, 2, 0, 29), (50, 256, 8, 0, 29), (40, 128, 4, 0, 5), (33, 256, 8, 2, 1),
                                               (17, 192, 4, 0, 29), (9, 512, 8, 0, 5)])
def test_attention_bwd_stage(native, B, d, H, q_first, n_q):
    g = torch.Generator().manual_seed(B + d + n_q)
    qkv = (torch.randn(B * 29, 3 * d, generator=g) * 0.7).half()
    n_live = torch.randint(0, 25, (B,), generator=g)
    kb = torch.zeros(B, 29)
    kb[:, 5:] = ((torch.arange(24)[None, :] < n_live[:, None]).float() - 1.0) * 16384.0
    go = (torch.randn(B * n_q, d, generator=g) * 0.5).half()
    qf = qkv.float().view(B, 29, 3 * d).requires_grad_(True)
    with torch.enable_grad():
        q, k, v = qf.split(d, -1)
        out = po.attention(q[:, q_first:q_first + n_q], k, v, kb, H)
        out.backward(go.float().view(B, n_q, d))
    gq = torch.empty(B * n_q, d, dtype=torch.float16, device="cuda")
    gkv = torch.empty(B * 29, 2 * d, dtype=torch.float16, device="cuda")
    qd, kbd, god = qkv.cuda(), kb.cuda(), go.cuda()
    native.check(native.lib.bsrl_attention_bwd(qd.data_ptr(), kbd.data_ptr(), B, d, H, q_first, n_q, god.data_ptr(),
                                               gq.data_ptr(), gkv.data_ptr(), _st()))
    ref = qf.grad
    torch.testing.assert_close(gq.float().cpu().view(B, n_q, d), ref[:, q_first:q_first + n_q, :d], atol=4e-3, rtol=4e-3)
    torch.testing.assert_close(gkv.float().cpu().view(B, 29, 2 * d), ref[:, :, d:], atol=4e-3, rtol=4e-3)


@pytest.mark.parametrize("case,B", [("tiny_plain", 130), ("tiny_geo_mixed", 45)])
def test_head_tail_bwd_stage(native, case, B):
    cfg, sd = golden_case(case)
    c = native.make_config(cfg.embed, cfg.n_heads, cfg.n_blocks, cfg.ffn_mult, cfg.trunk_dim, cfg.trunk_hidden,
                           cfg.value_bins, cfg.note_geo, cfg.head_gears, cfg.z_asinh, cfg.value_vmax, cfg.eps)
    pad, bins_pad = C.c_int32(), C.c_int32()
    first = (C.c_int32 * 29)()
    native.check(native.lib.bsrl_head_layout(C.byref(c), C.byref(pad), C.byref(bins_pad), first))
    g = torch.Generator().manual_seed(B)
    raw = (torch.randn(B, pad.value, generator=g) * 2).requires_grad_(True)
    vraw = (torch.randn(B, bins_pad.value, generator=g) * 3).requires_grad_(True)
    act = po.make_actions(B, cfg, 3)
    up = po.make_upstream(B, cfg, 4)
    gl = 0.1 * torch.randn(B, 29, cfg.k_max, generator=g) / B
    with torch.enable_grad():
        logits = torch.full((B, 29, cfg.k_max), -1e9)
        for j, k in enumerate(cfg.head_gears):
            logits[:, j, :k] = raw[:, first[j]:first[j] + k]
        logsm = torch.log_softmax(logits, -1)
        lp = logsm.gather(-1, act.long().unsqueeze(-1)).squeeze(-1).sum(-1)
        ent = -(logsm.exp() * logsm).sum(-1).sum(-1)
        vl = vraw[:, :cfg.value_bins]
        val = torch.softmax(vl, -1) @ po.value_centers(cfg)
        ((up["logprob"] * lp).sum() + (up["entropy"] * ent).sum() + (up["value"] * val).sum()
         + (up["value_logits"] * vl).sum() + (gl * logits).sum()).backward()
    ldh, ldb = 192, 128
    gh = torch.full((B, ldh), 7.0, dtype=torch.float16, device="cuda")
    gb = torch.full((B, ldb), 7.0, dtype=torch.float16, device="cuda")
    dev = {k: v.cuda() for k, v in up.items()}
    rawd, vrawd, actd, gld = raw.detach().cuda(), vraw.detach().cuda(), act.to(torch.int32).cuda(), gl.cuda()
    scale = 1024.0
    native.check(native.lib.bsrl_head_tail_bwd(C.byref(c), rawd.data_ptr(), vrawd.data_ptr(), B, actd.data_ptr(), native.I32,
                                               dev["logprob"].data_ptr(), dev["entropy"].data_ptr(), dev["value"].data_ptr(),
                                               dev["value_logits"].data_ptr(), gld.data_ptr(), scale, gh.data_ptr(), ldh,
                                               gb.data_ptr(), ldb, _st()))
    n_cols = sum(cfg.head_gears)
    torch.testing.assert_close(gh.float().cpu()[:, :n_cols] / scale, raw.grad[:, :n_cols], atol=2e-5, rtol=2e-3)
    assert float(gh[:, n_cols:].abs().max()) == 0.0                      # padding columns are zeroed for the GEMMs
    torch.testing.assert_close(gb.float().cpu()[:, :cfg.value_bins] / scale, vraw.grad[:, :cfg.value_bins], atol=2e-5, rtol=2e-3)
    assert float(gb[:, cfg.value_bins:].abs().max()) == 0.0


@pytest.mark.parametrize("engine", [0, 1])
@pytest.mark.parametrize("m,n,k", [(40, 64, 64), (1000, 128, 256), (5000, 1024, 256), (3333, 256, 1024), (129, 768, 256),
                                   (2048, 192, 192), (7777, 576, 192)])
def test_linear_bwd_stage(native, m, n, k, engine):
    """Weight gradient (split-K tcgen05 product over the token rows), bias gradient and input gradient of one Linear
    against fp32 matmuls on the same fp16 operands.  Engine 0 hands the operands to the tensor cores as they lie
    (the contraction index is their row: MN-major tiles); engine 1 is the warp-MMA engine on transposed copies."""
    native.lib.bsrl_set_engine(engine)
    g = torch.Generator().manual_seed(m + n + k)
    gy = (torch.randn(m, n, generator=g) * 0.5).half()
    x = torch.randn(m, k, generator=g).half()
    w = (torch.randn(n, k, generator=g) / k ** 0.5).half()
    nbytes = native.lib.bsrl_linear_bwd_scratch_bytes(m, n, k)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    gw, gb = torch.zeros(n, k, device="cuda"), torch.zeros(n, device="cuda")
    gx = torch.empty(m, k, device="cuda")
    gyd, xd, wd = gy.cuda(), x.cuda(), w.cuda()
    native.check(native.lib.bsrl_linear_bwd(gyd.data_ptr(), xd.data_ptr(), wd.data_ptr(), m, n, k, gw.data_ptr(), gb.data_ptr(),
                                            gx.data_ptr(), 1, scratch.data_ptr(), nbytes, _st()))
    native.lib.bsrl_set_engine(0)
    native.check(native.lib.bsrl_device_status())
    torch.testing.assert_close(gw.cpu(), gy.float().t() @ x.float(), atol=2e-3 * m ** 0.5, rtol=2e-3)
    torch.testing.assert_close(gb.cpu(), gy.float().sum(0), atol=1e-3 * m ** 0.5, rtol=1e-3)
    torch.testing.assert_close(gx.cpu(), gy.float() @ w.float(), atol=2e-3, rtol=2e-3)
