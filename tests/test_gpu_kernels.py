"""Single kernels through the C ABI against torch fp32 arithmetic on the same inputs."""
import ctypes as C

import pytest
import torch
import torch.nn.functional as F

from helpers import golden_case, make_cfg, po

pytestmark = pytest.mark.gpu


def _stream():
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("rows,d", [(1, 64), (37, 128), (1000, 256), (129, 512), (5, 1024)])
def test_layernorm(native, rows, d):
    g = torch.Generator().manual_seed(rows + d)
    x = (torch.randn(rows, d, generator=g) * 3 + 0.5).cuda()
    w = (1 + 0.1 * torch.randn(d, generator=g)).cuda()
    b = (0.1 * torch.randn(d, generator=g)).cuda()
    y = torch.empty(rows, d, dtype=torch.float16, device="cuda")
    native.check(native.lib.bsrl_layernorm(x.data_ptr(), w.data_ptr(), b.data_ptr(), 1e-5, rows, d,
                                           y.data_ptr(), d, _stream()))
    ref = F.layer_norm(x, (d,), w, b, 1e-5)
    # output is fp16: half an ulp of |ref| <= 8 is 4e-3
    torch.testing.assert_close(y.float(), ref, atol=4e-3, rtol=1e-3)


@pytest.mark.parametrize("engine", [0, 1])
@pytest.mark.parametrize("m,n,k,relu,resid,f32", [
    (1, 8, 32, 0, 0, 1), (127, 152, 64, 0, 0, 1), (129, 104, 512, 0, 0, 1), (1000, 768, 256, 0, 0, 0),
    (333, 1024, 256, 1, 0, 0), (260, 256, 1024, 0, 1, 1), (64, 512, 1280, 0, 0, 1), (4096, 256, 256, 0, 1, 1),
])
def test_linear(native, engine, m, n, k, relu, resid, f32):
    if engine == 1 and (k % 64 != 0 or n % 16 != 0):
        pytest.skip("shape outside the tcgen05 engine")
    g = torch.Generator().manual_seed(m * 7 + n)
    a = torch.randn(m, k, generator=g).half().cuda()
    w = (torch.randn(n, k, generator=g) / k ** 0.5).half().cuda()
    bias = torch.randn(n, generator=g).cuda()
    r = torch.randn(m, n, generator=g).cuda() if resid else None
    out = torch.empty(m, n, dtype=torch.float32 if f32 else torch.float16, device="cuda")
    rc = native.lib.bsrl_linear(a.data_ptr(), w.data_ptr(), bias.data_ptr(),
                                r.data_ptr() if resid else None, out.data_ptr(), f32, relu, m, n, k,
                                engine, _stream())
    if engine == 1 and rc == -5:
        pytest.skip("shape outside the tcgen05 engine: " + native.last_error())
    native.check(rc)
    native.check(native.lib.bsrl_device_status())     # no bounded wait ran out
    ref = a.float() @ w.float().t() + bias
    if relu:
        ref = ref.relu()
    if resid:
        ref = ref + r
    tol = dict(atol=2e-4, rtol=1e-4) if f32 else dict(atol=4e-3, rtol=1e-3)
    torch.testing.assert_close(out.float(), ref, **tol)


@pytest.mark.parametrize("B,d,H,q_first,n_q", [(1, 64, 2, 0, 29), (37, 256, 8, 0, 29), (50, 128, 4, 0, 5),
                                               (33, 256, 8, 2, 1), (9, 512, 8, 0, 29), (11, 192, 4, 0, 29)])
def test_attention(native, B, d, H, q_first, n_q):
    g = torch.Generator().manual_seed(B + d)
    qkv = torch.randn(B, 29, 3 * d, generator=g).half()
    n_live = torch.randint(0, 25, (B,), generator=g)
    n_live[0] = 0
    bias = torch.zeros(B, 29)
    bias[:, 5:] = ((torch.arange(24)[None, :] < n_live[:, None]).float() - 1.0) * 16384.0
    out = torch.empty(B * n_q, d, dtype=torch.float16, device="cuda")
    qkv_d, bias_d = qkv.cuda(), bias.cuda()
    native.check(native.lib.bsrl_attention(qkv_d.data_ptr(), bias_d.data_ptr(), B, d, H, q_first, n_q,
                                           out.data_ptr(), _stream()))
    q, k, v = qkv.float().split(d, -1)
    ref = po.attention(q[:, q_first:q_first + n_q], k, v, bias, H)
    torch.testing.assert_close(out.float().cpu().view(B, n_q, d), ref, atol=4e-3, rtol=2e-3)
    # masked keys carry exactly zero weight: junk in their k/v rows changes nothing
    junk = qkv.clone()
    dead = torch.cat([torch.zeros(B, 5, dtype=torch.bool), bias[:, 5:] < 0], 1)
    junk[..., d:][dead] = 77.0
    if q_first == 0 and n_q == 29:
        junk[..., :d][dead] = 0.5          # query rows of dead tokens may change their own output only
    out2 = torch.empty_like(out)
    junk_d = junk.cuda()
    native.check(native.lib.bsrl_attention(junk_d.data_ptr(), bias_d.data_ptr(), B, d, H, q_first, n_q,
                                           out2.data_ptr(), _stream()))
    o1 = out.view(B, n_q, d).cpu()
    o2 = out2.view(B, n_q, d).cpu()
    live_q = ~dead[:, q_first:q_first + n_q]
    assert torch.equal(o1[live_q], o2[live_q])


@pytest.mark.parametrize("T,d,H,q_first,n_q", [(17, 128, 4, 0, 17), (17, 128, 4, 0, 1), (33, 256, 8, 0, 33), (33, 256, 8, 0, 1),
                                                 (65, 512, 8, 0, 65), (65, 512, 8, 0, 1), (65, 256, 8, 0, 65),
                                                 (33, 128, 2, 0, 33), (33, 256, 8, 1, 32), (40, 256, 8, 0, 40), (33, 192, 4, 0, 33)])
def test_attention_tokens(native, T, d, H, q_first, n_q):
    """Token counts of the single-body-token layouts (the body token beside whole MMA tiles of object tokens) and a
    few shapes that take the padded kernel; masked keys carry exactly zero weight."""
    B = 37
    g = torch.Generator().manual_seed(T + d + n_q)
    qkv = torch.randn(B, T, 3 * d, generator=g).half()
    n_live = torch.randint(0, T, (B,), generator=g)
    n_live[0], n_live[1] = 0, T - 1
    bias = torch.zeros(B, T)
    bias[:, 1:] = ((torch.arange(T - 1)[None, :] < n_live[:, None]).float() - 1.0) * 16384.0
    out = torch.empty(B * n_q, d, dtype=torch.float16, device="cuda")
    qkv_d, bias_d = qkv.cuda(), bias.cuda()
    native.check(native.lib.bsrl_attention_tokens(qkv_d.data_ptr(), bias_d.data_ptr(), B, T, d, H, q_first, n_q,
                                                  out.data_ptr(), _stream()))
    q, k, v = qkv.float().split(d, -1)
    ref = po.attention(q[:, q_first:q_first + n_q], k, v, bias, H)
    torch.testing.assert_close(out.float().cpu().view(B, n_q, d), ref, atol=4e-3, rtol=2e-3)
    junk = qkv.clone()
    dead = bias < 0
    junk[..., d:][dead] = 77.0
    out2 = torch.empty_like(out)
    junk_d = junk.cuda()
    native.check(native.lib.bsrl_attention_tokens(junk_d.data_ptr(), bias_d.data_ptr(), B, T, d, H, q_first, n_q,
                                                  out2.data_ptr(), _stream()))
    assert torch.equal(out.cpu(), out2.cpu())


@pytest.mark.parametrize("case", ["tiny_plain", "tiny_geo_mixed"])
@pytest.mark.parametrize("obs_f16", [False, True])
def test_embed(native, case, obs_f16):
    cfg, sd = golden_case(case)
    from helpers import cuda_policy
    m = cuda_policy(cfg, sd)
    m.flatten_fp16()
    B = 19
    obs = po.make_obs(B, 77, padded=True)
    if obs_f16:
        obs = obs.half()
    obs_d = obs.cuda()
    x = torch.empty(B * 29, cfg.embed, device="cuda")
    kb = torch.empty(B, 29, device="cuda")
    ws = m._workspace(B, obs_d.device)
    native.check(native.lib.bsrl_embed(C.byref(m._cfg), m._arena.data_ptr(), obs_d.data_ptr(),
                                       1 if obs_f16 else 0, B, x.data_ptr(), kb.data_ptr(),
                                       ws.data_ptr(), ws.numel(), _stream()))
    tokens, bias = po.embed_tokens(sd, cfg, obs.float())
    torch.testing.assert_close(kb.cpu(), bias, atol=0, rtol=0)
    torch.testing.assert_close(x.cpu().view(B, 29, -1), tokens, atol=6e-3, rtol=5e-3)


@pytest.mark.parametrize("m,d,f,ln_out", [(128, 256, 1024, True), (1000, 256, 1024, True), (37, 128, 512, True),
                                          (5 * 77, 256, 1024, False), (20000, 192, 768, True), (40000, 256, 1024, True)])
def test_block_tail(native, m, d, f, ln_out):
    """Fused out-projection + LayerNorm + FFN kernel against the same chain in torch fp32 on the
    same fp16-rounded operands."""
    g = torch.Generator().manual_seed(m + d)
    att = torch.randn(m, d, generator=g).half().cuda()
    x = (torch.randn(m, d, generator=g) * 2).cuda()
    wo = (torch.randn(d, d, generator=g) / d ** 0.5).half().cuda()
    w0 = (torch.randn(f, d, generator=g) / d ** 0.5).half().cuda()
    w2 = (torch.randn(d, f, generator=g) / f ** 0.5).half().cuda()
    bo, b2 = torch.randn(d, generator=g).cuda() * 0.1, torch.randn(d, generator=g).cuda() * 0.1
    b0 = torch.randn(f, generator=g).cuda() * 0.1
    lg, lb = (1 + 0.1 * torch.randn(d, generator=g)).cuda(), (0.1 * torch.randn(d, generator=g)).cuda()
    og, ob = (1 + 0.1 * torch.randn(d, generator=g)).cuda(), (0.1 * torch.randn(d, generator=g)).cuda()
    x_out = torch.empty_like(x)
    out16 = torch.empty(m, d, dtype=torch.float16, device="cuda")
    native.check(native.lib.bsrl_block_tail(
        att.data_ptr(), x.data_ptr(), wo.data_ptr(), bo.data_ptr(), lg.data_ptr(), lb.data_ptr(),
        w0.data_ptr(), b0.data_ptr(), w2.data_ptr(), b2.data_ptr(), 1e-5, m, d, f, x_out.data_ptr(),
        out16.data_ptr(), og.data_ptr() if ln_out else None, ob.data_ptr() if ln_out else None, _stream()))
    native.check(native.lib.bsrl_device_status())
    x1 = x + att.float() @ wo.float().t() + bo
    h2 = F.layer_norm(x1, (d,), lg, lb, 1e-5).half().float()
    hid = (h2 @ w0.float().t() + b0).relu().half().float()
    xo = x1 + hid @ w2.float().t() + b2
    torch.testing.assert_close(x_out, xo, atol=3e-3, rtol=1e-3)
    ref16 = F.layer_norm(xo, (d,), og, ob, 1e-5) if ln_out else xo
    torch.testing.assert_close(out16.float(), ref16, atol=8e-3, rtol=2e-3)
    # in place on the residual stream, as the forward runs it
    x_in = x.clone()
    native.check(native.lib.bsrl_block_tail(
        att.data_ptr(), x_in.data_ptr(), wo.data_ptr(), bo.data_ptr(), lg.data_ptr(), lb.data_ptr(),
        w0.data_ptr(), b0.data_ptr(), w2.data_ptr(), b2.data_ptr(), 1e-5, m, d, f, x_in.data_ptr(),
        None, None, None, _stream()))
    native.check(native.lib.bsrl_device_status())
    assert torch.equal(x_in, x_out)


@pytest.mark.parametrize("B,d,H,q_first,n_q", [(1, 64, 2, 0, 29), (4, 256, 8, 0, 29), (37, 256, 8, 0, 29),
                                               (50, 128, 4, 0, 5), (33, 256, 8, 2, 1), (3000, 256, 8, 0, 29),
                                               # head_dim 48 (one head per group): the production shape
                                               (5, 192, 4, 0, 29), (1001, 192, 4, 0, 29), (70, 192, 4, 0, 5),
                                               (9, 192, 4, 2, 1),
                                               # head_dim 64 (one head per group, the h tile streamed): the wide policy
                                               (3, 64, 1, 0, 29), (50, 512, 8, 0, 29), (1001, 512, 8, 0, 29), (70, 512, 8, 0, 5),
                                               (9, 512, 8, 2, 1), (33, 256, 4, 0, 29)])
def test_qkv_attention(native, B, d, H, q_first, n_q):
    """Fused projection + attention kernel against torch fp32 on the same fp16 operands."""
    g = torch.Generator().manual_seed(B + d + n_q)
    h = torch.randn(B * 29, d, generator=g).half()
    w = (torch.randn(3 * d, d, generator=g) / d ** 0.5).half()
    bias = torch.randn(3 * d, generator=g) * 0.2
    n_live = torch.randint(0, 25, (B,), generator=g)
    kb = torch.zeros(B, 29)
    kb[:, 5:] = ((torch.arange(24)[None, :] < n_live[:, None]).float() - 1.0) * 16384.0
    # regroup per head group (two heads of 32, or one of 48): [q rows | k rows | v rows] of the group
    gd = 64 if d // H == 32 else d // H
    idx = []
    for grp in range(d // gd):
        for sct in range(3):
            idx += list(range(sct * d + grp * gd, sct * d + grp * gd + gd))
    idx = torch.tensor(idx)
    wg, bg = w[idx].contiguous().cuda(), bias[idx].contiguous().cuda()
    out = torch.empty(B * n_q, d, dtype=torch.float16, device="cuda")
    h_d, kb_d = h.cuda(), kb.cuda()
    native.check(native.lib.bsrl_qkv_attention(h_d.data_ptr(), wg.data_ptr(), bg.data_ptr(), kb_d.data_ptr(),
                                               B, d, H, q_first, n_q, out.data_ptr(), _stream()))
    native.check(native.lib.bsrl_device_status())
    qkv = (h.float() @ w.float().t() + bias).half().float().view(B, 29, 3 * d)
    q, k, v = qkv.split(d, -1)
    ref = po.attention(q[:, q_first:q_first + n_q], k, v, kb, H)
    torch.testing.assert_close(out.float().cpu().view(B, n_q, d), ref, atol=5e-3, rtol=3e-3)


@pytest.mark.parametrize("B,d,H,n_q", [(4, 64, 2, 33), (37, 128, 4, 33), (601, 256, 8, 33), (601, 256, 8, 1), (5, 128, 4, 1)])
def test_qkv_attention_body(native, B, d, H, n_q):
    """Fused projection + attention for 33-token envs (one body token + 32 object tokens): the object tokens are
    the kernel's tile rows, the body token is folded in from its own small projection.  Against torch fp32 on the
    same fp16 operands; masked object tokens carry exactly zero weight."""
    T = 33
    g = torch.Generator().manual_seed(B + d + n_q)
    h = torch.randn(B * T, d, generator=g).half()
    w = (torch.randn(3 * d, d, generator=g) / d ** 0.5).half()
    bias = torch.randn(3 * d, generator=g) * 0.2
    n_live = torch.randint(0, T, (B,), generator=g)
    n_live[0] = 0
    kb = torch.zeros(B, T)
    kb[:, 1:] = ((torch.arange(T - 1)[None, :] < n_live[:, None]).float() - 1.0) * 16384.0
    idx = []
    for grp in range(d // 64):
        for sct in range(3):
            idx += list(range(sct * d + grp * 64, sct * d + grp * 64 + 64))
    idx = torch.tensor(idx)
    wg, bg = w[idx].contiguous().cuda(), bias[idx].contiguous().cuda()
    qkv_ref = (h.float() @ w.float().t() + bias).half()
    qkv0 = qkv_ref.view(B, T, 3 * d)[:, 0].contiguous().cuda()          # the body rows' own projection
    out = torch.full((B * n_q, d), float("nan"), dtype=torch.float16, device="cuda")
    h_d, kb_d = h.cuda(), kb.cuda()
    native.check(native.lib.bsrl_qkv_attention_body(h_d.data_ptr(), wg.data_ptr(), bg.data_ptr(), qkv0.data_ptr(), kb_d.data_ptr(),
                                                    B, d, H, n_q, out.data_ptr(), _stream()))
    native.check(native.lib.bsrl_device_status())
    q, k, v = qkv_ref.float().view(B, T, 3 * d).split(d, -1)
    ref = po.attention(q[:, :n_q], k, v, kb, H)
    torch.testing.assert_close(out.float().cpu().view(B, n_q, d), ref, atol=5e-3, rtol=3e-3)


@pytest.mark.parametrize("m,n,k,in_place", [(128, 512, 512, False), (1000, 512, 512, True), (4099, 512, 256, False), (300, 256, 256, False),
                                            (77, 384, 128, True), (20000, 512, 512, True), (513, 64, 64, False)])
def test_linear_ln(native, m, n, k, in_place):
    """Projection + residual + LayerNorm kernel against fp32 torch on the same fp16 operands."""
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g).half()
    w = (torch.randn(n, k, generator=g) / k ** 0.5).half()
    bias = torch.randn(n, generator=g) * 0.3
    res = torch.randn(m, n, generator=g) * 2.0 + 0.5
    gamma, beta = 1.0 + 0.2 * torch.randn(n, generator=g), 0.1 * torch.randn(n, generator=g)
    ref_x = res + a.float() @ w.float().t() + bias
    ref_h = torch.nn.functional.layer_norm(ref_x, (n,), gamma, beta, 1e-5)
    res_d = res.cuda()
    x_out = res_d if in_place else torch.full((m, n), float("nan"), device="cuda")
    h = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
    a_d, w_d, b_d, g_d, be_d = a.cuda(), w.cuda(), bias.cuda(), gamma.cuda(), beta.cuda()
    native.check(native.lib.bsrl_linear_ln(a_d.data_ptr(), w_d.data_ptr(), b_d.data_ptr(), res_d.data_ptr(), g_d.data_ptr(),
                                           be_d.data_ptr(), 1e-5, m, n, k, x_out.data_ptr(), h.data_ptr(), _stream()))
    native.check(native.lib.bsrl_device_status())
    torch.testing.assert_close(x_out.cpu(), ref_x, atol=2e-3, rtol=1e-3)
    torch.testing.assert_close(h.float().cpu(), ref_h, atol=4e-3, rtol=2e-3)


def _native_cfg(native, cfg):
    return native.make_config(cfg.embed, cfg.n_heads, cfg.n_blocks, cfg.ffn_mult, cfg.trunk_dim,
                              cfg.trunk_hidden, cfg.value_bins, cfg.note_geo, cfg.head_gears,
                              cfg.z_asinh, cfg.value_vmax, cfg.eps, trunk_v2=(cfg.trunk_arch == "simbav2"))


@pytest.mark.parametrize("case,B", [("tiny_plain", 200), ("tiny_geo_mixed", 77), ("tiny_simbav2", 130)])
def test_trunk_heads_stage(native, case, B):
    """Readout trunk + packed heads alone (bsrl_trunk_heads) against the oracle's trunk and head
    Linears on the same fp16-rounded readout rows."""
    cfg, sd = golden_case(case)
    from helpers import cuda_policy
    m = cuda_policy(cfg, sd)
    m.flatten_fp16()
    c = m._cfg
    g = torch.Generator().manual_seed(B)
    lead = (torch.randn(B, 5 * cfg.embed, generator=g)).half()
    pad, bins_pad = C.c_int32(), C.c_int32()
    first = (C.c_int32 * 29)()
    native.check(native.lib.bsrl_head_layout(C.byref(c), C.byref(pad), C.byref(bins_pad), first))
    ws_n = native.lib.bsrl_workspace_bytes(C.byref(c), B)
    ws = torch.empty(ws_n, dtype=torch.uint8, device="cuda")
    raw = torch.empty(B, pad.value, device="cuda")
    h16 = torch.empty(B, cfg.trunk_dim, dtype=torch.float16, device="cuda")
    lead_d = lead.cuda()
    native.check(native.lib.bsrl_trunk_heads(C.byref(c), m._arena.data_ptr(), lead_d.data_ptr(), B, raw.data_ptr(),
                                             h16.data_ptr(), ws.data_ptr(), ws_n, _stream()))
    h_ref = po.trunk(sd, cfg, lead.float())
    torch.testing.assert_close(h16.float().cpu(), h_ref, atol=3e-2, rtol=2e-2)
    logits_ref = po.head_logits(sd, cfg, h_ref)                   # (B, 29, k_max) with -1e9 fill
    raw = raw.cpu()
    for j, k in enumerate(cfg.head_gears or (cfg.n_gears,) * 29):
        torch.testing.assert_close(raw[:, first[j]:first[j] + k], logits_ref[:, j, :k], atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("case,B", [("tiny_plain", 300), ("tiny_geo_mixed", 65)])
def test_head_tail_stage(native, case, B):
    """Head tail alone (bsrl_head_tail): fill, log-softmax, log-prob, entropy and HL-Gauss value are fp32
    arithmetic on given inputs, so they match the oracle to float rounding."""
    cfg, sd = golden_case(case)
    c = _native_cfg(native, cfg)
    gears = cfg.head_gears or (cfg.n_gears,) * 29
    pad, bins_pad = C.c_int32(), C.c_int32()
    first = (C.c_int32 * 29)()
    native.check(native.lib.bsrl_head_layout(C.byref(c), C.byref(pad), C.byref(bins_pad), first))
    g = torch.Generator().manual_seed(B)
    raw = torch.randn(B, pad.value, generator=g) * 2
    vraw = torch.randn(B, bins_pad.value, generator=g) * 3
    act = po.make_actions(B, cfg, 9)
    k_max = max(gears)
    out = dict(logits=torch.empty(B, 29, k_max), logprob=torch.empty(B), entropy=torch.empty(B),
               ent_head=torch.empty(B, 29), value=torch.empty(B))
    out = {k: v.cuda() for k, v in out.items()}
    raw_d, vraw_d, act_d = raw.cuda(), vraw.cuda(), act.to(torch.int32).cuda()
    native.check(native.lib.bsrl_head_tail(C.byref(c), raw_d.data_ptr(), vraw_d.data_ptr(), B, act_d.data_ptr(),
                                           native.I32, out["logits"].data_ptr(), out["logprob"].data_ptr(),
                                           out["entropy"].data_ptr(), out["ent_head"].data_ptr(),
                                           out["value"].data_ptr(), _stream()))
    ref_logits = torch.full((B, 29, k_max), -1e9)
    for j, k in enumerate(gears):
        ref_logits[:, j, :k] = raw[:, first[j]:first[j] + k]
    assert torch.equal(out["logits"].cpu(), ref_logits)
    lp, ent, ent_h = po.evaluate_actions(ref_logits, act)
    torch.testing.assert_close(out["logprob"].cpu(), lp, atol=2e-4, rtol=1e-5)
    torch.testing.assert_close(out["ent_head"].cpu(), ent_h, atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(out["entropy"].cpu(), ent, atol=2e-4, rtol=1e-5)
    val = torch.softmax(vraw[:, :cfg.value_bins], -1) @ po.value_centers(cfg)
    torch.testing.assert_close(out["value"].cpu(), val, atol=1e-5, rtol=1e-5)
