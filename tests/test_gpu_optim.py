"""Fused AdamW step + arena refresh against torch.optim.AdamW and a plain repack."""
import pytest
import torch

from helpers import cuda_policy, golden_case, po

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", ["tiny_plain", "tiny_vres"])
def test_adam_step_pack_matches_torch_adamw_and_a_repack(case):
    from beatsaberrl_b200.optim import PackedAdamW
    cfg, sd = golden_case(case)
    m = cuda_policy(cfg, sd)
    ref = cuda_policy(cfg, sd)                     # same masters, stepped by torch
    m.flatten_fp16()
    opt = PackedAdamW(m, lr=1e-2, betas=(0.9, 0.99), eps=1e-6, weight_decay=0.05, lr_scale={"critic_": 3.0})
    decay = [p for p in ref.parameters() if p.dim() >= 2]
    critic = {id(p) for n, p in ref.named_parameters() if n.startswith("critic_")}
    groups = []
    for is_c in (False, True):
        for dec in (False, True):
            ps = [p for p in ref.parameters() if (id(p) in critic) == is_c and (p.dim() >= 2) == dec]
            if ps:
                groups.append(dict(params=ps, lr=1e-2 * (3.0 if is_c else 1.0), weight_decay=0.05 if dec else 0.0))
    topt = torch.optim.AdamW(groups, betas=(0.9, 0.99), eps=1e-6)
    g = torch.Generator(device="cuda").manual_seed(1)
    frozen = "critic_ln.bias"
    obs = po.make_obs(64, 3).cuda()
    arena_ptr = m._arena.data_ptr()
    for step in range(3):
        for (n, p), (_, q) in zip(m.named_parameters(), ref.named_parameters()):
            if n == frozen:
                p.grad = None
                q.grad = None
                continue
            p.grad = torch.randn(p.shape, generator=g, device="cuda") * 0.1
            q.grad = p.grad.clone()
        opt.step()
        topt.step()
    for (n, p), (_, q) in zip(m.named_parameters(), ref.named_parameters()):
        torch.testing.assert_close(p, q, atol=2e-6, rtol=2e-5, msg=lambda s: f"{n}: {s}")
    assert m._arena.data_ptr() == arena_ptr
    # the arena the optimizer kernel wrote is what a full repack of the same masters writes, bit for bit
    fused_arena = m._arena.clone()
    logits_fused, v_fused = m.forward_stacked(obs)
    m.refresh_fp16_caches()
    assert torch.equal(fused_arena, m._arena)
    logits_re, v_re = m.forward_stacked(obs)
    assert torch.equal(logits_fused, logits_re) and torch.equal(v_fused, v_re)
    # a loss scaler's found_inf skips the update but leaves everything consistent
    before = [p.clone() for p in m.parameters()]
    opt.step(inv_scale=torch.tensor(0.5, device="cuda"), found_inf=torch.tensor(1.0, device="cuda"))
    for p, b in zip(m.parameters(), before):
        assert torch.equal(p, b)
    assert torch.equal(fused_arena, m._arena)
    # state round trip
    sd2 = opt.state_dict()
    opt2 = PackedAdamW(m, lr=1e-2)
    opt2.load_state_dict(sd2)
    assert opt2.step_count == opt.step_count and torch.equal(opt2.exp_avg[0], opt.exp_avg[0])
