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


def test_update_loop_learns_and_matches_a_torch_trained_twin():
    """The PPO update's pieces together: grad-mode recompute -> loss.backward() (the CUDA backward) -> PackedAdamW.step()
    (AdamW + arena refresh in one kernel), 30 times, on a behaviour-cloning objective: the log-probability of fixed
    target actions rises and the value regresses onto fixed targets.  A twin model -- the oracle's fp32 torch forward
    with torch.optim.AdamW -- is trained on the same data; the two loss curves stay together."""
    from beatsaberrl_b200.optim import PackedAdamW
    cfg, sd = golden_case("cfg1")
    m = cuda_policy(cfg, sd)
    m.flatten_fp16()
    opt = PackedAdamW(m, lr=3e-4, weight_decay=0.0)
    twin = {k: v.clone().requires_grad_(True) for k, v in sd.items()}
    topt = torch.optim.AdamW(list(twin.values()), lr=3e-4, weight_decay=0.0)
    B = 256
    obs = po.make_obs(B, 31, padded=True)
    act = po.make_actions(B, cfg, 32)
    vtarget = torch.linspace(-2.0, 2.0, B)
    obs_d, act_d, vt_d = obs.cuda(), act.cuda(), vtarget.cuda()

    def loss_of(lp, value):
        return -(lp.mean() / 29.0) + 0.5 * ((value - (vt_d if value.is_cuda else vtarget)) ** 2).mean()

    ours, theirs = [], []
    for step in range(30):
        with torch.enable_grad():
            _, lp, _, val = m.get_action_and_value(obs_d, act_d)
            loss = loss_of(lp, val)
            opt.zero_grad()
            loss.backward()
        opt.step()
        ours.append(float(loss.detach()))
        with torch.enable_grad():
            logits, value, _ = po.forward_stacked.__wrapped__(twin, cfg, obs, want=True)
            tlp, _, _ = po.evaluate_actions.__wrapped__(logits, act)
            tloss = loss_of(tlp, value)
            topt.zero_grad()
            tloss.backward()
        topt.step()
        theirs.append(float(tloss.detach()))
    m.check_device()
    # the fp32 twin's curve: the same to four digits for the first ten steps, within ten per cent later (rounding
    # differences grow along a training trajectory: 1-3 % by step 30 with the tcgen05 kernels, up to 6 % with the
    # warp-MMA cross-check engine, whose sums run in another order), and both end below 55 % of where they started
    for a, b in zip(ours[:10], theirs[:10]):
        assert abs(a - b) <= 2e-3 * abs(b), (ours, theirs)
    for a, b in zip(ours, theirs):
        assert abs(a - b) <= 0.10 * abs(b), (ours, theirs)
    assert ours[-1] < 0.55 * ours[0] and theirs[-1] < 0.55 * theirs[0], (ours, theirs)
    # the fp16 arena the forward reads is the one the optimizer kernel kept in step with the masters
    before = m._arena.clone()
    m.refresh_fp16_caches()
    assert torch.equal(before, m._arena)


def test_packed_muon_matches_a_per_matrix_implementation_and_a_repack():
    """The Muon half: Nesterov momentum -> five Newton-Schulz steps -> RMS-matched scale -> step, against a plain
    per-matrix fp32 implementation of the same recipe; the arena it leaves equals a full repack; AdamW with
    ``exclude`` leaves Muon's parameters alone."""
    import math
    from beatsaberrl_b200.optim import MUON_NS_COEFS, PackedAdamW, PackedMuon, muon_param_names
    cfg, sd = golden_case("tiny_plain")
    m = cuda_policy(cfg, sd)
    m.flatten_fp16()
    names = muon_param_names(m)
    assert "blocks.0.ffn.0.weight" in names and "trunk_fc1.weight" in names and "critic_mlp.0.weight" in names
    assert not any(n.startswith(("heads.", "note_mlp", "saber_mlp")) or n.endswith(".bias") for n in names)
    assert f"critic_mlp.{len(m.critic_mlp) - 1}.weight" not in names
    assert "note_mlp.2.weight" in muon_param_names(m, enc_hidden=True)
    muon = PackedMuon(m, names, lr=0.02, momentum=0.9)
    adam = PackedAdamW(m, lr=1e-3, exclude=names)
    named = dict(m.named_parameters())
    ref = {n: named[n].detach().clone() for n in names}
    bufs = {n: torch.zeros_like(ref[n]) for n in names}
    others = {n: p.detach().clone() for n, p in named.items() if n not in names}
    g = torch.Generator(device="cuda").manual_seed(5)
    for step in range(2):
        for n, p in named.items():
            p.grad = torch.randn(p.shape, generator=g, device="cuda") * 0.05
        for n in names:                                  # the recipe, one matrix at a time
            gr = named[n].grad
            bufs[n] = 0.9 * bufs[n] + gr
            u = gr + 0.9 * bufs[n]
            tall = u.shape[0] > u.shape[1]
            x = u.t() if tall else u
            x = x / (x.norm() + 1e-7)
            for a, b, c in MUON_NS_COEFS:
                s = x @ x.t()
                x = a * x + (b * s + c * (s @ s)) @ x
            x = x.t() if tall else x
            ref[n] = ref[n] - 0.02 * 0.2 * math.sqrt(max(u.shape)) * x
        muon.step()
        for n in names:
            torch.testing.assert_close(named[n], ref[n], atol=2e-6, rtol=2e-5, msg=lambda s, n=n: f"{n}: {s}")
        for n, before in others.items():                 # not Muon's: untouched by its step
            assert torch.equal(named[n], before), n
    arena = m._arena.clone()
    m.refresh_fp16_caches()
    assert torch.equal(arena, m._arena)
    # the Adam half ignores Muon's parameters and moves the rest
    snap = {n: p.detach().clone() for n, p in named.items()}
    adam.step()
    assert all(torch.equal(named[n], snap[n]) for n in names)
    assert any(not torch.equal(named[n], snap[n]) for n in others)
    arena = m._arena.clone()
    m.refresh_fp16_caches()
    assert torch.equal(arena, m._arena)
    sd2 = muon.state_dict()
    muon2 = PackedMuon(m, names)
    muon2.load_state_dict(sd2)
    assert torch.equal(muon2.bufs[0], muon.bufs[0])
