"""Graph-driver protocol on a GPU: capture and replay of the sampling / rollout entry points, weight
repacking under a live graph, the forward captured together with an in-place environment step
(the role of step_kernel in python/rollout_graph.py:45-74), and the workspace a graph holds on to."""
import pytest
import torch

from helpers import cuda_policy, golden_case, po

pytestmark = pytest.mark.gpu


def _warm(fn, n=3):
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(n):
            fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()


def test_sampling_graph_draws_new_actions_and_matches_eager():
    cfg, sd = golden_case("tiny_plain")
    m = cuda_policy(cfg, sd)
    m.flatten_fp16()
    obs = po.make_obs(192, 5).cuda()
    m.seed_sampler(77)
    _warm(lambda: m.get_action_and_value(obs))
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        ga, glp, gent, gv = m.get_action_and_value(obs)
    m.seed_sampler(77)                      # restart the counter: replay k must equal eager call k
    rng = m._rng_state
    draws = []
    for _ in range(3):
        g.replay()
        draws.append((ga.clone(), glp.clone(), gent.clone(), gv.clone()))
    assert int(rng[1]) == 3                 # the captured increment ran once per replay
    assert not torch.equal(draws[0][0], draws[1][0]) and not torch.equal(draws[1][0], draws[2][0])
    m.seed_sampler(77)
    for k in range(3):
        a, lp, ent, v = m.get_action_and_value(obs)
        assert torch.equal(a, draws[k][0]) and torch.equal(lp, draws[k][1])
        assert torch.equal(ent, draws[k][2]) and torch.equal(v, draws[k][3])


def test_rollout_step_graph_writes_rows_each_replay():
    cfg, sd = golden_case("tiny_geo_mixed")
    m = cuda_policy(cfg, sd)
    m.flatten_fp16()
    B = 96
    obs = po.make_obs(B, 6, padded=True).cuda()
    rows = dict(b_act=torch.zeros(B, 29, dtype=torch.uint8, device="cuda"),
                b_logp=torch.zeros(B, device="cuda"), b_val=torch.zeros(B, device="cuda"),
                b_obs=torch.zeros(B, 630, dtype=torch.float16, device="cuda"),
                ret_sig=torch.tensor(2.0, device="cuda"), ret_mu=torch.tensor(-0.5, device="cuda"))
    m.seed_sampler(5)
    _warm(lambda: m.rollout_step(obs, **rows))
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        ga, glp, _, gv = m.rollout_step(obs, **rows)
    m.seed_sampler(5)
    g.replay()
    a1 = ga.clone()
    assert torch.equal(rows["b_act"].long(), ga) and torch.equal(rows["b_logp"], glp)
    torch.testing.assert_close(rows["b_val"], gv * 2.0 - 0.5, atol=1e-6, rtol=1e-6)
    assert torch.equal(rows["b_obs"], obs.half())
    g.replay()
    assert not torch.equal(a1, ga) and torch.equal(rows["b_act"].long(), ga)
    m.seed_sampler(5)
    ea, elp, _, ev = m.get_action_and_value(obs)
    assert torch.equal(ea, a1)


def test_weight_repack_under_a_live_graph():
    from beatsaberrl_b200.graphs import GraphedForward
    from beatsaberrl_b200.policy import bump_weights_version
    cfg, sd = golden_case("tiny_plain")
    m = cuda_policy(cfg, sd)
    obs = po.make_obs(128, 9).cuda()
    gf = GraphedForward(m, 128)
    for _ in range(5):                      # warm-up calls, the capture, one replay
        l0, _ = gf(obs)
    assert gf.graph is not None
    l0 = l0.clone()
    with torch.no_grad():
        for p in m.heads.parameters():
            p.mul_(2.0)
    bump_weights_version()
    m.refresh_fp16_caches()                 # in place: the graph's arena pointer stays valid
    l1, _ = gf(obs)
    torch.testing.assert_close(l1, 2 * l0, atol=1e-2, rtol=1e-2)
    with pytest.raises(RuntimeError, match="static input expects"):
        gf(obs[:64])
    with pytest.raises(RuntimeError, match="static input expects"):
        gf(obs.half())


def test_forward_and_env_step_in_one_graph():
    """GraphedRollout: forward + sampling + an in-place env step as one graph; K replays reproduce K
    eager ticks from the same start state and sampling seed bit for bit."""
    from beatsaberrl_b200.graphs import GraphedRollout, StandInEnv
    cfg, sd = golden_case("tiny_plain")
    B, K = 160, 4
    m = cuda_policy(cfg, sd)
    env = StandInEnv(B, seed=3)
    obs0, st0 = env._obs.clone(), env._state.clone()
    m.seed_sampler(11)
    gr = GraphedRollout(m, env)
    # restart the env and the sampling stream (both in place: the graph holds their addresses), then replay
    env._obs.copy_(obs0); env._state.copy_(st0)
    m.seed_sampler(11)
    traj_g = []
    for _ in range(K):
        a, lp, v, rew, done = gr.step()
        traj_g.append((a.clone(), lp.clone(), v.clone(), env._obs.clone(), rew.clone(), done.clone()))
    # the same K ticks eagerly
    env._obs.copy_(obs0); env._state.copy_(st0)
    m.seed_sampler(11)
    traj_e = []
    for _ in range(K):
        a, lp, _, v = m.get_action_and_value(env._obs, need_entropy=False)
        env.step(a)
        traj_e.append((a.clone(), lp.clone(), v.clone(), env._obs.clone(), env._reward.clone(), env._done.clone()))
    for k in range(K):
        if k:
            assert not torch.equal(traj_e[k][3], traj_e[k - 1][3])      # the env really rewrites obs
            assert not torch.equal(traj_e[k][0], traj_e[k - 1][0])      # and each tick draws new actions
        for ge, ee in zip(traj_g[k], traj_e[k]):
            assert torch.equal(ge, ee)
    obs = env._obs                                                       # stand-in obs keep the input contract
    assert float(obs.abs().max()) <= 5.0
    mask = obs[:, po.OFF_MASK:po.OFF_MASK + 24]
    assert bool(((mask == 0) | (mask == 1)).all())
    # refresh() guards the captured stream mode (python/rollout_graph.py:76-97)
    m.fp16 = False
    with pytest.raises(RuntimeError, match="captured with policy.fp16=True"):
        gr.refresh()
    m.fp16 = True
    gr.refresh()


def test_graph_keeps_its_workspace_when_batch_size_changes():
    """A rollout graph captured at n_envs must survive forwards at other batch sizes (the PPO
    recompute on minibatches) and the allocations they make."""
    cfg, sd = golden_case("tiny_plain")
    m = cuda_policy(cfg, sd)
    m.flatten_fp16()
    obs = po.make_obs(128, 1).cuda()
    _warm(lambda: m.forward_stacked(obs))
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        gl, gv = m.forward_stacked(obs)
    ws128 = m._workspaces[(128, obs.device)][0]
    ptr128 = ws128.data_ptr()
    junk = []
    for b in (64, 32, 96, 200, 16):          # more batch sizes than the idle-workspace limit
        m.forward_stacked(po.make_obs(b, b).cuda())
        junk.append(torch.full((1 << 20,), 7.0, device="cuda"))          # would land in a freed workspace
    torch.cuda.synchronize()
    assert m._workspaces[(128, obs.device)][0].data_ptr() == ptr128
    assert len(m._workspaces) <= 1 + m._MAX_IDLE_WORKSPACES
    g.replay()
    el, ev = m.forward_stacked(obs)
    assert torch.equal(gl, el) and torch.equal(gv, ev)
    for j in junk:
        assert bool((j == 7.0).all())                                    # the replay wrote into nobody else's memory


def test_bounded_wait_runs_out_and_is_reported(native):
    """A wait that can never be satisfied gives up after its limit, the kernel returns, the status word
    says which kernel and role, the facade raises, and the next forward is fine."""
    cfg, sd = golden_case("tiny_plain")
    m = cuda_policy(cfg, sd)
    obs = po.make_obs(64, 2).cuda()
    l0, v0 = m.forward_stacked(obs)
    assert native.lib.bsrl_device_status() == 0
    st = torch.cuda.current_stream().cuda_stream
    native.check(native.lib.bsrl_selftest_wait_timeout(2000, st))
    torch.cuda.synchronize()                                             # the kernel returned by itself
    with pytest.raises(native.BsrlError) as ei:
        m.check_device()
    assert ei.value.status == -7 and "kernel 15, role 1" in str(ei.value)
    assert native.lib.bsrl_device_status() == 0                          # read-and-clear
    m.check_device()
    l1, v1 = m.forward_stacked(obs)
    assert torch.equal(l0, l1) and torch.equal(v0, v1)


def test_diag_stash_keeps_the_trunk_output():
    cfg, sd = golden_case("tiny_plain")
    m = cuda_policy(cfg, sd)
    obs = po.make_obs(50, 4)
    _, _, want = po.forward_stacked(sd, cfg, obs, want=True)
    m._diag_stash = True
    m.forward_stacked(obs.cuda())
    m._diag_stash = False
    assert m._diag_h.shape == (50, cfg.trunk_dim)
    torch.testing.assert_close(m._diag_h.float().cpu(), want["trunk"], atol=3e-2, rtol=2e-2)
