"""Benchmark of the policy forward: env-forwards/s on N B200s, with roofline and CPU baseline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg2]

One step = one ``forward_stacked`` over one batch of synthetic observations (65,536 envs per GPU
for the default ``cfg2`` workload: d=256, 4 blocks, 8 heads, Xavier init seed 1), replayed from a
CUDA graph captured after the warm-up, stage profiler off.  Under torchrun every rank runs the same
per-GPU batch (weak scaling, no collective on the path); timing is CUDA events bracketed by barrier
+ synchronize, max over ranks.  Rank 0 prints ONE JSON line, which also carries: the eager time of
the same step; per-stage times from a separate pass; ``e2e`` with host buffers; ``cfg5_recompute``
(131,072 envs per GPU through ``get_action_and_value(obs, int32 actions)``); the CPU baseline and,
on one GPU, ``reference_gpu`` (the reference's own fp16 GPU stream, if staged under ``baseline/_ref``).

``--impl reference`` times the reference algorithm's CPU implementation (the oracle port of
python/policy.py) on the host cores over a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "policy env-forwards/sec"
UNIT = "env-forwards/s"
WORKLOADS = {
    # name: (oracle config name, envs per GPU, weight seed, xavier, padded obs, obs seed)
    "cfg1": ("cfg1", 1024, 0, False, False, 0),
    "cfg2": ("cfg2", 65536, 1, True, False, 1),
    "cfg3": ("cfg3", 131072, 1, True, True, 2),
    "cfg4": ("cfg4", 32768, 3, False, False, 3),
    "cfg5": ("cfg5", 131072, 1, True, False, 1),
    # the reference's production shape (d 192, 6 blocks, 4 heads of 48, trunk 384, note-geo; python/train_batch.py:521-525)
    "recipe": ("recipe", 32768, 5, False, False, 5),
}
# the same BASELINE configurations in the single-body-token layout (T = 1 + n_obj tokens, GELU FFN, body-token
# readout; no counterpart in the reference): name -> (oracle config, envs per GPU, weight seed, xavier, padded, obs seed)
BODY_WORKLOADS = {
    "g_cfg1": ("cfg1", 1024, 0, False, False, 0),
    "g_cfg2": ("cfg2", 65536, 1, True, False, 1),
    "g_cfg3": ("cfg2", 131072, 1, True, True, 2),
    "g_cfg4": ("cfg4", 32768, 3, False, False, 3),
}


def read_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        j = json.loads(p.read_text())
        return dict(source="measured", hbm_gbs=j["hbm_gbs"], tflops_burst=j["bf16_tflops"],
                    tflops_sustained=j.get("bf16_tflops_sustained", j["bf16_tflops"]))
    return dict(source="fallback", hbm_gbs=6650.0, tflops_burst=1590.0, tflops_sustained=1400.0)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        top = [s for s in sm if s >= 0.5 * max(sm)] or sm     # samples under load
        return {"sm_mhz": statistics.median(top), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_forward_rate(cfg, sd, sample_envs, obs_seed, padded, reps, warm):
    """Oracle (port of the reference forward) on the host cores; best-of-reps env-forwards/s."""
    from oracle import policy_oracle as po
    torch.set_num_threads(os.cpu_count() or 1)
    obs = po.make_obs(sample_envs, obs_seed, padded=padded)
    for _ in range(warm):
        po.forward_stacked(sd, cfg, obs)
    best = float("inf")
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        po.forward_stacked(sd, cfg, obs)
        dt = time.perf_counter() - t0
        times.append(dt)
        best = min(best, dt)
    return sample_envs / best, times


def run_reference(args, rank, world):
    """The reference's CPU implementation of the path, rank 0 only."""
    if rank != 0:
        return
    from oracle import policy_oracle as po
    name, envs, wseed, xavier, padded, oseed = WORKLOADS[args.workload]
    cfg = po.named_config(name)
    sd = po.build_state_dict(cfg, wseed, xavier=xavier)
    sample = args.cpu_sample or max(64, min(envs, int(2.0e11 / (2 * po.mac_per_env(cfg)))))
    torch.set_num_threads(os.cpu_count() or 1)
    obs = po.make_obs(sample, oseed, padded=padded)
    for _ in range(args.warmup):
        po.forward_stacked(sd, cfg, obs)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        po.forward_stacked(sd, cfg, obs)
    dt = time.perf_counter() - t0
    rate = sample * args.steps / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": rate, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": f"{args.workload}: {describe(cfg)}, sample of {sample} envs per step"},
        "cpu_baseline": {"value": rate, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{sample} envs per step, torch fp32, all host threads"},
        "e2e": {"value": rate, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def describe(cfg):
    return (f"d={cfg.embed} L={cfg.n_blocks} H={cfg.n_heads} ffn={cfg.ffn_mult * cfg.embed} "
            f"trunk={cfg.trunk_dim} T=29 lead=5 gears={cfg.n_gears}")


def reference_gpu_leg(workload, timeout_s=420, update_envs=0):
    """The reference's own fp16 GPU stream on this GPU, in a process of its own (none of this library's
    kernels loaded there): ``baseline/ref_gpu_bench.py`` on the tree ``baseline/setup_ref.py`` staged."""
    script = ROOT / "baseline" / "ref_gpu_bench.py"
    if not (ROOT / "baseline" / "_ref" / "python" / "policy.py").exists():
        return {"unavailable": "baseline/_ref is not staged on this machine"}
    try:
        cmd = [sys.executable, str(script), "--workload", workload]
        if update_envs:
            cmd += ["--update", "--envs", str(update_envs)]
        r = subprocess.run(cmd, capture_output=True, text=True,
                           timeout=timeout_s, env=dict(os.environ, PYTHONDONTWRITEBYTECODE="1"))
    except subprocess.TimeoutExpired:
        return {"unavailable": f"reference GPU stream did not finish within {timeout_s} s"}
    for line in reversed(r.stdout.splitlines()):
        if line.startswith("{"):
            try:
                return json.loads(line)
            except ValueError:
                break
    return {"unavailable": ("no result line; stderr tail: " + r.stderr[-300:]).replace("\n", " ")}


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    from beatsaberrl_b200 import _native as nat
    from beatsaberrl_b200.policy import NotePolicy
    from oracle import policy_oracle as po   # weights / synthetic inputs / CPU baseline only

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    name, envs, wseed, xavier, padded, oseed = WORKLOADS[args.workload]
    if args.envs:
        envs = args.envs
    cfg = po.named_config(name)
    sd = po.build_state_dict(cfg, wseed, xavier=xavier)
    policy = NotePolicy(**cfg.ref_kwargs())
    policy.load_state_dict(sd)
    policy = policy.to(dev)
    policy.flatten_fp16()
    # each rank owns its own contiguous env range: independent seeds, no exchange
    obs_host = po.make_obs(envs, oseed + 1000 * rank, padded=padded).pin_memory()
    obs = obs_host.to(dev, non_blocking=True)
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed_ms(step, n):
        """n calls of step() between two events, barrier + synchronize on both sides, max over ranks."""
        barrier()
        e0.record()
        for _ in range(n):
            step()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1))

    # ---- device-resident throughput (value): CUDA-graph replays, stage profiler OFF -------------
    # Protocol of the reference's forward bench (python/bench_policy_forward.py:72-83): warm up, capture
    # the forward once, time the replays.  The same forward is also timed eagerly.
    for _ in range(args.warmup):
        policy.forward_stacked(obs)
    torch.cuda.synchronize()
    graph, timing = None, "eager launches"
    if not args.no_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                g_out = policy.forward_stacked(obs)
            timing = "CUDA-graph replays of one captured forward"
        except Exception as e:              # noqa: BLE001 -- report and fall back to eager launches
            graph, timing = None, f"eager launches (capture failed: {type(e).__name__})"
            torch.cuda.synchronize()
    step = graph.replay if graph is not None else (lambda: policy.forward_stacked(obs))
    for _ in range(max(3, args.warmup)):
        step()
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    ms = timed_ms(step, args.steps)
    clocks = sampler.stop()
    value = world * envs * args.steps / (ms * 1e-3)
    ms_eager = timed_ms(lambda: policy.forward_stacked(obs), args.steps)

    # ---- stage times: a separate pass with the library's per-launch events switched on ----------
    stage_steps = min(args.steps, 5)
    nat.check(nat.lib.bsrl_profile_enable(1))
    timed_ms(lambda: policy.forward_stacked(obs), stage_steps)
    stages = nat.profile_read()
    nat.check(nat.lib.bsrl_profile_enable(0))
    launches_per_step = int(sum(v["launches"] for v in stages.values())) // stage_steps

    # ---- end to end through the public API, host buffers (e2e) -----------------------
    # Every step copies its obs from pinned host memory, runs the forward and reads logits + value
    # back to pinned host memory.  The copies run on their own streams, double-buffered, so step
    # i+1's upload and step i-1's download overlap step i's kernels; all of it is inside the timed
    # region, which ends when the last download has landed.
    logits_host = [torch.empty(envs, 29, cfg.k_max, dtype=torch.float32).pin_memory() for _ in range(2)]
    value_host = [torch.empty(envs, dtype=torch.float32).pin_memory() for _ in range(2)]
    obs_dev = [torch.empty_like(obs) for _ in range(2)]
    up, down = torch.cuda.Stream(), torch.cuda.Stream()
    main = torch.cuda.current_stream()
    up_done = [torch.cuda.Event() for _ in range(2)]
    fwd_done = [torch.cuda.Event() for _ in range(2)]
    down_done = [torch.cuda.Event() for _ in range(2)]
    keep = [None, None]

    def e2e_run(n):
        for i in range(n):
            b = i & 1
            with torch.cuda.stream(up):
                up.wait_event(fwd_done[b])            # the forward that last read this buffer is done
                obs_dev[b].copy_(obs_host, non_blocking=True)
                up_done[b].record(up)
            main.wait_event(up_done[b])
            lg, vl = policy.forward_stacked(obs_dev[b])
            fwd_done[b].record(main)
            keep[b] = (lg, vl)                        # keep the outputs alive until they are downloaded
            with torch.cuda.stream(down):
                down.wait_event(fwd_done[b])
                logits_host[b].copy_(lg, non_blocking=True)
                value_host[b].copy_(vl, non_blocking=True)
                down_done[b].record(down)
            lg.record_stream(down)
            vl.record_stream(down)
        main.wait_stream(down)

    e2e_run(max(2, args.warmup // 2))
    barrier()
    e0.record()
    e2e_run(args.steps)
    e1.record()
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1))
    e2e_value = world * envs * args.steps / (ms_e2e * 1e-3)
    del obs_dev, keep, logits_host

    # ---- the PPO-recompute call at the sharded-rollout size: 131,072 envs per GPU through
    # get_action_and_value(obs, int32 actions) -- forward + fused log-softmax / log-prob / entropy ----
    recompute = None
    if args.workload == "cfg2" and not args.envs and not args.no_recompute:
        envs5 = WORKLOADS["cfg5"][1]
        obs5 = po.make_obs(envs5, oseed + 1000 * rank + 7).to(dev)
        act5 = po.make_actions(envs5, cfg, 4 + rank).to(torch.int32).to(dev)
        call = lambda: policy.get_action_and_value(obs5, act5)
        for _ in range(max(3, args.warmup)):
            call()
        ms5 = timed_ms(call, args.steps)
        recompute = {"workload": f"cfg5: {describe(cfg)}, {envs5} envs per GPU, get_action_and_value(obs, int32 actions)",
                     "value": world * envs5 * args.steps / (ms5 * 1e-3), "unit": UNIT,
                     "ms_per_step": ms5 / args.steps, "envs_per_gpu": envs5, "timing": "eager launches",
                     "outputs": "logprob, entropy, per-head entropy, value"}
        del obs5, act5

    # ---- the PPO update's recompute with gradients: forward in grad mode + backward to every parameter, on a
    # 16,384-env minibatch (python/train_batch.py:2669-2741; the reference's bench_policy_update.py protocol) ----
    update = None
    if args.workload == "cfg2" and not args.envs and not args.no_recompute:
        mb = 16384
        obs_u = po.make_obs(mb, oseed + 1000 * rank + 11).to(dev)
        act_u = po.make_actions(mb, cfg, 5 + rank).to(torch.uint8).to(dev)
        w_u = {k: v.to(dev) for k, v in po.make_upstream(mb, cfg, 6 + rank).items()}

        def update_step():
            with torch.enable_grad():
                _, lp, ent, val = policy.get_action_and_value(obs_u, act_u)
                loss = (w_u["logprob"] * lp).sum() + (w_u["entropy"] * ent).sum() + (w_u["value"] * val).sum() \
                    + (w_u["value_logits"] * policy._value_logits).sum()
                loss.backward()
            for p_ in policy.parameters():
                p_.grad = None
        for _ in range(3):
            update_step()
        ms_u = timed_ms(update_step, max(3, args.steps // 2))
        n_u = max(3, args.steps // 2)
        update = {"workload": f"cfg2 model, {mb}-env minibatch: get_action_and_value(obs, uint8 actions) in grad mode + "
                              "backward to every parameter",
                  "value": world * mb * n_u / (ms_u * 1e-3), "unit": "env-updates/s", "ms_per_step": ms_u / n_u,
                  "envs_per_gpu": mb, "flops_per_env": 6 * po.mac_per_env(cfg),
                  "tflops": 6.0 * po.mac_per_env(cfg) * mb * n_u / (ms_u * 1e-3) / 1e12}
        del obs_u, act_u

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peaks = read_peaks()
    mac = po.mac_per_env(cfg)
    fwd_tflops = 2.0 * mac * (value / world) / 1e12          # per GPU
    gemm = {k: v for k, v in stages.items() if v["flops"] > 0 and k != "attention"}
    top_name = max(gemm, key=lambda k: gemm[k]["ms"]) if gemm else None
    traffic = read_traffic_ratios()
    sm_mhz = clocks.get("sm_mhz")
    roofline = None
    if top_name:
        t = gemm[top_name]
        achieved = t["flops"] / (t["ms"] * 1e-3) / 1e12
        ms_launch = t["ms"] / t["launches"]
        tr = traffic.get(top_name)
        roofline = {"bound": "tensor", "kernel": top_name, "achieved": achieved,
                    "peak": peaks["tflops_burst"], "unit": "TFLOP/s",
                    "frac": achieved / peaks["tflops_burst"],
                    "peak_source": peaks["source"] + " (bf16 GEMM burst; the timed region is well under a second)",
                    "frac_of_sustained": achieved / peaks["tflops_sustained"], "peak_sustained": peaks["tflops_sustained"],
                    # clock-normalised: FLOP per SM per cycle at the SM clock sampled during the run, against
                    # the 8192 of one 128x256x16 f16 MMA every 128 cycles
                    "flop_per_sm_cycle": (t["flops"] / t["launches"]) / (ms_launch * 1e-3 * sm_mhz * 1e6 * 148) if sm_mhz else None,
                    "flop_per_sm_cycle_peak": 8192,
                    "traffic": (tr["ratio"] * t["bytes"] / t["launches"] if tr else None),
                    "traffic_source": (tr["source"] if tr else None),
                    "launches": t["launches"], "ms_per_launch": ms_launch,
                    "algorithmic_bytes_per_launch": t["bytes"] / t["launches"],
                    "forward_tflops": fwd_tflops,
                    "forward_frac_of_burst": fwd_tflops / peaks["tflops_burst"],
                    "forward_frac_of_sustained": fwd_tflops / peaks["tflops_sustained"],
                    "forward_frac_of_datasheet_2250": fwd_tflops / 2250.0,
                    "stage_ms_per_step": {k: round(v["ms"] / stage_steps, 4) for k, v in stages.items()},
                    "stage_pass": f"{stage_steps} eager steps with per-launch events, separate from the timed region"}
    cpu_baseline = None
    reference_gpu = None
    if world == 1:
        sample = args.cpu_sample or max(64, min(envs, int(6.0e11 / (2 * mac))))
        rate, times = cpu_forward_rate(cfg, sd, sample, oseed, padded, reps=3, warm=1)
        cpu_baseline = {"value": rate, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                        "sample": f"{sample} envs, best of 3 after 1 warm-up, torch fp32 on all host threads"}
        if not args.no_ref_gpu:
            del policy, obs
            torch.cuda.empty_cache()
            ref_wl = args.workload if args.workload in ("cfg1", "cfg2", "cfg4", "recipe") else "cfg2"
            reference_gpu = reference_gpu_leg(ref_wl)
            if update and "unavailable" not in reference_gpu:
                reference_gpu["update"] = reference_gpu_leg(ref_wl, update_envs=16384)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 operands, f32 accumulate",
        "data": "synthetic",
        "config": {"workload": f"{args.workload}: {describe(cfg)}, {envs} envs per GPU, "
                               f"{'Xavier' if xavier else 'default'} init seed {wseed}",
                   "l2": "inputs and activations larger than L2 (obs %.0f MB, token stream %.1f GB)"
                         % (envs * 630 * 4 / 1e6, envs * 29 * cfg.embed * 4 / 1e9),
                   "timing": timing, "mac_per_env": mac},
        "eager_ms_per_step": ms_eager / args.steps,
        "roofline": roofline, "cpu_baseline": cpu_baseline,
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": obs_host.numel() * 4,
                "d2h_bytes_per_step": (envs * 29 * cfg.k_max + envs) * 4},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
    }
    if recompute:
        line["cfg5_recompute"] = recompute
    if update:
        line["ppo_update"] = update
    if reference_gpu is not None:
        line["reference_gpu"] = reference_gpu
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def read_traffic_ratios():
    """{stage: {"ratio": measured DRAM bytes / algorithmic bytes, "source": ...}} written next to the ncu
    summaries when a kernel is profiled; traffic grows in proportion to the rows of a launch, so a
    full-size launch's traffic is the ratio times its algorithmic bytes."""
    p = ROOT / "profiles" / "traffic_ratios.json"
    try:
        return json.loads(p.read_text())
    except (OSError, ValueError):
        return {}


def run_body(args, rank, world, local_rank):
    """The single-body-token layout: device-resident forward_stacked, graph replays; one JSON line."""
    import torch.distributed as dist
    from beatsaberrl_b200.body_policy import BodyObjectPolicy
    from oracle import body_policy_oracle as bo
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    name, envs, wseed, xavier, padded, oseed = BODY_WORKLOADS[args.workload]
    envs = args.envs or envs
    cfg = bo.named_config(name)
    sd = bo.build_state_dict(cfg, wseed, xavier=xavier)
    policy = BodyObjectPolicy(**cfg.kwargs())
    policy.load_state_dict(sd)
    policy = policy.to(dev)
    policy.flatten_fp16()
    obs = bo.make_obs(envs, cfg, oseed + 1000 * rank, padded=padded).to(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        policy.forward_stacked(obs)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        policy.forward_stacked(obs)
    for _ in range(3):
        graph.replay()
    sampler = ClockSampler(local_rank)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.start()
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    stages, stage_steps = {}, 3
    if rank == 0:      # separate eager pass with the library's per-launch events: where the time goes
        from beatsaberrl_b200 import _native as nat
        nat.check(nat.lib.bsrl_profile_enable(1))
        for _ in range(stage_steps):
            policy.forward_stacked(obs)
        torch.cuda.synchronize()
        stages = nat.profile_read()
        nat.check(nat.lib.bsrl_profile_enable(0))
    if rank == 0:
        peaks = read_peaks()
        mac = bo.mac_per_env(cfg)
        value = world * envs * args.steps / (ms * 1e-3)
        tfl = 2.0 * mac * (value / world) / 1e12
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16 operands, f32 accumulate", "data": "synthetic",
            "config": {"workload": f"{args.workload}: single-body-token layout d={cfg.embed} L={cfg.n_blocks} H={cfg.n_heads} "
                                   f"ffn={cfg.ffn_mult * cfg.embed} GELU T={cfg.tokens} gears={cfg.n_gears}, {envs} envs per GPU",
                       "timing": "CUDA-graph replays of one captured forward", "mac_per_env": mac},
            "forward_tflops": tfl, "forward_frac_of_burst": tfl / peaks["tflops_burst"],
            "stage_ms_per_step": {k: round(v["ms"] / stage_steps, 4) for k, v in stages.items()}, "clocks": clocks}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_kernel(args):
    """Single-kernel microbenchmark through the C ABI (the small cases the ncu captures under
    profiles/ were taken on): block_tail, attn_block or linear on --rows token rows, d = --embed."""
    from beatsaberrl_b200 import _native as nat
    torch.cuda.set_device(0)
    d, rows = args.embed, args.rows
    f = 4 * d
    g = torch.Generator().manual_seed(1)
    rnd = lambda *shape, scale=1.0: (torch.randn(*shape, generator=g) * scale).cuda()
    st = torch.cuda.current_stream().cuda_stream
    if args.kernel == "block_tail":
        att, x = rnd(rows, d).half(), rnd(rows, d)
        wo, w0, w2 = rnd(d, d, scale=d ** -0.5).half(), rnd(f, d, scale=d ** -0.5).half(), rnd(d, f, scale=f ** -0.5).half()
        bo, b2, b0 = rnd(d, scale=0.1), rnd(d, scale=0.1), rnd(f, scale=0.1)
        lg, lb = torch.ones(d).cuda(), torch.zeros(d).cuda()
        out16 = torch.empty(rows, d, dtype=torch.float16, device="cuda")
        flops = 2.0 * rows * (d * d + 2 * d * f)
        nbytes = rows * d * (2 + 4 + 4 + 2)
        run = lambda: nat.check(nat.lib.bsrl_block_tail(
            att.data_ptr(), x.data_ptr(), wo.data_ptr(), bo.data_ptr(), lg.data_ptr(), lb.data_ptr(), w0.data_ptr(),
            b0.data_ptr(), w2.data_ptr(), b2.data_ptr(), 1e-5, rows, d, f, x.data_ptr(), out16.data_ptr(),
            lg.data_ptr(), lb.data_ptr(), st))
    elif args.kernel == "attn_block":
        envs = rows // 29
        h = rnd(envs * 29, d).half()
        w, bias = rnd(3 * d, d, scale=d ** -0.5).half(), rnd(3 * d, scale=0.1)
        kb = torch.zeros(envs, 29).cuda()
        out = torch.empty(envs * 29, d, dtype=torch.float16, device="cuda")
        flops = 2.0 * envs * 29 * 3 * d * d + 4.0 * envs * 29 * 29 * d
        nbytes = envs * 29 * d * 4
        heads = args.heads or d // 32                       # random weights: the per-group row order does not matter here
        n_q = args.nq or 29                                 # 5: the last block's lead rows; 1: the critic's query
        run = lambda: nat.check(nat.lib.bsrl_qkv_attention(h.data_ptr(), w.data_ptr(), bias.data_ptr(), kb.data_ptr(),
                                                           envs, d, heads, 0, n_q, out.data_ptr(), st))
    elif args.kernel == "linear_ln":      # out-projection + residual + LayerNorm for rows wider than the fused block tail
        n = k = d
        a, w, bias = rnd(rows, k).half(), rnd(n, k, scale=k ** -0.5).half(), rnd(n, scale=0.1)
        res = rnd(rows, n)
        lg, lb = torch.ones(n).cuda(), torch.zeros(n).cuda()
        h = torch.empty(rows, n, dtype=torch.float16, device="cuda")
        flops, nbytes = 2.0 * rows * n * k, rows * (k * 2 + n * 10)
        run = lambda: nat.check(nat.lib.bsrl_linear_ln(a.data_ptr(), w.data_ptr(), bias.data_ptr(), res.data_ptr(), lg.data_ptr(),
                                                       lb.data_ptr(), 1e-5, rows, n, k, res.data_ptr(), h.data_ptr(), st))
    elif args.kernel == "layernorm":
        x = rnd(rows, d)
        lg, lb = torch.ones(d).cuda(), torch.zeros(d).cuda()
        y = torch.empty(rows, d, dtype=torch.float16, device="cuda")
        flops, nbytes = 8.0 * rows * d, rows * d * 6
        run = lambda: nat.check(nat.lib.bsrl_layernorm(x.data_ptr(), lg.data_ptr(), lb.data_ptr(), 1e-5, rows, d, y.data_ptr(), d, st))
    elif args.kernel == "attention":
        envs = rows // 29
        qkv = rnd(envs * 29, 3 * d).half()
        kb = torch.zeros(envs, 29).cuda()
        out = torch.empty(envs * 29, d, dtype=torch.float16, device="cuda")
        flops, nbytes = 4.0 * envs * 29 * 29 * d, envs * 29 * d * 8
        run = lambda: nat.check(nat.lib.bsrl_attention(qkv.data_ptr(), kb.data_ptr(), envs, d, d // 32, 0, 29, out.data_ptr(), st))
    elif args.kernel == "attention_tokens":      # the single-body-token layout's attention: 33 tokens per env
        T = 33
        envs = rows // T
        qkv = rnd(envs * T, 3 * d).half()
        kb = torch.zeros(envs, T).cuda()
        out = torch.empty(envs * T, d, dtype=torch.float16, device="cuda")
        flops, nbytes = 4.0 * envs * T * T * d, envs * T * d * 8
        run = lambda: nat.check(nat.lib.bsrl_attention_tokens(qkv.data_ptr(), kb.data_ptr(), envs, T, d, d // 32, 0, T, out.data_ptr(), st))
    elif args.kernel == "wgrad":      # weight gradient of one Linear: g^T x over the token rows (split-K, MN-major operands)
        n, k = args.cols or 4 * d, d
        gy, x = rnd(rows, n, scale=0.5).half(), rnd(rows, k).half()
        gw = torch.zeros(n, k, device="cuda")
        n_s = nat.lib.bsrl_linear_bwd_scratch_bytes(rows, n, k)
        scratch = torch.empty(n_s, dtype=torch.uint8, device="cuda")
        flops, nbytes = 2.0 * rows * n * k, rows * (n + k) * 2 + n * k * 4
        run = lambda: nat.check(nat.lib.bsrl_linear_bwd(gy.data_ptr(), x.data_ptr(), None, rows, n, k, gw.data_ptr(), None, None, 0,
                                                        scratch.data_ptr(), n_s, st))
    elif args.kernel == "update":     # one PPO update step (grad-mode forward + backward) on rows / 29 envs of the cfg2 model
        from beatsaberrl_b200.policy import NotePolicy
        from oracle import policy_oracle as po
        cfg = po.named_config("cfg2")
        pol = NotePolicy(**cfg.ref_kwargs())
        pol.load_state_dict(po.build_state_dict(cfg, 1, xavier=True))
        pol = pol.cuda()
        pol.flatten_fp16()
        envs = rows // 29
        obs = po.make_obs(envs, 3).cuda()
        act = po.make_actions(envs, cfg, 5).to(torch.uint8).cuda()
        up = {k_: v.cuda() for k_, v in po.make_upstream(envs, cfg, 6).items()}
        flops, nbytes = 6.0 * po.mac_per_env(cfg) * envs, 0.0

        def run():
            with torch.enable_grad():
                _, lp, ent, val = pol.get_action_and_value(obs, act)
                loss = (up["logprob"] * lp).sum() + (up["entropy"] * ent).sum() + (up["value"] * val).sum() \
                    + (up["value_logits"] * pol._value_logits).sum()
                loss.backward()
            for p_ in pol.parameters():
                p_.grad = None
    elif args.kernel in ("embed", "head_tail"):
        import ctypes as C
        from beatsaberrl_b200.policy import NotePolicy
        from oracle import policy_oracle as po
        cfg = po.named_config("cfg2")
        pol = NotePolicy(**cfg.ref_kwargs()).cuda()
        pol.flatten_fp16()
        envs = rows // 29
        c = pol._cfg
        if args.kernel == "embed":      # tokenizer gather + fused encoders (x only)
            obs = po.make_obs(envs, 1).cuda()
            x = torch.empty(envs * 29, d, device="cuda")
            kbias = torch.empty(envs, 29, device="cuda")
            n_ws = nat.lib.bsrl_workspace_bytes(C.byref(c), envs)
            ws = torch.empty(n_ws, dtype=torch.uint8, device="cuda")
            flops = 2.0 * envs * 29 * d * (64 + d)
            nbytes = envs * (630 * 4 + 29 * 128 * 2 + 29 * d * 4)
            run = lambda: nat.check(nat.lib.bsrl_embed(C.byref(c), pol._arena.data_ptr(), obs.data_ptr(), nat.F32, envs, x.data_ptr(),
                                                       kbias.data_ptr(), ws.data_ptr(), n_ws, st))
        else:
            pad, bpad = C.c_int32(), C.c_int32()
            nat.check(nat.lib.bsrl_head_layout(C.byref(c), C.byref(pad), C.byref(bpad), None))
            raw, vraw = rnd(envs, pad.value), rnd(envs, bpad.value)
            act = po.make_actions(envs, cfg, 4).to(torch.int32).cuda()
            outs = [torch.empty(envs, 29, cfg.k_max, device="cuda"), torch.empty(envs, device="cuda"), torch.empty(envs, device="cuda"),
                    torch.empty(envs, 29, device="cuda"), torch.empty(envs, device="cuda")]
            flops = 60.0 * envs * 29 * cfg.k_max
            nbytes = envs * 4 * (pad.value + bpad.value + 29 * cfg.k_max + 29 + 3)
            run = lambda: nat.check(nat.lib.bsrl_head_tail(C.byref(c), raw.data_ptr(), vraw.data_ptr(), envs, act.data_ptr(), nat.I32,
                                                           outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(), outs[3].data_ptr(),
                                                           outs[4].data_ptr(), st))
    else:
        n, k = args.cols or 3 * d, d
        a, w, bias = rnd(rows, k).half(), rnd(n, k, scale=k ** -0.5).half(), rnd(n)
        out = torch.empty(rows, n, dtype=torch.float16, device="cuda")
        flops = 2.0 * rows * n * k
        nbytes = rows * k * 2 + n * k * 2 + rows * n * 2
        run = lambda: nat.check(nat.lib.bsrl_linear(a.data_ptr(), w.data_ptr(), bias.data_ptr(), None, out.data_ptr(),
                                                    0, 0, rows, n, k, 1, st))
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    nat.check(nat.lib.bsrl_device_status())
    ms = e0.elapsed_time(e1) / args.steps
    print(json.dumps({"kernel": args.kernel, "rows": rows, "embed": d, "ms_per_launch": ms,
                      "tflops": flops / ms / 1e9, "algorithmic_gbs": nbytes / ms / 1e6}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS) + sorted(BODY_WORKLOADS))
    ap.add_argument("--envs", type=int, default=0, help="envs per GPU (default: the workload's)")
    ap.add_argument("--cpu-sample", type=int, default=0, help="envs in the CPU sample")
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of CUDA-graph replays")
    ap.add_argument("--no-recompute", action="store_true", help="skip the cfg5 PPO-recompute sub-record")
    ap.add_argument("--no-ref-gpu", action="store_true", help="skip the reference's GPU stream (1-GPU runs)")
    ap.add_argument("--kernel", default="", choices=("", "block_tail", "attn_block", "linear", "layernorm", "attention", "embed", "head_tail",
                                                   "attention_tokens", "wgrad", "update", "linear_ln"),
                    help="time one kernel alone on --rows token rows instead of the whole forward")
    ap.add_argument("--rows", type=int, default=237568)
    ap.add_argument("--embed", type=int, default=256)
    ap.add_argument("--heads", type=int, default=0, help="heads of --kernel attn_block (default embed / 32)")
    ap.add_argument("--nq", type=int, default=0, help="query rows per env of --kernel attn_block (default 29)")
    ap.add_argument("--cols", type=int, default=0, help="output columns of --kernel linear (default 3 * embed)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        if args.workload in BODY_WORKLOADS:
            raise SystemExit("--impl reference: the single-body-token layout has no counterpart in the reference")
        run_reference(args, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the policy forward has no CPU path)")
    with torch.no_grad():          # the rollout / evaluation forward, as the reference's callers run it
        if args.kernel:
            run_kernel(args)
            return
        if args.workload in BODY_WORKLOADS:
            run_body(args, rank, world, local_rank)
            return
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
