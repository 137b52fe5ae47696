"""Times the reference's own fp16 GPU stream (its ``NotePolicy.forward_stacked`` with ``fp16=True``:
cuBLAS / cuBLASLt GEMMs, aten SDPA or its 29-token attention kernel, its LayerNorm and fused-FFN
kernels) on the GPU of this machine, from the tree staged by ``baseline/setup_ref.py``.

    python baseline/ref_gpu_bench.py [--workload cfg2|recipe|cfg1|cfg4] [--envs N] [--iters K] [--reps R]

Protocol of the reference's forward bench (python/bench_policy_forward.py:72-83): inputs resident on the
device, warm-up, best of R timed loops of K forwards, synchronised; eager and CUDA-graphed (its
``_Graphed`` driver).  Prints ONE JSON line; on any failure the line carries ``"unavailable"`` with the
reason.  None of this repository's kernels are loaded here.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
import types
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = HERE / "_ref" / "python"

# (embed, trunk_dim, n_blocks, n_heads, n_gears, note_geo, envs, xavier, seed)
SHAPES = {
    "cfg1": (128, 256, 2, 4, 5, False, 1024, False, 0),
    "cfg2": (256, 512, 4, 8, 5, False, 65536, True, 1),
    "cfg4": (512, 1024, 6, 8, 7, False, 32768, False, 3),
    "recipe": (192, 384, 6, 4, 5, True, 32768, False, 5),
}


def _stub_env_package():
    """The reference's ``beat_arena_env/__init__`` pulls in its Rust simulator and gymnasium; the policy
    only needs ``beat_arena_env.jit_cache`` and ``.constants``.  A bare package object pointing at the
    staged directory gives it those two without running the package's own ``__init__``."""
    pkg = types.ModuleType("beat_arena_env")
    pkg.__path__ = [str(REF / "beat_arena_env")]
    sys.modules["beat_arena_env"] = pkg
    cuda_env = types.ModuleType("beat_arena_env.cuda_env")
    cuda_env._toolchain_env = lambda: None          # only reached when an extension has to be rebuilt
    sys.modules["beat_arena_env.cuda_env"] = cuda_env


def run(args):
    import torch
    if not (REF / "policy.py").exists():
        return {"unavailable": "baseline/_ref is not staged (run baseline/setup_ref.py where the reference checkout is)"}
    if not torch.cuda.is_available():
        return {"unavailable": "no CUDA device"}
    sys.path.insert(0, str(REF))
    _stub_env_package()
    import fp16_linear as fl
    import fused_ln
    import policy as ref_policy
    from cuda_graphs import _Graphed

    embed, trunk, blocks, heads, gears, geo, envs, xavier, seed = SHAPES[args.workload]
    envs = args.envs or envs
    torch.manual_seed(seed)
    pol = ref_policy.NotePolicy(embed=embed, trunk_dim=trunk, n_blocks=blocks, n_heads=heads, n_gears=gears,
                                ffn_mult=4, note_geo=geo, head_gears=(gears,) * 29)
    if xavier:
        for m in pol.modules():
            if isinstance(m, torch.nn.Linear):
                torch.nn.init.xavier_uniform_(m.weight)
                torch.nn.init.zeros_(m.bias)
    pol = pol.cuda().eval()
    pol.fp16 = True
    if args.fused_ffn:
        pol.fused_ffn = pol.arch["fused_ffn"] = args.fused_ffn
    pol.flatten_fp16()
    g = torch.Generator().manual_seed(seed)
    obs = torch.randn(envs, ref_policy.OBS_DIM, generator=g).clamp_(-5, 5)
    obs[:, ref_policy.OFF_NOTE_MASK:ref_policy.OFF_NOTE_MASK + ref_policy.N_NOTE_SLOTS] = 1.0
    obs = obs.cuda()

    class GraphedForward(_Graphed):
        def __init__(self):
            super().__init__()
            self.s_obs = torch.zeros_like(obs)

        def _compute(self):
            with torch.no_grad():
                return pol.forward_stacked(self.s_obs)

        def __call__(self, o):
            self._copy_static(self.s_obs, o)
            return self._run()

    def eager():
        with torch.no_grad():
            return pol.forward_stacked(obs)

    def bench(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(args.reps):
            t0 = time.perf_counter()
            for _ in range(args.iters):
                fn()
            torch.cuda.synchronize()
            best = min(best, (time.perf_counter() - t0) / args.iters)
        return best

    if args.update:
        # forward in grad mode + backward of a PPO-like loss to every parameter: the reference's fp16 update stream
        # (its autograd.Functions and backward kernels), protocol of python/bench_policy_update.py
        gen = torch.Generator().manual_seed(seed + 1)
        act = torch.randint(0, gears, (envs, 29), generator=gen).to(torch.uint8).cuda()
        wl, we, wv = (torch.randn(envs, generator=gen) / envs).cuda(), (0.1 * torch.randn(envs, generator=gen) / envs).cuda(), \
            (torch.randn(envs, generator=gen) / envs).cuda()
        wvl = (0.2 * torch.randn(envs, pol.value_bins, generator=gen) / envs).cuda()
        pol.train()
        obs16 = obs.half()

        def update():
            _, lp, ent, val = pol.get_action_and_value(obs16, act)
            loss = (wl * lp.float()).sum() + (we * ent.float()).sum() + (wv * val.float()).sum() + (wvl * pol._value_logits.float()).sum()
            (loss * 1024.0).backward()
            for p_ in pol.parameters():
                p_.grad = None
        t = bench(update)
        return {"workload": args.workload, "envs": envs, "gpu": torch.cuda.get_device_name(0), "mode": "update (grad-mode forward + backward)",
                "ms_per_step": t * 1e3, "env_updates_s": envs / t, "fused_ffn_mode": pol.fused_ffn,
                "ln_kernel": "jit" if fused_ln._load() is not None else "torch fallback",
                "gemm_attn_kernels": "jit" if fl._load() is not None else "torch fallback",
                "protocol": f"best of {args.reps} x {args.iters} updates after {args.warmup} warm-ups, fp16 obs, loss scale 1024"}
    # The reference calls torch's scaled_dot_product_attention where its own 29-token kernel does not
    # engage; if the cuDNN backend refuses the shape (seen at 65,536 envs x 8 heads), fall back to torch's
    # other SDPA backends -- a torch setting, the reference's code is untouched.
    sdpa = "default backends"
    try:
        t_eager = bench(eager)
    except RuntimeError as e:
        if "mha_graph" not in str(e) and "cudnn" not in str(e).lower():
            raise
        torch.backends.cuda.enable_cudnn_sdp(False)
        sdpa = "cuDNN backend disabled after: " + str(e)[:120]
        t_eager = bench(eager)
    out = {"workload": args.workload, "envs": envs, "gpu": torch.cuda.get_device_name(0),
           "torch": torch.__version__, "eager_ms": t_eager * 1e3,
           "ln_kernel": "jit" if fused_ln._load() is not None else "torch fallback",
           "gemm_attn_kernels": "jit" if fl._load() is not None else "torch fallback",
           "fused_ffn_mode": pol.fused_ffn, "sdpa": sdpa, "dtype": "fp16 stream (reference --fp16)",
           "protocol": f"best of {args.reps} x {args.iters} forwards after {args.warmup} warm-ups, inputs resident"}
    try:
        gf = GraphedForward()
        t_graph = bench(lambda: gf(obs))
        out["graphed_ms"] = t_graph * 1e3
    except Exception as e:                      # capture can fail where eager works; keep the eager number
        out["graphed_ms"] = None
        out["graph_error"] = f"{type(e).__name__}: {e}"[:300]
    best = min(t for t in (t_eager, (out["graphed_ms"] or 1e30) / 1e3) if t)
    out["ms_per_step"] = best * 1e3
    out["env_forwards_s"] = envs / best
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="cfg2", choices=sorted(SHAPES))
    ap.add_argument("--envs", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--update", action="store_true", help="time the grad-mode forward + backward instead of the forward")
    ap.add_argument("--fused-ffn", default="", help="the reference's fused_ffn mode (off/on/up16/up16dn16)")
    args = ap.parse_args()
    try:
        line = run(args)
    except Exception as e:
        line = {"unavailable": f"{type(e).__name__}: {e}"[:500]}
    line["impl"] = "reference_gpu"
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
