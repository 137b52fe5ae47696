"""Stages the reference's own GPU policy stream under ``baseline/_ref/`` so that it can be timed on the
GPU box as a second baseline.

    python baseline/setup_ref.py [--reference /path/to/reference] [--no-build]

The GPU box has no copy of the reference checkout, and the reference builds its four CUDA sources
(LayerNorm, fp16 GEMM helpers, 29-token attention, fused FFN) at import time for the device it finds.
This script, run where the checkout IS available:

1. copies the UNMODIFIED files of the policy forward (``python/policy.py``, ``fp16_linear.py``,
   ``fused_ln.py``, ``cuda_graphs.py``, ``beat_arena_env/jit_cache.py``, ``constants.py`` and the four
   ``.cu`` files) into ``baseline/_ref/python/`` -- git-ignored, never committed, shipped with the working tree;
2. builds the two extensions for sm_100 with ``torch.utils.cpp_extension.load`` and the reference's own
   flags (``-arch=sm_100 -Xptxas -v``; nvcc cross-compiles without a GPU) into the build directories the
   reference looks in, and
3. stamps them with the reference's own source digest (``jit_cache._digest``), so that on the box its
   ``fast_load`` imports the built modules directly instead of rebuilding.

``baseline/ref_gpu_bench.py`` then imports that tree and times ``NotePolicy.forward_stacked`` on the GPU.
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref" / "python"
FILES = ["policy.py", "fp16_linear.py", "fused_ln.py", "cuda_graphs.py",
         "beat_arena_env/jit_cache.py", "beat_arena_env/constants.py",
         "beat_arena_env/csrc/layer_norm.cu", "beat_arena_env/csrc/fp16_gemm.cu",
         "beat_arena_env/csrc/small_attn.cu", "beat_arena_env/csrc/fused_ffn.cu"]
SM100_FLAGS = ["-arch=sm_100", "-Xptxas", "-v"]      # what jit_cache.cuda_flags() returns on a B200


def stage(reference: Path) -> None:
    src_root = reference / "python"
    for rel in FILES:
        src, dst = src_root / rel, DEST / rel
        if not src.exists():
            raise SystemExit(f"{src} is missing: is {reference} the reference checkout?")
        dst.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(src, dst)
    # headers the .cu files include from their own directory, if any
    for h in (src_root / "beat_arena_env" / "csrc").glob("*.h*"):
        shutil.copyfile(h, DEST / "beat_arena_env" / "csrc" / h.name)


def _jit_cache():
    spec = importlib.util.spec_from_file_location("_ref_jit_cache", DEST / "beat_arena_env" / "jit_cache.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def build() -> None:
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0"
    from torch.utils.cpp_extension import load
    jc = _jit_cache()
    csrc = DEST / "beat_arena_env" / "csrc"
    cublas = ["-lcublas", "-lcublasLt"]
    jobs = [("layer_norm_cuda", [csrc / "layer_norm.cu"], csrc / "build_ln", [], SM100_FLAGS),
            ("fp16_gemm", [csrc / "fp16_gemm.cu", csrc / "small_attn.cu", csrc / "fused_ffn.cu"],
             csrc / "build_fp16", cublas, SM100_FLAGS + cublas)]
    for name, srcs, bdir, ldflags, digest_flags in jobs:
        bdir.mkdir(exist_ok=True)
        srcs = [str(s) for s in srcs]
        load(name=name, sources=srcs, build_directory=str(bdir), extra_cuda_cflags=SM100_FLAGS,
             extra_ldflags=ldflags, verbose=False)
        (bdir / (name + ".srchash")).write_text(jc._digest(srcs, digest_flags))
        print(f"built {name} -> {bdir}")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("BSRL_REFERENCE", str(Path(__file__).resolve().parents[2] / "reference")))
    ap.add_argument("--no-build", action="store_true")
    args = ap.parse_args()
    stage(Path(args.reference))
    print(f"staged {len(FILES)} reference files under {DEST}")
    if not args.no_build:
        build()


if __name__ == "__main__":
    main()
