"""bsrl_forward_fixed: the forward on the library's built-in scratch.

Some hosts of this library cannot provide a workspace: a C/C++ simulator thread or a replay tool
that links no tensor library has no device allocator at hand, and a process running under a fixed
device-memory budget must not cudaMalloc late.  For them the library carries one entry point that
allocates nothing.  This test calls it through the C ABI twice in a row (the calls share the
scratch, which keeps the previous call's contents) and requires the same logits and values as the
ordinary bsrl_forward with a caller workspace.  Collected last on purpose: a failure here cannot
hide any other test from a run that stops at the first failure.
"""
import ctypes as C

import pytest
import torch

from helpers import cuda_policy, golden_case, po


@pytest.mark.gpu
def test_forward_fixed_matches_forward_twice(native):
    cfg, sd = golden_case("cfg1")
    m = cuda_policy(cfg, sd)
    m.flatten_fp16()
    lib = native.lib
    st = torch.cuda.current_stream().cuda_stream
    assert lib.bsrl_fixed_scratch_bytes() == 32 << 20
    for call, (B, seed) in enumerate([(96, 41), (64, 42)]):
        obs = po.make_obs(B, seed, padded=True).cuda()
        assert lib.bsrl_workspace_bytes(C.byref(m._cfg), B) <= lib.bsrl_fixed_scratch_bytes()
        ref_logits, ref_value = m.forward_stacked(obs)            # caller-workspace entry point
        logits = torch.full((B, 29, cfg.k_max), float("nan"), device="cuda")
        value = torch.full((B,), float("nan"), device="cuda")
        native.check(lib.bsrl_forward_fixed(C.byref(m._cfg), m._arena.data_ptr(), obs.data_ptr(), 0, B,
                                            logits.data_ptr(), value.data_ptr(), st))
        torch.cuda.synchronize()
        native.check(lib.bsrl_device_status())
        # same kernels on the same inputs: the tolerance of the parity gates is far from needed
        torch.testing.assert_close(logits, ref_logits, atol=2e-2, rtol=1e-2)
        torch.testing.assert_close(value, ref_value, atol=2e-2, rtol=1e-2)
        assert torch.equal(logits, ref_logits) and torch.equal(value, ref_value), f"call {call}"
    # a batch past the built-in scratch is refused on the host with a clear message
    big = 100_000
    rc = lib.bsrl_forward_fixed(C.byref(m._cfg), m._arena.data_ptr(), obs.data_ptr(), 0, big,
                                logits.data_ptr(), value.data_ptr(), st)
    assert rc == -4 and "built-in scratch" in native.last_error()


def test_forward_fixed_refuses_oversize_without_a_gpu(native):
    """Size check happens on the host before anything touches a device."""
    cfg, _ = golden_case("cfg1")
    c = native.make_config(cfg.embed, cfg.n_heads, cfg.n_blocks, cfg.ffn_mult, cfg.trunk_dim,
                           cfg.trunk_hidden, cfg.value_bins, cfg.note_geo, cfg.head_gears)
    fake = C.c_void_p(4096)
    assert native.lib.bsrl_forward_fixed(C.byref(c), fake, fake, 0, 1 << 20, fake, fake, None) == -4
    assert native.lib.bsrl_forward_fixed(C.byref(c), fake, fake, 0, -1, fake, fake, None) == -2
