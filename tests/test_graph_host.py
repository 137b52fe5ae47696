"""Host-side parts of the graph-driver protocol (no GPU needed)."""
import pytest
import torch

pytest.importorskip("beatsaberrl_b200._native", reason="libbsrl.so is not built")


def test_copy_static_refuses_shape_and_dtype_changes():
    from beatsaberrl_b200.graphs import copy_static
    static = torch.zeros(4, 630)
    copy_static(static, torch.ones(4, 630))
    assert float(static.sum()) == 4 * 630
    with pytest.raises(RuntimeError, match="static input expects"):
        copy_static(static, torch.ones(1, 630))          # would broadcast silently
    with pytest.raises(RuntimeError, match="static input expects"):
        copy_static(static, torch.ones(4, 630, dtype=torch.float64))   # would cast silently


def test_check_device_is_a_no_op_without_a_cuda_policy():
    from beatsaberrl_b200.policy import NotePolicy
    m = NotePolicy(embed=64, trunk_dim=128, n_blocks=2, n_heads=2, n_gears=5)
    m.check_device()                                     # parameters on the CPU: nothing to read
    with pytest.raises(RuntimeError, match="CUDA device only"):
        m.flatten_fp16()
