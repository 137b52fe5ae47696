"""C-ABI library on a host without a GPU: it loads, exports what the header declares, and its
host-side logic (configuration checks, parameter table, lane tables, sizes) is right.
No compute entry point is called here."""
import ctypes as C

import pytest
import torch

from helpers import make_cfg, po


def _cfg(native, cfg):
    return native.make_config(cfg.embed, cfg.n_heads, cfg.n_blocks, cfg.ffn_mult, cfg.trunk_dim,
                              cfg.trunk_hidden, cfg.value_bins, cfg.note_geo, cfg.head_gears,
                              cfg.z_asinh, cfg.value_vmax, cfg.eps)


def test_every_declared_symbol_is_exported(native):
    names = native.declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(native.lib, n), n
    assert native.lib.bsrl_abi_version() == 3


def test_token_lanes_match_oracle(native):
    for tok, name in enumerate(po.LEAD_ORDER):
        lanes = po.token_lanes(name)
        got = [native.lib.bsrl_token_lane(tok, k) for k in range(len(lanes))]
        assert got == lanes
        assert native.lib.bsrl_token_lane(tok, len(lanes)) == -1
    assert native.lib.bsrl_token_lane(5, 0) == -1


@pytest.mark.parametrize("name,geo", [("tiny", False), ("cfg1", True), ("cfg2", False), ("cfg4", False),
                                      ("recipe", True)])
def test_param_table_is_the_reference_state_dict(native, name, geo):
    cfg = make_cfg(name, geo)
    sd = po.build_state_dict(cfg, 0)
    table = native.param_table(_cfg(native, cfg))
    assert sorted(n for n, _, _ in table) == sorted(sd)
    for n, rows, cols in table:
        assert sd[n].numel() == rows * cols, n
        assert sd[n].shape[0] == rows, n


@pytest.mark.parametrize("name", ["cfg1", "cfg2", "cfg4"])
def test_mac_per_env_matches_oracle(native, name):
    cfg = make_cfg(name)
    assert native.lib.bsrl_mac_per_env(C.byref(_cfg(native, cfg))) == po.mac_per_env(cfg)


def test_sizes_grow_with_batch(native):
    c = _cfg(native, make_cfg("cfg2"))
    w1 = native.lib.bsrl_workspace_bytes(C.byref(c), 1024)
    w2 = native.lib.bsrl_workspace_bytes(C.byref(c), 2048)
    assert 0 < w1 < w2 <= 2 * w1 + 65536
    assert native.lib.bsrl_workspace_bytes(C.byref(c), 0) >= 0
    assert native.lib.bsrl_weights_bytes(C.byref(c)) > 2 * 5_000_000  # > fp16 copy of 5.7 M params


def test_config_errors_are_reported(native):
    good = make_cfg("cfg1")
    c = _cfg(native, good)
    assert native.lib.bsrl_config_validate(C.byref(c)) == 0
    c.embed = 100                      # not a multiple of 32
    assert native.lib.bsrl_config_validate(C.byref(c)) == -5
    assert "embed" in native.last_error()
    c = _cfg(native, good)
    c.n_heads = 3                      # 128 % 3 != 0
    assert native.lib.bsrl_config_validate(C.byref(c)) == -2
    c = _cfg(native, good)
    c.head_gears[4] = 9
    assert native.lib.bsrl_config_validate(C.byref(c)) == -2
    assert "head_gears" in native.last_error()
    c = _cfg(native, good)
    c.z_asinh = 0.0
    assert native.lib.bsrl_config_validate(C.byref(c)) == -2
    assert native.lib.bsrl_config_validate(None) == -1
    assert native.lib.bsrl_workspace_bytes(C.byref(c), 8) == -1


def test_null_and_size_checks_come_before_any_launch(native):
    """Bad arguments must be refused on the host (no device is present here at all)."""
    c = _cfg(native, make_cfg("tiny"))
    lib = native.lib
    assert lib.bsrl_forward(C.byref(c), None, None, 0, 4, None, None, None, None, 0, None) == -1
    assert lib.bsrl_pack_weights(C.byref(c), None, 0, None, 0, None) == -1
    assert lib.bsrl_linear(None, None, None, None, None, 0, 0, 8, 8, 32, 0, None) == -1
    fake = C.c_void_p(4096)            # never dereferenced: checks fail first
    assert lib.bsrl_linear(fake, fake, None, None, fake, 0, 0, 8, 8, 33, 0, None) == -2
    assert lib.bsrl_linear(C.c_void_p(4100), fake, None, None, fake, 0, 0, 8, 8, 32, 0, None) == -3
    assert lib.bsrl_attention(fake, fake, 4, 80, 2, 0, 29, fake, None) == -5   # head_dim 40
    assert lib.bsrl_attention(fake, fake, 4, 64, 2, 27, 5, fake, None) == -2   # queries past row 29
    # a workspace one byte short is refused
    need = lib.bsrl_workspace_bytes(C.byref(c), 4)
    assert lib.bsrl_forward(C.byref(c), C.c_void_p(256), fake, 0, 4, fake, fake, None,
                            C.c_void_p(512), need - 1, None) == -4


def test_policy_facade_host_side(native):
    from beatsaberrl_b200.policy import NotePolicy, bump_weights_version
    cfg = make_cfg("tiny", True, (5,) * 8 + (7,) + (5,) * 20)
    torch.manual_seed(9)
    m = NotePolicy(**cfg.ref_kwargs())
    sd = po.build_state_dict(cfg, 9)
    msd = m.state_dict()
    assert set(msd) == set(sd)
    for k in sd:                        # same creation order -> same seeded init as the reference
        assert torch.equal(msd[k], sd[k]), k
    assert m.k_max == 7 and m.n_lead == 5 and m.arch["head_gears"][8] == 7
    assert m.mac_per_env() == po.mac_per_env(cfg)
    with pytest.raises(RuntimeError):   # no CPU path
        m.forward_stacked(torch.zeros(2, 630))
    acc = NotePolicy(fp16_accum="all")      # a permission for cuBLAS in the reference: accepted, recorded, fp32 accumulation kept
    assert acc.arch["fp16_accum"] == "all" and acc.fp16_accum == "all"
    with pytest.raises(ValueError):
        NotePolicy(fp16_accum="sometimes")
    with pytest.raises(ValueError):
        NotePolicy(trunk_arch="mlp")
    with pytest.raises(ValueError):
        NotePolicy(z_asinh=0.0)
    bump_weights_version()
