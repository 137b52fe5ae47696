"""ctypes binding of libbsrl.so -- the only way Python reaches the kernels.

There is no fallback: if the library is missing the import of this module raises, and every
entry point turns a non-zero status into ``BsrlError`` carrying the library's message.
"""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = Path(__import__("os").environ.get("BSRL_LIB") or PKG / "_lib" / "libbsrl.so")   # BSRL_LIB: alternative build
HEADER = PKG.parent / "include" / "bsrl.h"

N_ACT_HEADS = 29
F32, F16, U8, I32, I64 = 0, 1, 2, 3, 4


class BsrlError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"bsrl status {status}: {message}")
        self.status = status


class Config(C.Structure):
    """Mirror of ``bsrl_config`` (include/bsrl.h)."""
    _fields_ = [("embed", C.c_int32), ("n_heads", C.c_int32), ("n_blocks", C.c_int32),
                ("ffn_mult", C.c_int32), ("trunk_dim", C.c_int32), ("trunk_hidden", C.c_int32),
                ("value_bins", C.c_int32), ("note_geo", C.c_int32),
                ("head_gears", C.c_int32 * N_ACT_HEADS),
                ("z_asinh", C.c_float), ("value_vmax", C.c_float), ("eps", C.c_float),
                ("emb_ln", C.c_int32), ("final_ln", C.c_int32), ("game_flux", C.c_int32),
                ("value_residual", C.c_int32), ("trunk_v2", C.c_int32)]


class GConfig(C.Structure):
    """Mirror of ``bsrl_gconfig`` (include/bsrl.h): the single-body-token layout."""
    _fields_ = [("embed", C.c_int32), ("n_heads", C.c_int32), ("n_blocks", C.c_int32), ("ffn_mult", C.c_int32),
                ("n_obj", C.c_int32), ("n_gears", C.c_int32), ("body_dim", C.c_int32), ("obj_dim", C.c_int32),
                ("eps", C.c_float)]


def make_config(embed, n_heads, n_blocks, ffn_mult, trunk_dim, trunk_hidden, value_bins, note_geo,
                head_gears, z_asinh=8.0, value_vmax=6.0, eps=1e-5, emb_ln=False, final_ln=False,
                game_flux=False, value_residual=False, trunk_v2=False) -> Config:
    c = Config()
    c.embed, c.n_heads, c.n_blocks, c.ffn_mult = embed, n_heads, n_blocks, ffn_mult
    c.trunk_dim, c.trunk_hidden, c.value_bins, c.note_geo = trunk_dim, trunk_hidden, value_bins, int(note_geo)
    for j, k in enumerate(head_gears):
        c.head_gears[j] = int(k)
    c.z_asinh, c.value_vmax, c.eps = z_asinh, value_vmax, eps
    c.emb_ln, c.final_ln, c.game_flux = int(emb_ln), int(final_ln), int(game_flux)
    c.value_residual = int(value_residual)
    c.trunk_v2 = int(trunk_v2)
    return c


def declared_symbols() -> list[str]:
    """Every function name ``include/bsrl.h`` declares."""
    text = HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bsrl_[a-z0-9_]+)\s*\(", text)))


if not LIB_PATH.exists():
    raise ImportError(f"{LIB_PATH} is missing: build it with `python -m beatsaberrl_b200.build` "
                      "(there is no CPU or torch fallback for the policy forward)")
lib = C.CDLL(str(LIB_PATH))

_P = C.c_void_p
_CFG = C.POINTER(Config)
_sig = {
    "bsrl_abi_version": (C.c_int, []),
    "bsrl_last_error": (C.c_char_p, []),
    "bsrl_config_validate": (C.c_int, [_CFG]),
    "bsrl_mac_per_env": (C.c_int64, [_CFG]),
    "bsrl_param_count": (C.c_int32, [_CFG]),
    "bsrl_param_desc": (C.c_int, [_CFG, C.c_int32, C.c_char_p, C.c_int32, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "bsrl_weights_bytes": (C.c_int64, [_CFG]),
    "bsrl_pack_weights": (C.c_int, [_CFG, C.POINTER(_P), C.c_int32, _P, C.c_int64, _P]),
    "bsrl_adam_step_pack": (C.c_int, [_CFG, C.POINTER(_P), C.POINTER(_P), C.POINTER(_P), C.POINTER(_P), C.c_int32,
                                      C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_float, C.c_float, C.c_float,
                                      C.c_int32, _P, _P, _P, C.c_int64, _P]),
    "bsrl_workspace_bytes": (C.c_int64, [_CFG, C.c_int64]),
    "bsrl_forward": (C.c_int, [_CFG, _P, _P, C.c_int32, C.c_int64, _P, _P, _P, _P, C.c_int64, _P]),
    "bsrl_train_save_bytes": (C.c_int64, [_CFG, C.c_int64]),
    "bsrl_backward_workspace_bytes": (C.c_int64, [_CFG, C.c_int64]),
    "bsrl_grad_floats": (C.c_int64, [_CFG, C.POINTER(C.c_int64), C.c_int32]),
    "bsrl_forward_train": (C.c_int, [_CFG, _P, _P, C.c_int32, C.c_int64, _P, C.c_int32, _P, _P, _P, _P, _P, _P,
                                     _P, C.c_int64, _P, C.c_int64, _P]),
    "bsrl_backward": (C.c_int, [_CFG, _P, C.c_int64, _P, C.c_int32, _P, C.c_int64, _P, _P, _P, _P, _P, C.c_float,
                                _P, C.c_int64, _P, C.c_int64, _P]),
    "bsrl_layernorm_bwd": (C.c_int, [_P, _P, C.c_float, _P, _P, C.c_int64, C.c_int32, _P, _P, _P, _P]),
    "bsrl_attention_bwd": (C.c_int, [_P, _P, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _P, _P, _P]),
    "bsrl_head_tail_bwd": (C.c_int, [_CFG, _P, _P, C.c_int64, _P, C.c_int32, _P, _P, _P, _P, _P, C.c_float, _P, C.c_int32,
                                     _P, C.c_int32, _P]),
    "bsrl_linear_bwd_scratch_bytes": (C.c_int64, [C.c_int64, C.c_int32, C.c_int32]),
    "bsrl_linear_bwd": (C.c_int, [_P, _P, _P, C.c_int64, C.c_int32, C.c_int32, _P, _P, _P, C.c_int32, _P, C.c_int64, _P]),
    "bsrl_g_config_validate": (C.c_int, [C.POINTER(GConfig)]),
    "bsrl_g_obs_dim": (C.c_int32, [C.POINTER(GConfig)]),
    "bsrl_g_mac_per_env": (C.c_int64, [C.POINTER(GConfig)]),
    "bsrl_g_param_count": (C.c_int32, [C.POINTER(GConfig)]),
    "bsrl_g_param_desc": (C.c_int, [C.POINTER(GConfig), C.c_int32, C.c_char_p, C.c_int32, C.POINTER(C.c_int64),
                                    C.POINTER(C.c_int64)]),
    "bsrl_g_weights_bytes": (C.c_int64, [C.POINTER(GConfig)]),
    "bsrl_g_pack_weights": (C.c_int, [C.POINTER(GConfig), C.POINTER(_P), C.c_int32, _P, C.c_int64, _P]),
    "bsrl_g_workspace_bytes": (C.c_int64, [C.POINTER(GConfig), C.c_int64]),
    "bsrl_g_forward": (C.c_int, [C.POINTER(GConfig), _P, _P, C.c_int64, _P, C.c_int32, _P, _P, _P, _P, _P, _P,
                                 C.c_int64, _P]),
    "bsrl_fixed_scratch_bytes": (C.c_int64, []),
    "bsrl_forward_fixed": (C.c_int, [_CFG, _P, _P, C.c_int32, C.c_int64, _P, _P, _P]),
    "bsrl_forward_act": (C.c_int, [_CFG, _P, _P, C.c_int32, C.c_int64, _P, C.c_int32, _P, _P, _P, _P, _P, _P,
                                   _P, C.c_int64, _P]),
    "bsrl_forward_sample": (C.c_int, [_CFG, _P, _P, C.c_int32, C.c_int64, _P, _P, _P, _P, _P, _P, _P, _P, C.c_int64, _P]),
    "bsrl_forward_rollout": (C.c_int, [_CFG, _P, _P, C.c_int32, C.c_int64, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
                                       _P, C.c_int64, _P]),
    "bsrl_token_lane": (C.c_int32, [C.c_int32, C.c_int32]),
    "bsrl_device_status": (C.c_int, []),
    "bsrl_set_engine": (C.c_int, [C.c_int32]),
    "bsrl_profile_enable": (C.c_int, [C.c_int32]),
    "bsrl_profile_stage_count": (C.c_int32, []),
    "bsrl_profile_stage_name": (C.c_char_p, [C.c_int32]),
    "bsrl_profile_stage": (C.c_int, [C.c_int32, C.POINTER(C.c_double), C.POINTER(C.c_int64),
                                     C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "bsrl_embed": (C.c_int, [_CFG, _P, _P, C.c_int32, C.c_int64, _P, _P, _P, C.c_int64, _P]),
    "bsrl_trunk_heads": (C.c_int, [_CFG, _P, _P, C.c_int64, _P, _P, _P, C.c_int64, _P]),
    "bsrl_head_tail": (C.c_int, [_CFG, _P, _P, C.c_int64, _P, C.c_int32, _P, _P, _P, _P, _P, _P]),
    "bsrl_head_layout": (C.c_int, [_CFG, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "bsrl_workspace_region": (C.c_int, [_CFG, C.c_int64, C.c_char_p, C.POINTER(C.c_int64), C.POINTER(C.c_int64),
                                        C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_int32)]),
    "bsrl_standin_env_step": (C.c_int, [_P, C.c_int64, _P, _P, _P, _P, _P]),
    "bsrl_selftest_wait_timeout": (C.c_int, [C.c_int32, _P]),
    "bsrl_layernorm": (C.c_int, [_P, _P, _P, C.c_float, C.c_int64, C.c_int32, _P, C.c_int64, _P]),
    "bsrl_linear": (C.c_int, [_P, _P, _P, _P, _P, C.c_int32, C.c_int32, C.c_int64, C.c_int32, C.c_int32,
                              C.c_int32, _P]),
    "bsrl_block_tail": (C.c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, C.c_float, C.c_int64, C.c_int32,
                                  C.c_int32, _P, _P, _P, _P, _P]),
    "bsrl_qkv_attention": (C.c_int, [_P, _P, _P, _P, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _P]),
    "bsrl_attention": (C.c_int, [_P, _P, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _P]),
    "bsrl_apply_updates_pack": (C.c_int, [_CFG, C.POINTER(_P), C.POINTER(_P), C.c_int32, _P, _P, C.c_int64, _P]),
    "bsrl_linear_ln": (C.c_int, [_P, _P, _P, _P, _P, _P, C.c_float, C.c_int64, C.c_int32, C.c_int32, _P, _P, _P]),
    "bsrl_qkv_attention_body": (C.c_int, [_P, _P, _P, _P, _P, C.c_int64, C.c_int32, C.c_int32, C.c_int32, _P, _P]),
    "bsrl_attention_tokens": (C.c_int, [_P, _P, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _P]),
}
for _name, (_res, _args) in _sig.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args

import os as _os
if _os.environ.get("BSRL_ENGINE", "") == "mma":      # cross-check runs: warp-MMA kernels only
    lib.bsrl_set_engine(1)


def last_error() -> str:
    return (lib.bsrl_last_error() or b"").decode()


def check(status: int) -> None:
    if status != 0:
        raise BsrlError(status, last_error())


def param_table(cfg: Config):
    """[(state_dict name, rows, cols), ...] in the order ``bsrl_pack_weights`` expects."""
    n = lib.bsrl_param_count(C.byref(cfg))
    if n < 0:
        raise BsrlError(n, last_error())
    out = []
    buf = C.create_string_buffer(128)
    r, c = C.c_int64(), C.c_int64()
    for i in range(n):
        check(lib.bsrl_param_desc(C.byref(cfg), i, buf, 128, C.byref(r), C.byref(c)))
        out.append((buf.value.decode(), r.value, c.value))
    return out


def profile_read():
    """{stage: dict(ms, launches, flops, bytes)} accumulated since bsrl_profile_enable(1);
    the caller synchronises the stream first."""
    out = {}
    for i in range(lib.bsrl_profile_stage_count()):
        ms, n, fl, by = C.c_double(), C.c_int64(), C.c_double(), C.c_double()
        check(lib.bsrl_profile_stage(i, C.byref(ms), C.byref(n), C.byref(fl), C.byref(by)))
        if n.value:
            out[lib.bsrl_profile_stage_name(i).decode()] = dict(ms=ms.value, launches=n.value,
                                                                flops=fl.value, bytes=by.value)
    return out
