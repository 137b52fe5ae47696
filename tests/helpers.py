"""Shared test helpers: golden cases, oracle-backed policies, parity gates."""
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from oracle import policy_oracle as po  # noqa: E402

# must mirror tests/golden/make_golden.py CASES
GOLDEN_CASES = {
    "tiny_plain": dict(cfg="tiny", geo=False, hg=None, xavier=False, seed=11, jitter=0.0),
    "tiny_geo_mixed": dict(cfg="tiny", geo=True, hg=(5,) * 8 + (7,) + (5,) * 6 + (7,) + (5,) * 13,
                           xavier=True, seed=12, jitter=0.1),
    "cfg1": dict(cfg="cfg1", geo=False, hg=None, xavier=False, seed=0, jitter=0.0),
    "tiny_options": dict(cfg="tiny", geo=True, hg=None, xavier=False, seed=13, jitter=0.1,
                         opts=dict(emb_ln=True, final_ln=True, game="flux")),
    "tiny_vres": dict(cfg="tiny", geo=False, hg=None, xavier=False, seed=14, jitter=0.1,
                      opts=dict(value_residual=True, n_blocks=3)),
    "tiny_simbav2": dict(cfg="tiny", geo=False, hg=None, xavier=False, seed=15, jitter=0.1,
                         opts=dict(trunk_arch="simbav2")),
}


def make_cfg(name, geo=False, hg=None, opts=None):
    cfg = po.named_config(name)
    cfg.note_geo = geo
    cfg.head_gears = hg
    for k, v in (opts or {}).items():
        setattr(cfg, k, v)
    cfg.__post_init__()
    return cfg


def golden_case(name):
    c = GOLDEN_CASES[name]
    cfg = make_cfg(c["cfg"], c["geo"], c["hg"], c.get("opts"))
    sd = po.build_state_dict(cfg, c["seed"], xavier=c["xavier"], ln_jitter=c["jitter"])
    return cfg, sd


def cuda_policy(cfg, sd, device="cuda"):
    """The product's NotePolicy with the oracle's weights loaded."""
    from beatsaberrl_b200.policy import NotePolicy
    m = NotePolicy(**cfg.ref_kwargs())
    m.load_state_dict(sd)
    return m.to(device)


# parity gates of the forward: |a-b| <= ATOL + RTOL*|b| on every logit and value,
# argmax over gears equal on >= 99.9% of the (B x 29) heads
ATOL, RTOL, ARGMAX_MIN = 2e-2, 1e-2, 0.999


def assert_parity(logits, value, ref_logits, ref_value, argmax_min=ARGMAX_MIN):
    rep = po.parity_report(logits.float().cpu(), value.float().cpu(), ref_logits, ref_value, ATOL, RTOL)
    assert rep["logit_within"] == 1.0, rep
    assert rep["value_within"] == 1.0, rep
    assert rep["argmax_agree"] >= argmax_min, rep
    return rep
