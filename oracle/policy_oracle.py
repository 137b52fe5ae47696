"""CPU oracle for the batched transformer-policy forward (TEST INFRASTRUCTURE).

This file is the checker, not the product.  Only tests, the smoke check and
the CPU-baseline leg of the benchmark may import it; the CUDA path never does.

It restates, in plain torch fp32 on the CPU, the arithmetic of the reference's
``NotePolicy`` forward (reference ``python/policy.py``):

* obs lane routing               -> ``python/policy.py:174-275`` and ``:1099-1105``
* hand-relative note geometry    -> ``python/policy.py:329-404``
* four token encoders            -> ``python/policy.py:940-952`` and ``:1224-1249``
* additive key mask              -> ``python/policy.py:422-428`` and ``:1257-1260``
* pre-LN transformer block       -> ``python/policy.py:524-715`` (fp32 record path
  ``:686-690``), residual+LN pass ``python/fused_ln.py:140-164``
* final block on the lead rows   -> ``python/policy.py:593-631`` and ``:1302-1305``
* SimBa readout trunk            -> ``python/policy.py:1107-1138``
* packed action heads + fill     -> ``python/policy.py:1311-1344``
* adapool critic + HL-Gauss      -> ``python/policy.py:1346-1403`` and ``:931-935``
* log-softmax / log-prob / entropy tail -> ``python/policy.py:1467-1516``

Parity pin: ``tests/test_oracle_vs_reference.py`` compares this restatement with
the reference module itself (when the reference checkout is importable) and
``tests/golden/`` holds vectors generated from the reference by
``tests/golden/make_golden.py``; the CPU suite checks the oracle against them.

The weights are addressed by the reference's ``state_dict`` names, so a
``NotePolicy.state_dict()`` can be fed in unchanged.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn as nn
import torch.nn.functional as F

# ----------------------------------------------------------------------------
# Observation layout (facts of the reference's obs contract, python/policy.py:147-275)
# ----------------------------------------------------------------------------
OBS_DIM = 630
N_SLOTS = 24                    # entity window
NOTE_FEAT = 18
N_LEAD = 5                      # saber_L, saber_R, torso, leg_L, leg_R
N_TOKENS = N_LEAD + N_SLOTS     # 29
N_HEADS_ACT = 29                # factored action heads
MASK_BIAS = 16384.0             # python/policy.py:428
MASKED_LOGIT = -1e9             # python/policy.py:434
GEO_FEAT = 22                   # python/policy.py:316

# named obs blocks: name -> (first lane, count)
_BLOCKS = {
    "root": (0, 15),
    "q_spine": (15, 3), "q_arm_l": (18, 8), "q_arm_r": (26, 8),
    "q_leg_l": (34, 6), "q_leg_r": (40, 6),
    "qd_spine": (46, 3), "qd_arm_l": (49, 7), "qd_arm_r": (56, 7),
    "qd_leg_l": (63, 6), "qd_leg_r": (69, 6),
    "hand_l": (75, 11), "hand_r": (86, 11),
    "head": (97, 3), "contact": (100, 2),
    "notes": (102, N_SLOTS * NOTE_FEAT),
    "mask": (534, N_SLOTS),
    "ground_l": (558, 2), "ground_r": (560, 2),
    "pts_elbow_l": (562, 3), "pts_elbow_r": (565, 3),
    "pts_knee_l": (568, 3), "pts_knee_r": (571, 3),
    "pts_foot_l": (574, 3), "pts_foot_r": (577, 3),
    "vel_elbow_l": (580, 3), "vel_elbow_r": (583, 3),
    "vel_knee_l": (586, 3), "vel_knee_r": (589, 3),
    "vel_foot_l": (592, 3), "vel_foot_r": (595, 3),
    "prev_l": (598, 5), "prev_r": (603, 5),
    "tau_spine": (608, 3), "tau_arm": (611, 7), "tau_leg": (618, 6),
    "tip_l": (624, 3), "tip_r": (627, 3),
}
OFF_NOTES = _BLOCKS["notes"][0]
OFF_MASK = _BLOCKS["mask"][0]
OBS_HEAD_Z = 99                 # python/policy.py:321

# which blocks feed which lead token, in lane order
TOKEN_BLOCKS = {
    "saber_l": ["q_arm_l", "qd_arm_l", "hand_l", "pts_elbow_l", "vel_elbow_l",
                "prev_l", "tau_arm", "tip_l"],
    "saber_r": ["q_arm_r", "qd_arm_r", "hand_r", "pts_elbow_r", "vel_elbow_r",
                "prev_r", "tau_arm", "tip_r"],
    "torso": ["root", "q_spine", "qd_spine", "head", "contact", "tau_spine"],
    "leg_l": ["q_leg_l", "qd_leg_l", "ground_l", "pts_knee_l", "pts_foot_l",
              "vel_knee_l", "vel_foot_l", "tau_leg"],
    "leg_r": ["q_leg_r", "qd_leg_r", "ground_r", "pts_knee_r", "pts_foot_r",
              "vel_knee_r", "vel_foot_r", "tau_leg"],
}
LEAD_ORDER = ("saber_l", "saber_r", "torso", "leg_l", "leg_r")


def token_segments(name: str):
    """[(first lane, count), ...] of one lead token, merged where adjacent."""
    segs = []
    for b in TOKEN_BLOCKS[name]:
        s, n = _BLOCKS[b]
        if segs and segs[-1][0] + segs[-1][1] == s:
            segs[-1] = (segs[-1][0], segs[-1][1] + n)
        else:
            segs.append((s, n))
    return segs


def token_lanes(name: str):
    """Flat obs lane list of one lead token."""
    return [s + i for s, n in token_segments(name) for i in range(n)]


SABER_FEAT = len(token_lanes("saber_l"))     # 47
TORSO_FEAT = len(token_lanes("torso"))       # 29
LEG_FEAT = len(token_lanes("leg_l"))         # 32
assert (SABER_FEAT, TORSO_FEAT, LEG_FEAT) == (47, 29, 32)


@dataclass
class PolicyConfig:
    """Hyper-parameters that shape the forward (reference ctor, python/policy.py:795-806)."""
    embed: int = 128
    trunk_dim: int = 256
    n_blocks: int = 3
    n_heads: int = 4
    n_gears: int = 5
    ffn_mult: int = 4
    note_geo: bool = False
    value_bins: int = 101
    value_vmax: float = 6.0
    trunk_hidden: int | None = None
    z_asinh: float = 8.0
    head_gears: tuple | None = None
    eps: float = 1e-5
    emb_ln: bool = False        # LayerNorm on the token embeddings (python/policy.py:962, :1261-1262)
    final_ln: bool = False      # LayerNorm on the lead rows leaving the last block (:969, :1306-1307)
    game: str = "standard"      # "flux": bar slots aim the geometry lanes at lanes 12, 13 (:357-360)
    value_residual: bool = False  # blocks after the first mix block 0's values in: v <- a v + b v0 (:512-520, :611)
    trunk_arch: str = "simba"    # "simbav2": hyperspherical trunk (python/policy.py:984-1021, :1140-1155)

    def __post_init__(self):
        if self.head_gears is None:
            self.head_gears = (self.n_gears,) * N_HEADS_ACT
        self.head_gears = tuple(int(k) for k in self.head_gears)
        assert len(self.head_gears) == N_HEADS_ACT
        assert all(3 <= k <= 7 for k in self.head_gears)
        assert self.embed % self.n_heads == 0
        if self.trunk_hidden is None:
            self.trunk_hidden = self.trunk_dim

    @property
    def k_max(self) -> int:
        return max(self.head_gears)

    @property
    def note_in(self) -> int:
        return NOTE_FEAT + (GEO_FEAT if self.note_geo else 0)

    def ref_kwargs(self) -> dict:
        """Keyword arguments that build the same network with the reference ctor."""
        return dict(embed=self.embed, trunk_dim=self.trunk_dim, n_blocks=self.n_blocks,
                    n_heads=self.n_heads, n_gears=self.n_gears, ffn_mult=self.ffn_mult,
                    note_geo=self.note_geo, value_bins=self.value_bins,
                    value_vmax=self.value_vmax, trunk_hidden=self.trunk_hidden,
                    z_asinh=self.z_asinh, head_gears=self.head_gears, emb_ln=self.emb_ln,
                    final_ln=self.final_ln, game=self.game, value_residual=self.value_residual,
                    trunk_arch=self.trunk_arch)


# the five benchmark configurations in reference-drop-in form (T = 29, n_lead = 5)
def named_config(name: str) -> PolicyConfig:
    table = {
        "cfg1": dict(embed=128, trunk_dim=256, n_blocks=2, n_heads=4, n_gears=5),
        "cfg2": dict(embed=256, trunk_dim=512, n_blocks=4, n_heads=8, n_gears=5),
        "cfg4": dict(embed=512, trunk_dim=1024, n_blocks=6, n_heads=8, n_gears=7),
        "tiny": dict(embed=64, trunk_dim=128, n_blocks=2, n_heads=2, n_gears=5),
        "recipe": dict(embed=192, trunk_dim=384, n_blocks=6, n_heads=4, n_gears=5,
                       note_geo=True),
    }
    table["cfg3"] = table["cfg2"]
    table["cfg5"] = table["cfg2"]
    return PolicyConfig(**table[name])


# ----------------------------------------------------------------------------
# Weights: the reference's parameter names, creation order and default init
# ----------------------------------------------------------------------------
def linear_specs(cfg: PolicyConfig):
    """(state_dict prefix, in_features, out_features) of every Linear, in the order
    the reference ctor creates them (python/policy.py:940-1067) -- the order fixes the
    RNG stream of a seeded init."""
    d, D, Hh = cfg.embed, cfg.trunk_dim, cfg.trunk_hidden
    s = []

    def mlp(prefix, sizes):
        for i in range(len(sizes) - 1):
            s.append((f"{prefix}.{2 * i}", sizes[i], sizes[i + 1]))

    mlp("note_mlp", [cfg.note_in, d, d])
    mlp("saber_mlp", [SABER_FEAT + 2, d, d])
    mlp("torso_mlp", [TORSO_FEAT, d, d])
    mlp("leg_mlp", [LEG_FEAT + 2, d, d])
    for i in range(cfg.n_blocks):
        p = f"blocks.{i}"
        for nm in ("q_proj", "k_proj", "v_proj", "out_proj"):
            s.append((f"{p}.{nm}", d, d))
        mlp(f"{p}.ffn", [d, cfg.ffn_mult * d, d])
    if cfg.trunk_arch == "simbav2":
        s += [("trunk_in", N_LEAD * d, D), ("trunk_w1", D, Hh), ("trunk_w2", Hh, D)]
    else:
        s += [("trunk_proj", N_LEAD * d, D), ("trunk_fc1", D, Hh), ("trunk_fc2", Hh, D)]
    for j, k in enumerate(cfg.head_gears):
        s.append((f"heads.{j}", D, k))
    for nm in ("critic_q", "critic_k", "critic_v", "critic_out"):
        s.append((nm, d, d))
    mlp("critic_mlp", [d + D, D, D, cfg.value_bins])
    return s


def layernorm_specs(cfg: PolicyConfig):
    """(prefix, width) of every LayerNorm (their init draws no random numbers, so the order is free)."""
    out = []
    for i in range(cfg.n_blocks):
        out += [(f"blocks.{i}.ln_attn", cfg.embed), (f"blocks.{i}.ln_ffn", cfg.embed)]
    if cfg.trunk_arch != "simbav2":
        out += [("trunk_ln1", cfg.trunk_dim), ("trunk_ln2", cfg.trunk_dim)]
    out.append(("critic_ln", cfg.embed))
    if cfg.emb_ln:
        out.append(("emb_ln", cfg.embed))
    if cfg.final_ln:
        out.append(("final_ln", cfg.embed))
    return out


def build_state_dict(cfg: PolicyConfig, seed: int, xavier: bool = False,
                     ln_jitter: float = 0.0) -> dict:
    """Seeded weights with the reference's names.  ``torch.manual_seed(seed)`` followed
    by default ``nn.Linear`` init in ctor order reproduces ``NotePolicy(...)`` after the
    same seed; ``xavier`` then re-draws every Linear weight with ``xavier_uniform_`` in
    ``modules()`` order and zeroes the biases.  ``ln_jitter`` > 0 perturbs the LayerNorm
    affine parameters (they are 1/0 at init) so tests exercise them."""
    torch.manual_seed(seed)
    sd = {}
    lins = []
    for prefix, fin, fout in linear_specs(cfg):
        m = nn.Linear(fin, fout)
        lins.append((prefix, m))
        if prefix == "trunk_w2":
            # SimBaV2: orthogonal init of the three trunk matrices right after their creation (the
            # draws sit at this point of the RNG stream), zero frozen biases, rows projected onto the
            # unit sphere (python/policy.py:1003-1021, :1165-1177)
            for _, tm in lins[-3:]:
                nn.init.orthogonal_(tm.weight)
                nn.init.zeros_(tm.bias)
            with torch.no_grad():
                for _, tm in lins[-3:]:
                    tm.weight.div_(tm.weight.norm(dim=1, keepdim=True).clamp_min(1e-12))
    if xavier:
        # reference modules() order == ctor registration order for the Linears
        for _, m in lins:
            nn.init.xavier_uniform_(m.weight)
            nn.init.zeros_(m.bias)
    for prefix, m in lins:
        sd[prefix + ".weight"] = m.weight.detach().clone()
        sd[prefix + ".bias"] = m.bias.detach().clone()
    g = torch.Generator().manual_seed(seed + 7919)
    if cfg.trunk_arch == "simbav2":
        D, Hh = cfg.trunk_dim, cfg.trunk_hidden
        sd["trunk_s_in"] = torch.full((D,), math.sqrt(2.0 / D))
        sd["trunk_s_1"] = torch.full((Hh,), math.sqrt(2.0 / Hh))
        sd["trunk_alpha"] = torch.full((D,), 1.0 / math.sqrt(D))
        if ln_jitter > 0:
            for k in ("trunk_s_in", "trunk_s_1", "trunk_alpha"):
                sd[k] = sd[k] * (1.0 + ln_jitter * torch.randn(sd[k].shape, generator=g))
    if cfg.value_residual:   # (a, b) = (1, 0) at init; the jitter moves them so tests exercise the mix
        for i in range(1, cfg.n_blocks):
            sd[f"blocks.{i}.vres_a"] = torch.ones(1)
            sd[f"blocks.{i}.vres_b"] = torch.zeros(1)
            if ln_jitter > 0:
                sd[f"blocks.{i}.vres_a"] += ln_jitter * torch.randn(1, generator=g)
                sd[f"blocks.{i}.vres_b"] += 0.3 + ln_jitter * torch.randn(1, generator=g)
    for prefix, w in layernorm_specs(cfg):
        sd[prefix + ".weight"] = torch.ones(w)
        sd[prefix + ".bias"] = torch.zeros(w)
        if ln_jitter > 0:
            sd[prefix + ".weight"] += ln_jitter * torch.randn(w, generator=g)
            sd[prefix + ".bias"] += ln_jitter * torch.randn(w, generator=g)
    return sd


# ----------------------------------------------------------------------------
# Synthetic inputs (same recipe the benchmark and the tests use)
# ----------------------------------------------------------------------------
def make_obs(B: int, seed: int, padded: bool = False, note_geo_safe: bool = True):
    """obs ~ N(0,1) clipped to +-5, fp32 (B, 630).  Mask lanes are 1.0 everywhere, or,
    when ``padded``, a per-env count n ~ U{0..24} of live slots (first n live) with the
    dead slots' 18 feature lanes zeroed.  The is_wall lane (14) of every note is forced
    to {0,1} so the geometry lanes see the values the simulator writes."""
    g = torch.Generator().manual_seed(seed)
    obs = torch.randn(B, OBS_DIM, generator=g).clamp_(-5.0, 5.0)
    mask = torch.ones(B, N_SLOTS)
    if padded:
        n = torch.randint(0, N_SLOTS + 1, (B,), generator=g)
        mask = (torch.arange(N_SLOTS)[None, :] < n[:, None]).float()
    notes = obs[:, OFF_NOTES:OFF_MASK].view(B, N_SLOTS, NOTE_FEAT)
    if note_geo_safe:
        notes[:, :, 14] = (notes[:, :, 14] > 0.5).float()
    notes *= mask[:, :, None]
    obs[:, OFF_MASK:OFF_MASK + N_SLOTS] = mask
    return obs


def make_actions(B: int, cfg: PolicyConfig, seed: int):
    g = torch.Generator().manual_seed(seed)
    a = torch.stack([torch.randint(0, k, (B,), generator=g) for k in cfg.head_gears], 1)
    return a.to(torch.int32)


# ----------------------------------------------------------------------------
# Forward
# ----------------------------------------------------------------------------
def make_upstream(B: int, cfg: PolicyConfig, seed: int):
    """Upstream gradients of a PPO-like loss for the gradient parity tests: seeded, of the size a
    mean-reduced loss hands back (1 / B per env)."""
    g = torch.Generator().manual_seed(seed)
    return {"logprob": torch.randn(B, generator=g) / B, "entropy": 0.1 * torch.randn(B, generator=g) / B,
            "value": torch.randn(B, generator=g) / B,
            "value_logits": 0.2 * torch.randn(B, cfg.value_bins, generator=g) / B}


def frozen_params(cfg) -> tuple:
    """Parameters the reference keeps out of training: the SimBaV2 trunk's three biases are created zero with
    requires_grad False (python/policy.py:1003-1009), so their gradient is None there."""
    if cfg.trunk_arch == "simbav2":
        return ("trunk_in.bias", "trunk_w1.bias", "trunk_w2.bias")
    return ()


def grad_stats(name: str, g):
    """[norm, four fixed random projections] of a gradient tensor, float64; the projection vectors are
    seeded by the parameter's name, so they are the same wherever this runs."""
    seed = sum((i + 1) * ord(ch) for i, ch in enumerate(name)) % (2 ** 31)
    gen = torch.Generator().manual_seed(seed)
    g = g.detach().double().reshape(-1).cpu()
    r = torch.randn(4, g.numel(), generator=gen, dtype=torch.float64)
    return torch.cat([g.norm().reshape(1), r @ g])


def _lin(sd, name, x):
    return F.linear(x, sd[name + ".weight"], sd[name + ".bias"])


def _ln(sd, name, x, eps):
    return F.layer_norm(x, (x.shape[-1],), sd[name + ".weight"], sd[name + ".bias"], eps)


def _mlp2(sd, name, x):
    return _lin(sd, name + ".2", F.relu(_lin(sd, name + ".0", x)))


def note_geo(notes, sabers, z_asinh: float, z_off, flux: bool = False):
    """22 derived lanes per (env, slot): per hand [dx/2, dy/2, asinh(dz/8), asinh(|dp|/8),
    t_plane/3, vhat.cut, blade.cut] then per hand [along, perp, cut-plane distance,
    v_tip.cut] (python/policy.py:329-404; ``flux`` = the Flux game's variant).  notes (B,24,18), sabers
    (B,2,47), z_off (B,) -> (B,24,22), all fp32."""
    XN, YN, ZS, VN, HANDLE = 1.0, 0.75, 8.0, 6.0, 0.16
    z_m = torch.sinh(notes[..., 2]) * float(z_asinh)
    tx, ty = notes[..., 0], notes[..., 1]
    if flux:   # a bar slot is aimed at where it must be crossed (python/policy.py:357-360)
        is_bar = notes[..., 9] > 0.5
        tx = torch.where(is_bar, notes[..., 12], tx)
        ty = torch.where(is_bar, notes[..., 13], ty)
    npos = torch.stack([tx * XN, ty * YN, z_m], -1)
    cut = torch.stack([notes[..., 6], notes[..., 7], torch.zeros_like(z_m)], -1)
    live = 1.0 - notes[..., 14:15]
    speed = (-notes[..., 3:4] * ZS).clamp_min(1e-3)
    zrel = z_m - (z_off * XN)[:, None]
    tpl = (zrel[..., None] / speed).clamp(-0.5, 3.0) / 3.0
    first, second = [], []
    for hand in range(2):
        w = sabers[:, hand]
        wpos = torch.stack([w[:, 15] * XN, w[:, 16] * YN, w[:, 17]], -1)
        dpm = npos - wpos[:, None]
        dp = dpm * 0.5
        dist = dp.norm(dim=-1, keepdim=True)
        dp = torch.cat([dp[..., :2], torch.asinh(dp[..., 2:3] * 2.0 / 8.0)], -1)
        dist = torch.asinh(dist * 2.0 / 8.0)
        v = w[:, 18:21] * VN
        vhat = v / (v.norm(dim=-1, keepdim=True) + 0.05)
        vdot = (vhat[:, None] * cut).sum(-1, keepdim=True) * live
        b = w[:, 21:24]
        bdot = (b[:, None] * cut).sum(-1, keepdim=True) * live
        first += [dp, dist, tpl, vdot, bdot]
        ab = (dpm * b[:, None]).sum(-1, keepdim=True)
        along = torch.asinh((ab - HANDLE) * 0.5)
        perp = torch.asinh((dpm - ab * b[:, None]).norm(dim=-1, keepdim=True) * 0.5)
        vt = w[:, 44:47]
        pn = torch.linalg.cross(b, vt * VN)
        nhat = pn / (pn.norm(dim=-1, keepdim=True) + 0.05)
        cpd = torch.asinh((dpm * nhat[:, None]).sum(-1, keepdim=True) * 0.5)
        vtdot = (vt[:, None] * cut).sum(-1, keepdim=True) * live
        second += [along, perp, cpd, vtdot]
    return torch.cat(first + second, -1)


def token_features(cfg: PolicyConfig, obs):
    """obs (B,630) -> dict of per-encoder input rows and the key mask."""
    B = obs.shape[0]
    eye = torch.eye(2, dtype=obs.dtype).expand(B, 2, 2)
    sab = torch.stack([obs[:, token_lanes("saber_l")], obs[:, token_lanes("saber_r")]], 1)
    legs = torch.stack([obs[:, token_lanes("leg_l")], obs[:, token_lanes("leg_r")]], 1)
    notes = obs[:, OFF_NOTES:OFF_MASK].reshape(B, N_SLOTS, NOTE_FEAT)
    if cfg.note_geo:
        notes = torch.cat([notes, note_geo(notes, sab, cfg.z_asinh, obs[:, OBS_HEAD_Z], cfg.game == "flux")], -1)
    return dict(saber=torch.cat([sab, eye], -1), torso=obs[:, token_lanes("torso")],
                leg=torch.cat([legs, eye], -1), note=notes,
                mask=obs[:, OFF_MASK:OFF_MASK + N_SLOTS])


def embed_tokens(sd, cfg: PolicyConfig, obs):
    """(B,630) -> tokens (B,29,d) in the order [saber_L, saber_R, torso, leg_L, leg_R,
    slot_0..23] and the additive key bias (B,29)."""
    f = token_features(cfg, obs)
    tokens = torch.cat([_mlp2(sd, "saber_mlp", f["saber"]),
                        _mlp2(sd, "torso_mlp", f["torso"]).unsqueeze(1),
                        _mlp2(sd, "leg_mlp", f["leg"]),
                        _mlp2(sd, "note_mlp", f["note"])], 1)
    bias = F.pad((f["mask"] - 1.0) * MASK_BIAS, (N_LEAD, 0))
    return tokens, bias


def attention(q, k, v, bias, n_heads: int):
    """softmax(q k^T / sqrt(dh) + bias) v, heads concatenated.  q (B,Tq,d), k/v (B,T,d),
    bias (B,T) additive on keys."""
    B, Tq, d = q.shape
    T = k.shape[1]
    dh = d // n_heads
    qh = q.view(B, Tq, n_heads, dh).transpose(1, 2)
    kh = k.view(B, T, n_heads, dh).transpose(1, 2)
    vh = v.view(B, T, n_heads, dh).transpose(1, 2)
    s = qh @ kh.transpose(-2, -1) / (dh ** 0.5) + bias[:, None, None, :]
    return (torch.softmax(s, -1) @ vh).transpose(1, 2).reshape(B, Tq, d)


def block_forward(sd, cfg: PolicyConfig, i: int, x, bias, n_queries: int = 0, v0=None, want_v: bool = False):
    """One resolved pre-LN block.  ``x`` is the resolved residual stream entering the
    block (the reference defers the previous FFN's residual add into this block's LN
    pass; in fp32 that is the same sum).  Returns the resolved stream leaving the block,
    restricted to the first ``n_queries`` rows when > 0.  ``v0``: block 0's attention values,
    mixed into this block's (value residual); ``want_v``: also return this block's own values."""
    p = f"blocks.{i}"
    h = _ln(sd, p + ".ln_attn", x, cfg.eps)
    k, v = _lin(sd, p + ".k_proj", h), _lin(sd, p + ".v_proj", h)
    v_own = v
    if v0 is not None:
        v = sd[p + ".vres_a"] * v + sd[p + ".vres_b"] * v0
    if n_queries:
        x, h = x[:, :n_queries], h[:, :n_queries]
    q = _lin(sd, p + ".q_proj", h)
    att = _lin(sd, p + ".out_proj", attention(q, k, v, bias, cfg.n_heads))
    x = x + att
    h2 = _ln(sd, p + ".ln_ffn", x, cfg.eps)
    out = x + _mlp2(sd, p + ".ffn", h2)
    return (out, v_own) if want_v else out


def trunk_v2(sd, cfg: PolicyConfig, z):
    """SimBaV2 readout trunk (python/policy.py:1140-1155): x = l2n(s_in W_in z);
    y = l2n(W2 relu(s_1 W1 x)); x = l2n(x + alpha (y - x)); h = sqrt(D) x, alpha = 0.5 sqrt(D) trunk_alpha."""
    D = cfg.trunk_dim
    l2n = lambda v: F.normalize(v, dim=-1, eps=1e-6)
    x = l2n(_lin(sd, "trunk_in", z) * sd["trunk_s_in"])
    u = F.relu(_lin(sd, "trunk_w1", x) * sd["trunk_s_1"])
    y = l2n(_lin(sd, "trunk_w2", u))
    alpha = sd["trunk_alpha"] * (0.5 * math.sqrt(D))
    x = l2n(x + alpha * (y - x))
    return x * math.sqrt(D)


def trunk(sd, cfg: PolicyConfig, lead):
    """(B, 5d) -> (B, D): proj -> LN1 -> fc1 -> ReLU -> fc2 -> +res -> LN2 (or the SimBaV2 trunk)."""
    if cfg.trunk_arch == "simbav2":
        return trunk_v2(sd, cfg, lead)
    x = _lin(sd, "trunk_proj", lead)
    u = _ln(sd, "trunk_ln1", x, cfg.eps)
    dlt = _lin(sd, "trunk_fc2", F.relu(_lin(sd, "trunk_fc1", u)))
    return _ln(sd, "trunk_ln2", x + dlt, cfg.eps)


def value_centers(cfg: PolicyConfig):
    return torch.linspace(-float(cfg.value_vmax), float(cfg.value_vmax), cfg.value_bins)


def critic(sd, cfg: PolicyConfig, x_res, h, bias):
    """adapool critic: LN, torso-token query, 1-query MHA over all tokens, out-proj,
    3-layer MLP on [pooled, trunk], softmax-expectation over the bin centres."""
    hv = _ln(sd, "critic_ln", x_res, cfg.eps)
    q = _lin(sd, "critic_q", hv[:, 2:3])
    k, v = _lin(sd, "critic_k", hv), _lin(sd, "critic_v", hv)
    a = _lin(sd, "critic_out", attention(q, k, v, bias, cfg.n_heads)[:, 0])
    z = torch.cat([a, h], -1)
    z = F.relu(_lin(sd, "critic_mlp.0", z))
    z = F.relu(_lin(sd, "critic_mlp.2", z))
    vlogits = _lin(sd, "critic_mlp.4", z)
    return torch.softmax(vlogits, -1) @ value_centers(cfg), vlogits


def head_logits(sd, cfg: PolicyConfig, h):
    """(B, D) -> (B, 29, k_max); lanes past a head's gear count hold MASKED_LOGIT."""
    B = h.shape[0]
    out = h.new_full((B, N_HEADS_ACT, cfg.k_max), MASKED_LOGIT)
    for j, k in enumerate(cfg.head_gears):
        out[:, j, :k] = _lin(sd, f"heads.{j}", h)
    return out


@torch.no_grad()
def forward_stacked(sd, cfg: PolicyConfig, obs, want: bool = False):
    """obs (B,630) fp32 -> logits (B,29,k_max) fp32, value (B,) fp32.  With ``want`` also
    returns a dict of intermediates keyed by stage name."""
    obs = obs.float()
    B = obs.shape[0]
    keep = {}
    x, bias = embed_tokens(sd, cfg, obs)
    if cfg.emb_ln:
        x = _ln(sd, "emb_ln", x, cfg.eps)
    keep["tokens"], keep["key_bias"] = x, bias
    v0 = None
    for i in range(cfg.n_blocks - 1):
        if cfg.value_residual and i == 0:
            x, v0 = block_forward(sd, cfg, i, x, bias, want_v=True)
        else:
            x = block_forward(sd, cfg, i, x, bias, v0=v0)
        keep[f"x{i + 1}"] = x
    lead = block_forward(sd, cfg, cfg.n_blocks - 1, x, bias, n_queries=N_LEAD, v0=v0)
    if cfg.final_ln:
        lead = _ln(sd, "final_ln", lead, cfg.eps)
    keep["lead"] = lead
    h = trunk(sd, cfg, lead.reshape(B, -1))
    keep["trunk"] = h
    logits = head_logits(sd, cfg, h)
    value, vlogits = critic(sd, cfg, x, h, bias)
    keep["value_logits"] = vlogits
    return (logits, value, keep) if want else (logits, value)


@torch.no_grad()
def evaluate_actions(logits, actions, need_entropy: bool = True):
    """log-softmax tail for given actions: logprob (B,), per-head entropy (B,29) and its
    sum (B,) (python/policy.py:1473-1516)."""
    logsm = torch.log_softmax(logits, -1)
    lp = logsm.gather(-1, actions.long().unsqueeze(-1)).squeeze(-1).sum(-1)
    if not need_entropy:
        return lp, None, None
    ent_h = -(logsm.exp() * logsm).sum(-1)
    return lp, ent_h.sum(-1), ent_h


def mac_per_env(cfg: PolicyConfig) -> int:
    """Algorithmic multiply-accumulates of one env-forward (dense over all T keys)."""
    d, L, T, l, D = cfg.embed, cfg.n_blocks, N_TOKENS, N_LEAD, cfg.trunk_dim
    Hh = cfg.trunk_hidden
    f = cfg.ffn_mult
    enc = d * (N_SLOTS * cfg.note_in + 2 * (SABER_FEAT + 2) + TORSO_FEAT
               + 2 * (LEG_FEAT + 2)) + T * d * d
    blk = (4 + 2 * f) * T * d * d + 2 * T * T * d
    last = 2 * T * d * d + (2 + 2 * f) * l * d * d + 2 * l * T * d
    tr = l * d * D + 2 * D * Hh
    heads = D * sum(cfg.head_gears)
    cr = 2 * T * d * d + 2 * d * d + 2 * T * d + (d + D) * D + D * D + cfg.value_bins * D
    return enc + (L - 1) * blk + last + tr + heads + cr


def parity_report(logits, value, ref_logits, ref_value, atol=2e-2, rtol=1e-2):
    """Gate metrics: element tolerance |a-b| <= atol + rtol|b| on logits (live lanes) and
    value, and argmax agreement over the (B x 29) heads."""
    live = ref_logits > -1e8
    err = (logits - ref_logits).abs()
    ok = (err <= atol + rtol * ref_logits.abs()) | ~live
    verr = (value - ref_value).abs()
    vok = verr <= atol + rtol * ref_value.abs()
    agree = (logits.argmax(-1) == ref_logits.argmax(-1)).float().mean().item()
    return dict(logit_max_err=float(err[live].max()), logit_within=float(ok.float().mean()),
                value_max_err=float(verr.max()), value_within=float(vok.float().mean()),
                argmax_agree=agree)
