"""Generates tests/golden/body_policy_golden.npz for the single-body-token layout.

    python tests/golden/make_golden_g.py [/path/to/reference]

The layout's tokenizer and readout do not exist in the reference, but its blocks do: each case builds the
reference's own ``policy.Block`` modules (python/policy.py:483-715) with ``ffn[1]`` swapped to ``nn.GELU()``,
puts them between two ``nn.Linear`` encoders and the ``heads`` / ``value`` Linears created in the order
``oracle/body_policy_oracle.build_state_dict`` uses, loads the oracle's seeded weights into them, and runs the
reference Block code on a stored obs batch in fp32 on the CPU, following the calling protocol of the
reference's forward (python/policy.py:1263-1305: deferred FFN residual handed to the next block as ``delta``,
last block on the first row).  Stored: obs, actions, logits, value, log-prob, entropy, parameter checksums.
"""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.nn as nn

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
from oracle import body_policy_oracle as bo  # noqa: E402
from oracle import policy_oracle as po  # noqa: E402

CASES = [  # name, config, weight seed, xavier, ln_jitter, B, padded, obs seed
    ("gtiny", "gtiny", 31, False, 0.1, 16, True, 41),
    ("gtiny_xavier", "gtiny", 32, True, 0.0, 16, False, 42),
    ("cfg1", "cfg1", 0, False, 0.0, 8, True, 43),
]


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("BSRL_REFERENCE", str(Path(__file__).resolve().parents[3] / "reference"))
    sys.dont_write_bytecode = True
    sys.path.insert(0, os.path.join(ref, "python"))
    import policy as rp  # the reference module

    out = {}
    for name, cfg_name, seed, xav, jit, B, padded, oseed in CASES:
        cfg = bo.named_config(cfg_name)
        sd = bo.build_state_dict(cfg, seed, xavier=xav, ln_jitter=jit)
        d = cfg.embed
        blocks = []
        for i in range(cfg.n_blocks):
            blk = rp.Block(d, cfg.n_heads, cfg.ffn_mult).eval()
            blk.ffn[1] = nn.GELU()
            blk.load_state_dict({k[len(f"blocks.{i}."):]: v for k, v in sd.items() if k.startswith(f"blocks.{i}.")})
            blocks.append(blk)
        obs = bo.make_obs(B, cfg, oseed, padded=padded)
        act = bo.make_actions(B, cfg, oseed + 1)
        N = cfg.n_obj
        with torch.no_grad():
            body = obs[:, :cfg.body_dim]
            objs = obs[:, cfg.body_dim: cfg.body_dim + N * cfg.obj_dim].reshape(B, N, cfg.obj_dim)
            live = obs[:, cfg.body_dim + N * cfg.obj_dim:]
            lin = lambda nm, x: torch.nn.functional.linear(x, sd[nm + ".weight"], sd[nm + ".bias"])
            tokens = torch.cat([lin("body_enc", body)[:, None], lin("obj_enc", objs)], 1)
            attn_bias = torch.nn.functional.pad((live - 1.0) * rp.MASK_BIAS, (1, 0)).unsqueeze(1)   # (B, 1, T)
            delta = delta_b = None
            for blk in blocks[:-1]:
                tokens, delta, delta_b = blk(tokens, None, attn_bias=attn_bias, delta=delta, delta_bias=delta_b)
            lead = blocks[-1](tokens, None, n_queries=1, attn_bias=attn_bias, delta=delta, delta_bias=delta_b)
            h = lead[:, 0]
            logits = lin("heads", h).view(B, 29, cfg.n_gears)
            value = lin("value", h)[:, 0]
            lp, ent, ent_h = po.evaluate_actions(logits, act)
        out[f"{name}/obs"] = obs.numpy()
        out[f"{name}/actions"] = act.numpy()
        out[f"{name}/logits"] = logits.numpy()
        out[f"{name}/value"] = value.numpy()
        out[f"{name}/logprob"] = lp.numpy()
        out[f"{name}/entropy"] = ent.numpy()
        names = sorted(sd)
        out[f"{name}/param_sums"] = np.array([[float(sd[k].double().sum()), float(sd[k].double().abs().sum())] for k in names])
        out[f"{name}/param_names"] = np.array(names)
    np.savez_compressed(HERE / "body_policy_golden.npz", **out)
    print("wrote", HERE / "body_policy_golden.npz", sum(v.nbytes for v in out.values()), "bytes raw")


if __name__ == "__main__":
    main()
