"""The oracle against the live reference module (runs only where the reference checkout is)."""
import sys

import pytest
import torch

from conftest import REFERENCE
from helpers import make_cfg, po

pytestmark = pytest.mark.skipif(not (REFERENCE / "python" / "policy.py").exists(),
                                reason="reference checkout not present")


@pytest.fixture(scope="module")
def ref_policy():
    sys.dont_write_bytecode = True
    sys.path.insert(0, str(REFERENCE / "python"))
    import policy as rp
    return rp


@pytest.mark.parametrize("name,geo,xavier,seed", [("tiny", False, False, 5), ("tiny", True, True, 6),
                                                  ("cfg1", True, False, 7)])
def test_oracle_equals_reference(ref_policy, name, geo, xavier, seed):
    cfg = make_cfg(name, geo)
    torch.manual_seed(seed)
    m = ref_policy.NotePolicy(**cfg.ref_kwargs()).eval()
    if xavier:
        for mod in m.modules():
            if isinstance(mod, torch.nn.Linear):
                torch.nn.init.xavier_uniform_(mod.weight)
                torch.nn.init.zeros_(mod.bias)
    sd = po.build_state_dict(cfg, seed, xavier=xavier)
    rsd = m.state_dict()
    assert set(sd) == set(rsd)
    for k in sd:
        assert torch.equal(sd[k], rsd[k]), k
    obs = po.make_obs(32, seed, padded=True)
    act = po.make_actions(32, cfg, seed)
    with torch.no_grad():
        rl, rv = m.forward_stacked(obs)
        _, rlp, rent, _ = m.get_action_and_value(obs, act)
    l, v = po.forward_stacked(sd, cfg, obs)
    lp, ent, _ = po.evaluate_actions(l, act)
    torch.testing.assert_close(l, rl, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(v, rv, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(lp, rlp, atol=5e-5, rtol=1e-5)
    torch.testing.assert_close(ent, rent, atol=5e-5, rtol=1e-5)


def test_lane_tables(ref_policy):
    assert tuple(po.token_lanes("saber_l")) == ref_policy._SABER_L_IDX
    assert tuple(po.token_lanes("saber_r")) == ref_policy._SABER_R_IDX
    assert tuple(po.token_lanes("torso")) == ref_policy._TORSO_IDX
    assert tuple(po.token_lanes("leg_l")) == ref_policy._LEG_L_IDX
    assert tuple(po.token_lanes("leg_r")) == ref_policy._LEG_R_IDX
