"""CPU tests of the Maferax design: configuration parsing and the oracle's own consistency (portions against whole
prompts, the router's grouped choice)."""
import copy

import pytest
import torch

from maferax_util import MIXED, config, dense, gla, latent, moe, tokens
from oracle.maferax_oracle import MaferaxOracle, random_weights, route, tensor_shapes
from smoltts_b200.lm_config import MaferaxConfig


def test_config_round_trip_and_shapes():
    cfg = MaferaxConfig.from_dict(MIXED)
    assert MaferaxConfig.from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    assert cfg.layer_runs() == [0, 1, 2, 3]
    ranks = {i: L["mixer"]["_rank"] for i, L in enumerate(MIXED["layers"]) if L["type"] == "gla"}
    assert cfg.tensor_shapes(ranks) == tensor_shapes(MIXED)
    with pytest.raises(ValueError):
        MaferaxConfig.from_dict(config([{"type": "conv", "mixer": {}, "mlp": None}]))
    with pytest.raises(ValueError):
        MaferaxConfig.from_dict(config([gla(mlp=moe(experts=5, identity=2, groups=3))]))          # 7 outputs, 3 groups
    with pytest.raises(ValueError):
        MaferaxConfig.from_dict(config([gla(mlp=moe(experts=6, identity=2, top=3, groups=4, keep=1))]))   # 3 choices from one group of 2


def test_registry_names_the_design(tmp_path):
    from smoltts_b200 import registry

    MaferaxConfig.from_dict(MIXED).save(str(tmp_path / "config.json"))
    assert registry.design_of(str(tmp_path)) == "Maferax"
    assert registry.registered()["Maferax"] == ("smoltts_b200.lm", "MaferaxLM")


def test_oracle_portions_equal_the_whole_prompt():
    w = random_weights(MIXED, 3)
    orc = MaferaxOracle(MIXED, w)
    toks = tokens(40, MIXED["vocab"])
    whole = orc.forward(toks)
    cache, parts = orc.new_cache(), []
    for lo, hi in ((0, 7), (7, 9), (9, 10), (10, 33), (33, 40)):
        parts.append(orc.forward(toks[lo:hi], cache))
    assert float((torch.cat(parts) - whole).abs().max()) < 1e-9


def test_router_groups_corrections_and_weights():
    """Eight outputs in four groups of two, two groups kept.  The best single score sits in a group whose other member is
    poor -- still its group's score is its best member, so it is kept; an output with a good score in a dropped group is
    not chosen; the correction moves the choice but not the weights."""
    router = {"experts": 6, "identity": 2, "top": 2, "groups": {"count": 4, "keep": 2}, "scale": 2.0}
    logits = torch.tensor([[3.0, -5.0, 2.5, 2.4, 2.45, 0.0, -1.0, -2.0]], dtype=torch.float64)
    w = {"router": torch.eye(8, dtype=torch.float64), "correction": torch.zeros(8, dtype=torch.float64)}
    ids, wts = route(logits, w, "", router)
    assert ids.tolist() == [[0, 2]]                      # groups {0,1} and {2,3} are kept; 4 (group 2) is out though it beats 3
    s = torch.softmax(logits[0], 0)
    assert torch.allclose(wts[0], s[[0, 2]] / s[[0, 2]].sum() * 2.0)
    w["correction"][3] = 0.5                             # lifts output 3 above 2 for the choice only
    ids2, wts2 = route(logits, w, "", router)
    assert ids2.tolist() == [[3, 0]]
    assert torch.allclose(wts2[0], s[[3, 0]] / s[[3, 0]].sum() * 2.0)
    w["correction"] = torch.tensor([0.0, 0.0, -2.0, -2.0, 0.0, 0.0, 0.0, 0.0], dtype=torch.float64)   # negative choice scores
    ids3, _ = route(logits, w, "", router)
    assert ids3.tolist() == [[0, 4]]                     # group {2,3} falls behind group {4,5}


def test_identity_outputs_hand_the_input_on():
    cfg = config([gla(mlp=moe(experts=0, identity=4, top=2, groups=2, keep=1, scale=3.0))])
    w = random_weights(cfg, 1)
    orc = MaferaxOracle(cfg, w)
    from oracle.maferax_oracle import expert_mixture

    h = torch.randn(5, cfg["width"], dtype=torch.float64)
    out = expert_mixture(h, orc.w, "l0.mlp.", cfg["layers"][0]["mlp"])
    assert torch.allclose(out, 3.0 * h)                  # the weights of the chosen outputs sum to the scale
