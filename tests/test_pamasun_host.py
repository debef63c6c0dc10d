"""CPU tests of the Pamasun path: configuration, pools, scheduling logic against a recording stand-in of the engine,
and the oracle's own consistency (whole prompt == portions == token by token)."""
import json

import pytest
import torch

from oracle.pamasun_oracle import PamasunOracle, layer_runs, random_weights
from pamasun_util import MIXED, attn, config, delta, tokens
from smoltts_b200.lm_config import PamasunConfig
from smoltts_b200.pool import PagePool, SlotPool
from smoltts_b200.registry import design_of, registered


def test_config_round_trip_and_runs(tmp_path):
    cfg = PamasunConfig.from_dict(MIXED)
    assert cfg.layer_runs() == [0, 1, 2, 1, 2, 3] == layer_runs(MIXED)
    assert PamasunConfig.from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    assert PamasunConfig.from_dict(config([attn()])).layer_runs() == [0]
    three = config([attn(), delta(), attn()], loop={"start": 0, "stop": 3, "times": 3})
    assert PamasunConfig.from_dict(three).layer_runs() == [0, 1, 2] * 3
    shapes = cfg.tensor_shapes({0: 8, 3: 5})
    assert shapes["l3.mix.w1"] == (5, 64) and shapes["l1.mix.k"] == (32, 64) and "l2.mlp.up" not in shapes
    assert set(shapes) == set(random_weights(MIXED))
    (tmp_path / "config.json").write_text(json.dumps(MIXED))
    assert design_of(str(tmp_path)) == "Pamasun"
    assert {"Pamasun", "dual_ar"} <= set(registered())
    with pytest.raises(ValueError):
        PamasunConfig.from_dict(config([{"type": "conv", "mixer": {}, "mlp": None}]))


def test_pools_reuse_lifo_and_reject_double_free():
    p = PagePool(4, 16)
    a = p.allocate(3)
    assert a == [0, 1, 2] and len(p) == 1 and p.pages_for(17) == 2 and p.pages_for(16) == 1
    p.free([1])
    assert p.allocate(1) == [1]
    with pytest.raises(Exception):
        p.allocate(2)
    p.free(a)
    with pytest.raises(ValueError):
        p.free([0])
    s = SlotPool(2)
    assert s.allocate(2) == [0, 1]
    with pytest.raises(Exception):
        s.allocate(1)


class _Seq:
    def __init__(self, uid):
        self.uid, self.pages, self.length = uid, [], 0


class _FakeEngine:
    """Records the engine steps a scheduler makes; logits row = (uid, position) so that order and positions can be checked."""

    def __init__(self, max_step_tokens=8, max_seqs=2, pages=64, page_size=4, vocab=7):
        self.max_step_tokens, self.max_seqs = max_step_tokens, max_seqs
        self.page_pool, self.slot_pool = PagePool(pages, page_size), SlotPool(max_seqs)
        self.device = torch.device("cpu")
        self.config = type("C", (), {"vocab": vocab})()
        self.calls = []

    def open_sequence(self, uid):
        s = _Seq(uid)
        s.slot = self.slot_pool.allocate(1)[0]
        return s

    def close_sequence(self, s):
        self.page_pool.free(s.pages)
        self.slot_pool.free([s.slot])
        s.pages = []

    def forward(self, entries, trace=False):
        rows = []
        self.calls.append([(s.uid, list(t), list(w)) for s, t, w in entries])
        assert sum(len(t) for _, t, _ in entries) <= self.max_step_tokens and len(entries) <= self.max_seqs
        for s, t, w in entries:
            need = self.page_pool.pages_for(s.length + len(t)) - len(s.pages)
            s.pages += self.page_pool.allocate(need) if need > 0 else []
            rows += [[float(s.uid), float(s.length + i)] + [0.0] * 5 for i in w]
            s.length += len(t)
        return torch.tensor(rows).reshape(len(rows), 7)

    def sample(self, logits, *a, **k):
        return (logits[:, 1].to(torch.int32) + 1) % 7            # "next token" = position + 1


def test_feed_cuts_large_steps_and_keeps_row_order():
    from smoltts_b200.serving import TokenBatcher

    eng = _FakeEngine()
    b = TokenBatcher(eng)
    out = b.feed([(1, list(range(11)), [10, 0, 7]), (2, [5, 5, 5], [2])], end=[2])
    # 14 tokens through steps of 8: request 1 is cut at 8, request 2 rides in the second step
    assert [[(u, len(t)) for u, t, _ in c] for c in eng.calls] == [[(1, 8)], [(1, 3), (2, 3)]]
    assert out[:, :2].tolist() == [[1, 10], [1, 0], [1, 7], [2, 2]]
    assert len(eng.slot_pool) == 1 and len(eng.page_pool) == 64 - 3
    out = b.feed([(1, [3], [0])], end=[1])
    assert out[:, :2].tolist() == [[1, 11]] and len(eng.page_pool) == 64 and len(eng.slot_pool) == 2


def test_batcher_mixes_decode_tokens_with_prompt_portions_and_recycles():
    from smoltts_b200.serving import TokenBatcher

    eng = _FakeEngine(max_step_tokens=6, max_seqs=2, pages=8, page_size=4)
    b = TokenBatcher(eng)
    outs = b.generate([[1, 2, 3], list(range(10)), [4]], max_new_tokens=3)
    assert [len(o) for o in outs] == [3, 3, 3]
    assert outs[0] == [3, 4, 5] and outs[2] == [1, 2, 3]        # position + 1 of the last token fed
    # some step carried a single decoded token of one request beside a prompt portion of another
    assert any(len(c) == 2 and {len(t) for _, t, _ in c} != {1} and 1 in {len(t) for _, t, _ in c} for c in eng.calls)
    assert len(eng.page_pool) == 8 and len(eng.slot_pool) == 2 and b.stats["retired"] == 3


def test_oracle_portions_equal_whole():
    cfg = MIXED
    orc = PamasunOracle(cfg, random_weights(cfg, 3))
    toks = tokens(23, cfg["vocab"])
    whole = orc.forward(toks)
    cache = orc.new_cache()
    parts = [orc.forward(toks[a:b], cache) for a, b in ((0, 5), (5, 7), (7, 8), (8, 20), (20, 23))]
    assert torch.allclose(torch.cat(parts), whole, atol=1e-9)
