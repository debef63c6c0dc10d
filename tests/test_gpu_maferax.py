"""GPU tests of the Maferax engine against the CPU oracle (float64, written from the design's equations).

Small configurations and seeded random weights; fp32 engines are held to 3e-4 of the logits' spread, bf16 engines to
8e-2.  Where random weights would hide a fault the weights are edited so that it shows (sharp attention that reaches far
back, slowly decaying recurrent state, router scores that make the grouped choice bite)."""
import copy

import pytest
import torch

from maferax_util import MIXED, TOL, config, dense, engine_and_oracle, gla, latent, moe, rel_err, row_errs, tokens

pytestmark = pytest.mark.gpu
F32, BF16 = torch.float32, torch.bfloat16


def run_whole(model, toks, want=None, trace=False):
    from smoltts_b200.serving import TokenBatcher

    b = TokenBatcher(model)
    want = list(range(len(toks))) if want is None else want
    out = b.feed([("w", toks, want)], end=["w"], trace=trace)
    model.check_device_errors()
    return out


def peaky(w):
    """Sharp attention that can reach far back; recurrent state that decays slowly."""
    for k in list(w):
        if k.endswith(("mix.uq", "mix.dkv")):
            w[k] = (w[k] * 2.5).bfloat16().float()
        if k.endswith("mix.a2.b"):
            w[k] = (w[k] + 3.0).bfloat16().float()


LAYERS = {
    "latent": [latent()],
    "latent-1head": [latent(heads=1, dim=8, rot_dim=2, vdim=8, q_rank=8, kv_rank=16)],
    "latent-unaligned": [latent(heads=3, dim=12, rot_dim=6, vdim=20, q_rank=10, kv_rank=20, scale=0.3)],
    "latent-wide": [latent(heads=2, dim=40, rot_dim=16, vdim=72, q_rank=48, kv_rank=136, scale=0.1)],
    "latent-rank260": [latent(heads=2, dim=24, rot_dim=12, vdim=16, q_rank=16, kv_rank=260, scale=0.1)],
    "latent-12heads": [latent(heads=12, dim=8, rot_dim=8, vdim=8, q_rank=32, kv_rank=32, scale=0.25)],
    "latent-norot": [latent(heads=2, dim=16, rot_dim=0, vdim=16, q_rank=16, kv_rank=32)],
    "latent-part-rotated": [latent(heads=2, dim=8, rot_dim=12, rot_dims=8, vdim=8, q_rank=16, kv_rank=20, scale=0.3, base=30.0)],
    "gla": [gla()],
    "gla-1head-32": [gla(heads=1, dim=32, vdim=8, rank=3)],
    "gla-odd": [gla(heads=2, dim=6, vdim=10, tau=1.0, rank=7)],
    "gla-20x130": [gla(heads=2, dim=20, vdim=130, tau=4.0)],
    "gla-64x64": [gla(heads=2, dim=64, vdim=64, tau=16.0, rank=16)],
    "gla-128x40": [gla(heads=1, dim=128, vdim=40, tau=2.0)],
    "gla-160": [gla(heads=1, dim=160, vdim=16, rank=4)],
    "gla-256": [gla(heads=2, dim=256, vdim=24, rank=12)],
    "dense": [gla(mlp=dense(52))],
    "moe": [gla(mlp=moe())],
    "moe-one-group-top1": [gla(mlp=moe(experts=5, identity=0, top=1, groups=1, keep=1, scale=1.0, ff=20))],
    "moe-all-kept-top4": [latent(mlp=moe(experts=4, identity=5, top=4, groups=3, keep=3, scale=0.5, ff=10))],
    "moe-identity-only": [gla(mlp=moe(experts=0, identity=4, top=2, groups=2, keep=1, scale=3.0))],
    "moe-many": [latent(mlp=moe(experts=30, identity=2, top=6, groups=8, keep=3, scale=2.0, ff=12))],
}


@pytest.mark.parametrize("name", list(LAYERS))
@pytest.mark.parametrize("dtype", [F32, BF16], ids=["f32", "bf16"])
def test_each_mechanism_alone(name, dtype):
    cfg = config(LAYERS[name], vocab=61, width=72)
    model, orc, _ = engine_and_oracle(cfg, seed=1, dtype=dtype)
    toks = tokens(37, 61)
    logits, traces = run_whole(model, toks, trace=True)
    col = []
    want = orc.forward(toks, collect=col)
    if dtype == BF16 and "moe" in name:
        # among many experts a token's last choice can be a close call, which bf16 inputs may turn the other way: the fp32
        # engine is held to every row, the bf16 engine to all rows but two
        assert int((row_errs(logits, want) > TOL[dtype]).sum()) <= 2
        return
    assert rel_err(traces[0][0], col[0]) < TOL[dtype]
    assert rel_err(logits, want) < TOL[dtype]


@pytest.mark.parametrize("dtype", [F32, BF16], ids=["f32", "bf16"])
def test_every_layer_of_a_hybrid_and_the_depth_average(dtype):
    model, orc, w = engine_and_oracle(MIXED, seed=2, dtype=dtype)
    toks = tokens(50, MIXED["vocab"], 1)
    logits, traces = run_whole(model, toks, trace=True)
    col = []
    want = orc.forward(toks, collect=col)
    assert traces[0].shape[0] == len(col) == 4
    for n, c in enumerate(col):
        assert rel_err(traces[0][n], c) < TOL[dtype], f"layer {n}"
    assert rel_err(logits, want) < TOL[dtype]
    if dtype == F32:
        # the test sees the depth average, the stream's scale before the sum, and the logit scale
        from oracle.maferax_oracle import MaferaxOracle

        w2 = copy.deepcopy(w)
        w2["l2.dwa"][0] += 0.5
        assert rel_err(MaferaxOracle(MIXED, w2).forward(toks), want) > 30 * TOL[F32]
        other = dict(MIXED, postln_alpha=1.0)
        assert rel_err(MaferaxOracle(other, w).forward(toks), want) > 30 * TOL[F32]
        slow = copy.deepcopy(MIXED)
        slow["layers"][0]["mixer"]["tau"] = 2.0 * MIXED["layers"][0]["mixer"]["tau"]      # ... and the decay's exponent
        assert rel_err(MaferaxOracle(slow, w).forward(toks), want) > 30 * TOL[F32]
        w3 = copy.deepcopy(w)
        w3["l1.mix.g"] = torch.zeros_like(w["l1.mix.g"])                                  # ... and the per-head output gate
        assert rel_err(MaferaxOracle(MIXED, w3).forward(toks), want) > 30 * TOL[F32]


@pytest.mark.parametrize("dtype", [F32, BF16], ids=["f32", "bf16"])
def test_odd_width_and_vocabulary(dtype):
    """Sizes that are multiples of nothing: no 16-byte pieces anywhere, every kernel on its element-wise form."""
    from smoltts_b200.serving import TokenBatcher

    cfg = config([gla(heads=1, dim=10, vdim=6, rank=3, mlp=moe(experts=3, identity=0, top=2, groups=1, keep=1, ff=9)),
                  latent(heads=3, dim=6, rot_dim=2, vdim=5, q_rank=7, kv_rank=9, mlp=dense(11))], vocab=37, width=50)
    model, orc, _ = engine_and_oracle(cfg, seed=14, dtype=dtype)
    toks = tokens(45, 37, 41)
    want = orc.forward(toks)
    b = TokenBatcher(model)
    got = torch.cat([b.feed([("w", toks[:30], list(range(30)))])] + [b.feed([("w", [t], [0])]) for t in toks[30:]])
    b.close()
    assert rel_err(got, want) < TOL[dtype]


@pytest.mark.parametrize("dtype", [F32, BF16], ids=["f32", "bf16"])
def test_wide_stream_rows(dtype):
    from smoltts_b200.serving import TokenBatcher

    cfg = config([latent(heads=2, dim=8, rot_dim=4, vdim=8, q_rank=8, kv_rank=16, mlp=dense(24)), gla(heads=1, dim=16, vdim=8)], vocab=43, width=2120)
    model, orc, _ = engine_and_oracle(cfg, seed=12, dtype=dtype)
    toks = tokens(21, 43, 40)
    want = orc.forward(toks)
    b = TokenBatcher(model)
    got = torch.cat([b.feed([("w", toks[:12], list(range(12)))])] + [b.feed([("w", [t], [0])]) for t in toks[12:]])
    b.close()
    assert rel_err(got, want) < TOL[dtype]


@pytest.mark.parametrize("dtype", [F32, BF16], ids=["f32", "bf16"])
def test_prefill_against_token_by_token_and_portions(dtype):
    from smoltts_b200.serving import TokenBatcher

    model, orc, _ = engine_and_oracle(MIXED, seed=3, edit=peaky, dtype=dtype)
    toks = tokens(90, MIXED["vocab"], 2)
    want = orc.forward(toks)
    whole = run_whole(model, toks)
    assert rel_err(whole, want) < TOL[dtype]
    b = TokenBatcher(model)
    one = torch.cat([b.feed([("d", [t], [0])]) for t in toks])
    b.feed([("d", [0], [])], end=["d"])
    assert rel_err(one, want) < TOL[dtype] and rel_err(one, whole) < (1e-4 if dtype == F32 else TOL[dtype])
    for sizes in ([2] * 45, [17, 2, 31, 3, 2, 16, 15, 2, 2], [15, 1, 16, 16, 1, 1, 33, 7], [64, 26], [9, 8, 8, 9, 56]):
        assert sum(sizes) == 90
        outs, at = [], 0
        for n in sizes:
            outs.append(b.feed([("p", toks[at:at + n], list(range(n)))], end=["p"] if at + n == 90 else []))
            at += n
        got = torch.cat(outs)
        assert rel_err(got, want) < TOL[dtype], sizes
        assert rel_err(got, whole) < (1e-4 if dtype == F32 else TOL[dtype]), sizes
    assert len(model.page_pool) == model.page_pool.n and len(model.slot_pool) == model.slot_pool.n


@pytest.mark.parametrize("dtype", [F32, BF16], ids=["f32", "bf16"])
def test_unequal_batches_equal_each_alone_with_reused_pages_and_slots(dtype):
    """Four requests of different lengths share steps: portions beside single tokens, requests that pause, finish and are
    replaced.  The pool holds fewer pages than all requests together need, so pages and slots are used again, and the
    pools are filled with garbage first: nothing may depend on what a page or slot held before."""
    from smoltts_b200.serving import TokenBatcher

    model, orc, _ = engine_and_oracle(MIXED, seed=4, edit=peaky, max_tokens=208, max_seqs=3, dtype=dtype)
    model._kv_pool.view(dtype).fill_(1e4)
    model._state_pool.view(torch.float32).fill_(-3e3)
    V = MIXED["vocab"]
    reqs = {"a": tokens(70, V, 10), "b": tokens(33, V, 11), "c": tokens(5, V, 12), "d": tokens(64, V, 13), "e": tokens(49, V, 17)}
    want = {k: orc.forward(v) for k, v in reqs.items()}
    plan = [[("a", 16), ("b", 2), ("c", 1)], [("a", 3), ("b", 29), ("c", 4)], [("a", 13), ("b", 1), ("d", 2)],
            [("a", 1), ("b", 1), ("d", 30)], [("a", 1), ("d", 1)], [("a", 33), ("d", 31), ("e", 17)], [("a", 1), ("e", 2)],
            [("a", 1), ("e", 30)], [("a", 1)]]
    b, at, got = TokenBatcher(model), {k: 0 for k in reqs}, {k: [] for k in reqs}
    for step in plan:
        entries, end = [], []
        for k, n in step:
            entries.append((k, reqs[k][at[k]:at[k] + n], list(range(n))))
            at[k] += n
            if at[k] == len(reqs[k]):
                end.append(k)
        out = b.feed(entries, end=end)
        lo = 0
        for k, n in step:
            got[k].append(out[lo:lo + n])
            lo += n
    model.check_device_errors()
    assert at == {k: len(v) for k, v in reqs.items()}
    for k in reqs:
        assert rel_err(torch.cat(got[k]), want[k]) < TOL[dtype], k
    assert len(model.page_pool) == model.page_pool.n and len(model.slot_pool) == 3


@pytest.mark.parametrize("dtype", [F32, BF16], ids=["f32", "bf16"])
def test_far_keys_page_borders_first_tokens_and_rotation(dtype):
    """Attention sharp enough that single keys decide the output.  The oracle shows that the wanted positions depend on
    the very first tokens, on keys several pages back and on the rotation's positions; the engine must agree at and
    around every page border, in a prompt and when decoding."""
    from oracle.maferax_oracle import MaferaxOracle
    from smoltts_b200.serving import TokenBatcher

    cfg = config([latent(heads=4, dim=16, rot_dim=16, vdim=16, q_rank=32, kv_rank=32, scale=0.5, base=50.0),
                  latent(heads=2, dim=8, rot_dim=24, vdim=8, q_rank=16, kv_rank=24, scale=0.4, base=3000.0, mlp=dense(40))], vocab=53)
    model, orc, w = engine_and_oracle(cfg, seed=5, dtype=dtype, edit=peaky, page_size=16, max_tokens=512)
    toks = tokens(200, 53, 3)
    want = orc.forward(toks)
    for far in (0, 1, 15, 16, 17):                          # first tokens, and keys at a page's edge
        other = list(toks)
        other[far] = (other[far] + 7) % 53
        moved = rel_err(orc.forward(other)[150:], want[150:])
        assert moved > 50 * TOL[F32], f"test is blind to key {far} ({moved})"
    still = copy.deepcopy(cfg)
    still["layers"][0]["mixer"]["rot"]["base"] = 51.0
    assert rel_err(MaferaxOracle(still, w).forward(toks)[150:], want[150:]) > 50 * TOL[F32], "test is blind to the rotation"
    assert rel_err(run_whole(model, toks), want) < TOL[dtype]
    b = TokenBatcher(model)
    head = b.feed([("x", toks[:100], list(range(100)))])
    tail = torch.cat([b.feed([("x", [t], [0])]) for t in toks[100:]])
    b.feed([("x", [1], [])], end=["x"])
    got = torch.cat([head, tail])
    edges = [0, 1, 2, 15, 16, 17, 31, 32, 33, 111, 112, 113, 127, 128, 129, 191, 192, 193, 199]
    assert rel_err(got[edges], want[edges]) < TOL[dtype]
    assert rel_err(got, want) < TOL[dtype]


def test_grouped_choice_identity_outputs_and_corrections_show():
    """Router weights large enough that the choice is clear-cut, corrections large enough to change it: ignoring the groups,
    the corrections or the identity outputs moves the oracle's logits far beyond the tolerance."""
    from oracle.maferax_oracle import MaferaxOracle

    def edit(w):
        w["l0.mlp.router"] = (w["l0.mlp.router"] * 3.0).bfloat16().float()
        w["l0.mlp.correction"] = (w["l0.mlp.correction"] * 6.0).bfloat16().float()

    cfg = config([gla(mlp=moe(experts=9, identity=3, top=3, groups=4, keep=2, scale=2.5, ff=20))], vocab=41)
    model, orc, w = engine_and_oracle(cfg, seed=6, edit=edit)
    toks = tokens(60, 41, 4)
    want = orc.forward(toks)
    free = copy.deepcopy(cfg)
    free["layers"][0]["mlp"]["router"]["groups"] = {"count": 1, "keep": 1}
    assert rel_err(MaferaxOracle(free, w).forward(toks), want) > 100 * TOL[F32], "groups"
    w2 = dict(w)
    w2["l0.mlp.correction"] = torch.zeros_like(w["l0.mlp.correction"])
    assert rel_err(MaferaxOracle(cfg, w2).forward(toks), want) > 100 * TOL[F32], "corrections"
    none = copy.deepcopy(cfg)
    none["layers"][0]["mlp"]["router"].update(experts=12, identity=0)
    w3 = dict(w)
    for e in (9, 10, 11):
        for nm in ("gate", "up", "down"):
            w3[f"l0.mlp.e{e}.{nm}"] = torch.zeros_like(w[f"l0.mlp.e0.{nm}"])
    assert rel_err(MaferaxOracle(none, w3).forward(toks), want) > 100 * TOL[F32], "identity outputs"
    assert rel_err(run_whole(model, toks), want) < TOL[F32]


def test_long_decoding_keeps_the_state():
    """300 single-token steps after a short prompt, slow decays: the recurrent state and the cache are carried exactly."""
    from smoltts_b200.serving import TokenBatcher

    cfg = config([gla(heads=2, dim=16, vdim=16, tau=32.0, mlp=dense(32)), latent(mlp=moe()), gla(heads=1, dim=32, vdim=24, tau=64.0)], vocab=67)
    model, orc, _ = engine_and_oracle(cfg, seed=7, edit=peaky, max_tokens=384)
    toks = tokens(310, 67, 5)
    want = orc.forward(toks)
    b = TokenBatcher(model)
    outs = [b.feed([("l", toks[:10], list(range(10)))])] + [b.feed([("l", [t], [0])]) for t in toks[10:]]
    b.close()
    got = torch.cat(outs)
    assert rel_err(got[-5:], want[-5:]) < TOL[F32] and rel_err(got, want) < TOL[F32]
    # the test sees a lost state: the last logits depend on the first token through the recurrence and the cache
    other = [(toks[0] + 1) % 67] + toks[1:]
    assert rel_err(orc.forward(other)[-20:], want[-20:]) > 3 * TOL[F32]


def test_greedy_generation_through_the_batcher():
    """The scheduler's own loop: admission, chunked prefill beside decoding, the library's sampler, retirement."""
    from smoltts_b200.serving import TokenBatcher

    model, orc, _ = engine_and_oracle(MIXED, seed=8, max_tokens=160, max_seqs=2, max_step_tokens=24)
    V = MIXED["vocab"]
    prompts = [tokens(30, V, 20), tokens(3, V, 21), tokens(41, V, 22), tokens(1, V, 23)]
    b = TokenBatcher(model, step_tokens=24)
    got = b.generate(prompts, max_new_tokens=6)
    for p, g in zip(prompts, got):
        seq = list(p)
        for tok in g:
            logits = orc.forward(seq)[-1]
            top = torch.topk(logits, 2).values
            if float(top[0] - top[1]) > 1e-3 * float(logits.std()):      # a near-tie may go either way
                assert tok == int(logits.argmax()), (p, g)
            seq.append(tok)
    assert len(model.page_pool) == model.page_pool.n and len(model.slot_pool) == 2 and b.stats["retired"] == 4


def test_generation_and_trace_through_the_registry(tmp_path):
    """A checkpoint folder on disk: the registry picks the design's class by config.json, the command line generates."""
    import json
    import subprocess
    import sys

    from smoltts_b200.registry import load_model

    model, orc, w = engine_and_oracle(MIXED, seed=8)
    model.save_pretrained(str(tmp_path))
    again = load_model(str(tmp_path), dtype=F32, max_tokens=256, max_seqs=2, page_size=16)
    assert type(again).__name__ == "MaferaxLM"
    toks = tokens(20, MIXED["vocab"], 30)
    assert rel_err(run_whole(again, toks), orc.forward(toks)) < TOL[F32]
    out = subprocess.run([sys.executable, "-m", "smoltts_b200", "generate", "--model", str(tmp_path), "--dtype", "float32",
                          "--prompt", ",".join(map(str, toks)), "--max-new-tokens", "3"], capture_output=True, text=True, check=True)
    rec = json.loads(out.stdout.strip().splitlines()[-1])
    assert rec["prompt"] == toks and len(rec["tokens"]) == 3


def test_batched_and_grouped_products_against_torch():
    """The per-head (strided, batched) and per-expert (gathered, grouped) forms of the matrix products, through models
    whose only large products are those: many heads and experts, rows far beyond one tile."""
    cfg = config([latent(heads=5, dim=24, rot_dim=8, vdim=40, q_rank=40, kv_rank=72, scale=0.15,
                         mlp=moe(experts=7, identity=1, top=3, groups=2, keep=2, scale=1.0, ff=56))], vocab=89, width=96)
    toks = tokens(300, 89, 9)
    for dtype in (F32, BF16):
        model, orc, _ = engine_and_oracle(cfg, seed=13, dtype=dtype, page_size=64, max_tokens=512, max_step_tokens=512)
        assert rel_err(run_whole(model, toks), orc.forward(toks)) < TOL[dtype]


@pytest.mark.parametrize("dtype", [F32, BF16], ids=["f32", "bf16"])
def test_long_portions_take_the_large_tile_path(dtype):
    """Steps of several hundred tokens (the matrix products change kernels with the row count) against the oracle, against
    short portions of the same prompt, and beside a decoding request in the same step."""
    from smoltts_b200.serving import TokenBatcher

    cfg = config([gla(heads=2, dim=32, vdim=48, rank=8, mlp=dense(160)),
                  latent(heads=4, dim=32, rot_dim=16, vdim=24, q_rank=64, kv_rank=64, scale=0.2, mlp=moe(experts=6, identity=2, ff=64))],
                 vocab=131, width=128)
    model, orc, _ = engine_and_oracle(cfg, seed=11, dtype=dtype, edit=peaky, page_size=64, max_tokens=1024, max_step_tokens=512)
    toks, other = tokens(700, 131, 30), tokens(40, 131, 31)
    want, want_o = orc.forward(toks), orc.forward(other)
    b = TokenBatcher(model)
    b.feed([("o", other[:30], [])])
    got = [b.feed([("a", toks[:300], list(range(300)))])]
    out = b.feed([("a", toks[300:690], list(range(390))), ("o", other[30:31], [0])])
    got.append(out[:390])
    assert rel_err(out[390:], want_o[30:31]) < TOL[dtype]
    got.append(b.feed([("a", toks[690:], list(range(10)))], end=["a", "o"]))
    long = torch.cat(got)
    # bf16: of 700 rows a few may sit on a close call of the router and take another expert than the oracle
    flips = 0 if dtype == F32 else 4
    assert int((row_errs(long, want) > TOL[dtype]).sum()) <= flips
    short = torch.cat([b.feed([("s", toks[lo:lo + 100], list(range(100)))], end=["s"] if lo == 600 else []) for lo in range(0, 700, 100)])
    assert int((row_errs(short, want) > TOL[dtype]).sum()) <= flips
    assert int((row_errs(long, short) > (1e-4 if dtype == F32 else TOL[dtype])).sum()) <= flips
    model.check_device_errors()
