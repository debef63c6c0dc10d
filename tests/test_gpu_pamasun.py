"""GPU tests of the Pamasun engine against the CPU oracle (float64, written from the design's equations).

Small configurations and seeded random weights; fp32 engines are held to 3e-4 of the logits' spread, bf16 engines to
8e-2.  Where random weights would hide a fault the weights are edited so that it shows (peaky attention, strong sinks,
slow decays)."""
import pytest
import torch

from pamasun_util import MIXED, TOL, attn, config, delta, engine_and_oracle, rel_err, tokens

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
    """Sharp attention that can reach far back, a sink that matters, slowly decaying recurrent state."""
    for k in list(w):
        if k[-5:] in ("mix.q", "mix.k") and k[:-1] + "sink" in w:
            w[k] = (w[k] * 3.0).bfloat16().float()
        if k.endswith("mix.r1"):
            w[k] = (w[k] * 0.1).bfloat16().float()
        if k.endswith("mix.sink"):
            w[k] = (w[k] + 2.0).bfloat16().float()
        if k.endswith("mix.w0"):
            w[k] = (w[k] - 4.0).bfloat16().float()


# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("layers", [
    [attn(ff=0)], [delta(ff=0)], [attn(heads=1, kv_heads=1, dim=8, vdim=8, ff=40)], [delta(heads=1, dim=32, ff=0, rank=3)],
    [attn(heads=6, kv_heads=2, dim=24, vdim=40, scale=0.2, ff=0)], [delta(heads=2, dim=48, ff=0, rank=16)],
    [delta(heads=1, dim=128, ff=0)], [attn(heads=3, kv_heads=1, dim=12, vdim=20, scale=0.3, ff=0)],
    [attn(heads=2, kv_heads=1, dim=128, vdim=64, scale=0.09, ff=0)], [attn(heads=2, kv_heads=2, dim=40, vdim=136, scale=0.15, ff=0)],
    [delta(heads=1, dim=160, ff=0, rank=4)], [delta(heads=2, dim=256, ff=0, rank=12)], [delta(heads=2, dim=20, ff=0, rank=7)]],
    ids=["attention", "delta", "mha+mlp", "delta32", "gqa-odd", "delta48", "delta128", "attn-unaligned", "attn128", "attn-wide-v",
         "delta160", "delta256", "delta20-odd-rank"])
@pytest.mark.parametrize("dtype", [F32, BF16], ids=["f32", "bf16"])
def test_each_mechanism_alone(layers, dtype):
    cfg = config(layers, vocab=61, width=72)
    model, orc, _ = engine_and_oracle(cfg, seed=1, dtype=dtype)
    toks = tokens(37, 61)
    logits, traces = run_whole(model, toks, trace=True)
    col = []
    want = orc.forward(toks, collect=col)
    assert rel_err(traces[0][0], col[0]) < TOL[dtype]
    assert rel_err(logits, want) < TOL[dtype]


@pytest.mark.parametrize("dtype", [F32, BF16], ids=["f32", "bf16"])
def test_wide_residual_rows(dtype):
    """A width beyond what the norm kernels keep in registers (their shared-memory form), prompt and decoding."""
    from smoltts_b200.serving import TokenBatcher

    cfg = config([attn(heads=2, kv_heads=1, dim=16, vdim=16, ff=40), delta(heads=1, dim=16, ff=0)], vocab=43, width=2120)
    model, orc, _ = engine_and_oracle(cfg, seed=12, dtype=dtype)
    toks = tokens(21, 43, 40)
    want = orc.forward(toks)
    b = TokenBatcher(model)
    got = torch.cat([b.feed([("w", toks[:12], list(range(12)))])] + [b.feed([("w", [t], [0])]) for t in toks[12:]])
    b.close()
    assert rel_err(got, want) < TOL[dtype]


@pytest.mark.parametrize("dtype", [F32, BF16], ids=["f32", "bf16"])
def test_every_layer_run_of_a_looped_hybrid(dtype):
    model, orc, _ = engine_and_oracle(MIXED, seed=2, dtype=dtype)
    toks = tokens(50, MIXED["vocab"], 1)
    logits, traces = run_whole(model, toks, trace=True)
    col = []
    want = orc.forward(toks, collect=col)
    assert traces[0].shape[0] == len(col) == 6
    for n, c in enumerate(col):
        assert rel_err(traces[0][n], c) < TOL[dtype], f"layer run {n}"
    assert rel_err(logits, want) < TOL[dtype]


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
    for sizes in ([2] * 45, [17, 2, 31, 3, 2, 16, 15, 2, 2], [15, 1, 16, 16, 1, 1, 33, 7], [64, 26]):
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
def test_far_keys_page_borders_and_first_tokens(dtype):
    """Attention sharp enough that single keys decide the output.  The oracle shows that the wanted positions depend on
    the very first tokens and on keys several pages back; the engine must agree at and around every page border, in a
    prompt and when decoding."""
    from smoltts_b200.serving import TokenBatcher

    cfg = config([attn(heads=4, kv_heads=2, dim=16, vdim=16, scale=0.5, ff=0), attn(heads=2, kv_heads=1, dim=32, vdim=8, scale=0.4)], vocab=53)
    model, orc, _ = engine_and_oracle(cfg, seed=5, dtype=dtype, edit=peaky, page_size=16, max_tokens=512)
    toks = tokens(200, 53, 3)
    want = orc.forward(toks)
    for far in (0, 1, 15, 16, 17):                          # first tokens, and keys at a page's edge
        other = list(toks)
        other[far] = (other[far] + 7) % 53
        moved = rel_err(orc.forward(other)[150:], want[150:])
        assert moved > 50 * TOL[F32], f"test is blind to key {far} ({moved})"
    assert rel_err(run_whole(model, toks), want) < TOL[dtype]
    b = TokenBatcher(model)
    head = b.feed([("x", toks[:100], list(range(100)))])
    tail = torch.cat([b.feed([("x", [t], [0])]) for t in toks[100:]])
    b.feed([("x", [1], [])], end=["x"])
    got = torch.cat([head, tail])
    edges = [0, 1, 2, 15, 16, 17, 31, 32, 33, 111, 112, 113, 127, 128, 129, 191, 192, 193, 199]
    assert rel_err(got[edges], want[edges]) < TOL[dtype]
    assert rel_err(got, want) < TOL[dtype]


def test_sink_and_distance_penalty_show():
    """A model whose sink and penalty are strong: leaving either out moves the oracle's logits far beyond the tolerance."""
    import copy

    from oracle.pamasun_oracle import PamasunOracle

    cfg = config([attn(ff=0)], vocab=41)
    model, orc, w = engine_and_oracle(cfg, seed=6, edit=peaky)
    toks = tokens(60, 41, 4)
    want = orc.forward(toks)
    for name, value in (("l0.mix.sink", -30.0), ("l0.mix.r1", 0.0)):
        w2 = copy.deepcopy(w)
        w2[name] = torch.full_like(w2[name], value)
        assert rel_err(PamasunOracle(cfg, w2).forward(toks), want) > 100 * TOL[F32], name
    assert rel_err(run_whole(model, toks), want) < TOL[F32]


def test_long_decoding_keeps_the_state():
    """300 single-token steps after a short prompt, slow decays: the recurrent state and the cache are carried exactly."""
    from smoltts_b200.serving import TokenBatcher

    cfg = config([delta(heads=2, dim=16), attn(), delta(heads=1, dim=32, ff=0)], vocab=67, loop={"start": 0, "stop": 2, "times": 2})
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
    # sampled generation is reproducible and differs between requests
    s1 = TokenBatcher(model, temp=1.0, top_k=20, seed=5).generate([prompts[0], prompts[0]], 5)
    s2 = TokenBatcher(model, temp=1.0, top_k=20, seed=5).generate([prompts[0], prompts[0]], 5)
    assert s1 == s2 and s1[0] != s1[1]


def test_linear_kernels_against_torch():
    model, _, _ = engine_and_oracle(config([attn(ff=0)]), seed=9)
    modelb, _, _ = engine_and_oracle(config([attn(ff=0)]), seed=9, dtype=BF16)
    g = torch.Generator(device="cuda").manual_seed(0)
    for M, N, K in ((1, 200, 72), (5, 33, 40), (17, 64, 256), (70, 130, 100), (300, 96, 35), (129, 257, 64),
                    (3, 700, 512), (8, 1300, 264), (2, 768, 4608), (4, 100, 8),      # few rows: 2, 1, 2 and 4 warps per column
                    (260, 333, 72), (515, 96, 64), (1024, 768, 256), (300, 100, 136), (257, 97, 1000)):      # 257 rows and more: tcgen05 tiles
        a = torch.randn(M, K, device="cuda", generator=g)
        w = torch.randn(N, K, device="cuda", generator=g)
        ref = a.double() @ w.double().T
        assert float((model.linear(a, w).double() - ref).abs().max()) < 1e-4 * K ** 0.5
        ab, wb = a.bfloat16(), w.bfloat16()
        refb = ab.double() @ wb.double().T
        assert float((modelb.linear(ab, wb).double() - refb).abs().max()) < 1e-4 * K ** 0.5


@pytest.mark.parametrize("dtype", [F32, BF16], ids=["f32", "bf16"])
def test_long_portions_take_the_large_tile_path(dtype):
    """Steps of several hundred tokens (the matrix products change kernels with the row count) against the oracle, against
    short portions of the same prompt, and beside a decoding request in the same step."""
    from smoltts_b200.serving import TokenBatcher

    cfg = config([delta(heads=2, dim=32, ff=160, rank=8), attn(heads=4, kv_heads=2, dim=32, vdim=24, scale=0.2, ff=104)], vocab=131, width=128)
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
    assert rel_err(long, want) < TOL[dtype]
    short = torch.cat([b.feed([("s", toks[lo:lo + 100], list(range(100)))], end=["s"] if lo == 600 else []) for lo in range(0, 700, 100)])
    assert rel_err(short, want) < TOL[dtype]
    assert rel_err(long, short) < (1e-4 if dtype == F32 else TOL[dtype])
    model.check_device_errors()


def test_capacity_errors_are_raised_not_faulted():
    from smoltts_b200._errors import SmolError
    from smoltts_b200.serving import TokenBatcher

    model, _, _ = engine_and_oracle(config([attn(ff=0)]), seed=10, max_tokens=32, max_seqs=2, page_size=16)
    b = TokenBatcher(model)
    b.feed([("a", [1] * 20, [])])
    with pytest.raises(SmolError):
        b.feed([("b", [1] * 20, [])])                       # 2 + 2 pages > 2
    b.feed([("a", [1], [0])], end=["a", "b"])
    b.feed([("c", [1] * 32, [31])], end=["c"])
    assert len(model.page_pool) == 2 and len(model.slot_pool) == 2
