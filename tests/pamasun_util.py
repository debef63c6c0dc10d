"""Shared helpers of the Pamasun tests: small configurations, seeded weights, engine + oracle pairs."""
from __future__ import annotations

import torch

from oracle.pamasun_oracle import PamasunOracle, random_weights


def attn(heads=4, kv_heads=2, dim=16, vdim=8, scale=0.25, ff=48):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def delta(heads=2, dim=16, ff=48, rank=8):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "_rank": rank}, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(layers, vocab=97, width=64, scale=4.0, eps=1e-5, loop=None):
    return {"architecture": "Pamasun", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps},
            "layers": layers, "loop": loop or {"start": 0, "stop": 0, "times": 1}}


MIXED = config([delta(), attn(), attn(heads=2, kv_heads=2, dim=8, vdim=16, ff=0), delta(heads=3, dim=8, rank=5)],
               loop={"start": 1, "stop": 3, "times": 2})


def tokens(n, vocab, seed=0):
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


_CACHE = {}


def engine_and_oracle(cfg, seed=0, dtype=torch.float32, spread=1.0, edit=None, **engine):
    """(engine, oracle, weights) on identical seeded weights.  ``edit(weights)`` may change them first."""
    from smoltts_b200.lm import PamasunLM
    from smoltts_b200.lm_config import PamasunConfig

    key = (repr(cfg), seed, dtype, spread, edit, tuple(sorted(engine.items())))
    if key not in _CACHE:
        w = random_weights(cfg, seed, spread)
        if edit is not None:
            edit(w)
        kw = dict(max_tokens=1024, max_seqs=4, page_size=16, max_step_tokens=256)
        kw.update(engine)
        model = PamasunLM(PamasunConfig.from_dict(cfg), dtype=dtype, **kw)
        model.load_state_dict(w)
        _CACHE[key] = (model, PamasunOracle(cfg, w), w)
    return _CACHE[key]


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    """Largest row error of ``got`` against ``want`` relative to the rows' spread (mean taken off both)."""
    got, want = got.double().cpu(), want.double().cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    spread = (want - want.mean(-1, keepdim=True)).pow(2).mean().sqrt()
    return float(d.pow(2).mean(-1).sqrt().max() / spread)


TOL = {torch.float32: 3e-4, torch.bfloat16: 8e-2}
