"""Shared helpers of the Maferax tests: small configurations, seeded weights, engine + oracle pairs."""
from __future__ import annotations

import torch

from oracle.maferax_oracle import MaferaxOracle, random_weights


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, identity=2, top=2, groups=4, keep=2, scale=1.5, ff=24):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "identity": identity, "top": top, "groups": {"count": groups, "keep": keep}, "scale": scale}}


def latent(heads=4, dim=16, rot_dim=8, vdim=12, q_rank=24, kv_rank=40, scale=0.2, base=5000.0, mlp=None, rot_dims=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
                      "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}}


def gla(heads=2, dim=16, vdim=24, tau=8.0, rank=8, mlp=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "_rank": rank}, "mlp": mlp}


def config(layers, vocab=97, width=64, eps=1e-5, alpha=1.5, logit_scale=0.7):
    return {"architecture": "Maferax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "postln_alpha": alpha,
            "logit_scale": logit_scale, "layers": layers}


MIXED = config([gla(mlp=dense()), latent(mlp=moe()), latent(heads=2, dim=8, rot_dim=4, vdim=20, q_rank=12, kv_rank=24, scale=0.3),
                gla(heads=3, dim=8, vdim=12, tau=3.0, rank=5, mlp=moe(experts=3, identity=1, top=3, groups=2, keep=2, scale=1.0, ff=16))])


def tokens(n, vocab, seed=0):
    g = torch.Generator().manual_seed(2000 + seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


_CACHE = {}


def engine_and_oracle(cfg, seed=0, dtype=torch.float32, spread=1.0, edit=None, **engine):
    """(engine, oracle, weights) on identical seeded weights.  ``edit(weights)`` may change them first."""
    from smoltts_b200.lm import MaferaxLM
    from smoltts_b200.lm_config import MaferaxConfig

    key = (repr(cfg), seed, dtype, spread, edit, tuple(sorted(engine.items())))
    if key not in _CACHE:
        w = random_weights(cfg, seed, spread)
        if edit is not None:
            edit(w)
        kw = dict(max_tokens=1024, max_seqs=4, page_size=16, max_step_tokens=256)
        kw.update(engine)
        model = MaferaxLM(MaferaxConfig.from_dict(cfg), dtype=dtype, **kw)
        model.load_state_dict(w)
        _CACHE[key] = (model, MaferaxOracle(cfg, w), w)
    return _CACHE[key]


def row_errs(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Every row's error of ``got`` against ``want`` relative to the rows' spread (mean taken off both)."""
    got, want = got.double().cpu(), want.double().cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    spread = (want - want.mean(-1, keepdim=True)).pow(2).mean().sqrt()
    return d.pow(2).mean(-1).sqrt() / spread


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    """Largest row error."""
    return float(row_errs(got, want).max())


TOL = {torch.float32: 3e-4, torch.bfloat16: 8e-2}
