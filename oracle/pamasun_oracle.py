"""CPU oracle of the Pamasun hybrid language model -- TEST INFRASTRUCTURE, never imported by the product.

A plain, slow restatement in torch CPU ops (float64 by default), one function per mechanism, token by token where a
mechanism is recurrent.  Shares no code with ``smoltts_b200``.  Inputs are a parsed ``config.json`` dictionary and a
``name -> tensor`` dictionary in the checkpoint's naming (``l<i>.mix.*``, ``l<i>.mlp.*``, ``embed``, ``head``,
``final.norm``).

Notation: x residual stream [T, D]; h a sublayer's input; H query heads, G key/value heads, d key size, dv value size;
t, j positions counted from 0 in a sequence.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

DECAY_FLOOR = math.exp(-0.5)      # decay = exp(-DECAY_FLOOR * sigmoid(.)) lies in (exp(-e^-1/2), 1)
UNIT_KEY_EPS = 1e-6


def rms_divide(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def norm_one_plus(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight is an offset from one."""
    return rms_divide(x, eps) * (1.0 + w)


def norm_plain(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_divide(x, eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def poly_norm(z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    """a N(z) + b N(z^2) + c N(z^3) + e with N the RMS division over a token's feed-forward vector."""
    a, b, c, e = [coef[i] for i in range(4)]
    return a * rms_divide(z, eps) + b * rms_divide(z ** 2, eps) + c * rms_divide(z ** 3, eps) + e


def dense_mlp(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, eps: float) -> torch.Tensor:
    z = h @ w[pre + "up"].T
    return poly_norm(z, w[pre + "act"], eps) @ w[pre + "down"].T


def sink_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, mixer: dict, eps: float,
                   past_k: Optional[torch.Tensor] = None, past_v: Optional[torch.Tensor] = None):
    """Causal grouped-query attention with per-head q/k RMS norm, a logarithmic distance penalty, a key-less sink in the
    softmax denominator and a sigmoid output gate.  ``h`` [T, D] continues a sequence whose normed keys / values so far
    are ``past_k`` [P, G, d] / ``past_v`` [P, G, dv].  Returns (out [T, D], keys [P+T, G, d], values [P+T, G, dv])."""
    H, G, d, dv, scale = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"], mixer["scale"]
    T = h.shape[0]
    q = norm_plain((h @ w[pre + "q"].T).view(T, H, d), w[pre + "q.norm"], eps)
    k = norm_plain((h @ w[pre + "k"].T).view(T, G, d), w[pre + "k.norm"], eps)
    v = (h @ w[pre + "v"].T).view(T, G, dv)
    if past_k is not None:
        k = torch.cat([past_k, k], 0)
        v = torch.cat([past_v, v], 0)
    P = k.shape[0] - T
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        i = P + t
        dist = (i - torch.arange(i + 1)).to(h.dtype)
        for hh in range(H):
            g = hh // (H // G)
            s = (k[: i + 1, g] @ q[t, hh]) * scale - w[pre + "r1"][hh] * torch.log1p(w[pre + "r2"][hh] * dist)
            m = torch.maximum(s.max(), w[pre + "sink"][hh])
            e = torch.exp(s - m)
            out[t, hh] = (e[:, None] * v[: i + 1, g]).sum(0) / (e.sum() + torch.exp(w[pre + "sink"][hh] - m))
    gate = torch.sigmoid(h @ w[pre + "g"].T)
    return (out.reshape(T, H * dv) * gate) @ w[pre + "o"].T, k, v


def general_delta(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, mixer: dict, eps: float,
                  state: Optional[torch.Tensor] = None):
    """Delta-rule recurrence with a per-channel decay and a per-channel removal rate along the unit key:
    S <- diag(w) S - (a * u)(u^T S) + k v^T (both corrections read the old S), o = S^T r.  ``state`` [H, d, d]."""
    H, d = mixer["heads"], mixer["dim"]
    T = h.shape[0]
    r = (h @ w[pre + "r"].T).view(T, H, d)
    k = (h @ w[pre + "k"].T).view(T, H, d)
    v = (h @ w[pre + "v"].T).view(T, H, d)
    decay = torch.exp(-DECAY_FLOOR * torch.sigmoid(torch.tanh(h @ w[pre + "w1"].T) @ w[pre + "w2"].T + w[pre + "w0"])).view(T, H, d)
    rate = torch.sigmoid(h @ w[pre + "a"].T + w[pre + "a.b"]).view(T, H, d)
    u = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + UNIT_KEY_EPS)
    S = torch.zeros(H, d, d, dtype=h.dtype) if state is None else state.clone()
    o = torch.zeros(T, H, d, dtype=h.dtype)
    for t in range(T):
        for hh in range(H):
            old = S[hh]
            seen = u[t, hh] @ old                                          # [d] over value columns
            S[hh] = decay[t, hh][:, None] * old - torch.outer(rate[t, hh] * u[t, hh], seen) + torch.outer(k[t, hh], v[t, hh])
            o[t, hh] = S[hh].T @ r[t, hh]
    o = rms_divide(o, eps).reshape(T, H * d) * w[pre + "norm"]
    return (o * torch.sigmoid(h @ w[pre + "g"].T)) @ w[pre + "o"].T, S


def layer_runs(cfg: dict) -> List[int]:
    """Layer index of every layer run: layers start..stop-1 repeat ``times`` times in a row, then the rest."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = loop["start"], loop["stop"], loop["times"]
    if b <= a:
        return list(range(n))
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


class PamasunOracle:
    """Whole model, with an explicit per-sequence cache (one entry per layer run) so that a prompt can be fed in portions."""

    def __init__(self, cfg: dict, weights: Dict[str, torch.Tensor], dtype=torch.float64):
        self.cfg = cfg
        self.dtype = dtype
        self.w = {k: v.to(dtype) for k, v in weights.items()}
        self.eps = cfg["norm"]["eps"]
        self.runs = layer_runs(cfg)

    def new_cache(self) -> list:
        return [None] * len(self.runs)

    def forward(self, tokens, cache: Optional[list] = None, collect: Optional[list] = None) -> torch.Tensor:
        """tokens: the next ids of one sequence; returns logits [T, vocab] and updates ``cache`` in place."""
        cfg, w, eps = self.cfg, self.w, self.eps
        if cache is None:
            cache = self.new_cache()
        x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
        for n, li in enumerate(self.runs):
            L, pre = cfg["layers"][li], f"l{li}."
            h = norm_one_plus(x, w[pre + "norm1"], eps)
            if L["type"] == "attention":
                pk, pv = cache[n] if cache[n] is not None else (None, None)
                y, k, v = sink_attention(h, w, pre + "mix.", L["mixer"], eps, pk, pv)
                cache[n] = (k, v)
            elif L["type"] == "general_delta":
                y, S = general_delta(h, w, pre + "mix.", L["mixer"], eps, cache[n])
                cache[n] = S
            else:
                raise ValueError(L["type"])
            x = x + norm_one_plus(y, w[pre + "norm1b"], eps) * w[pre + "ls1"]
            if L.get("mlp"):
                y = dense_mlp(norm_one_plus(x, w[pre + "norm2"], eps), w, pre + "mlp.", eps)
                x = x + norm_one_plus(y, w[pre + "norm2b"], eps) * w[pre + "ls2"]
            if collect is not None:
                collect.append(x.clone())
        return norm_one_plus(x, w["final.norm"], eps) @ w["head"].T


def random_weights(cfg: dict, seed: int = 0, spread: float = 1.0) -> Dict[str, torch.Tensor]:
    """bf16-representable random weights for a configuration, in the checkpoint's naming."""
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]

    def mat(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * (s * spread / math.sqrt(i))).bfloat16().float()

    def vec(n, s=0.1, base=0.0):
        return (base + torch.randn(n, generator=g) * s).bfloat16().float()

    w = {"embed": (torch.randn(V, D, generator=g) * 0.06).bfloat16().float(), "head": mat(V, D), "final.norm": vec(D)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for nm in ("norm1", "norm1b"):
            w[p + nm] = vec(D)
        w[p + "ls1"] = vec(D, 0.2, 0.7)
        if L["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w.update({p + "mix.q": mat(H * d, D), p + "mix.k": mat(G * d, D), p + "mix.v": mat(G * dv, D),
                      p + "mix.g": mat(H * dv, D), p + "mix.o": mat(D, H * dv),
                      p + "mix.q.norm": vec(d, 0.2, 1.0), p + "mix.k.norm": vec(d, 0.2, 1.0),
                      p + "mix.r1": (torch.rand(H, generator=g) * 0.8 + 0.1).bfloat16().float(),
                      p + "mix.r2": (torch.rand(H, generator=g) * 1.5 + 0.05).bfloat16().float(),
                      p + "mix.sink": vec(H, 1.0)})
        else:
            H, d = m["heads"], m["dim"]
            rank = m.get("_rank", 8)
            for nm in ("r", "k", "v", "g", "a"):
                w[p + "mix." + nm] = mat(H * d, D)
            w.update({p + "mix.a.b": vec(H * d, 0.5), p + "mix.w1": mat(rank, D), p + "mix.w2": mat(H * d, rank, 2.0),
                      p + "mix.w0": vec(H * d, 1.0), p + "mix.norm": vec(H * d, 0.2, 1.0), p + "mix.o": mat(D, H * d)})
        if L.get("mlp"):
            F = L["mlp"]["ff"]
            for nm in ("norm2", "norm2b"):
                w[p + nm] = vec(D)
            w.update({p + "ls2": vec(D, 0.2, 0.7), p + "mlp.up": mat(F, D), p + "mlp.down": mat(D, F),
                      p + "mlp.act": torch.tensor([0.6, 0.3, 0.15, 0.05]).bfloat16().float() + vec(4, 0.05)})
    return w
