"""CPU oracle of the Maferax hybrid language model -- TEST INFRASTRUCTURE, never imported by the product.

A plain, slow restatement in torch CPU ops (float64 by default), one function per mechanism, token by token where a
mechanism is recurrent.  Shares no code with ``smoltts_b200``.  Inputs are a parsed ``config.json`` dictionary and a
``name -> tensor`` dictionary in the checkpoint's naming (``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.dwa``, ``embed``,
``embed.norm``, ``head``, ``final.norm``).

Notation: x the stream [T, D]; h a sublayer's input; H heads; d the unrotated and r the rotated query/key size of a
latent-attention head, dv its value size, c the cached latent [kv_rank]; for the gated linear recurrence d key channels
and dv value channels per head, S the state [d, dv]; t, j positions counted from 0 in a sequence.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_divide(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def scalar_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS division times ONE number for all coordinates."""
    return rms_divide(x, eps) * g.reshape(())


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rotate_interleaved(v: torch.Tensor, pos: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """Rotary positions on the first ``dims`` coordinates of the last axis, coordinate 2i paired with 2i+1:
    (a, b) -> (a cos - b sin, b cos + a sin) with angle pos * base^(-2i/dims).  ``pos`` [T] broadcasts from the first axis."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    ang = pos.to(torch.float64)[:, None] * base ** (-2.0 * i / dims)            # [T, dims/2]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [dims // 2]
    cos, sin = ang.cos().view(shape).to(v.dtype), ang.sin().view(shape).to(v.dtype)
    out = v.clone()
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * cos - b * sin
    out[..., 1:dims:2] = b * cos + a * sin
    return out


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, mixer: dict, eps: float, pos0: int = 0,
                     past_c: Optional[torch.Tensor] = None, past_kr: Optional[torch.Tensor] = None):
    """Causal softmax attention whose keys and values are expanded from a cached latent.  ``h`` [T, D] continues a
    sequence that holds ``pos0`` positions with latents ``past_c`` [pos0, kv_rank] and rotated shared key parts
    ``past_kr`` [pos0, r].  Returns (out [T, D], latents, rotated parts) with the new positions appended."""
    H, d, r, dv, rank = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"], mixer["kv_rank"]
    rot = mixer["rot"]
    T = h.shape[0]
    pos = torch.arange(pos0, pos0 + T)
    cq = rms_divide(h @ w[pre + "dq"].T, eps) * w[pre + "dq.norm"]
    q = (cq @ w[pre + "uq"].T).view(T, H, d + r)
    q_plain, q_rot = q[..., :d], rotate_interleaved(q[..., d:], pos, rot["base"], rot["dims"])
    kv = h @ w[pre + "dkv"].T
    c = rms_divide(kv[:, :rank], eps) * w[pre + "dkv.norm"]
    kr = rotate_interleaved(kv[:, rank:], pos, rot["base"], rot["dims"])
    if past_c is not None and past_c.shape[0]:
        c, kr = torch.cat([past_c, c], 0), torch.cat([past_kr, kr], 0)
    k_plain = (c @ w[pre + "uk"].T).view(-1, H, d)
    v = (c @ w[pre + "uv"].T).view(-1, H, dv)
    gate = torch.sigmoid(h @ w[pre + "g"].T)                                    # [T, H]
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        n = pos0 + t + 1
        for hh in range(H):
            s = (k_plain[:n, hh] @ q_plain[t, hh] + kr[:n] @ q_rot[t, hh]) * mixer["scale"]
            out[t, hh] = torch.softmax(s, 0) @ v[:n, hh] * gate[t, hh]
    return out.reshape(T, H * dv) @ w[pre + "o"].T, c, kr


def gated_linear_recurrence(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, mixer: dict, eps: float,
                            state: Optional[torch.Tensor] = None):
    """S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head, with a per-key-channel decay
    a = sigmoid(z)^(1/tau), z from a low-rank projection with a bias.  ``state`` [H, d, dv] (None: zeros).
    Returns (out [T, D], state)."""
    H, d, dv, tau = mixer["heads"], mixer["dim"], mixer["vdim"], mixer["tau"]
    T = h.shape[0]
    q = (h @ w[pre + "q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w[pre + "k"].T).view(T, H, d)
    v = (h @ w[pre + "v"].T).view(T, H, dv)
    z = (h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "a2.b"]
    decay = torch.exp(torch.nn.functional.logsigmoid(z) / tau).view(T, H, d)
    S = torch.zeros(H, d, dv, dtype=h.dtype) if state is None else state.clone()
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_divide(o, eps) * w[pre + "norm"]
    out = (o.reshape(T, H * dv) * silu(h @ w[pre + "g"].T)) @ w[pre + "o"].T
    return out, S


def gated_mlp(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, act) -> torch.Tensor:
    return (act(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def route(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, router: dict):
    """Per token: the chosen outputs of the router (ids [T, top], in decreasing choice score) and their weights."""
    E, top = router["experts"] + router["identity"], router["top"]
    s = torch.softmax(h @ w[pre + "router"].T, -1)                               # [T, E]
    choice = s + w[pre + "correction"]
    n_groups, keep = router["groups"]["count"], router["groups"]["keep"]
    size = E // n_groups
    ids = torch.zeros(h.shape[0], top, dtype=torch.long)
    wts = torch.zeros(h.shape[0], top, dtype=h.dtype)
    for t in range(h.shape[0]):
        group_score = [choice[t, g * size:(g + 1) * size].max().item() for g in range(n_groups)]
        kept = sorted(range(n_groups), key=lambda g: (-group_score[g], g))[:keep]
        allowed = [e for e in range(E) if e // size in kept]
        allowed.sort(key=lambda e: (-choice[t, e].item(), e))
        chosen = allowed[:top]
        ids[t] = torch.tensor(chosen)
        sc = s[t, chosen]
        wts[t] = sc / (sc.sum() + 1e-20) * router["scale"]
    return ids, wts


def expert_mixture(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, mlp: dict) -> torch.Tensor:
    router = mlp["router"]
    ids, wts = route(h, w, pre, router)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(ids[t].tolist(), wts[t]):
            if e >= router["experts"]:
                out[t] += g * h[t]                                               # an identity output hands the input on
            else:
                out[t] += g * gated_mlp(h[t:t + 1], w, f"{pre}e{e}.", silu)[0]
    return out


class MaferaxOracle:
    """Whole model; ``forward`` continues a cache, so prompts can be fed in portions or token by token."""

    def __init__(self, cfg: dict, weights: Dict[str, torch.Tensor], dtype=torch.float64):
        self.cfg = cfg
        self.dtype = dtype
        self.w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}

    def new_cache(self) -> dict:
        return {"pos": 0, "layers": [None] * len(self.cfg["layers"])}

    def forward(self, tokens, cache: Optional[dict] = None, collect: Optional[list] = None) -> torch.Tensor:
        """Logits [T, vocab] of the tokens; ``collect`` receives the stream after every layer [T, D]."""
        cfg, w = self.cfg, self.w
        cache = cache if cache is not None else self.new_cache()
        eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
        x = scalar_norm(w["embed"][torch.as_tensor(tokens, dtype=torch.long)], w["embed.norm"], eps)
        results = [x]
        for i, L in enumerate(cfg["layers"]):
            p = f"l{i}."
            if L["type"] == "latent_attention":
                past = cache["layers"][i] or (None, None)
                y, c, kr = latent_attention(x, w, p + "mix.", L["mixer"], eps, cache["pos"], past[0], past[1])
                cache["layers"][i] = (c, kr)
            elif L["type"] == "gla":
                y, cache["layers"][i] = gated_linear_recurrence(x, w, p + "mix.", L["mixer"], eps, cache["layers"][i])
            else:
                raise ValueError(L["type"])
            x = scalar_norm(alpha * x + y, w[p + "norm1"], eps)
            mlp = L.get("mlp")
            if mlp:
                y = gated_mlp(x, w, p + "mlp.", gelu_tanh) if mlp["kind"] == "dense" else expert_mixture(x, w, p + "mlp.", mlp)
                x = scalar_norm(alpha * x + y, w[p + "norm2"], eps)
            results.append(x)
            x = sum(w[p + "dwa"][j] * results[j] for j in range(i + 2))
            if collect is not None:
                collect.append(x)
        cache["pos"] += len(tokens)
        return scalar_norm(x, w["final.norm"], eps) @ w["head"].T * cfg["logit_scale"]


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    D, V = cfg["width"], cfg["vocab"]
    out: Dict[str, tuple] = {"embed": (V, D), "embed.norm": (), "head": (V, D), "final.norm": ()}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = ()
        out[p + "dwa"] = (i + 2,)
        if L["type"] == "latent_attention":
            H, d, r, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
            out.update({p + "mix.dq": (m["q_rank"], D), p + "mix.dq.norm": (m["q_rank"],), p + "mix.uq": (H * (d + r), m["q_rank"]),
                        p + "mix.dkv": (m["kv_rank"] + r, D), p + "mix.dkv.norm": (m["kv_rank"],), p + "mix.uk": (H * d, m["kv_rank"]),
                        p + "mix.uv": (H * dv, m["kv_rank"]), p + "mix.g": (H, D), p + "mix.o": (D, H * dv)})
        else:
            H, d, dv, rank = m["heads"], m["dim"], m["vdim"], m.get("_rank", 8)
            out.update({p + "mix.q": (H * d, D), p + "mix.k": (H * d, D), p + "mix.v": (H * dv, D), p + "mix.g": (H * dv, D),
                        p + "mix.o": (D, H * dv), p + "mix.norm": (dv,), p + "mix.a1": (rank, D), p + "mix.a2": (H * d, rank),
                        p + "mix.a2.b": (H * d,)})
        mlp = L.get("mlp")
        if mlp:
            out[p + "norm2"] = ()
            if mlp["kind"] == "dense":
                out.update({p + "mlp.gate": (mlp["ff"], D), p + "mlp.up": (mlp["ff"], D), p + "mlp.down": (D, mlp["ff"])})
            else:
                R, F = mlp["router"], mlp["expert"]["ff"]
                for e in range(R["experts"]):
                    out.update({f"{p}mlp.e{e}.gate": (F, D), f"{p}mlp.e{e}.up": (F, D), f"{p}mlp.e{e}.down": (D, F)})
                out.update({p + "mlp.router": (R["experts"] + R["identity"], D), p + "mlp.correction": (R["experts"] + R["identity"],)})
    return out


def random_weights(cfg: dict, seed: int = 0, spread: float = 1.0) -> Dict[str, torch.Tensor]:
    """Seeded weights, rounded to bfloat16 values (so that a bf16 engine and the oracle hold the same numbers)."""
    g = torch.Generator().manual_seed(seed)
    sd: Dict[str, torch.Tensor] = {}
    for k, s in tensor_shapes(cfg).items():
        if len(s) == 2:
            t = torch.randn(*s, generator=g) * spread * s[1] ** -0.5
            if k == "embed":
                t = torch.randn(*s, generator=g)
            elif k.endswith("mlp.router"):
                t = t * 4.0                                                      # spread-out router scores: few close calls
        elif k.endswith(("norm1", "norm2", "embed.norm", "final.norm")):
            t = 1.0 + 0.2 * torch.rand((), generator=g)
        elif k.endswith("dwa"):
            t = torch.rand(*s, generator=g) * 0.3
            t[-1] = 1.0
        elif k.endswith(("dq.norm", "dkv.norm", "mix.norm")):
            t = 1.0 + 0.1 * torch.randn(*s, generator=g)
        elif k.endswith("a2.b"):
            t = 2.0 + torch.randn(*s, generator=g)
        elif k.endswith("correction"):
            t = 0.05 * torch.randn(*s, generator=g)
        else:
            t = 0.1 * torch.randn(*s, generator=g)
        sd[k] = t.to(torch.bfloat16).to(torch.float32)
    return sd
