"""Plain, slow restatement of the Pomipel design in torch, one function per mechanism, for the tests to compare the
framework against.  It shares no code with the package: it takes the parsed ``config.json`` dictionary and a
``{tensor name: tensor}`` dictionary and recomputes every position from the whole token list (no cache, no batch).

Notation: ``d`` model width, ``H`` heads, ``dk`` / ``dv`` per-head query-key / value sizes, ``r`` latent size.
``dtype`` is the storage / matrix-product dtype (float32, float64 or bfloat16); what the design computes in 32-bit
(softmax, norms, router, the residual stream) is computed in at least float32 whatever ``dtype`` is.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def _hi(dtype: torch.dtype) -> torch.dtype:
    return torch.float64 if dtype == torch.float64 else torch.float32


def linear(x: torch.Tensor, w: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """y = W x with weights stored (out, in); operands in ``dtype``, accumulation at least 32-bit."""
    if dtype == torch.bfloat16:
        return (x.to(dtype).float() @ w.to(dtype).float().t()).to(dtype)
    return x.to(dtype) @ w.to(dtype).t()


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_plain(x: torch.Tensor, w: torch.Tensor, eps: float, dtype: torch.dtype) -> torch.Tensor:
    """x / rms(x) * w, statistics in 32-bit."""
    hi = _hi(dtype)
    return (rms_unit(x.to(hi), eps) * w.to(hi)).to(dtype)


def norm_zero_centred(x: torch.Tensor, w: torch.Tensor, eps: float, hi: torch.dtype) -> torch.Tensor:
    """x / rms(x) * (1 + w): the block and final norm, result left in 32-bit."""
    return rms_unit(x.to(hi), eps) * (1.0 + w.to(hi))


def embed(tokens: List[int], weights: Dict[str, torch.Tensor], scale: float, hi: torch.dtype, start: int = 0) -> torch.Tensor:
    idx = torch.tensor(tokens, dtype=torch.long)
    pos = torch.arange(start, start + len(tokens))
    return weights["embed"].to(hi)[idx] * scale + weights["pos"].to(hi)[pos]


def latent_of(h: torch.Tensor, weights: Dict[str, torch.Tensor], prefix: str, eps: float, dtype: torch.dtype) -> torch.Tensor:
    """The cached latent c = norm(W_dkv h) of an attention layer that owns one."""
    return norm_plain(linear(h, weights[prefix + "dkv"], dtype), weights[prefix + "dkv.norm"], eps, dtype)


def latent_attention(h: torch.Tensor, c: torch.Tensor, weights: Dict[str, torch.Tensor], prefix: str, mixer: dict, eps: float,
                     dtype: torch.dtype) -> torch.Tensor:
    """h (T, d) in ``dtype``; c (T, r) the latents of the same positions (own or borrowed).  Causal, full softmax."""
    hi = _hi(dtype)
    H, dk, dv = mixer["heads"], mixer["dim"], mixer["vdim"]
    T = h.shape[0]
    cq = norm_plain(linear(h, weights[prefix + "dq"], dtype), weights[prefix + "dq.norm"], eps, dtype)
    q = linear(cq, weights[prefix + "uq"], dtype).view(T, H, dk)
    k = linear(c, weights[prefix + "uk"], dtype).view(T, H, dk)
    v = linear(c, weights[prefix + "uv"], dtype).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=hi)
    for i in range(T):
        for hh in range(H):
            s = (k[: i + 1, hh].to(hi) @ q[i, hh].to(hi)) * mixer["scale"]
            p = torch.softmax(s, dim=0)
            out[i, hh] = p @ v[: i + 1, hh].to(hi)
    return linear(out.to(dtype).reshape(T, H * dv), weights[prefix + "o"], dtype)


def route(h: torch.Tensor, weights: Dict[str, torch.Tensor], prefix: str, router: dict, hi: torch.dtype):
    """-> (chosen expert ids (T, top), their weights (T, top)).  Sigmoid scores; the choice uses score + correction
    restricted to the best groups (a group's rank is the sum of its two largest corrected scores); the weights are
    the uncorrected scores, not renormalised."""
    E, top = router["experts"], router["top"]
    G, keep = router["groups"]["count"], router["groups"]["keep"]
    z = h.to(hi) @ weights[prefix + "router"].to(hi).t()
    s = torch.sigmoid(z)
    choice = s + weights[prefix + "correction"].to(hi)
    T = h.shape[0]
    per = E // G
    ids = torch.zeros(T, top, dtype=torch.long)
    wts = torch.zeros(T, top, dtype=hi)
    for t in range(T):
        grp = choice[t].view(G, per)
        rank = torch.sort(grp, dim=1, descending=True).values[:, : min(2, per)].sum(dim=1)
        kept = torch.sort(rank, descending=True, stable=True).indices[:keep].tolist()
        allowed = torch.full((E,), -math.inf, dtype=hi)
        for g in kept:
            allowed[g * per : (g + 1) * per] = choice[t, g * per : (g + 1) * per]
        pick = torch.sort(allowed, descending=True, stable=True).indices[:top]
        ids[t] = pick
        wts[t] = s[t, pick]
    return ids, wts


def moe(h: torch.Tensor, weights: Dict[str, torch.Tensor], prefix: str, mlp: dict, dtype: torch.dtype) -> torch.Tensor:
    hi = _hi(dtype)
    ids, wts = route(h, weights, prefix, mlp["router"], hi)
    T = h.shape[0]
    out = torch.zeros(T, weights[prefix + "e0.down"].shape[0], dtype=hi)
    for t in range(T):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            u = linear(h[t : t + 1], weights[f"{prefix}e{e}.up"], dtype)
            a = torch.relu(u.to(hi)) ** 2
            y = linear(a.to(dtype), weights[f"{prefix}e{e}.down"], dtype)
            out[t] += wts[t, j] * y[0].to(hi)
    return out


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype: torch.dtype = torch.float32,
            return_layers: bool = False):
    """Logits (T, vocab) in 32-bit (or 64-bit for dtype float64) of one sequence starting at position 0."""
    hi = _hi(dtype)
    eps = config["norm"]["eps"]
    x = embed(tokens, weights, config["embedding"]["scale"], hi)
    latents: Dict[int, torch.Tensor] = {}
    layers = []
    for i, layer in enumerate(config["layers"]):
        assert layer["type"] == "latent_attention"
        p = f"l{i}."
        mixer = layer["mixer"]
        h = x.to(dtype)
        src = mixer.get("kv_from")
        if src is None:
            latents[i] = latent_of(h, weights, p + "mix.", eps, dtype)
            c = latents[i]
        else:
            c = latents[src]
        m = latent_attention(h, c, weights, p + "mix.", mixer, eps, dtype)
        x = x + norm_zero_centred(m, weights[p + "norm1"], eps, hi)
        if layer.get("mlp") is not None:
            f = moe(x.to(dtype), weights, p + "mlp.", layer["mlp"], dtype)
            x = x + norm_zero_centred(f, weights[p + "norm2"], eps, hi)
        layers.append(x.clone())
    xn = norm_zero_centred(x, weights["final.norm"], eps, hi).to(dtype)
    logits = linear(xn, weights["head"], dtype).to(hi) * config["logit_scale"]
    if return_layers:
        return logits, torch.stack(layers)
    return logits
