"""Plain, slow restatement of the Lefalix design in torch, one function per mechanism, for the tests to compare the
framework against.  It shares no code with the package: it takes the parsed ``config.json`` dictionary and a
``{tensor name: tensor}`` dictionary and recomputes every position from the whole token list (no state, no batch).

Everything runs in float64 on the CPU: the comparison tolerances of the tests are what the framework's bfloat16 / float32
arithmetic may lose against exact arithmetic.

Notation: ``T`` tokens, ``d`` width, ``H`` value (or query) heads, ``G`` key heads, ``dk`` / ``dv`` per-head key / value sizes,
``n`` taps of a short convolution.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w


def causal_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u (T, C), w (C, n): y[t] = sum_j w[:, j] * u[t - (n - 1) + j], zero for negative times."""
    T, C = u.shape
    n = w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(n):
            src = t - (n - 1) + j
            if src >= 0:
                y[t] += w[:, j] * u[src]
    return y


def rotary_frequencies(rot: dict) -> torch.Tensor:
    dims, base = rot["dims"], rot["base"]
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    sc = rot.get("scaling")
    if not sc:
        return f
    def index_of(turns):
        return dims * math.log(sc["original"] / (2 * math.pi * turns)) / (2 * math.log(base))
    lo = max(math.floor(index_of(sc["fast"])), 0)
    hi = min(math.ceil(index_of(sc["slow"])), dims - 1)
    i = torch.arange(dims // 2, dtype=F64)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
    return f / sc["factor"] * ramp + f * (1 - ramp)


def rotate(x: torch.Tensor, rot: Optional[dict], first_position: int = 0) -> torch.Tensor:
    """x (T, heads, dk): pairs (2i, 2i + 1) of the first rot.dims dimensions turned by position * frequency_i."""
    if not rot or rot["dims"] == 0:
        return x
    f = rotary_frequencies(rot)
    mag = 0.1 * math.log(rot["scaling"]["factor"]) + 1 if rot.get("scaling") else 1.0
    out = x.clone()
    for t in range(x.shape[0]):
        ang = (first_position + t) * f
        c, s = torch.cos(ang) * mag, torch.sin(ang) * mag
        a, b = x[t, :, 0 : rot["dims"] : 2], x[t, :, 1 : rot["dims"] : 2]
        out[t, :, 0 : rot["dims"] : 2] = a * c - b * s
        out[t, :, 1 : rot["dims"] : 2] = b * c + a * s
    return out


def window_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv(h @ W[p + "q"].T + W[p + "q.b"], W[p + "q.conv"]).view(T, H, dk)
    k = causal_conv(h @ W[p + "k"].T + W[p + "k.b"], W[p + "k.conv"]).view(T, G, dk)
    v = causal_conv(h @ W[p + "v"].T + W[p + "v.b"], W[p + "v.conv"]).view(T, G, dv)
    q = unit_rms(rotate(q, m.get("rot")), eps)
    k = unit_rms(rotate(k, m.get("rot")), eps)
    window = m["mask"]["size"]
    out = torch.zeros(T, H, dv, dtype=F64)
    for i in range(T):
        lo = max(0, i - window + 1)
        for hh in range(H):
            g = hh // (H // G)
            s = (k[lo : i + 1, g] @ q[i, hh]) * m["scale"]
            e = torch.exp(s - s.max())
            denom = e.sum() + torch.exp(W[p + "sink"][hh] - s.max())
            out[i, hh] = (e / denom) @ v[lo : i + 1, g]
    return out.reshape(T, H * dv) @ W[p + "o"].T + W[p + "o.b"]


def delta_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor) -> torch.Tensor:
    """One head.  q, k (T, dk), v (T, dv), g (T,) or (T, dk), beta (T,).  Decay, error-corrected write, then read."""
    T, dk = q.shape
    S = torch.zeros(dk, v.shape[1], dtype=F64)
    o = torch.zeros(T, v.shape[1], dtype=F64)
    for t in range(T):
        S = S * (g[t][:, None] if g.dim() == 2 else g[t])
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        o[t] = S.T @ q[t]
    return o


def delta_mixer(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float, channel: bool) -> torch.Tensor:
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    silu = torch.nn.functional.silu
    q = silu(causal_conv(h @ W[p + "q"].T, W[p + "q.conv"])).view(T, G, dk)
    k = silu(causal_conv(h @ W[p + "k"].T, W[p + "k.conv"])).view(T, G, dk)
    v = silu(causal_conv(h @ W[p + "v"].T, W[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[p + "b"].T)
    rate = torch.exp(W[p + "A_log"])
    if channel:
        step = torch.nn.functional.softplus((h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]).view(T, H, dk)
        g = torch.exp(-rate[None, :, None] * step)
        gate = torch.sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T).view(T, H, dv)
    else:
        g = torch.exp(-rate[None, :] * torch.nn.functional.softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))
        gate = silu(h @ W[p + "g"].T).view(T, H, dv)
    o = torch.stack([delta_scan(q[:, hh // (H // G)], k[:, hh // (H // G)], v[:, hh], g[:, hh], beta[:, hh]) for hh in range(H)], dim=1)
    o = unit_rms(o, eps) * W[p + "norm"] * gate
    return o.reshape(T, H * dv) @ W[p + "o"].T


def route(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, router: dict):
    """-> (ids (T, top), weights (T, top)): softmax scores over all experts; only experts of the `keep` groups with the largest
    best score are eligible; the weights are the chosen scores as they are."""
    E, top = router["experts"], router["top"]
    groups = router.get("groups") or {}
    count = groups.get("count", 1)
    keep = groups.get("keep", count)
    s = torch.softmax(h @ W[p + "router"].T, dim=-1)
    best = s.view(-1, count, E // count).max(dim=-1).values
    kept = best.topk(keep, dim=-1).indices
    eligible = torch.zeros_like(best, dtype=torch.bool).scatter(1, kept, True).repeat_interleave(E // count, dim=1)
    ids = s.masked_fill(~eligible, -1.0).topk(top, dim=-1).indices
    return ids, s.gather(1, ids)


def feed_forward(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, f: dict) -> torch.Tensor:
    if f["kind"] == "dense":
        return torch.nn.functional.gelu(h @ W[p + "up"].T) @ W[p + "down"].T
    ids, wts = route(h, W, p, f["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(ids[t].tolist(), wts[t]):
            q = f"{p}e{e}."
            out[t] += s * ((torch.nn.functional.silu(h[t] @ W[q + "gate"].T) * (h[t] @ W[q + "up"].T)) @ W[q + "down"].T)
    return out


def layer_runs(cfg: dict) -> List[tuple]:
    """(layer index, the embedding re-enters first) for every layer run, in order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    runs = [(i, False) for i in range(loop["start"])]
    for rep in range(loop["times"]):
        runs += [(i, rep > 0 and i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, False) for i in range(loop["stop"], n)]


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], return_layers: bool = False):
    """-> logits (T, vocab) in float64 (and the residual stream after every layer run)."""
    W = {k: v.to(F64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x0 = W["embed"][torch.tensor(tokens, dtype=torch.long)]
    x = x0.clone()
    seen = []
    for i, reenter in layer_runs(cfg):
        if reenter:
            x = x + x0
        layer, p = cfg["layers"][i], f"l{i}."
        h = norm(x, W[p + "norm1"], eps)
        if layer["type"] == "parallel":
            a = window_attention(h, W, p + "mix.left.", layer["mixer"]["left"], eps)
            b = delta_mixer(h, W, p + "mix.right.", layer["mixer"]["right"], eps, channel=False)
            y = 0.5 * (norm(a, W[p + "mix.left.out"], eps) + norm(b, W[p + "mix.right.out"], eps))
        else:
            y = delta_mixer(h, W, p + "mix.", layer["mixer"], eps, channel=True)
        x = x + norm(y, W[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            x = x + norm(feed_forward(norm(x, W[p + "norm2"], eps), W, p + "mlp.", layer["mlp"]), W[p + "norm2b"], eps)
        seen.append(x.clone())
    logits = norm(x, W["final.norm"], eps) @ W["head"].T
    return (logits, seen) if return_layers else logits
