"""A plain, slow restatement of the Tizodra design, one function per mechanism, in torch on the CPU.

It shares nothing with the engine: it reads a dict of tensors by name and the raw config.json dict, runs a
whole sequence from its first token, and returns logits for every token.  Everything is computed in the
dtype the caller asks for (float64 by default).

Notation: T tokens, D = width.  Attention: H query heads, G key/value heads, d per-head query/key size, e
per-head value size.  Delta mixer: H value heads, G query/key heads, d and e as above, S a [d, e] matrix a head.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


# ---------------------------------------------------------------------------------------------------
# token-local pieces
def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def relu_squared(z):
    r = torch.clamp(z, min=0.0)
    return r * r


def dense_ff(h, w_up, w_down):
    return relu_squared(h @ w_up.T) @ w_down.T


def sinusoid(positions: torch.Tensor, width: int, dtype=torch.float64) -> torch.Tensor:
    """[T, width]: column 2i = sin(p * base^(-2i / width)), column 2i + 1 = cos of the same angle, base 10000."""
    out = torch.zeros(positions.shape[0], width, dtype=dtype)
    p = positions.to(dtype)
    for c in range(width):
        i = c // 2
        angle = p * (10000.0 ** (-2.0 * i / width))
        out[:, c] = torch.sin(angle) if c % 2 == 0 else torch.cos(angle)
    return out


# ---------------------------------------------------------------------------------------------------
# attention with a window that keeps the first tokens, a distance bias, a sink, a gate a head
def head_slopes(H: int) -> List[float]:
    return [2.0 ** (-8.0 * (h + 1) / H) for h in range(H)]


def visible(i: int, j: int, size: int, keep_first: int) -> bool:
    """Whether the token at place i reads the token at place j.  size 0: no window."""
    if j > i:
        return False
    return size <= 0 or i - j < size or j < keep_first


def sink_attention(h, w: Dict[str, torch.Tensor], m: dict, eps: float, first_position: int = 0):
    """h [T, D] (one sequence, its first row at place `first_position`) -> [T, D].  `w`: the mixer's tensors by
    their short names (q, q.b, k, k.b, v, v.b, temp, sink, g, o); `m`: the mixer's entry of config.json."""
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    mask = m.get("mask") or {}
    size, keep = int(mask.get("size") or 0), int(mask.get("keep_first") or 0)
    T = h.shape[0]
    q = (h @ w["q"].T + w["q.b"]).view(T, H, d)
    k = (h @ w["k"].T + w["k.b"]).view(T, G, d)
    v = rms((h @ w["v"].T + w["v.b"]).view(T, G, e), eps)             # the value is kept normalised
    gate = torch.sigmoid(h @ w["g"].T)                                # [T, H]
    slopes = head_slopes(H)
    out = torch.zeros(T, H, e, dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        for t in range(T):
            i = first_position + t
            js = torch.tensor([j for j in range(T) if visible(i, first_position + j, size, keep)], dtype=torch.long)
            s = (k[js, g] @ q[t, a]) * m["scale"] * w["temp"][a] - slopes[a] * (t - js).to(h.dtype)
            top = torch.maximum(s.max(), w["sink"][a])
            p = torch.exp(s - top)
            denom = p.sum() + torch.exp(w["sink"][a] - top)           # the sink: a weight without a value
            out[t, a] = (p[:, None] * v[js, g]).sum(dim=0) / denom
    out = out * gate[:, :, None]
    return out.reshape(T, H * e) @ w["o"].T


# ---------------------------------------------------------------------------------------------------
# gated delta rule
def causal_conv(u, w):
    """u [T, C], w [C, taps] (the last column weighs the current token); zeros before the first token."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], dim=0)
    out = torch.zeros_like(u)
    for j in range(taps):
        out = out + padded[j:j + T] * w[:, j]
    return out


def unit(x):
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


def delta_mixer(h, w: Dict[str, torch.Tensor], m: dict, eps: float, keep_states: Optional[list] = None):
    """h [T, D] (one sequence from its first token) -> [T, D].  `w`: the mixer's tensors by their short names
    (q, q.conv, k, k.conv, v, v.conv, b, a, A_log, dt_bias, norm, g, o)."""
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(causal_conv(h @ w["q"].T, w["q.conv"])).view(T, G, d)
    k = silu(causal_conv(h @ w["k"].T, w["k.conv"])).view(T, G, d)
    v = silu(causal_conv(h @ w["v"].T, w["v.conv"])).view(T, H, e)
    q = unit(q) * d ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ w["b"].T)                                            # [T, H]
    decay = torch.exp(-torch.exp(w["A_log"]) * softplus(h @ w["a"].T + w["dt_bias"]))   # [T, H]
    o = torch.zeros(T, H, e, dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        S = torch.zeros(d, e, dtype=h.dtype)
        for t in range(T):
            S = decay[t, a] * S
            u = beta[t, a] * (v[t, a] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            o[t, a] = S.T @ q[t, g]                                               # reads this token's write
        if keep_states is not None:
            keep_states.append(S)
    y = rms(o, eps) * w["norm"] * silu(h @ w["g"].T).view(T, H, e)
    return y.reshape(T, H * e) @ w["o"].T


# ---------------------------------------------------------------------------------------------------
# the whole model
def run_order(cfg: dict) -> List[tuple]:
    """[(layer index, first of a pass)]: the layers of `loop` run `times` times in a row, the rest once."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    order = [(i, False) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        order += [(i, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return order + [(i, False) for i in range(loop["stop"], n)]


def sub(w: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def forward(weights: Dict[str, torch.Tensor], cfg: dict, tokens, dtype=torch.float64, streams: Optional[list] = None):
    """Logits [T, vocab] of one sequence from its first token.  `streams`: receives the residual stream after
    every layer run."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    D, eps = cfg["width"], cfg["norm"]["eps"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    T = ids.shape[0]
    x0 = w["embed"][ids] + sinusoid(torch.arange(T), D, dtype)
    x = x0
    for i, first in run_order(cfg):
        L, p = cfg["layers"][i], f"l{i}."
        if first:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T
        hn = rms(x, eps) * w[p + "norm1"]
        if L["type"] == "attention":
            x = x + sink_attention(hn, sub(w, p + "mix."), L["mixer"], eps)
        elif L["type"] == "delta":
            x = x + delta_mixer(hn, sub(w, p + "mix."), L["mixer"], eps)
        else:
            raise ValueError(f"layer type {L['type']}")
        if L.get("mlp"):
            x = x + dense_ff(rms(x, eps) * w[p + "norm2"], w[p + "mlp.up"], w[p + "mlp.down"])
        if streams is not None:
            streams.append(x.clone())
    return (rms(x, eps) * w["final.norm"]) @ w["head"].T * cfg.get("logit_scale", 1.0)


def greedy(weights, cfg, prompt, n_new: int, dtype=torch.float64):
    """(tokens, margins): greedy continuation of `prompt`, and at each new token the best logit's lead over the
    second."""
    toks, margins = list(prompt), []
    for _ in range(n_new):
        top = forward(weights, cfg, toks, dtype)[-1].topk(2)
        margins.append(float(top.values[0] - top.values[1]))
        toks.append(int(top.indices[0]))
    return toks, margins
