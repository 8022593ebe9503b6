"""A plain, slow restatement of the Fokisun design, one function per mechanism, whole sequences only, on the CPU.

It shares no code with the engine: weights come as a dict name -> tensor, the configuration as the parsed
config.json.  Everything is computed in `dtype` (float64 by default), so it is the yardstick for both of the
engine's precisions.

    layer:    h = dyt(x);  X = x + m (mixer(h) + ff(h));  x = sum_j dwa[j] X_j  (X_0 = the embedding's output)
    dyt:      tanh(alpha x) w + b
    mixers:   latent attention | hgrn2 | windowed attention with a unit sink
    ff:       dense gated (gelu_tanh) | sigmoid-routed experts with groups and a shared expert
"""
from __future__ import annotations

import math

import torch


def dyt(x, w, b, alpha):
    return torch.tanh(alpha * x) * w + b


def rms(x, w, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def _angles(pos, base, dims, factor, dtype):
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims) / factor
    a = pos.to(dtype)[:, None] * f[None, :]                    # [T, dims / 2]
    return torch.cos(a), torch.sin(a)


def rotate_halves(x, pos, base, dims, factor=1.0):
    """x [T, heads, n]: element i turns with element i + dims / 2, i < dims / 2; the rest passes."""
    c, s = _angles(pos, base, dims, factor, x.dtype)
    c, s = c[:, None, :], s[:, None, :]
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def rotate_interleaved(x, pos, base, dims, factor=1.0):
    """x [T, heads, n]: element 2i turns with element 2i + 1, 2i + 1 < dims; the rest passes."""
    c, s = _angles(pos, base, dims, factor, x.dtype)
    c, s = c[:, None, :], s[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def latent_attention(h, W, p, m, eps):
    """Queries through a normed latent; keys and values from a normed latent plus one rotated key part for all heads."""
    T = h.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms(h @ W[p + "dq"].T, W[p + "dq.norm"], eps)
    q = (cq @ W[p + "uq"].T).view(T, H, d + r)
    q_plain, q_rot = q[..., :d], q[..., d:]
    kv = h @ W[p + "dkv"].T
    c = rms(kv[:, :rank], W[p + "dkv.norm"], eps)
    k_rot = kv[:, rank:].view(T, 1, r)
    rot = m["rot"]
    q_rot = rotate_halves(q_rot, pos, rot["base"], rot["dims"])
    k_rot = rotate_halves(k_rot, pos, rot["base"], rot["dims"])
    k_plain = (c @ W[p + "uk"].T).view(T, H, d)
    v = (c @ W[p + "uv"].T).view(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot[:, 0])) * m["scale"]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    s = s.masked_fill(~(j <= i), float("-inf"))
    o = torch.einsum("hij,jhd->ihd", torch.softmax(s, dim=-1), v)
    g = torch.sigmoid(h @ W[p + "g"].T)                          # [T, H]
    return (o * g[:, :, None]).reshape(T, H * dv) @ W[p + "o"].T


def hgrn2(h, W, p, m, eps):
    """S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t; f bounded below by `lower`."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ W[p + "q"].T).view(T, H, d)
    v = (h @ W[p + "v"].T).view(T, H, dv)
    low = W[p + "lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ W[p + "f"].T + W[p + "f.b"])).view(T, H, d)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hde,hd->he", S, q[t])
    out = rms(out, W[p + "norm"], eps)
    return out.reshape(T, H * dv) @ W[p + "o"].T


def attention(h, W, p, m, eps, v_first):
    """Grouped heads, biases, one norm over all of q (and of k), interleaved rotation, a window, a sink of score 0,
    values mixed with the first such layer's, a gate element by element.  Returns (output, this layer's values as
    they are cached)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rms(h @ W[p + "q"].T + W[p + "q.b"], W[p + "q.norm"], eps).view(T, H, d)
    k = rms(h @ W[p + "k"].T + W[p + "k.b"], W[p + "k.norm"], eps).view(T, G, d)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).view(T, G, dv)
    rot = m.get("rot")
    if rot:
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        q = rotate_interleaved(q, pos, rot["base"], rot["dims"], factor)
        k = rotate_interleaved(k, pos, rot["base"], rot["dims"], factor)
    if m.get("v_mix") and v_first is not None:
        lam = W[p + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    kx = k.repeat_interleave(H // G, dim=1)
    vx = v.repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kx) * m["scale"]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = j <= i
    window = (m.get("mask") or {}).get("size", 0)
    if window:
        seen = seen & (i - j < window)
    e = torch.exp(s - 0.0).masked_fill(~seen, 0.0)               # scores are small here; the sink's weight is exp(0)
    pr = e / (1.0 + e.sum(dim=-1, keepdim=True))
    o = torch.einsum("hij,jhd->ihd", pr, vx).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T + W[p + "o.b"], v


def gated_ff(h, W, p, act):
    return (act(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def route(h, W, p, router, margins_out=None):
    """(chosen experts [T, top], their weights [T, top]).  margins_out: a list that receives, per token, how far
    the choice is from turning (the last open group's lead over the first closed one, the last chosen score's over
    the first one left out; the smaller of the two)."""
    E, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    s = torch.sigmoid(h @ W[p + "router"].T)
    per = E // groups["count"]
    gs = s.view(-1, groups["count"], per).topk(min(2, per), dim=-1).values.sum(dim=-1)
    kept = gs.topk(groups["keep"], dim=-1).indices
    open_ = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, kept, True)
    masked = s.masked_fill(~open_.repeat_interleave(per, dim=1), float("-inf"))
    ids = masked.topk(top, dim=-1).indices
    w = s.gather(1, ids)
    if margins_out is not None:
        inf = torch.full((s.shape[0],), float("inf"), dtype=s.dtype)
        gsort = gs.sort(dim=-1, descending=True).values
        gm = gsort[:, groups["keep"] - 1] - gsort[:, groups["keep"]] if groups["keep"] < groups["count"] else inf
        msort = masked.sort(dim=-1, descending=True).values
        em = msort[:, top - 1] - msort[:, top] if top < per * groups["keep"] else inf
        margins_out.append(torch.minimum(gm, em))
    return ids, w / (w.sum(dim=-1, keepdim=True) + 1e-20) * router["scale"]


def moe_ff(h, W, p, f, margins_out=None):
    ids, w = route(h, W, p, f["router"], margins_out)
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, we in zip(ids[t].tolist(), w[t]):
            out[t] += we * gated_ff(h[t:t + 1], W, f"{p}e{e}.", silu)[0]
    if f.get("shared"):
        out = out + gated_ff(h, W, p + "shared.", silu)
    return out


def forward(cfg, weights, tokens, dtype=torch.float64, margins_out=None):
    """(logits [T, vocab], the stream behind every layer [L, T, width]).  margins_out: see `route`, one entry a
    routed layer."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, m_res = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    history, streams = [x], []
    v_first = None
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = dyt(x, W[p + "norm1"], W[p + "norm1.b"], W[p + "norm1.alpha"])
        if l["type"] == "latent_attention":
            a = latent_attention(h, W, p + "mix.", l["mixer"], eps)
        elif l["type"] == "hgrn2":
            a = hgrn2(h, W, p + "mix.", l["mixer"], eps)
        elif l["type"] == "attention":
            a, v = attention(h, W, p + "mix.", l["mixer"], eps, v_first)
            if l["mixer"].get("v_mix") and v_first is None:
                v_first = v
        else:
            raise ValueError(l["type"])
        f = l.get("mlp")
        if f:
            a = a + (gated_ff(h, W, p + "mlp.", gelu_tanh) if f["kind"] == "dense" else moe_ff(h, W, p + "mlp.", f, margins_out))
        history.append(x + m_res * a)
        coef = W[p + "dwa"]
        x = sum(coef[j] * history[j] for j in range(i + 2))
        streams.append(x)
    h = dyt(x, W["final.norm"], W["final.norm.b"], W["final.norm.alpha"])
    return (h @ W["embed"].T) * cfg.get("logit_scale", 1.0), torch.stack(streams)
