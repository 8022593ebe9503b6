"""Softmax attention without a rotation, whose positions enter through a distance bias, with a window that keeps
the first tokens, a sink in the softmax and a gate per head:

    q = W_q h + b_q,  k = W_k h + b_k,  v = W_v h + b_v         (H query heads of d; G key/value heads of d and e)
    v <- v / rms(v) per head, no weight; it is cached so
    s(i, j) = (q_i . k_j) * scale * temp[h] - slope[h] * (i - j),    slope[h] = 2^(-slope_bits (h + 1) / H)
    i reads j  iff  j <= i and (i - j < window or j < keep_first)    (window 0: every j <= i)
    p(i, j) = exp(s(i, j)) / (exp(sink[h]) + sum_j' exp(s(i, j')))   the sink has no key and no value
    out = W_o concat_h(sigmoid(W_g h)_h * sum_j p(i, j) v_j)

Query head h reads key/value head h / (H / G).  A token's key and normalised value lie side by side in one cache
row, so the two may differ in size.  Scores, weights, the value norm and the gate are float32.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .attention import ATTENTION_WORK
from .base import KVRequest, Mixer


def distance_slopes(heads: int, bits: float):
    """slope[h] = 2^(-bits (h + 1) / heads) for h = 0 .. heads - 1."""
    return [2.0 ** (-float(bits) * (h + 1) / heads) for h in range(heads)]


class SinkWindowAttention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, value_dim, scale, window (0: all keys), keep_first,
    eps (of the value norm), slope_bits (None or 0: no distance bias), bias (q, k, v have one: default True),
    temperature, sink, gate (the three per-head extras: default True; a design without one leaves it out).
    tensors: q, k, v, o, and q_bias, k_bias, v_bias, temp [H], sink [H], g [H, hidden]."""

    adds_in_place = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.H, self.G = int(p["num_heads"]), int(p["num_kv_heads"])
        self.d, self.e = int(p["head_dim"]), int(p["value_dim"])
        if self.H % self.G:
            raise ValueError(f"attention: {self.H} heads are not a multiple of {self.G} kv heads")
        if not (0 < self.d <= 256 and 0 < self.e <= 256):
            raise ValueError(f"attention: head sizes {self.d} / {self.e} must be within 1 .. 256")
        self.scale = float(p["scale"]) if p.get("scale") is not None else float(self.d) ** -0.5
        self.window, self.keep_first = int(p.get("window") or 0), int(p.get("keep_first") or 0)
        if self.window < 0 or self.keep_first < 0:
            raise ValueError("attention: window and keep_first must not be negative")
        self.eps = float(p["eps"])
        self.slope_bits = float(p.get("slope_bits") or 0.0)
        self.has_bias = bool(p.get("bias", True))
        self.has_temp, self.has_sink, self.has_gate = (bool(p.get(n, True)) for n in ("temperature", "sink", "gate"))
        self.w_in = self.w_o = self.bias = self.temp = self.sink = self.slope = None

    def tensor_specs(self):
        t, Hd, Gd, Ge = self.spec.tensors, self.H * self.d, self.G * self.d, self.G * self.e
        specs = [TensorSpec(t["q"], (Hd, self.hidden)), TensorSpec(t["k"], (Gd, self.hidden)),
                 TensorSpec(t["v"], (Ge, self.hidden)), TensorSpec(t["o"], (self.hidden, self.H * self.e))]
        if self.has_bias:
            specs += [TensorSpec(t["q_bias"], (Hd,), std=0.1), TensorSpec(t["k_bias"], (Gd,), std=0.1),
                      TensorSpec(t["v_bias"], (Ge,), std=0.1)]
        if self.has_temp:
            specs.append(TensorSpec(t["temp"], (self.H,), mean=1.0, std=0.2))
        if self.has_sink:
            specs.append(TensorSpec(t["sink"], (self.H,), std=1.0))
        if self.has_gate:
            specs.append(TensorSpec(t["g"], (self.H, self.hidden)))
        return specs

    def load(self, source):
        t = self.spec.tensors
        ws = [source.get(t[n]) for n in ("q", "k", "v")] + ([source.get(t["g"])] if self.has_gate else [])
        dt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_in = torch.cat([w.to(dt) for w in ws], dim=0).contiguous()        # [q | k | v | gate logits]
        self.w_o = source.get(t["o"])
        f32 = lambda name: source.get(t[name]).float().contiguous()
        if self.has_bias:
            self.bias = torch.cat([f32("q_bias"), f32("k_bias"), f32("v_bias")]).contiguous()
        self.temp = f32("temp") if self.has_temp else None
        self.sink = f32("sink") if self.has_sink else None
        if self.slope_bits:
            self.slope = torch.tensor(distance_slopes(self.H, self.slope_bits), dtype=torch.float32,
                                      device=self.env.device)

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o))

    def flops(self, tokens, keys=0.0):
        if self.window > 0:
            keys = min(keys, float(self.window + self.keep_first))
        proj = 2.0 * tokens * self.hidden * (self.w_in.shape[0] + self.H * self.e)
        return proj + 2.0 * tokens * keys * self.H * (self.d + self.e)

    def cache_request(self):
        return KVRequest(self.G, self.d + self.e, self.window, planes=1, keep_first=self.keep_first if self.window else 0)

    def step_planner(self):
        return ATTENTION_WORK

    def forward(self, h, ctx, cache, add_to=None):
        proj = ops.linear(h, self.w_in, torch.float32, ctx.err)
        if not self.has_gate:
            raise NotImplementedError("attention without a gate: the prepare kernel reads the gate's logits")
        q, gate = ops.sink_attn_prepare(proj, self.bias, cache.k_pages, ctx, cache.block_table, self.H, self.G, self.d,
                                        self.e, self.eps, write=cache.writes)
        a = ops.sink_attention(q, cache.k_pages, gate, self.temp, self.slope, self.sink, ctx, ctx.plan(ATTENTION_WORK),
                               cache.block_table, self.e, self.scale, self.window, self.keep_first)
        a = a.view(a.shape[0], self.H * self.e)
        if add_to is not None and ops.linear_add(add_to, a, self.w_o):
            return None
        return ops.linear_parts(a, self.w_o, ctx.err)
