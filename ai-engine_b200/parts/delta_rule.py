"""The gated delta rule: a linear attention whose state is corrected towards each token's value along its key
instead of only added to, and decays by one number per token and head:

    q, k = W_q h, W_k h  (G heads of d);  v = W_v h  (H heads of e);  head h reads q/k head h / (H / G)
    q, k, v <- silu(causal convolution over time, per channel, `taps` taps, no bias)
    q <- q / sqrt(|q|^2 + unit_eps) * d^(-1/2),  k <- k / sqrt(|k|^2 + unit_eps)          per head
    beta = sigmoid(W_b h);  g = exp(-exp(A_log) * softplus(W_a h + dt_bias))              per head
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q                          S [d, e] float32
    out = W_o (o / rms(o) * w * silu(W_g h))                                              rms per head, w [e]

The state and the convolution's last taps - 1 inputs live in the request's slot, so a portion of a prompt or a
decoded token continues where the previous step stopped.  Everything behind the convolution's activation is float32.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Mixer, StateRequest


class GatedDeltaRule(Mixer):
    """params: hidden_size, num_heads (H), num_qk_heads (G), key_dim (d), value_dim (e), taps, eps (of the output
    norm), unit_eps (default 1e-6).  tensors: q, k [G d, hidden], v, g [H e, hidden], b, a [H, hidden],
    q_conv, k_conv [G d, taps], v_conv [H e, taps], a_log, dt_bias [H], norm [e], o [hidden, H e]."""

    adds_in_place = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.H, self.G = int(p["hidden_size"]), int(p["num_heads"]), int(p["num_qk_heads"])
        self.d, self.e, self.taps = int(p["key_dim"]), int(p["value_dim"]), int(p["taps"])
        self.eps, self.unit_eps = float(p["eps"]), float(p.get("unit_eps") or 1e-6)
        if self.H % self.G:
            raise ValueError(f"delta rule: {self.H} heads are not a multiple of {self.G} query/key heads")
        if self.taps < 1:
            raise ValueError(f"delta rule: taps must be >= 1, got {self.taps}")
        if not 0 < self.d <= 256:
            raise ValueError(f"delta rule: key_dim {self.d} must be within 1 .. 256")
        self.channels = 2 * self.G * self.d + self.H * self.e
        self.w_in = self.w_o = self.w_conv = self.a_log = self.dt_bias = self.norm_w = None

    def tensor_specs(self):
        t, Gd, He = self.spec.tensors, self.G * self.d, self.H * self.e
        return [TensorSpec(t["q"], (Gd, self.hidden)), TensorSpec(t["k"], (Gd, self.hidden)),
                TensorSpec(t["v"], (He, self.hidden)), TensorSpec(t["g"], (He, self.hidden)),
                TensorSpec(t["b"], (self.H, self.hidden)), TensorSpec(t["a"], (self.H, self.hidden)),
                TensorSpec(t["q_conv"], (Gd, self.taps), std=0.4), TensorSpec(t["k_conv"], (Gd, self.taps), std=0.4),
                TensorSpec(t["v_conv"], (He, self.taps), std=0.4),
                TensorSpec(t["a_log"], (self.H,), mean=-0.5, std=0.5), TensorSpec(t["dt_bias"], (self.H,), mean=-1.0, std=0.5),
                TensorSpec(t["norm"], (self.e,), init="ones"), TensorSpec(t["o"], (self.hidden, He))]

    def load(self, source):
        t = self.spec.tensors
        ws = [source.get(t[n]) for n in ("q", "k", "v", "g", "b", "a")]
        dt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_in = torch.cat([w.to(dt) for w in ws], dim=0).contiguous()        # [q | k | v | gate | beta | decay]
        self.w_o = source.get(t["o"])
        f32 = lambda name: source.get(t[name]).float().contiguous()
        self.w_conv = torch.cat([f32("q_conv"), f32("k_conv"), f32("v_conv")], dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm_w = f32("a_log"), f32("dt_bias"), f32("norm")

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o))

    def flops(self, tokens, keys=0.0):
        proj = 2.0 * tokens * self.hidden * (self.w_in.shape[0] + self.H * self.e)
        return proj + 6.0 * tokens * self.H * self.d * self.e

    def state_request(self):
        return {"tail": StateRequest((self.taps - 1, self.channels), torch.float32),
                "S": StateRequest((self.H, self.d, self.e), torch.float32)}

    def forward(self, h, ctx, cache, add_to=None):
        Gd, He, C = self.G * self.d, self.H * self.e, self.channels
        proj = ops.linear(h, self.w_in, torch.float32, ctx.err)
        qkv = ops.causal_conv(proj[:, :C], self.w_conv, None, cache.state["tail"], ctx, torch.float32, activation="silu")
        o = ops.delta_rule(qkv[:, :Gd], qkv[:, Gd:2 * Gd], qkv[:, 2 * Gd:], proj[:, C + He:C + He + self.H],
                           proj[:, C + He + self.H:C + He + 2 * self.H], self.a_log, self.dt_bias,
                           float(self.d) ** -0.5, self.unit_eps, cache.state["S"], ctx, self.H, self.G, self.d, self.e,
                           chunked=self.env.dtype != torch.float32)
        y = ops.head_norm_gate(o, proj[:, C:C + He], self.norm_w, self.eps, self.env.dtype)
        if add_to is not None and ops.linear_add(add_to, y, self.w_o):
            return None
        return ops.linear_parts(y, self.w_o, ctx.err)
