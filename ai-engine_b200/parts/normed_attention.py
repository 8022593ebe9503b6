"""Grouped-query softmax attention whose queries and keys are normed over the whole projection and rotated, with
a sliding window, a softmax that leaks into a sink, values mixed across layers and a gate on every output element:

    q = W_q h + b_q,  k = W_k h + b_k,  v = W_v h + b_v           (H query heads of d; G key/value heads of d and e)
    q <- q / rms(q) * w_q over all H d elements at once, k likewise over G d       (before the split into heads)
    the first rot_dims elements of every head of q and k are rotated by the position
    v <- (1 - lambda) v + lambda v_src        in every layer that mixes but the one that provides v_src: its own v
                                               of the same token; the mixed v is what is cached
    s(i, j) = (q_i . k_j) * scale over the keys j <= i with i - j < window (window 0: all)
    p(i, j) = exp(s(i, j)) / (exp(sink) + sum_j' exp(s(i, j')))      sink = 0: one is added to the denominator
    out = W_o (concat_h(sum_j p(i, j) v_j) * sigmoid(W_g h)) + b_o

Query head h reads key/value head h / (H / G).  A token's key and value lie side by side in one cache row, so the
two may differ in size.  Norms, angles, scores, weights, the mix and the gate are float32.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .attention import ATTENTION_WORK
from .base import KVRequest, Mixer


class NormedGatedAttention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, value_dim, scale, window (0: all keys), eps (of the
    q and k norms), qk_norm (default True), bias (q, k, v and o have one: default True), sink (the score of the
    softmax's sink; None: none), position_encoding (name of a rotary encoding, either layout; None: no rotation),
    value_mix (None | "source": this layer's values are kept for the step | "mix": they are mixed with the
    source's), value_mix_key (names the source among several).  tensors: q, k, v, g, o, and q_bias, k_bias, v_bias,
    o_bias, q_norm [H d], k_norm [G d], lambda (one number; read by "mix" layers, tolerated in a "source")."""

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
        self.window = int(p.get("window") or 0)
        self.eps = float(p["eps"])
        self.qk_norm, self.has_bias = bool(p.get("qk_norm", True)), bool(p.get("bias", True))
        self.sink_score = p.get("sink")
        pe = p.get("position_encoding")
        self.rope = env.position_encodings[pe] if pe else None
        if self.rope is not None and self.rope.rot_dim > self.d:
            raise ValueError("attention: the rotation is wider than a head")
        self.value_mix = p.get("value_mix")
        if self.value_mix not in (None, "source", "mix"):
            raise ValueError(f"attention: value_mix `{self.value_mix}` is not known (source, mix)")
        self.mix_key = "mixed_values_" + str(p.get("value_mix_key") or "")
        self.w_in = self.w_o = self.bias = self.o_bias = self.q_w = self.k_w = self.lam = self.sink = None

    def tensor_specs(self):
        t, Hd, Gd, Ge, He = self.spec.tensors, self.H * self.d, self.G * self.d, self.G * self.e, self.H * self.e
        specs = [TensorSpec(t["q"], (Hd, self.hidden)), TensorSpec(t["k"], (Gd, self.hidden)),
                 TensorSpec(t["v"], (Ge, self.hidden)), TensorSpec(t["g"], (He, self.hidden)),
                 TensorSpec(t["o"], (self.hidden, He))]
        if self.has_bias:
            specs += [TensorSpec(t["q_bias"], (Hd,), std=0.1), TensorSpec(t["k_bias"], (Gd,), std=0.1),
                      TensorSpec(t["v_bias"], (Ge,), std=0.1), TensorSpec(t["o_bias"], (self.hidden,), std=0.1)]
        if self.qk_norm:
            specs += [TensorSpec(t["q_norm"], (Hd,), init="ones"), TensorSpec(t["k_norm"], (Gd,), init="ones")]
        if self.value_mix is not None:
            specs.append(TensorSpec(t["lambda"], (), mean=0.4, std=0.1))
        return specs

    def load(self, source):
        t = self.spec.tensors
        ws = [source.get(t[n]) for n in ("q", "k", "v", "g")]
        dt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_in = torch.cat([w.to(dt) for w in ws], dim=0).contiguous()        # [q | k | v | gate logits]
        self.w_o = source.get(t["o"])
        f32 = lambda name: source.get(t[name]).float().contiguous()
        if self.has_bias:
            self.bias = torch.cat([f32("q_bias"), f32("k_bias"), f32("v_bias")]).contiguous()
            self.o_bias = f32("o_bias")
        if self.qk_norm:
            self.q_w, self.k_w = f32("q_norm"), f32("k_norm")
        if self.value_mix is not None:
            self.lam = f32("lambda").reshape(1)
        if self.sink_score is not None:
            self.sink = torch.full((self.H,), float(self.sink_score), dtype=torch.float32, device=self.env.device)

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o))

    def flops(self, tokens, keys=0.0):
        if self.window > 0:
            keys = min(keys, float(self.window))
        proj = 2.0 * tokens * self.hidden * (self.w_in.shape[0] + self.H * self.e)
        return proj + 2.0 * tokens * keys * self.H * (self.d + self.e)

    def cache_request(self):
        return KVRequest(self.G, self.d + self.e, self.window, planes=1)

    def step_planner(self):
        return ATTENTION_WORK

    def forward(self, h, ctx, cache, add_to=None):
        proj = ops.linear(h, self.w_in, torch.float32, ctx.err)
        rot = self.rope.rotation() if self.rope is not None else None
        mix_from = None
        if self.value_mix == "mix":
            mix_from = getattr(ctx, self.mix_key, None)
            if mix_from is None or mix_from.shape[0] != h.shape[0]:
                raise RuntimeError("attention: a layer mixes its values, but no earlier layer of the step provided any")
        q, kept = ops.normed_attn_prepare(proj, self.bias, self.q_w, self.k_w, self.eps, rot[0] if rot else None,
                                          rot[1] if rot else 0, rot is not None and not self.rope.interleaved,
                                          cache.k_pages, ctx, cache.block_table, self.H, self.G, self.d, self.e,
                                          mix_from=mix_from, mix_lambda=self.lam if mix_from is not None else None,
                                          keep_values=self.value_mix == "source", write=cache.writes)
        if kept is not None:
            setattr(ctx, self.mix_key, kept)
        a = ops.sink_attention(q, cache.k_pages, None, None, None, self.sink, ctx, ctx.plan(ATTENTION_WORK),
                               cache.block_table, self.e, self.scale, self.window, 0)
        a = a.view(a.shape[0], self.H * self.e)
        n = self.H * self.d + self.G * (self.d + self.e)
        ops.sigmoid_gate_mul_(a, proj[:, n:n + self.H * self.e], 1)
        y = ops.linear_parts(a, self.w_o, ctx.err)
        return ops.add_bias_(y, self.o_bias) if self.o_bias is not None else y
