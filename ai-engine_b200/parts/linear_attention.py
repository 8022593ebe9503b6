"""Linear attention with a decaying matrix state per head and no softmax:

    S_t = diag(a_t) S_(t-1) + k_t v_t^T,    o_t = S_t^T q_t        (S: [key_dim, value_dim], float32)

The decay a_t is a constant per head (retention) or depends on the token and the key channel through a
low-rank projection, a_t = sigmoid(W_2 (W_1 h_t) + b)^(1 / tau) (gated linear attention).  Each head's output
is divided by its root mean square (with or without a weight), multiplied by silu(W_g h) and projected by
W_o.  The state starts at zero and is carried from token to token in the request's slot, so prompts in
portions and decoded tokens continue one another.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Mixer, StateRequest


class DecayLinearAttention(Mixer):
    """params: hidden_size, num_heads, key_dim, value_dim, eps; decay: a list of one constant per head, or None
    with tau and decay_rank (the rank random weights get; a file's tensors decide theirs); scale_on: "q" | "k"
    (which of the two is multiplied by key_dim^-1/2); norm_weight (bool: the output norm has a weight [value_dim]
    shared by the heads).  tensors: q, k [H d, hidden], v, g [H dv, hidden], o [hidden, H dv], norm, and for a
    gated decay a1 [r, hidden], a2 [H d, r], a2_bias [H d]."""

    adds_in_place = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.H = int(p["hidden_size"]), int(p["num_heads"])
        self.d, self.dv, self.eps = int(p["key_dim"]), int(p["value_dim"]), float(p["eps"])
        self.decay = None if p.get("decay") is None else [float(x) for x in p["decay"]]
        if self.decay is not None and len(self.decay) != self.H:
            raise ValueError("linear attention: one decay per head")
        self.tau = float(p.get("tau") or 0.0)
        self.decay_rank = int(p.get("decay_rank") or 16)
        if self.decay is None and self.tau <= 0:
            raise ValueError("linear attention: a gated decay needs tau > 0")
        if p.get("scale_on") not in ("q", "k"):
            raise ValueError("linear attention: scale_on is q or k")
        s = float(self.d) ** -0.5
        self.q_scale, self.k_scale = (s, 1.0) if p["scale_on"] == "q" else (1.0, s)
        self.norm_weight = bool(p.get("norm_weight"))
        self.w_in = self.w_o = self.w_a2 = self.a2_bias = self.out_weight = self.decay_head = None
        self.r = 0

    def tensor_specs(self):
        t, Hd, Hv = self.spec.tensors, self.H * self.d, self.H * self.dv
        specs = [TensorSpec(t["q"], (Hd, self.hidden)), TensorSpec(t["k"], (Hd, self.hidden)),
                 TensorSpec(t["v"], (Hv, self.hidden)), TensorSpec(t["g"], (Hv, self.hidden)),
                 TensorSpec(t["o"], (self.hidden, Hv))]
        if self.norm_weight:
            specs.append(TensorSpec(t["norm"], (self.dv,), init="ones"))
        if self.decay is None:
            specs += [TensorSpec(t["a1"], (self.decay_rank, self.hidden), free=(0,)),
                      TensorSpec(t["a2"], (Hd, self.decay_rank), free=(1,)),
                      TensorSpec(t["a2_bias"], (Hd,), mean=3.0, std=1.0)]
        return specs

    def load(self, source):
        t = self.spec.tensors
        ws = [source.get(t[n]) for n in ("q", "k", "v", "g")]
        if self.decay is None:
            a1 = source.get(t["a1"])
            self.w_a2 = source.get(t["a2"])
            self.r = a1.shape[0]
            if self.w_a2.shape[1] != self.r:
                raise ValueError(f"linear attention: {t['a1']} has {self.r} rows but {t['a2']} {self.w_a2.shape[1]} columns")
            ws.append(a1)
            self.a2_bias = source.get(t["a2_bias"]).float().contiguous()
        else:
            self.decay_head = torch.tensor(self.decay, dtype=torch.float32, device=self.env.device)
        dt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_in = torch.cat([w.to(dt) for w in ws], dim=0).contiguous()
        self.w_o = source.get(t["o"])
        if self.norm_weight:
            self.out_weight = source.get(t["norm"]).float().contiguous()

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o, self.w_a2) if w is not None)

    def flops(self, tokens, keys=0.0):
        proj = 2.0 * tokens * self.hidden * (self.w_in.shape[0] + self.H * self.dv) + 2.0 * tokens * self.r * self.H * self.d
        return proj + 4.0 * tokens * self.H * self.d * self.dv

    def state_request(self):
        return StateRequest((self.H, self.d, self.dv), torch.float32)

    def forward(self, h, ctx, cache, add_to=None):
        Hd, Hv = self.H * self.d, self.H * self.dv
        proj = ops.linear(h, self.w_in, torch.float32, ctx.err)
        q, k = proj[:, :Hd], proj[:, Hd:2 * Hd]
        v, g = proj[:, 2 * Hd:2 * Hd + Hv], proj[:, 2 * Hd + Hv:2 * Hd + 2 * Hv]
        decay_tok = None
        if self.decay is None:
            T = h.shape[0]
            z = torch.empty((T, Hd), dtype=torch.float32, device=h.device)
            ops.gemm_f32_ex(proj[:, 2 * Hd + 2 * Hv:], self.w_a2, z, T, Hd, self.r, proj.stride(0), Hd)
            decay_tok = ops.gated_decay(z, self.a2_bias, self.tau)
        o = ops.linear_recurrence(q, k, v, decay_tok, self.decay_head, self.q_scale, self.k_scale, cache.state, ctx,
                                  self.H, self.d, self.dv)
        y = ops.head_norm_gate(o, g, self.out_weight, self.eps, self.env.dtype)
        if add_to is not None and ops.linear_add(add_to, y, self.w_o):
            return None
        return ops.linear_parts(y, self.w_o, ctx.err)


class ForgetGateLinearAttention(Mixer):
    """Linear attention without keys, in which the forget gate also decides what is written (HGRN2):

        q = silu(W_q h),  v = W_v h,  f = l + (1 - l) sigmoid(W_f h + b_f)          (l: a lower bound per channel)
        S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T,    o_t = S_t^T q_t                (S: [key_dim, value_dim], float32)

    Each head's output is divided by its root mean square over value_dim, times a weight shared by the heads, and
    projected by W_o.  The gate, its complement and the query's activation are made in float32 from the projection's
    float32 output inside the recurrence kernel, as the tokens' rows are staged.

    params: hidden_size, num_heads, key_dim, value_dim, eps.  tensors: q, f [H d, hidden], f_bias, lower [H d],
    v [H dv, hidden], norm [dv], o [hidden, H dv]."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.H = int(p["hidden_size"]), int(p["num_heads"])
        self.d, self.dv, self.eps = int(p["key_dim"]), int(p["value_dim"]), float(p["eps"])
        self.w_in = self.w_o = self.f_bias = self.lower = self.out_weight = None

    def tensor_specs(self):
        t, Hd, Hv = self.spec.tensors, self.H * self.d, self.H * self.dv
        return [TensorSpec(t["q"], (Hd, self.hidden)), TensorSpec(t["f"], (Hd, self.hidden)),
                TensorSpec(t["f_bias"], (Hd,), mean=1.0, std=1.0), TensorSpec(t["lower"], (Hd,), mean=0.3, std=0.1),
                TensorSpec(t["v"], (Hv, self.hidden)), TensorSpec(t["norm"], (self.dv,), init="ones"),
                TensorSpec(t["o"], (self.hidden, Hv))]

    def load(self, source):
        t = self.spec.tensors
        ws = [source.get(t[n]) for n in ("q", "f", "v")]
        dt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_in = torch.cat([w.to(dt) for w in ws], dim=0).contiguous()          # [q | f | v]
        self.f_bias = source.get(t["f_bias"]).float().contiguous()
        self.lower = source.get(t["lower"]).float().contiguous()
        self.out_weight = source.get(t["norm"]).float().contiguous()
        self.w_o = source.get(t["o"])

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o))

    def flops(self, tokens, keys=0.0):
        return 2.0 * tokens * self.hidden * (self.w_in.shape[0] + self.H * self.dv) + 4.0 * tokens * self.H * self.d * self.dv

    def state_request(self):
        return StateRequest((self.H, self.d, self.dv), torch.float32)

    def forward(self, h, ctx, cache, add_to=None):
        Hd = self.H * self.d
        proj = ops.linear(h, self.w_in, torch.float32, ctx.err)
        q, z, v = proj[:, :Hd], proj[:, Hd:2 * Hd], proj[:, 2 * Hd:]
        o = ops.linear_recurrence(q, None, v, z, None, 1.0, 1.0, cache.state, ctx, self.H, self.d, self.dv,
                                  forget_lower=self.lower, forget_bias=self.f_bias)
        y = ops.head_norm_gate(o, None, self.out_weight, self.eps, self.env.dtype)
        return ops.linear_parts(y, self.w_o, ctx.err)
