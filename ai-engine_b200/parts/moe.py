"""Mixtures of small gated feed-forwards.  `TableMoE`: the experts are chosen by a table, not by a router;
`RoutedMoE` (below): by a softmax router with a correction for the choice, groups of experts, and experts that
hand their input on unchanged.

TableMoE: row `id` of the
table [vocab, top] names the experts of a token with that id, each weighing 1 / top.  An expert is

    g = min(W_gate h, limit),  u = clamp(W_up h, -limit, limit),  y = g * sigmoid(alpha g) * (u + shift),  W_down y

without biases.  An optional shared expert of the same form (its own width and limit) runs for every token and
is added, multiplied by sigmoid(w_sg . h), one number per token.

A step's (token, choice) pairs are grouped by expert on the device (tiles of 64 rows, each expert's rows padded
to whole tiles), the two products run once per tile with the tile's expert's weights, and a last kernel sums
each token's rows in the order of its choices: no row's result depends on which other tokens are in the step.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import FeedForward


class TableMoE(FeedForward):
    """params: hidden_size, vocab_size, num_experts, top, intermediate_size, limit, alpha (default 1.702), shift
    (default 1), shared_intermediate_size (0: none), shared_limit.  tensors: table; gate, up, down as patterns with
    `{e}` for the expert's index; shared_gate, shared_up, shared_down, shared_sg [1, hidden]."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.vocab = int(p["hidden_size"]), int(p["vocab_size"])
        self.E, self.top, self.F = int(p["num_experts"]), int(p["top"]), int(p["intermediate_size"])
        self.limit, self.alpha, self.shift = float(p["limit"]), float(p.get("alpha", 1.702)), float(p.get("shift", 1.0))
        self.Fs, self.shared_limit = int(p.get("shared_intermediate_size") or 0), float(p.get("shared_limit") or 0.0)
        self.table = self.w_gu = self.w_down = self.w_shared_in = self.w_shared_down = None

    def tensor_specs(self):
        t, D = self.spec.tensors, self.hidden
        specs = [TensorSpec(t["table"], (self.vocab, self.top), init="distinct", high=self.E)]
        for e in range(self.E):
            specs += [TensorSpec(t["gate"].format(e=e), (self.F, D)), TensorSpec(t["up"].format(e=e), (self.F, D)),
                      TensorSpec(t["down"].format(e=e), (D, self.F))]
        if self.Fs:
            specs += [TensorSpec(t["shared_gate"], (self.Fs, D)), TensorSpec(t["shared_up"], (self.Fs, D)),
                      TensorSpec(t["shared_down"], (D, self.Fs)), TensorSpec(t["shared_sg"], (1, D))]
        return specs

    def load(self, source):
        t = self.spec.tensors
        self.table = source.get(t["table"]).to(torch.int32).contiguous()
        gu, down = [], []
        for e in range(self.E):
            gu += [source.get(t["gate"].format(e=e)), source.get(t["up"].format(e=e))]
            down.append(source.get(t["down"].format(e=e)))
        dt = torch.float32 if any(w.dtype == torch.float32 for w in gu + down) else gu[0].dtype
        self.w_gu = torch.stack([w.to(dt) for w in gu]).view(self.E, 2 * self.F, self.hidden).contiguous()
        self.w_down = torch.stack([w.to(dt) for w in down]).contiguous()                  # [E, hidden, F]
        if self.Fs:
            ws = [source.get(t[n]) for n in ("shared_gate", "shared_up", "shared_sg")]
            sdt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
            # [2 Fs + 1, hidden], with zero rows up to a multiple of 8: an odd row count would leave the rows of
            # the product's output unaligned, which the library's fast kernels do not take
            pad = (-(2 * self.Fs + 1)) % 8
            ws.append(torch.zeros((pad, self.hidden), dtype=sdt, device=ws[0].device))
            self.w_shared_in = torch.cat([w.to(sdt) for w in ws], dim=0).contiguous()
            self.w_shared_down = source.get(t["shared_down"])

    def weight_bytes(self):
        """What a step of many tokens reads: every expert once."""
        return sum(w.numel() * w.element_size() for w in (self.w_gu, self.w_down, self.w_shared_in, self.w_shared_down)
                   if w is not None)

    def flops(self, tokens, keys=0.0):
        return 2.0 * tokens * 3 * self.hidden * (self.top * self.F + self.Fs)

    def forward(self, h, ctx):
        T, D, F = h.shape[0], self.hidden, self.F
        row_token, pair_row, tile_expert = ops.expert_plan(ctx.token_ids, self.table, self.E, ctx.err)
        gu = ops.grouped_linear(h, self.w_gu, tile_expert, torch.float32, ctx.err, row_src=row_token)
        act = ops.clamped_glu(gu, F, self.limit, self.alpha, self.shift, self.env.dtype)
        y = ops.grouped_linear(act, self.w_down, tile_expert, torch.float32, ctx.err)
        shared = gate = None
        if self.Fs:
            sp = ops.linear(h, self.w_shared_in, torch.float32, ctx.err)
            sa = ops.clamped_glu(sp, self.Fs, self.shared_limit, self.alpha, self.shift, self.env.dtype)
            shared = ops.linear(sa, self.w_shared_down, torch.float32, ctx.err)
            gate = sp[:, 2 * self.Fs]
        return ops.expert_combine(y, pair_row, self.top, 1.0 / self.top, shared, gate, T)


class RoutedMoE(FeedForward):
    """A mixture of gated feed-forwards W_down (act(W_gate h) * (W_up h)) chosen by a router, per token:

        s = softmax(W_router h)                     over all router outputs, float32
        choice = s + correction                     only the choice uses the correction
        the outputs form `groups` equal groups of neighbours; a group counts as its best choice value, and only
        members of the `keep` best groups can be chosen; the `top` largest choice values among them are taken
        out = sum over the chosen e of s_e * expert_e(h)            (the weights are not renormalised)

    The router's last `identity` outputs have no tensors: such an expert's output is h itself.

    Variants, each a parameter: `score` "sigmoid": s_e = sigmoid(z_e), every output on its own; `group_top` n: a group
    counts as the sum of its n largest choice values; `normalise`: the chosen weights are divided by their sum
    (+ 1e-20); `route_scale` multiplies them; no tensor `correction`: the choice is made on s itself; a shared
    expert of the same form (`shared_intermediate_size`) runs for every token and is added.

    params: hidden_size, num_experts (with tensors), identity (default 0), top, intermediate_size, groups
    (default 1), keep (default 1), activation (default "silu"), score (default "softmax"), group_top (default 1),
    normalise (default False), route_scale (default 1), shared_intermediate_size (default 0).  tensors: router
    [num_experts + identity, hidden], correction [num_experts + identity] (optional); gate, up, down as patterns with
    `{e}` for the expert's index; shared_gate, shared_up, shared_down."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.E, self.ident = int(p["hidden_size"]), int(p["num_experts"]), int(p.get("identity") or 0)
        self.top, self.F = int(p["top"]), int(p["intermediate_size"])
        self.groups, self.keep = int(p.get("groups") or 1), int(p.get("keep") or 1)
        self.activation = p.get("activation") or "silu"
        total = self.E + self.ident
        if self.activation != "silu":
            raise ValueError("routed experts: the experts' activation is silu")
        if total % self.groups or not 1 <= self.keep <= self.groups or not 1 <= self.top <= total // self.groups * self.keep:
            raise ValueError(f"routed experts: {total} router outputs do not divide into {self.groups} groups of which "
                             f"{self.keep} are kept for {self.top} choices")
        self.score = p.get("score") or "softmax"
        if self.score not in ("softmax", "sigmoid"):
            raise ValueError(f"routed experts: score `{self.score}` is not known (softmax, sigmoid)")
        self.group_top, self.normalise = int(p.get("group_top") or 1), bool(p.get("normalise"))
        self.route_scale = float(p.get("route_scale") if p.get("route_scale") is not None else 1.0)
        self.has_correction = "correction" in spec.tensors
        self.Fs = int(p.get("shared_intermediate_size") or 0)
        self.shared = None
        if self.Fs:
            from .registry import lookup
            from .spec import PartSpec
            t = spec.tensors
            self.shared = lookup("feed_forward", "swiglu")(PartSpec("swiglu", dict(
                hidden_size=self.hidden, intermediate_size=self.Fs, activation=self.activation),
                dict(gate=t["shared_gate"], up=t["shared_up"], down=t["shared_down"])), env)
        self.w_router = self.correction = self.w_gu = self.w_down = None

    def sub_parts(self):
        return {"shared": self.shared} if self.shared is not None else {}

    def tensor_specs(self):
        t, D, total = self.spec.tensors, self.hidden, self.E + self.ident
        specs = [TensorSpec(t["router"], (total, D), std=0.3)]
        if self.has_correction:
            specs.append(TensorSpec(t["correction"], (total,), std=0.05))
        for e in range(self.E):
            specs += [TensorSpec(t["gate"].format(e=e), (self.F, D)), TensorSpec(t["up"].format(e=e), (self.F, D)),
                      TensorSpec(t["down"].format(e=e), (D, self.F))]
        return specs + (self.shared.tensor_specs() if self.shared is not None else [])

    def load(self, source):
        t = self.spec.tensors
        self.w_router = source.get(t["router"])
        if self.w_router.dtype == torch.bfloat16 and self.w_router.shape[0] % 8:
            # zero rows up to a multiple of 8: the tensor-core products want rows of the output 16 bytes apart
            pad = torch.zeros(((-self.w_router.shape[0]) % 8, self.hidden), dtype=torch.bfloat16, device=self.w_router.device)
            self.w_router = torch.cat([self.w_router, pad], dim=0).contiguous()
        if self.has_correction:
            self.correction = source.get(t["correction"]).float().contiguous()
        if self.shared is not None:
            self.shared.load(source)
        gu, down = [], []
        for e in range(self.E):
            gu += [source.get(t["gate"].format(e=e)), source.get(t["up"].format(e=e))]
            down.append(source.get(t["down"].format(e=e)))
        if self.E:
            dt = torch.float32 if any(w.dtype == torch.float32 for w in gu + down) else gu[0].dtype
            self.w_gu = torch.stack([w.to(dt) for w in gu]).view(self.E, 2 * self.F, self.hidden).contiguous()
            self.w_down = torch.stack([w.to(dt) for w in down]).contiguous()              # [E, hidden, F]

    def weight_bytes(self):
        """What a step of many tokens reads: every expert once."""
        return sum(w.numel() * w.element_size() for w in (self.w_router, self.w_gu, self.w_down) if w is not None) \
            + (self.shared.weight_bytes() if self.shared is not None else 0)

    def flops(self, tokens, keys=0.0):
        return 2.0 * tokens * self.hidden * (3 * self.top * self.F + self.E + self.ident) \
            + (self.shared.flops(tokens, keys) if self.shared is not None else 0.0)

    def forward(self, h, ctx):
        # the router in float32 on the sublayer's input as the experts see it: products of bfloat16 values are exact
        # in float32, so the tensor-core product with float32 sums is a float32 product of those inputs
        if h.dtype == torch.bfloat16 and self.w_router.dtype == torch.bfloat16:
            logits = ops.linear(h, self.w_router, torch.float32, ctx.err)[:, :self.E + self.ident]
        else:
            logits = ops.gemm_f32(ops.cast(h, torch.float32), self.w_router)
        ids, weights = ops.route_topk(logits, self.correction, self.groups, self.keep, self.top, score=self.score,
                                      group_top=self.group_top, normalise=self.normalise, weight_scale=self.route_scale)
        shared = self.shared.forward(h, ctx) if self.shared is not None else None
        if not self.E:
            y = torch.zeros((1, self.hidden), dtype=torch.float32, device=h.device)
            pair_row = torch.full((ids.numel(),), -2, dtype=torch.int32, device=h.device)
            return ops.expert_combine_weighted(y, pair_row, weights, h, shared)
        row_token, pair_row, tile_expert = ops.expert_plan(None, ids, self.E, ctx.err, identity=self.ident)
        gu = ops.grouped_linear(h, self.w_gu, tile_expert, torch.float32, ctx.err, row_src=row_token)
        act = ops.clamped_glu(gu, self.F, float("inf"), 1.0, 0.0, self.env.dtype)       # silu(gate) * up
        y = ops.grouped_linear(act, self.w_down, tile_expert, torch.float32, ctx.err)
        return ops.expert_combine_weighted(y, pair_row, weights, h, shared)
