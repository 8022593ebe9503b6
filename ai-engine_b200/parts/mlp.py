"""SwiGLU feed-forward (crates/ai-engine-runtime/src/arch/ffn.rs:50-54):
down(silu(gate(x)) * up(x)), no bias, silu(z) = z * sigmoid(z) in float32."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import FeedForward


class SwiGLU(FeedForward):
    """params: hidden_size, intermediate_size, activation (default "silu"; "relu" and "gelu_tanh" give
    down(act(gate(x)) * up(x)) with that act).  tensors: gate, up [F, hidden], down [hidden, F].  gate and up
    are fused into one [2F, hidden] weight at load."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.activation = spec.params.get("activation") or "silu"
        if self.activation not in ops.GLU_ACTIVATIONS:
            raise ValueError(f"gated feed-forward: activation `{self.activation}` is not known "
                             f"({', '.join(ops.GLU_ACTIVATIONS)})")
        self.w_gu = self.w_down = None
        self.block = 0

    def tensor_specs(self):
        t = self.spec.tensors
        return [TensorSpec(t["gate"], (self.inter, self.hidden)),
                TensorSpec(t["up"], (self.inter, self.hidden)),
                TensorSpec(t["down"], (self.hidden, self.inter))]

    def load(self, source):
        t = self.spec.tensors
        g, u = source.get(t["gate"]), source.get(t["up"])
        dt = torch.float32 if torch.float32 in (g.dtype, u.dtype) else g.dtype
        # bfloat16: 64 gate rows then their 64 up rows, tile by tile, so that a 128-row
        # weight tile of the tensor-core kernel holds both halves of 64 outputs
        self.block = ops.TC_SWIGLU_BLOCK if (dt == torch.bfloat16 and self.inter % ops.TC_SWIGLU_BLOCK == 0
                                             and self.activation == "silu") else 0
        if self.block:
            b = self.block
            self.w_gu = torch.stack([g.view(-1, b, self.hidden), u.view(-1, b, self.hidden)], dim=1) \
                .reshape(2 * self.inter, self.hidden).contiguous()
        else:
            self.w_gu = torch.cat([g.to(dt), u.to(dt)], dim=0).contiguous()
        self.w_down = source.get(t["down"])

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_gu, self.w_down))

    def flops(self, tokens, keys=0.0):
        return 2.0 * tokens * 3 * self.inter * self.hidden

    adds_in_place = True

    def forward(self, h, ctx, add_to=None):
        err = ctx.err if ctx is not None else None
        a = ops.linear_swiglu(h, self.w_gu, self.block, err, self.activation)
        if add_to is not None and ops.linear_add(add_to, a, self.w_down):
            return None
        return ops.linear_parts(a, self.w_down, err)   # joins the residual in float32, inside the next norm


class PolyNormFF(FeedForward):
    """down(act(up(x))) with act = a N(z) + b N(z^2) + c N(z^3) + e: powers element by element, N the division of
    a token's vector of intermediate values by its root mean square (float32).  params: hidden_size,
    intermediate_size, eps.  tensors: up [F, hidden], down [hidden, F], act [4] = (a, b, c, e)."""

    adds_in_place = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden, self.inter = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        self.eps = float(spec.params["eps"])
        self.w_up = self.w_down = self.coef = None

    def tensor_specs(self):
        t = self.spec.tensors
        return [TensorSpec(t["up"], (self.inter, self.hidden)), TensorSpec(t["down"], (self.hidden, self.inter)),
                TensorSpec(t["act"], (4,), mean=0.3, std=0.1)]

    def load(self, source):
        t = self.spec.tensors
        self.w_up, self.w_down = source.get(t["up"]), source.get(t["down"])
        self.coef = source.get(t["act"]).float().contiguous()

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_up, self.w_down))

    def flops(self, tokens, keys=0.0):
        return 2.0 * tokens * 2 * self.inter * self.hidden

    def forward(self, h, ctx, add_to=None):
        z = ops.linear(h, self.w_up, torch.float32, ctx.err)
        a = ops.polynorm(z, self.coef, self.eps, self.env.dtype)
        if add_to is not None and ops.linear_add(add_to, a, self.w_down):
            return None
        return ops.linear_parts(a, self.w_down, ctx.err)


class DenseFF(FeedForward):
    """down(act(up(x))) without a gate.  params: hidden_size, intermediate_size, activation (relu_squared, the
    default; relu, silu, gelu_tanh).  tensors: up [F, hidden], down [hidden, F].  The activation is worked out in
    float32 from the product's output."""

    adds_in_place = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden, self.inter = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        self.activation = spec.params.get("activation") or "relu_squared"
        if self.activation not in ops.PLAIN_ACTIVATIONS:
            raise ValueError(f"feed-forward: activation `{self.activation}` is not known "
                             f"({', '.join(ops.PLAIN_ACTIVATIONS)})")
        self.w_up = self.w_down = None

    def tensor_specs(self):
        t = self.spec.tensors
        return [TensorSpec(t["up"], (self.inter, self.hidden)), TensorSpec(t["down"], (self.hidden, self.inter))]

    def load(self, source):
        t = self.spec.tensors
        self.w_up, self.w_down = source.get(t["up"]), source.get(t["down"])

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_up, self.w_down))

    def flops(self, tokens, keys=0.0):
        return 2.0 * tokens * 2 * self.inter * self.hidden

    def forward(self, h, ctx, add_to=None):
        err = ctx.err if ctx is not None else None
        a = ops.linear_activated(h, self.w_up, self.activation, err)
        if add_to is not None and ops.linear_add(add_to, a, self.w_down):
            return None
        return ops.linear_parts(a, self.w_down, err)
