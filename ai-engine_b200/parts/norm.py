"""RMSNorm (crates/ai-engine-runtime/src/arch/rmsnorm.rs:29-42)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Norm


class RMSNorm(Norm):
    """params: size, eps; offset (default 0): the stored weight is the scale's distance from `offset`, the
    row is scaled by offset + w (a weight stored around zero has offset 1); output (default "compute"):
    "float32" returns the normalised rows in float32 whatever the compute dtype (for a consumer that goes on
    in 32-bit).  tensors: weight [size].  y = (x / sqrt(mean(x^2) + eps)) * (offset + w), statistics in
    float32; the add of a pending branch is fused in."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.offset = float(spec.params.get("offset") or 0.0)
        self.out_dtype = torch.float32 if spec.params.get("output") == "float32" else env.dtype
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.spec.tensors["weight"], (self.size,), init="zeros" if self.offset else "ones")]

    def load(self, source):
        self.weight = source.get(self.spec.tensors["weight"])
        if self.offset:       # the sum in float32: 1 + w keeps every bit of a bfloat16 w near zero
            self.weight = (self.weight.float() + self.offset).contiguous()

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def forward(self, x, delta=None, rows=None, write_back=True):
        return ops.add_rmsnorm(x, delta, self.weight, self.eps, self.out_dtype, rows=rows,
                               write_back=write_back)


class DynamicTanh(Norm):
    """A norm that computes no mean and no variance: y = tanh(alpha x) * w + b, element by element in float32.
    params: size; output (default "compute", or "float32").  tensors: weight [size], bias [size], alpha (one number).
    The add of a pending branch is fused in.  `ahead()` hands (weight, bias, alpha) to a kernel that already holds
    the stream's new value and can make this norm's output on the way."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = int(spec.params["size"])
        self.out_dtype = torch.float32 if spec.params.get("output") == "float32" else env.dtype
        self.weight = self.bias = self.alpha = None

    def tensor_specs(self):
        t = self.spec.tensors
        return [TensorSpec(t["weight"], (self.size,), init="ones"), TensorSpec(t["bias"], (self.size,), init="zeros"),
                TensorSpec(t["alpha"], (), mean=0.5, std=0.05)]

    def load(self, source):
        t = self.spec.tensors
        self.weight = source.get(t["weight"]).float().contiguous()
        self.bias = source.get(t["bias"]).float().contiguous()
        self.alpha = source.get(t["alpha"]).float().reshape(1).contiguous()

    def weight_bytes(self):
        return 2 * self.size * 4

    def ahead(self):
        return self.weight, self.bias, self.alpha

    def forward(self, x, delta=None, rows=None, write_back=True):
        return ops.add_dyt(x, delta, self.weight, self.bias, self.alpha, self.out_dtype, rows=rows, write_back=write_back)
