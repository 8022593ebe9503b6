"""Fixed sinusoidal position vectors, added to the residual stream behind the embedding:

    column 2i of the vector for place p = sin(p * base^(-2i / size)),  column 2i + 1 = cos of the same angle.

Only the frequencies are kept; the kernel makes float(p) * f_i in float32 for the places of a step's tokens, so no
table bounds the context."""
from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from .base import PositionEncoding


def sinusoid_frequencies(size: int, base: float) -> np.ndarray:
    """base^(-2i / size) for i = 0 .. ceil(size / 2) - 1, worked out in double and rounded to float32."""
    i = np.arange((size + 1) // 2, dtype=np.float64)
    return np.power(float(base), -2.0 * i / float(size)).astype(np.float32)


class SinusoidalPositions(PositionEncoding):
    """params: size (the stream's width), base (default 10000)."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = int(spec.params["size"])
        self.base = float(spec.params.get("base") or 10000.0)
        self.freq_host = sinusoid_frequencies(self.size, self.base)
        self.freq = None

    def load(self, source):
        self.freq = torch.from_numpy(self.freq_host.copy()).to(self.env.device)

    def add_to(self, x, ctx) -> None:
        ops.add_sinusoid(x, ctx.positions, self.freq)
