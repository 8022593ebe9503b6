"""The pre-norm residual block (crates/ai-engine-runtime/src/arch/block.rs:13-27):
x = x + mixer(norm(x)); x = x + ffn(norm(x)).

The residual stream stays float32.  A branch's output is not added by a kernel
of its own: it travels as `pending` into the next norm, which adds it in
float32, stores the sum and normalises it in one pass over the row.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Block


class PreNormBlock(Block):
    """x = x + mixer(norm(x)); x = x + ffn(norm(x)).  The feed-forward with its norm is optional.

    With the tensor `input_mix` [hidden, 2 hidden], the block first replaces the stream by a projection of the
    stream and the embedding's output side by side, x <- W [x ; x0] (a layer that opens a pass over a group of
    layers which is run several times: every pass starts from the running stream and the embedding together).  The
    projection reads both in the compute dtype and writes the new float32 stream."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "ffn_norm": "norm", "ffn": "feed_forward"}
    optional_roles = ("ffn_norm", "ffn")

    def __init__(self, spec, env, parts):
        super().__init__(spec, env)
        self.mixer_norm, self.mixer = parts["mixer_norm"], parts["mixer"]
        self.ffn_norm, self.ffn = parts.get("ffn_norm"), parts.get("ffn")
        if (self.ffn is None) != (self.ffn_norm is None):
            raise ValueError("pre-norm block: a feed-forward comes with its norm")
        self.hidden = env.hidden_size
        self.w_mix = None
        self.needs_embedding_output = "input_mix" in spec.tensors

    def tensor_specs(self):
        name = self.spec.tensors.get("input_mix")
        return [TensorSpec(name, (self.hidden, 2 * self.hidden))] if name else []

    def load(self, source):
        name = self.spec.tensors.get("input_mix")
        if name:
            self.w_mix = source.get(name)

    def weight_bytes(self):
        return self.w_mix.numel() * self.w_mix.element_size() if self.w_mix is not None else 0

    def flops(self, tokens, keys=0.0):
        return 4.0 * tokens * self.hidden * self.hidden if self.w_mix is not None else 0.0

    def forward(self, x, pending, ctx, caches):
        if self.w_mix is not None:
            both = ops.join_streams(x, pending, ctx.embedding_output, self.env.dtype)
            x, pending = ops.linear(both, self.w_mix, torch.float32, ctx.err), None
        h = self.mixer_norm.forward(x, pending)
        if self.mixer.adds_in_place:      # a large step's output projection adds to the stream itself: a is None then
            a = self.mixer.forward(h, ctx, caches.get("mixer"), add_to=x)
        else:
            a = self.mixer.forward(h, ctx, caches.get("mixer"))
        if self.ffn is None:
            return x, a
        h = self.ffn_norm.forward(x, a)
        if self.ffn.adds_in_place:
            return x, self.ffn.forward(h, ctx, add_to=x)
        return x, self.ffn.forward(h, ctx)


class DepthAveragedBlock(Block):
    """A pre-norm block whose sublayers read their input through a filter over time, and whose result is
    averaged with the results of all earlier layers:

        h = filter(norm(x));  x = x + mixer(h);  h = filter(norm(x));  x = x + ffn(h)          -> X_(depth + 1)
        x = sum_{j = 0 .. depth + 1} coef[j] * X_j        (X_0: the stream the first layer received)

    The filters and the feed-forward (with its norm) are optional roles.  params: depth (number of layers
    before this one), levels (layers of the model + 1).  tensors: coef [depth + 2] (absent: no averaging).
    The streams X_j of a step live in one float32 buffer [levels, T, hidden] that the first layer makes
    and hangs on the step context; norms hand float32 rows to the filters."""

    roles = {"mixer_norm": "norm", "mixer_filter": "filter", "mixer": "mixer",
             "ffn_norm": "norm", "ffn_filter": "filter", "ffn": "feed_forward"}
    optional_roles = ("mixer_filter", "ffn_norm", "ffn_filter", "ffn")

    def __init__(self, spec, env, parts):
        super().__init__(spec, env)
        self.p = parts
        self.depth, self.levels = int(spec.params["depth"]), int(spec.params["levels"])
        if "ffn" in parts and "ffn_norm" not in parts:
            raise ValueError("depth-averaged block: a feed-forward needs its norm")
        self.coef = None

    def tensor_specs(self):
        name = self.spec.tensors.get("coef")
        n = self.depth + 2
        return [TensorSpec(name, (n,), mean=1.0 / n, std=0.1 / n)] if name else []

    def load(self, source):
        name = self.spec.tensors.get("coef")
        if name:
            self.coef = source.get(name).float().contiguous()

    def _filtered(self, role, h, ctx, caches):
        f = self.p.get(role)
        if f is None:
            return ops.cast(h, self.env.dtype)
        return f.forward(h, ctx, caches[role])

    def forward(self, x, pending, ctx, caches):
        h = self.p["mixer_norm"].forward(x, pending)
        if self.coef is not None:
            if self.depth == 0:
                ctx.depth_history = torch.empty((self.levels,) + tuple(x.shape), dtype=torch.float32, device=x.device)
                ctx.depth_history[0].copy_(x)
            history = ctx.depth_history
        h = self._filtered("mixer_filter", h, ctx, caches)
        mixer = self.p["mixer"]
        if mixer.adds_in_place:
            a = mixer.forward(h, ctx, caches.get("mixer"), add_to=x)
        else:
            a = mixer.forward(h, ctx, caches.get("mixer"))
        ffn = self.p.get("ffn")
        if ffn is not None:
            h = self.p["ffn_norm"].forward(x, a)
            h = self._filtered("ffn_filter", h, ctx, caches)
            a = ffn.forward(h, ctx, add_to=x) if ffn.adds_in_place else ffn.forward(h, ctx)
        if self.coef is None:
            return x, a
        ops.depth_average(x, a, history, self.coef, self.depth + 1)
        return x, None


class SandwichNormBlock(Block):
    """A block that normalises each sublayer's input and its output:

        x = x + post_norm(mixer(norm(x)));   x = x + ffn_post_norm(ffn(ffn_norm(x)))

    The feed-forward with its two norms is optional.  A post-norm reads the branch in float32 and hands its
    float32 result on as the pending branch, which the next norm adds to the stream."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "mixer_post_norm": "norm",
             "ffn_norm": "norm", "ffn": "feed_forward", "ffn_post_norm": "norm"}
    optional_roles = ("ffn_norm", "ffn", "ffn_post_norm")

    def __init__(self, spec, env, parts):
        super().__init__(spec, env)
        self.p = parts
        if ("ffn" in parts) != ("ffn_norm" in parts) or ("ffn" in parts) != ("ffn_post_norm" in parts):
            raise ValueError("sandwich block: a feed-forward comes with both of its norms")

    @staticmethod
    def _normed(norm, y):
        """norm(y) in float32 for a branch y [T, D] (any dtype) or float32 [parts, T, D] (summed first)."""
        if y.dim() == 3:
            return norm.forward(y[0], y[1:] if y.shape[0] > 1 else None, write_back=False)
        return norm.forward(ops.cast(y, torch.float32), None, write_back=False)

    def forward(self, x, pending, ctx, caches):
        h = self.p["mixer_norm"].forward(x, pending)
        pending = self._normed(self.p["mixer_post_norm"], self.p["mixer"].forward(h, ctx, caches.get("mixer")))
        ffn = self.p.get("ffn")
        if ffn is not None:
            h = self.p["ffn_norm"].forward(x, pending)
            pending = self._normed(self.p["ffn_post_norm"], ffn.forward(h, ctx))
        return x, pending


class ParallelBlock(Block):
    """A block whose mixer and feed-forward read the same normed input and are added together:

        h = norm(x);   X = x + mult * (mixer(h) + ffn(h))                                 -> X_(depth + 1)
        x = sum_{j = 0 .. depth + 1} coef[j] * X_j        (X_0: the stream the first layer received)

    The feed-forward is optional, and so is the averaging (no tensor `coef`: x = X).  params: mult (default 1),
    depth (number of layers before this one), levels (layers of the model + 1).  tensors: coef [depth + 2].
    The two branch outputs, the stream and the earlier streams meet in one kernel.  `norm_ahead` (set by the model
    builder's order of layers through `set_next_norm`): when the norm that reads the stream next is one without
    statistics, that kernel writes its output too and hangs it on the step for the next block to pick up."""

    roles = {"norm": "norm", "mixer": "mixer", "ffn": "feed_forward"}
    optional_roles = ("ffn",)

    def __init__(self, spec, env, parts):
        super().__init__(spec, env)
        self.norm, self.mixer, self.ffn = parts["norm"], parts["mixer"], parts.get("ffn")
        self.mult = float(spec.params.get("mult", 1.0))
        self.depth, self.levels = int(spec.params.get("depth") or 0), int(spec.params.get("levels") or 0)
        self.coef = None
        self.next_norm = None

    def tensor_specs(self):
        name = self.spec.tensors.get("coef")
        n = self.depth + 2
        return [TensorSpec(name, (n,), mean=1.0 / n, std=0.1 / n)] if name else []

    def load(self, source):
        name = self.spec.tensors.get("coef")
        if name:
            self.coef = source.get(name).float().contiguous()

    def first_norm(self):
        return self.norm

    def set_next_norm(self, norm) -> None:
        """The norm that reads the stream after this block (the next block's, or the model's last); used only if it
        can be made ahead (`ahead()`) and hands on the compute dtype."""
        self.next_norm = norm if hasattr(norm, "ahead") else None

    def forward(self, x, pending, ctx, caches):
        ahead = getattr(ctx, "normed_ahead", None)
        if pending is None and ahead is not None and ahead[0] is self.norm:
            h = ahead[1]
        else:
            h = self.norm.forward(x, pending)
        ctx.normed_ahead = None
        history = None
        if self.coef is not None:
            if self.depth == 0:
                ctx.depth_history = torch.empty((self.levels,) + tuple(x.shape), dtype=torch.float32, device=x.device)
                ctx.depth_history[0].copy_(x)
            history = ctx.depth_history
        a = self.mixer.forward(h, ctx, caches.get("mixer"))
        b = self.ffn.forward(h, ctx) if self.ffn is not None else None
        a, b = ops.cast(a, torch.float32), (ops.cast(b, torch.float32) if b is not None else None)
        nxt = self.next_norm
        made = ops.parallel_residual(x, a, b, self.mult, history, self.coef, self.depth + 1,
                                     norm_ahead=nxt.ahead() if nxt is not None else None,
                                     out_dtype=nxt.out_dtype if nxt is not None else None)
        if made is not None:
            ctx.normed_ahead = (nxt, made)
        return x, None
