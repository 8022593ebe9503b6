"""Attention whose cache holds one compressed vector per token.

Per token the layer projects a latent c [kv_rank] (RMS-normalised with a weight) and one rotated key part
kr [rot_dim] that all heads share; only [c | kr] is cached.  Head h has the key [W_uk,h c | kr] and the
value W_uv,h c, and a query [q_plain,h | q_rot,h]; score = (q_plain . W_uk c + q_rot . kr) * scale, softmax
over the keys the mask shows (all earlier ones, or the last `window`), output W_o on the concatenated heads.

The up-projections never touch the cache: W_uk is folded into the query (qa_h = W_uk,h^T q_plain,h, so
qa_h . c = q_plain,h . W_uk,h c) and W_uv is applied to the attention-weighted sum of latents
(sum_j p_j W_uv c_j = W_uv sum_j p_j c_j).  The attention kernel then reads the cache rows as they are, as
one key/value head for all query heads, for prompts and decoded tokens alike.

The queries may go through a latent of their own (`q_rank`): c_q = RMSnorm(W_dq h) with a weight, q = W_uq c_q.  A
gate per head (`head_gate`) multiplies head h's output by sigmoid(W_g h)_h; it is applied to the head's values before
the output projection.  The rotation pairs neighbours or halves, as its encoding says.

A layer may read another layer's cache (`shares_cache`): it has no latent projection of its own and writes
nothing; the run order names the layer whose rows it reads.
"""
from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import KVRequest, Mixer, StepPlanner


class LatentWork(StepPlanner):
    """The work list of the tensor-core kernel: `tiles` [n, 2] = (request row, offset among the tokens it brings)
    of units of `tq` consecutive tokens of one request, which share the cache rows they gather.  A step in which
    every request brings one token has units of one token, all others units of four."""

    key = "latent"

    def plan(self, ctx):
        tq = 1 if ctx.max_q_len <= 1 else 4
        tiles = [(r, off) for r, n in enumerate(ctx.h_q_len.tolist()) for off in range(0, n, tq)]
        return dict(tiles=np.asarray(tiles, dtype=np.int32).reshape(-1, 2)), dict(tq=tq)


LATENT_WORK = LatentWork()


class LatentAttention(Mixer):
    """params: hidden_size, num_heads, head_dim (unrotated part), rot_dim, value_dim, kv_rank, scale, window
    (0 = all keys), cache_window (the window the cached rows must outlive: the widest of all layers that read
    them; default = window), eps (of the latents' norms), position_encoding (name of a rotary encoding over rot_dim
    or fewer elements, either layout), shares_cache, q_rank (0: the queries are projected directly), head_gate.
    tensors: q [H (d + rot), hidden] (or, with q_rank: dq [q_rank, hidden], dq_norm [q_rank], uq [H (d + rot),
    q_rank]), dkv [kv_rank + rot, hidden], dkv_norm [kv_rank], uk [H d, kv_rank], uv [H dv, kv_rank], o [hidden,
    H dv], g [H, hidden]."""

    adds_in_place = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.H = int(p["hidden_size"]), int(p["num_heads"])
        self.d, self.rot, self.dv, self.rank = int(p["head_dim"]), int(p["rot_dim"]), int(p["value_dim"]), int(p["kv_rank"])
        self.scale = float(p["scale"])
        self.window = int(p.get("window") or 0)
        self.cache_window = int(p["cache_window"]) if p.get("cache_window") is not None else self.window
        self.eps = float(p["eps"])
        self.shares_cache = bool(p.get("shares_cache"))
        pe = p.get("position_encoding")
        self.rope = env.position_encodings[pe] if pe else None
        if self.rope is not None and self.rope.rot_dim > self.rot:
            raise ValueError("latent attention: the rotation is wider than rot_dim")
        self.halves = self.rope is not None and not getattr(self.rope, "interleaved", False)
        self.q_rank, self.head_gate = int(p.get("q_rank") or 0), bool(p.get("head_gate"))
        if (self.q_rank or self.head_gate) and self.shares_cache:
            raise ValueError("latent attention: a layer that reads another's cache has neither a query latent nor a gate")
        self.w_uq = self.cq_weight = None
        self.w_in = self.w_ukT = self.w_uv = self.w_o = self.c_weight = self._no_rope = None

    def tensor_specs(self):
        t, dq = self.spec.tensors, self.d + self.rot
        if self.q_rank:
            specs = [TensorSpec(t["dq"], (self.q_rank, self.hidden)), TensorSpec(t["dq_norm"], (self.q_rank,), init="ones"),
                     TensorSpec(t["uq"], (self.H * dq, self.q_rank))]
        else:
            specs = [TensorSpec(t["q"], (self.H * dq, self.hidden))]
        if self.head_gate:
            specs.append(TensorSpec(t["g"], (self.H, self.hidden)))
        if not self.shares_cache:
            specs += [TensorSpec(t["dkv"], (self.rank + self.rot, self.hidden)),
                      TensorSpec(t["dkv_norm"], (self.rank,), init="ones")]
        return specs + [TensorSpec(t["uk"], (self.H * self.d, self.rank)),
                        TensorSpec(t["uv"], (self.H * self.dv, self.rank)),
                        TensorSpec(t["o"], (self.hidden, self.H * self.dv))]

    def load(self, source):
        t = self.spec.tensors
        q = source.get(t["dq"] if self.q_rank else t["q"])
        if self.q_rank:
            self.w_uq = source.get(t["uq"])
            self.cq_weight = source.get(t["dq_norm"]).float().contiguous()
        if self.shares_cache:
            self.w_in = q
        else:
            # one product for everything that reads h: [q or its latent | latent | key part | gate logits]
            ws = [q, source.get(t["dkv"])] + ([source.get(t["g"])] if self.head_gate else [])
            dt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else q.dtype
            pad = (-sum(w.shape[0] for w in ws)) % 8     # rows of the product's output stay 16 bytes apart
            if pad:
                ws.append(torch.zeros((pad, self.hidden), dtype=dt, device=q.device))
            self.w_in = torch.cat([w.to(dt) for w in ws], dim=0).contiguous()
            self.c_weight = source.get(t["dkv_norm"]).float().contiguous()
        # [H, kv_rank, d]: the folding product reads W_uk,h transposed
        self.w_ukT = source.get(t["uk"]).view(self.H, self.d, self.rank).transpose(1, 2).contiguous()
        self.w_uv = source.get(t["uv"]).view(self.H, self.dv, self.rank).contiguous()
        self.w_o = source.get(t["o"])
        self._no_rope = torch.zeros(0, dtype=torch.float32, device=self.env.device)

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_uq, self.w_ukT, self.w_uv, self.w_o)
                   if w is not None)

    def flops(self, tokens, keys=0.0):
        if self.window:
            keys = min(keys, float(self.window))
        proj = 2.0 * tokens * (self.w_in.shape[0] * self.hidden + self.H * self.dv * self.hidden
                               + self.H * self.rank * (self.d + self.dv) + self.q_rank * self.H * (self.d + self.rot))
        return proj + 2.0 * tokens * keys * self.H * (2 * self.rank + self.rot)

    def cache_request(self):
        return KVRequest(1, self.rank + self.rot, self.cache_window, planes=1)

    def step_planner(self):
        return LATENT_WORK

    def forward(self, h, ctx, cache, add_to=None):
        T = h.shape[0]
        rot = self.rope.rotation() if self.rope is not None else None
        inv_freq = rot[0] if rot is not None else self._no_rope
        proj = ops.linear(h, self.w_in, torch.float32, ctx.err)
        kv, first = None, self.H * (self.d + self.rot)
        if self.q_rank:
            # the queries' latent, normed in float32, then the queries: a second product, its output is what the
            # prepare kernel reads the queries from; the latent and the key part stay in the first product's
            cq = ops.slice_rmsnorm(proj[:, :self.q_rank], self.cq_weight, self.eps, self.env.dtype)
            kv, first = proj[:, self.q_rank:], self.q_rank
            q_src = ops.linear(cq, self.w_uq, torch.float32, ctx.err)
        else:
            q_src = proj
        q_plain, q_full = ops.latent_prepare(q_src, self.H, self.d, self.rot, self.rank, self.c_weight, self.eps,
                                             inv_freq, cache.k_pages, ctx, cache.block_table, self.env.dtype,
                                             write=cache.writes and not self.shares_cache, kv=kv, halves=self.halves)
        ops.head_linear(q_plain, self.w_ukT, q_full)
        mixed = ops.latent_attention(q_full, cache.k_pages, ctx, cache.block_table, self.rank, self.scale,
                                     self.window, self.env.dtype, ctx.plan(LATENT_WORK))
        a = torch.empty((T, self.H, self.dv), dtype=self.env.dtype, device=h.device)
        ops.head_linear(mixed, self.w_uv, a)
        a = a.view(T, self.H * self.dv)
        if self.head_gate:
            g0 = first + self.rank + self.rot
            ops.sigmoid_gate_mul_(a, proj[:, g0:g0 + self.H], self.dv)
        if add_to is not None and ops.linear_add(add_to, a, self.w_o):
            return None
        return ops.linear_parts(a, self.w_o, ctx.err)
