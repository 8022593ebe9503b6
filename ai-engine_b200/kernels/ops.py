"""Python faces of the CUDA kernels: each takes torch tensors on the device,
checks what the kernel cannot check itself, and launches on torch's current
stream.  Shapes and dtypes a kernel does not take are refused with an error.
"""
from __future__ import annotations

import math
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from .loader import KernelError, check, library, require_cuda
from .profile import enabled as _profiling, region

F32, BF16 = 0, 1


def dtype_code(t) -> int:
    dt = t if isinstance(t, torch.dtype) else t.dtype
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {dt} is not taken by the kernels (float32, bfloat16)")


def _p(t: Optional[torch.Tensor]):
    return c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current stream of device 0 as a handle for the launchers (the raw query costs a fraction
    of a microsecond; `torch.cuda.current_stream()` several, once per kernel launch)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(0))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _nb(*ts) -> int:
    """Bytes of the given tensors (what a kernel that touches each once has to move)."""
    return sum(t.numel() * t.element_size() for t in ts if t is not None)


def _dev(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            require_cuda()
            raise KernelError("kernel operands must live on the CUDA device")
        if t is not None and not t.is_contiguous():
            raise KernelError("kernel operands must be contiguous")


_SMS = [0]


def sm_count() -> int:
    """SMs of the device (148 on a B200), asked once: grids and split counts are sized by it."""
    if not _SMS[0]:
        _SMS[0] = int(torch.cuda.get_device_properties(0).multi_processor_count)
    return _SMS[0]


# ---------------------------------------------------------------------------
def embed_gather(ids: torch.Tensor, table: torch.Tensor, err: torch.Tensor,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x[t] = float32(table[ids[t]]); an id outside the table sets the error word."""
    _dev(ids, table, err)
    T, (V, D) = ids.shape[0], table.shape
    if out is None:
        out = torch.empty((T, D), dtype=torch.float32, device=table.device)
    lib = library("elementwise.cu")
    with region("embed_gather", T * D * table.element_size() + _nb(out)):
        check(lib.aie_embed_gather(_p(ids), _p(table), c_int(dtype_code(table)), _p(out), c_int(T),
                                   c_int(D), c_int(V), _p(err), _stream()), "embed_gather")
    return out


def take_sampled_ids(ids: torch.Tensor, src: torch.Tensor, last: torch.Tensor, err: torch.Tensor) -> None:
    """ids[t] = last[src[t]] where src[t] >= 0 (int32, in place): tokens that the previous step
    sampled and the host has not read yet."""
    _dev(ids, src, last, err)
    lib = library("elementwise.cu")
    check(lib.aie_take_sampled_ids(_p(ids), _p(src), _p(last), c_int(ids.shape[0]), c_int(last.shape[0]),
                                   _p(err), _stream()), "take_sampled_ids")


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
                write_back: bool = True, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """s = x (+ delta); out = (s / sqrt(mean(s^2) + eps)) * weight.  `x` is the
    float32 residual stream and receives s when `write_back`; `rows` picks rows.
    `delta` may be [parts, T, D]: the parts of a split product, added here in order."""
    _dev(x, delta, weight, rows)
    if x.dtype != torch.float32:
        raise KernelError("add_rmsnorm: the residual stream must be float32")
    D = x.shape[-1]
    if weight.shape != (D,):
        raise KernelError(f"add_rmsnorm: weight shape {tuple(weight.shape)} != ({D},)")
    parts, part_stride = 1, 0
    if delta is not None and delta.dim() == 3:        # [parts, T, D]: parts of a split product
        parts, part_stride = delta.shape[0], delta.stride(0)
        if delta.shape[1:] != x.shape:
            raise KernelError("add_rmsnorm: delta parts differ in shape from x")
    elif delta is not None and delta.shape != x.shape:
        raise KernelError("add_rmsnorm: delta shape differs from x")
    n = x.shape[0] if rows is None else rows.shape[0]
    if out is None:
        out = torch.empty((n, D), dtype=out_dtype, device=x.device)
    lib = library("elementwise.cu")
    stored = write_back and rows is None and delta is not None      # without a branch to add, the stream is as it was
    with region("add_rmsnorm", n * D * 4 * (2 if stored else 1) + (_nb(delta) if rows is None else 0) + _nb(out)):
        check(lib.aie_add_rmsnorm(_p(x), _p(delta), c_int(dtype_code(delta) if delta is not None else 0),
                                  _p(weight), c_int(dtype_code(weight)), _p(out),
                                  c_int(dtype_code(out)), _p(rows), c_int(n), c_int(D), c_float(eps),
                                  c_int(1 if stored else 0), c_int(parts),
                                  c_longlong(part_stride), _stream()),
              "add_rmsnorm")
    return out


GLU_ACTIVATIONS = {"silu": 0, "relu": 1, "gelu_tanh": 2}


def silu_mul(gu: torch.Tensor, out: Optional[torch.Tensor] = None, block: int = 0, activation: str = "silu") -> torch.Tensor:
    """a[t, f] = act(gate) * up, act = silu unless `activation` names another (relu, gelu_tanh).  block == 0:
    gu[t] = [gate (F) | up (F)]; block > 0: gu[t] is in groups of `block` gate columns followed by their `block`
    up columns."""
    _dev(gu)
    T, F2 = gu.shape
    F = F2 // 2
    if out is None:
        out = torch.empty((T, F), dtype=gu.dtype, device=gu.device)
    lib = library("elementwise.cu")
    with region("silu_mul", _nb(gu, out)):
        check(lib.aie_silu_mul(_p(gu), _p(out), c_int(dtype_code(gu)), c_int(T), c_int(F), c_int(block),
                               c_int(GLU_ACTIVATIONS[activation]), _stream()), "silu_mul")
    return out


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if x.dtype == dtype:
        return x
    _dev(x)
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    lib = library("elementwise.cu")
    with region("cast", _nb(x, out)):
        check(lib.aie_cast(_p(x), c_int(dtype_code(x)), _p(out), c_int(dtype_code(out)),
                           c_longlong(x.numel()), _stream()), "cast")
    return out


# ---------------------------------------------------------------------------
def gemm_f32(a: torch.Tensor, w: torch.Tensor, rows: Optional[torch.Tensor] = None,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M, N] = a[M, K] . w[N, K]^T in true float32 (FMA on CUDA cores)."""
    _dev(a, w, rows)
    if a.dtype != torch.float32:
        raise KernelError("gemm_f32: activations must be float32")
    K = a.shape[1]
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm_f32: inner sizes differ ({K} vs {w.shape[1]})")
    M = a.shape[0] if rows is None else rows.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    lib = library("gemm_f32.cu")
    with region("gemm_f32", _nb(w, out) + M * K * 4, 2.0 * M * N * K):
        check(lib.aie_gemm_f32(_p(a), _p(w), c_int(dtype_code(w)), _p(out), _p(rows), c_int(M), c_int(N),
                               c_int(K), c_int(out.stride(0)), _stream()), "gemm_f32")
    return out


def tc_tile(T: int) -> int:
    """Token tile of the tcgen05 product: the smallest of 16 .. 256 that holds T, else 256."""
    for bn in (16, 32, 64, 128, 256):
        if T <= bn:
            return bn
    return 256


def tc_splits(T: int, N: int, K: int, bn: int) -> int:
    """Parts to cut K into.  A weight with fewer 128-row tiles than the machine has SMs is
    cut so that the grid comes close to three CTAs per SM (what fits beside each other with
    4-stage rings), each part at least 12 K blocks of 64: measured inside whole decode steps
    of 1 to 64 tokens, K = 4096 is best cut into 5 parts (fewer leave SMs idle, more pay for
    their unjoined float32 parts, which the consumer reads).  A weight with more tiles is not cut."""
    tiles = ((N + 127) // 128) * ((T + bn - 1) // bn)
    kb = (K + 63) // 64
    if tiles >= sm_count():
        return 1
    return max(1, min((_TC_CTAS_PER_SM * sm_count()) // tiles, kb // _TC_MIN_KB))


# split K: at least this many K blocks of 64 a part, at most this many CTAs an SM.  Swept inside whole decode steps
# of 1, 8 and 64 requests (8B shape): (12, 3) and (12, 2) are equal and best; 8 or 6 blocks a part cost 0-2 %,
# 20 / 32 / 56 blocks a part 2 / 7 / 20 %, four CTAs an SM 4-7 %.
_TC_MIN_KB = 12
_TC_CTAS_PER_SM = 3
TC_SWIGLU_BLOCK = 64     # gate/up rows per half of a 128-row weight tile


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, err: torch.Tensor,
            bn: Optional[int] = None, splits: Optional[int] = None, swiglu: bool = False,
            raw_parts: bool = False):
    """bfloat16 x . w^T on tcgen05 tensor cores fed by TMA; None when the sizes are not
    taken (K not a multiple of 8).  swiglu: w is the fused gate/up weight [2F, K] in tiles
    of 64 gate rows + their 64 up rows; the result is silu(gate) * up, [T, F].
    raw_parts: the parts of a split K are not joined: the result is float32
    [splits, T, N] and whoever reads it adds the parts (the norm and rotary kernels do)."""
    T, K = x.shape
    N = w.shape[0]
    if K % 8 or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or (swiglu and N % 128):
        return None
    _dev(x, w, err)
    bn = bn or tc_tile(T)
    splits = splits or tc_splits(T, N, K, bn)
    if swiglu:
        splits = 1 if raw_parts else min(splits, 8)
    kb = (K + 63) // 64
    splits = max(1, min(splits, kb))
    splits = -(-kb // -(-kb // splits))      # no part without K blocks: 64 blocks in 9 parts of 8 are 8 parts
    if raw_parts and splits > 1:
        out = torch.empty((splits, T, N), dtype=torch.float32, device=x.device)
    else:
        raw_parts = False
        splits = min(splits, 8)              # joined inside a cluster of at most 8 CTAs
        out = torch.empty((T, N // 2 if swiglu else N), dtype=out_dtype, device=x.device)
    lib = library("gemm_tc.cu")
    with region("gemm_tc_swiglu" if swiglu else "gemm_tc", _nb(x, w, out), 2.0 * T * N * K):
        check(lib.aie_gemm_tc(_p(x), _p(w), _p(out), c_int(dtype_code(out)), c_int(T), c_int(N), c_int(K),
                              c_int(out.stride(-2)), c_int(bn), c_int(splits), c_int(1 if swiglu else 0),
                              c_int(1 if raw_parts else 0), _p(err), _stream()), "gemm_tc")
    return out


TC_MAX_TOKENS = 64       # up to here the tcgen05 kernel of this package; above, the library product
TC_ROPE_MAX_TOKENS = 16  # up to here the q/k/v product rotates and writes the cache in its epilogue


def linear_parts(x: torch.Tensor, w: torch.Tensor, err: Optional[torch.Tensor] = None,
                 out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """x . w^T for a consumer that can add parts (the next norm, the rotary kernel): float32
    [parts, T, N] when a small bfloat16 step cut K and left the parts unjoined, else [T, N]
    in `out_dtype`."""
    if (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] <= TC_MAX_TOKENS
            and err is not None):
        y = gemm_tc(x, w, torch.float32, err, raw_parts=True)
        if y is not None:
            return y
    return linear(x, w, out_dtype, err)


def linear_add(stream: torch.Tensor, x: torch.Tensor, w: torch.Tensor) -> bool:
    """stream [T, N] float32 += x . w^T in place, the sum taken in float32 inside the library product (its
    epilogue reads the stream and writes it back), for bfloat16 steps of more than 64 tokens: the branch
    output never travels through memory on its own.  False when the step is not of that kind (nothing
    was done): the caller takes `linear_parts` and lets the next norm add."""
    if (x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or stream.dtype != torch.float32
            or x.shape[0] <= TC_MAX_TOKENS or stream.shape != (x.shape[0], w.shape[0]) or not stream.is_contiguous()):
        return False
    _dev(x, w, stream)
    with region("gemm_library", _nb(x, w) + 2 * _nb(stream), 2.0 * x.shape[0] * w.shape[0] * w.shape[1]):
        torch.addmm(stream, x, w.t(), out_dtype=torch.float32, out=stream)
    return True


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           err: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x . w^T.  float32 activations (or a weight stored in 32-bit) take the true
    float32 kernel.  bfloat16 x bfloat16: steps of up to 64 tokens take this package's
    tcgen05 kernel (a weight stream); more tokens take the library matrix product, as the
    reference's engine does for its products
    (crates/ai-engine-candle/src/paged/transformer.rs:153-155)."""
    out_dtype = out_dtype or x.dtype
    if x.dtype == torch.float32 or w.dtype == torch.float32:
        y = gemm_f32(cast(x, torch.float32), w)
        return cast(y, out_dtype)
    if x.shape[0] <= TC_MAX_TOKENS and err is not None:
        y = gemm_tc(x, w, out_dtype, err)
        if y is not None:
            return y
    _dev(x, w)
    with region("gemm_library", _nb(x, w) + x.shape[0] * w.shape[0] * (4 if out_dtype == torch.float32 else 2),
                2.0 * x.shape[0] * w.shape[0] * w.shape[1]):
        if out_dtype == torch.float32:
            return torch.mm(x, w.t(), out_dtype=torch.float32)
        return torch.mm(x, w.t())


def linear_swiglu(x: torch.Tensor, w_gu: torch.Tensor, block: int = 0,
                  err: Optional[torch.Tensor] = None, activation: str = "silu") -> torch.Tensor:
    """silu(x . gate^T) * (x . up^T) for the fused gate/up weight [2F, K]; [T, F] in x's
    dtype.  block == 0: rows [0, F) are gate, [F, 2F) up.  block == 64: tiles of 64 gate
    rows + their 64 up rows, which lets the tcgen05 kernel apply the activation in its
    epilogue when the step is small."""
    if (block == TC_SWIGLU_BLOCK and x.dtype == torch.bfloat16 and w_gu.dtype == torch.bfloat16
            and x.shape[0] <= TC_MAX_TOKENS and err is not None and activation == "silu"):
        y = gemm_tc(x, w_gu, x.dtype, err, swiglu=True)
        if y is not None:
            return y
    return silu_mul(linear(x, w_gu, x.dtype, err), block=block, activation=activation)


def linear_rope_kv(x: torch.Tensor, w_qkv: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                   positions: torch.Tensor, token_req: torch.Tensor, block_table: torch.Tensor,
                   inv_freq: torch.Tensor, H: int, K: int, d: int, err: torch.Tensor,
                   write: bool = True) -> Optional[torch.Tensor]:
    """The q/k/v projection of a small bfloat16 step with the rotation and the cache write in
    its epilogue (one kernel instead of product + rotary kernel); returns q [T, H, d], or None
    when the sizes are not taken: more than 16 tokens, a head size that does not divide 128,
    a partial rotation, K not a multiple of 8."""
    T, Kin = x.shape
    N = w_qkv.shape[0]
    if (T > TC_ROPE_MAX_TOKENS or x.dtype != torch.bfloat16 or w_qkv.dtype != torch.bfloat16
            or k_pages.dtype != torch.bfloat16 or Kin % 8 or d % 2 or 128 % d or N % 128
            or N != (H + 2 * K) * d or inv_freq.shape[0] * 2 != d):
        return None
    _dev(x, w_qkv, k_pages, v_pages, positions, token_req, block_table, inv_freq, err)
    num_pages, Kp, P, dp = k_pages.shape
    if (Kp, dp) != (K, d) or v_pages.shape != k_pages.shape:
        raise KernelError("linear_rope_kv: page shape does not fit (K, d)")
    bn = tc_tile(T)
    kb = (Kin + 63) // 64
    splits = max(1, min(8, kb // 8, (3 * sm_count()) // max(1, N // 128)))
    splits = -(-kb // -(-kb // splits))
    q_out = torch.empty((T, H, d), dtype=torch.bfloat16, device=x.device)
    lib = library("gemm_tc.cu")
    with region("gemm_tc_rope", _nb(x, w_qkv) + T * N * 2, 2.0 * T * N * Kin):
        check(lib.aie_gemm_tc_rope(_p(x), _p(w_qkv), c_int(T), c_int(N), c_int(Kin), c_int(bn), c_int(splits),
                                   _p(q_out), _p(k_pages), _p(v_pages), _p(positions), _p(token_req),
                                   _p(block_table), c_int(block_table.shape[1]), c_int(num_pages), c_int(P),
                                   c_int(H), c_int(K), c_int(d), _p(inv_freq), c_int(1 if write else 0), _p(err),
                                   _stream()), "gemm_tc_rope")
    return q_out


# ---------------------------------------------------------------------------
def rope_kv_write(qkv: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                  positions: torch.Tensor, token_req: torch.Tensor, block_table: torch.Tensor,
                  inv_freq: torch.Tensor, H: int, K: int, d: int, err: torch.Tensor,
                  q_out: Optional[torch.Tensor] = None, write: bool = True) -> torch.Tensor:
    """Rotate q and k by position, write k and v to their pages; returns q [T, H, d].
    k_pages / v_pages: [num_pages, K, page, d] of one layer."""
    _dev(qkv, k_pages, v_pages, positions, token_req, block_table, inv_freq, err)
    parts, part_stride = 1, 0
    if qkv.dim() == 3:            # [parts, T, width] float32: parts of a split product, added here
        parts, part_stride = qkv.shape[0], qkv.stride(0)
    T = qkv.shape[-2]
    if qkv.shape[-1] != (H + 2 * K) * d:
        raise KernelError("rope_kv_write: qkv width differs from (H + 2K) * d")
    num_pages, Kp, P, dp = k_pages.shape
    if (Kp, dp) != (K, d) or v_pages.shape != k_pages.shape:
        raise KernelError("rope_kv_write: page shape does not fit (K, d)")
    if qkv.dtype != k_pages.dtype and qkv.dtype != torch.float32:
        raise KernelError("rope_kv_write: qkv must be in the cache's dtype or float32")
    rot = inv_freq.shape[0] * 2
    if q_out is None:
        q_out = torch.empty((T, H, d), dtype=k_pages.dtype, device=qkv.device)
    lib = library("rope_kv.cu")
    with region("rope_kv_write", _nb(qkv) + T * (H + 2 * K) * d * k_pages.element_size()):
        check(lib.aie_rope_kv_write(_p(qkv), c_int(dtype_code(qkv)), c_int(parts), c_longlong(part_stride),
                                    _p(q_out), _p(k_pages), _p(v_pages), c_int(dtype_code(k_pages)),
                                    _p(positions), _p(token_req), _p(block_table),
                                    c_int(block_table.shape[1]), c_int(num_pages), c_int(P), c_int(T),
                                    c_int(H), c_int(K), c_int(d), c_int(rot), _p(inv_freq),
                                    c_int(1 if write else 0), _p(err), _stream()), "rope_kv_write")
    return q_out


def paged_attention_plain(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                          positions: torch.Tensor, token_req: torch.Tensor,
                          block_table: torch.Tensor, scale: float, window: int, err: torch.Tensor,
                          out: Optional[torch.Tensor] = None,
                          token_list: Optional[torch.Tensor] = None, cost=(0.0, 0.0)) -> torch.Tensor:
    """softmax(q.k * scale over keys j <= pos (and j > pos - window)) . v per query
    token and head, keys read through the block table.  q, out: [T, H, d].
    `token_list`: only these tokens are computed (the others' rows of out are left)."""
    _dev(q, k_pages, v_pages, positions, token_req, block_table, err, token_list)
    T, H, d = q.shape
    num_pages, K, P, dp = k_pages.shape
    if dp != d or H % K:
        raise KernelError("paged_attention: head sizes do not fit")
    if d > 256:
        raise KernelError(f"paged_attention: head_dim {d} > 256 is not supported")
    if out is None:
        out = torch.empty_like(q)
    lib = library("attention_plain.cu")
    with region("attention_plain", *cost):
        check(lib.aie_paged_attention_plain(_p(q), _p(k_pages), _p(v_pages), _p(out),
                                            c_int(dtype_code(q)), _p(positions), _p(token_req),
                                            _p(block_table), c_int(block_table.shape[1]),
                                            c_int(num_pages), c_int(P),
                                            c_int(T if token_list is None else token_list.shape[0]),
                                            c_int(H), c_int(K), c_int(d), c_int(window), c_float(scale),
                                            _p(token_list), _p(err), _stream()),
              "paged_attention_plain")
    return out


def decode_splits(n_dec: int, kv_heads: int, group: int, max_keys: int, bt_width: int = 0) -> int:
    """How many parts to cut each decode request's keys into so that the grid fills
    the machine (two CTAs fit on each SM), with parts of at least 128
    keys, and no part spanning more block-table entries than a CTA keeps."""
    ctas = n_dec * kv_heads * ((group + 7) // 8)
    want = max(1, (2 * sm_count()) // ctas)   # rounded down: one full wave, no short second one
    s = max(1, min(want, (max_keys + 127) // 128, 64))
    return max(s, (bt_width + 1999) // 2000)


_DECODE_COUNTERS = {}        # device -> zeroed int32 tickets of the decode kernel (they return to zero)


def _decode_counters(device, n: int):
    t = _DECODE_COUNTERS.get(device)
    if t is None or t.numel() < n:
        t = torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device)
        _DECODE_COUNTERS[device] = t
    return t


def paged_attention_decode(q, k_pages, v_pages, dec_tokens, positions, token_req, block_table,
                           scale: float, window: int, splits: int, err, out,
                           join_in_kernel: bool = False, cost=(0.0, 0.0)) -> None:
    """bfloat16 split-KV attention for the tokens in `dec_tokens` (requests that bring
    one token).  Head sizes 64 and 128.  Uses scratch for the parts when splits > 1; they are
    joined by a second kernel, or (join_in_kernel) by whichever CTA finishes last — measured
    slightly slower in a decode step, kept for callers that want one launch."""
    _dev(q, k_pages, v_pages, dec_tokens, positions, token_req, block_table, err, out)
    T, H, d = q.shape
    num_pages, K, P, _ = k_pages.shape
    n = dec_tokens.shape[0]
    part_o = part_lse = counters = None
    if splits > 1:
        part_o = torch.empty((n, H, splits, d), dtype=torch.float32, device=q.device)
        part_lse = torch.empty((n, H, splits), dtype=torch.float32, device=q.device)
        if join_in_kernel:
            counters = _decode_counters(q.device, n * K * ((H // K + 7) // 8))
    lib = library("attention_fast.cu")
    with region("attention_decode", *cost):
        check(lib.aie_paged_attention_decode(_p(q), _p(k_pages), _p(v_pages), _p(out), _p(part_o),
                                             _p(part_lse), _p(dec_tokens), c_int(n), _p(positions),
                                             _p(token_req), _p(block_table), c_int(block_table.shape[1]),
                                             c_int(num_pages), c_int(P), c_int(H), c_int(K), c_int(d),
                                             c_int(window), c_float(scale), c_int(splits), _p(counters),
                                             _p(err), _stream()), "paged_attention_decode")


PREFILL_TILE = 128       # query tokens per CTA of the tensor-core attention kernel


def paged_attention_prefill(q, k_pages, v_pages, tiles, q_start, q_len, ctx_len, block_table,
                            scale: float, window: int, err, out, cost=(0.0, 0.0)) -> None:
    """bfloat16 tensor-core attention for requests that bring more than one token.
    `tiles`: int32 [n, 2] = (request row, offset of a PREFILL_TILE-token tile in its tokens).
    Head sizes 64 and 128."""
    _dev(q, k_pages, v_pages, tiles, q_start, q_len, ctx_len, block_table, err, out)
    T, H, d = q.shape
    num_pages, K, P, _ = k_pages.shape
    lib = library("attention_fast.cu")
    with region("attention_prefill_mma", *cost):
        check(lib.aie_paged_attention_prefill(_p(q), _p(k_pages), _p(v_pages), _p(out), _p(tiles),
                                              c_int(tiles.shape[0]), _p(q_start), _p(q_len), _p(ctx_len),
                                              _p(block_table), c_int(block_table.shape[1]),
                                              c_int(num_pages), c_int(P), c_int(H), c_int(K), c_int(d),
                                              c_int(window), c_float(scale), _p(err), _stream()),
              "paged_attention_prefill")


def paged_attention_prefill_tc(q, k_pages, v_pages, tiles, q_start, q_len, ctx_len, block_table,
                               scale: float, window: int, err, out, cost=(0.0, 0.0), pair: bool = False) -> bool:
    """The tcgen05 version of paged_attention_prefill (scores and outputs in tensor memory,
    operands by TMA).  Takes head sizes 64 and 128, pages of 8 .. 128 keys that divide 128, no window; returns
    False when it does not take the sizes (nothing was launched).  `pair`: the kernel whose CTAs take two tiles
    each; `tiles` then lists units of 2 * PREFILL_TILE tokens (request row, offset of the unit)."""
    _dev(q, k_pages, v_pages, tiles, q_start, q_len, ctx_len, block_table, err, out)
    T, H, d = q.shape
    num_pages, K, P, _ = k_pages.shape
    if d not in (64, 128) or window > 0 or P < 8 or P > 128 or 128 % P:
        return False
    lib = library("attention_prefill_tc.cu")
    fn = lib.aie_paged_attention_prefill_tc_pair if pair else lib.aie_paged_attention_prefill_tc
    with region("attention_prefill_tcgen05", *cost):
        rc = fn(_p(q), _p(k_pages), _p(v_pages), _p(out), _p(tiles), c_int(tiles.shape[0]), _p(q_start), _p(q_len),
                _p(ctx_len), _p(block_table), c_int(block_table.shape[1]), c_int(num_pages), c_int(P), c_int(T),
                c_int(H), c_int(K), c_int(d), c_int(window), c_float(scale), _p(err), _stream())
    if rc == -2:
        return False
    check(rc, "paged_attention_prefill_tc")
    return True


def prefill_takes_pairs(n_tiles: int, n_units: int, heads: int) -> bool:
    """Whether the tcgen05 prompt kernel with two query tiles per CTA is the faster one for a step with `n_tiles`
    tiles in `n_units` units of two.  Measured on heads of 128 and of 64: it takes 0.80-0.86 of the one-tile
    kernel's time when nearly all units are whole and its CTAs (units x heads) fill the SMs in whole rounds about as
    well as the one-tile kernel's; with a lone tile in a unit it runs at half speed, and with fewer CTAs than SMs
    the longest CTA decides, which is twice as long."""
    if n_units == 0 or n_tiles < 1.8 * n_units:
        return False
    sms = sm_count()
    w1, w2 = n_tiles * heads / sms, n_units * heads / sms
    if w2 <= 1.0:
        return False
    return 0.86 * math.ceil(w2) / w2 < math.ceil(w1) / w1


def paged_attention(q, k_pages, v_pages, ctx, work, block_table, scale: float, window: int):
    """Attention of a step's query tokens over the cache.  `ctx` gives the step's generic arrays
    (positions, token_req, q_start, q_len, ctx_len, R), `work` the attention work lists derived from
    them (decode_tokens, prefill_tiles, n_decode, max_decode_len).  float32 takes the plain
    kernel.  bfloat16 with a head size of 64 or 128: requests that bring one token
    take the split-KV decode kernel, the others a tensor-core kernel for portions of
    prompts (tcgen05 for head size 128 without a window, else mma.sync); other head sizes
    take the plain kernel."""
    T, H, d = q.shape
    K = k_pages.shape[1]
    fast = q.dtype == torch.bfloat16 and d in (64, 128)
    dec_cost = pre_cost = (0.0, 0.0)
    if _profiling() and hasattr(ctx, "h_q_len"):      # keys read and products done, from the host's lengths
        ql, cl = ctx.h_q_len.astype(float), ctx.h_ctx_len.astype(float)
        if window > 0:
            cl = cl.clip(max=float(window))
        es = k_pages.element_size()
        lone = ql == 1
        keys = float((cl[lone] + 1).sum())
        dec_cost = (keys * K * d * 2 * es, 4.0 * keys * H * d)
        pairs = float((ql[~lone] * cl[~lone] + ql[~lone] * (ql[~lone] + 1) / 2).sum())
        pre_cost = (float((cl[~lone] + ql[~lone]).sum()) * K * d * 2 * es + float(ql[~lone].sum()) * H * d * 2 * es,
                    4.0 * pairs * H * d)
    if not fast:
        return paged_attention_plain(q, k_pages, v_pages, ctx.positions, ctx.token_req, block_table,
                                     scale, window, ctx.err,
                                     cost=(dec_cost[0] + pre_cost[0], dec_cost[1] + pre_cost[1]))
    out = torch.empty_like(q)
    if work.n_decode:
        keys = work.max_decode_len if window <= 0 else min(window, work.max_decode_len)
        paged_attention_decode(q, k_pages, v_pages, work.decode_tokens, ctx.positions, ctx.token_req,
                               block_table, scale, window,
                               decode_splits(work.n_decode, K, H // K, keys, block_table.shape[1]),
                               ctx.err, out, cost=dec_cost)
    if work.n_decode < ctx.R:
        pairs = getattr(work, "prefill_pairs", None)
        if pairs is not None and prefill_takes_pairs(work.prefill_tiles.shape[0], pairs.shape[0], H):
            took = paged_attention_prefill_tc(q, k_pages, v_pages, pairs, ctx.q_start, ctx.q_len, ctx.ctx_len,
                                              block_table, scale, window, ctx.err, out, cost=pre_cost, pair=True)
        else:
            took = paged_attention_prefill_tc(q, k_pages, v_pages, work.prefill_tiles, ctx.q_start, ctx.q_len,
                                              ctx.ctx_len, block_table, scale, window, ctx.err, out, cost=pre_cost)
        if not took:
            paged_attention_prefill(q, k_pages, v_pages, work.prefill_tiles, ctx.q_start, ctx.q_len,
                                    ctx.ctx_len, block_table, scale, window, ctx.err, out, cost=pre_cost)
    return out


# ---------------------------------------------------------------------------
# true-float32 products with strides, batches and per-tile weights
def gemm_f32_ex(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, M: int, N: int, K: int, lda: int, ldc: int,
                batch: int = 1, a_bs: int = 0, w_bs: int = 0, c_bs: int = 0,
                a_rows: Optional[torch.Tensor] = None, tile_w: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[m, n] = sum_k a[m, k] * w[n, k] on the CUDA cores, float32 sums in the order k = 0 .. K-1, operands
    float32 or bfloat16 (widened), result rounded once to out's dtype.  `a`, `w`, `out` are the tensors that
    hold the first operand of the batch at their data pointer; rows are lda / K / ldc elements apart and the
    operands of a batch a_bs / w_bs / c_bs elements.  a_rows: row gather (-1 reads zeros).  tile_w: weight
    index per tile of 64 rows (-1 skips the tile), the weights w_bs elements apart."""
    for t in (a, w, out, a_rows, tile_w):
        if t is not None and not t.is_cuda:
            require_cuda()
            raise KernelError("kernel operands must live on the CUDA device")
    lib = library("gemm_f32.cu")
    with region("gemm_f32", (N * K * w.element_size() + M * K * a.element_size() + M * N * out.element_size()) * batch,
                2.0 * M * N * K * batch):
        check(lib.aie_gemm_f32_ex(_p(a), c_int(dtype_code(a)), _p(w), c_int(dtype_code(w)), _p(out),
                                  c_int(dtype_code(out)), _p(a_rows), _p(tile_w), c_int(M), c_int(N), c_int(K),
                                  c_int(lda), c_int(ldc), c_int(batch), c_longlong(a_bs), c_longlong(w_bs),
                                  c_longlong(c_bs), _stream()), "gemm_f32_ex")
    return out


def head_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Per-head projection: out[t, h, :] = w[h] . x[t, h, :] with x [T, H, K] (the last axis contiguous, any
    strides before it), w [H, N, K], out [T, H, >= N] (written into its first N columns of the last axis)."""
    T, H, K = x.shape
    N = w.shape[1]
    if w.shape != (H, N, K) or out.shape[:2] != (T, H) or out.shape[2] < N:
        raise KernelError("head_linear: shapes do not fit")
    if x.stride(2) != 1 or out.stride(2) != 1 or not w.is_contiguous():
        raise KernelError("head_linear: the last axis must be contiguous")
    if T > TC_MAX_TOKENS and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        # many tokens: the library's batched product, as for the other projections of a prompt step
        with region("gemm_library", _nb(x, w) + T * H * N * out.element_size(), 2.0 * T * H * N * K):
            dst = out[:, :, :N].transpose(0, 1)          # [H, T, N] view: the product is written in place
            if out.dtype == torch.float32:
                torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out_dtype=torch.float32, out=dst)
            else:
                torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out=dst)
        return out
    return gemm_f32_ex(x, w, out, T, N, K, x.stride(0), out.stride(0), batch=H, a_bs=x.stride(1), w_bs=N * K,
                       c_bs=out.stride(1))


# ---------------------------------------------------------------------------
# parts that carry state or normalise over other axes than the stream's width
def short_conv(h: torch.Tensor, w: torch.Tensor, state: torch.Tensor, ctx, out_dtype: torch.dtype) -> torch.Tensor:
    """out = h + causal convolution of h over each request's tokens, per channel.  h [T, D] float32; w [D, taps]
    float32; state [max_seqs, taps - 1, D] float32: each request's last taps - 1 inputs, read for the first
    tokens of its portion and replaced by the portion's last ones."""
    _dev(h, w, state)
    T, D = h.shape
    taps = w.shape[1]
    if h.dtype != torch.float32 or w.dtype != torch.float32 or state.dtype != torch.float32:
        raise KernelError("short_conv: inputs, taps and state are float32")
    if w.shape[0] != D or state.shape[1:] != (max(taps - 1, 0), D):
        raise KernelError("short_conv: shapes do not fit")
    out = torch.empty((T, D), dtype=out_dtype, device=h.device)
    lib = library("sequence_ops.cu")
    with region("short_conv", _nb(h, out)):
        check(lib.aie_short_conv(_p(h), _p(w), _p(state), _p(out), c_int(dtype_code(out)), _p(ctx.q_start),
                                 _p(ctx.q_len), _p(ctx.slots), _p(ctx.token_req), c_int(T), c_int(D), c_int(taps),
                                 c_int(state.shape[0]), _p(ctx.err), _stream()), "short_conv")
    return out


def depth_average(x: torch.Tensor, delta: Optional[torch.Tensor], history: torch.Tensor, coef: torch.Tensor,
                  depth: int) -> None:
    """X = x (+ delta, or the sum of its parts); history[depth] = X; x = sum_{j <= depth} coef[j] history[j],
    in place.  x [T, D] float32; history [levels, T, D] float32; coef float32 [>= depth + 1]."""
    _dev(x, delta, history, coef)
    if x.dtype != torch.float32 or history.dtype != torch.float32 or coef.dtype != torch.float32:
        raise KernelError("depth_average: stream, history and weights are float32")
    if history.shape[1:] != x.shape or depth >= history.shape[0] or coef.shape[0] < depth + 1:
        raise KernelError("depth_average: shapes do not fit")
    parts, stride = 0, 0
    if delta is not None:
        parts, stride = (delta.shape[0], delta.stride(0)) if delta.dim() == 3 else (1, 0)
        if delta.shape[-2:] != x.shape:
            raise KernelError("depth_average: delta differs in shape from x")
    lib = library("sequence_ops.cu")
    with region("depth_average", (depth + 3) * _nb(x) + _nb(delta)):
        check(lib.aie_depth_average(_p(x), _p(delta), c_int(dtype_code(delta) if delta is not None else 0),
                                    c_int(parts), c_longlong(stride), _p(history), _p(coef), c_int(depth),
                                    c_longlong(x.numel()), _stream()), "depth_average")


def polynorm(z: torch.Tensor, coef: torch.Tensor, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """a N(z) + b N(z^2) + c N(z^3) + e per row, N = division by the root mean square; coef = (a, b, c, e)."""
    _dev(z, coef)
    if z.dtype != torch.float32 or coef.dtype != torch.float32 or coef.numel() != 4:
        raise KernelError("polynorm: float32 input and four float32 coefficients")
    T, F = z.shape
    out = torch.empty((T, F), dtype=out_dtype, device=z.device)
    lib = library("sequence_ops.cu")
    with region("polynorm", _nb(z, out)):
        check(lib.aie_polynorm(_p(z), _p(coef), _p(out), c_int(dtype_code(out)), c_int(T), c_int(F), c_float(eps),
                               _stream()), "polynorm")
    return out


def head_norm_gate(o: torch.Tensor, gate: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float,
                   out_dtype: torch.dtype) -> torch.Tensor:
    """Per (token, head): o / rms(o) (* weight) (* silu(gate)).  o [T, H, dv] float32; gate [T, H * dv] float32,
    rows gate.stride(0) apart, or None (no gate); weight [dv] float32 or None.  Returns [T, H * dv]."""
    _dev(o, weight)
    T, H, dv = o.shape
    if o.dtype != torch.float32 or (gate is not None and (gate.dtype != torch.float32 or gate.stride(1) != 1
                                                          or gate.shape != (T, H * dv))):
        raise KernelError("head_norm_gate: shapes or dtypes do not fit")
    out = torch.empty((T, H * dv), dtype=out_dtype, device=o.device)
    lib = library("sequence_ops.cu")
    with region("head_norm_gate", 2 * _nb(o) + _nb(out)):
        check(lib.aie_head_norm_gate(_p(o), _p(gate), c_int(gate.stride(0) if gate is not None else 0), _p(weight), _p(out),
                                     c_int(dtype_code(out)), c_int(T), c_int(H), c_int(dv), c_float(eps), _stream()),
              "head_norm_gate")
    return out


def clamped_glu(gu: torch.Tensor, F: int, limit: float, alpha: float, shift: float,
                out_dtype: torch.dtype) -> torch.Tensor:
    """g = min(gate, limit), u = clamp(up, +-limit): g * sigmoid(alpha g) * (u + shift).  gu [T, >= 2F] float32
    with the gate in columns [0, F) and up in [F, 2F)."""
    if gu.dtype != torch.float32 or gu.stride(1) != 1 or gu.shape[1] < 2 * F:
        raise KernelError("clamped_glu: float32 [T, >= 2F] input")
    T = gu.shape[0]
    out = torch.empty((T, F), dtype=out_dtype, device=gu.device)
    lib = library("sequence_ops.cu")
    with region("clamped_glu", 2 * T * F * 4 + _nb(out)):
        check(lib.aie_clamped_glu(_p(gu), c_int(gu.stride(0)), _p(out), c_int(dtype_code(out)), c_longlong(T),
                                  c_int(F), c_float(limit), c_float(alpha), c_float(shift), _stream()), "clamped_glu")
    return out


def gated_decay(z: torch.Tensor, bias: Optional[torch.Tensor], tau: float) -> torch.Tensor:
    """sigmoid(z + bias)^(1 / tau) in float32, z [T, N] contiguous."""
    _dev(z, bias)
    if z.dtype != torch.float32:
        raise KernelError("gated_decay: float32 logits")
    out = torch.empty_like(z)
    lib = library("sequence_ops.cu")
    with region("gated_decay", 2 * _nb(z)):
        check(lib.aie_gated_decay(_p(z), _p(bias), _p(out), c_longlong(z.shape[0]), c_int(z.shape[1]), c_float(tau),
                                  _stream()), "gated_decay")
    return out


EXPERT_TILE = 64         # rows per tile of the grouped products


def expert_plan(token_ids: Optional[torch.Tensor], table: torch.Tensor, experts: int, err: torch.Tensor,
                identity: int = 0):
    """Group the (token, choice) pairs of a step by expert: (row_token [tiles * 64], pair_row [T * top],
    tile_expert [tiles]); the sizes depend on T alone.  token_ids None: `table` [T, top] holds each token's
    choices (a router's).  Choices experts .. experts + identity - 1 get no row; their pairs are marked -2."""
    _dev(token_ids, table, err)
    V, top = table.shape
    T = token_ids.shape[0] if token_ids is not None else V
    tiles = (T * top + EXPERT_TILE - 1) // EXPERT_TILE + experts
    dev = table.device
    row_token = torch.empty(tiles * EXPERT_TILE, dtype=torch.int32, device=dev)
    pair_row = torch.empty(T * top, dtype=torch.int32, device=dev)
    tile_expert = torch.empty(tiles, dtype=torch.int32, device=dev)
    lib = library("sequence_ops.cu")
    check(lib.aie_expert_plan(_p(token_ids), _p(table), c_int(T), c_int(V), c_int(top), c_int(experts),
                              c_int(identity), c_int(EXPERT_TILE), c_int(tiles), _p(row_token), _p(pair_row), _p(tile_expert), _p(err),
                              _stream()), "expert_plan")
    return row_token, pair_row, tile_expert


def expert_combine(y: torch.Tensor, pair_row: torch.Tensor, top: int, weight: float,
                   shared: Optional[torch.Tensor], gate: Optional[torch.Tensor], T: int) -> torch.Tensor:
    """out[t] = weight * sum_s y[pair_row[t top + s]] (+ shared[t] * sigmoid(gate[t])), float32 [T, D];
    gate: a [T] float32 view (any stride)."""
    _dev(y, pair_row, shared)
    D = y.shape[1]
    if y.dtype != torch.float32 or (shared is not None and (shared.dtype != torch.float32 or gate is None or
                                                            gate.dtype != torch.float32)):
        raise KernelError("expert_combine: float32 operands")
    out = torch.empty((T, D), dtype=torch.float32, device=y.device)
    lib = library("sequence_ops.cu")
    with region("expert_combine", (top + 2) * T * D * 4):
        check(lib.aie_expert_combine(_p(y), _p(pair_row), c_int(top), c_float(weight), _p(shared), _p(gate),
                                     c_int(gate.stride(0) if gate is not None else 0), _p(out), c_int(T), c_int(D),
                                     _stream()), "expert_combine")
    return out


def latent_prepare(proj: torch.Tensor, H: int, d: int, rot: int, rank: int, c_weight: Optional[torch.Tensor],
                   eps: float, inv_freq: torch.Tensor, pages: torch.Tensor, ctx, block_table: torch.Tensor,
                   q_dtype: torch.dtype, write: bool, kv: Optional[torch.Tensor] = None, halves: bool = False):
    """From the fused projection [q heads (d plain | rot rotated) | latent (rank) | shared key part (rot)] of a
    step: (q_plain [T, H, d] in q_dtype, q_full [T, H, rank + rot] float32 whose last rot columns hold the
    rotated query parts); with `write`, the normalised latent and the rotated key part go into the tokens'
    cache rows.  pages [num_pages, 1, P, rank + rot].  kv: the latent and the key part come from this float32 view
    [T, >= rank + rot] (rows any stride) instead of the columns behind the queries.  halves: the rotation pairs
    element i with i + rot_dims / 2 instead of 2i with 2i + 1."""
    _dev(proj, c_weight, inv_freq, pages, block_table)
    T, ld = proj.shape
    need = H * (d + rot) + ((rank + rot) if write and kv is None else 0)
    if kv is not None and (kv.dtype != torch.float32 or kv.stride(1) != 1 or kv.shape[0] != T or kv.shape[1] < rank + rot):
        raise KernelError("latent_prepare: the latent projection is a float32 view [T, >= rank + rot]")
    if proj.dtype != torch.float32 or ld < need or pages.shape[1] != 1 or pages.shape[3] != rank + rot:
        raise KernelError("latent_prepare: shapes or dtypes do not fit")
    q_plain = torch.empty((T, H, d), dtype=q_dtype, device=proj.device)
    q_full = torch.empty((T, H, rank + rot), dtype=torch.float32, device=proj.device)
    lib = library("latent_attention.cu")
    with region("latent_prepare", _nb(proj, q_plain) + T * H * rot * 4):
        check(lib.aie_latent_prepare(_p(proj), c_int(ld), c_int(T), c_int(H), c_int(d), c_int(rot), c_int(rank),
                                     c_int(2 * inv_freq.shape[0]), c_int(1 if write else 0), _p(c_weight),
                                     c_float(eps), _p(inv_freq), _p(q_plain), c_int(dtype_code(q_plain)), _p(q_full),
                                     _p(pages), c_int(dtype_code(pages)), _p(ctx.positions), _p(ctx.token_req),
                                     _p(block_table), c_int(block_table.shape[1]), c_int(pages.shape[0]),
                                     c_int(pages.shape[2]), _p(ctx.err), _p(kv), c_int(kv.stride(0) if kv is not None else 0),
                                     c_int(1 if halves else 0), _stream()), "latent_prepare")
    return q_plain, q_full


def latent_attention(q_full: torch.Tensor, pages: torch.Tensor, ctx, block_table: torch.Tensor, rank: int,
                     scale: float, window: int, out_dtype: torch.dtype, work=None) -> torch.Tensor:
    """softmax over the visible cache rows of (q_full . row) * scale, times the rows' first `rank` elements:
    [T, H, rank].  q_full [T, H, dk] float32; pages [num_pages, 1, P, dk].  `work`: the step's units of tokens
    (`tiles` [n, 2], `tq`) for the tensor-core kernel, which bfloat16 takes when the sizes fit (a latent of
    64 .. 512 in steps of 64, rows a multiple of 16); everything else takes the plain kernel."""
    _dev(q_full, pages, block_table)
    T, H, dk = q_full.shape
    if q_full.dtype != torch.float32 or pages.shape[3] != dk or pages.shape[1] != 1:
        raise KernelError("latent_attention: shapes or dtypes do not fit")
    out = torch.empty((T, H, rank), dtype=out_dtype, device=q_full.device)
    cost = (float(_nb(q_full, out)), 0.0)
    if _profiling() and hasattr(ctx, "h_q_len"):      # cache rows read once per request, products per (query, key) pair
        pairs = rows = 0.0
        for n, c in zip(ctx.h_q_len.tolist(), ctx.h_ctx_len.tolist()):
            seen = [min(c + i + 1, window) if window > 0 else c + i + 1 for i in range(n)]
            pairs += float(sum(seen))
            rows += float(min(c + n, (window + n) if window > 0 else c + n))
        cost = (cost[0] + rows * dk * pages.element_size(), 2.0 * pairs * H * (dk + rank))
    if (work is not None and pages.dtype == torch.bfloat16 and out_dtype == torch.bfloat16 and rank % 64 == 0
            and 64 <= rank <= 512 and dk % 16 == 0 and dk <= 1024
            and (work.tq * 16 + 64) * (dk + 8) * 2 + work.tq * 7000 <= 220 * 1024):
        # tensor cores; a step of few tokens cuts each token's keys into parts so that the grid fills the machine
        keys = ctx.bt_width * ctx.page_size if ctx.bucketed else ctx.max_total_len
        if window > 0:
            keys = min(keys, window + 63)
        ctas = work.tiles.shape[0] * ((H + 15) // 16)
        splits = max(1, min(64, (keys + 63) // 64, (2 * sm_count()) // ctas))
        part_o = part_ml = None
        if splits > 1:
            part_o = torch.empty((T, H, splits, rank), dtype=torch.float32, device=q_full.device)
            part_ml = torch.empty((T, H, splits, 2), dtype=torch.float32, device=q_full.device)
        lib = library("latent_attention_tc.cu")
        with region("latent_attention_tc", *cost):
            check(lib.aie_latent_attention_tc(_p(q_full), _p(pages), _p(out), _p(part_o), _p(part_ml), _p(work.tiles),
                                              c_int(work.tiles.shape[0]), c_int(work.tq), _p(ctx.q_start),
                                              _p(ctx.q_len), _p(ctx.ctx_len), _p(block_table), c_int(block_table.shape[1]),
                                              c_int(pages.shape[0]), c_int(pages.shape[2]), c_int(T), c_int(H),
                                              c_int(rank), c_int(dk), c_int(window), c_float(scale), c_int(splits),
                                              _p(ctx.err), _stream()), "latent_attention_tc")
        return out
    lib = library("latent_attention.cu")
    with region("latent_attention", *cost):
        check(lib.aie_latent_attention(_p(q_full), _p(pages), c_int(dtype_code(pages)), _p(out),
                                       c_int(dtype_code(out)), _p(ctx.positions), _p(ctx.token_req), _p(block_table),
                                       c_int(block_table.shape[1]), c_int(pages.shape[0]), c_int(pages.shape[2]),
                                       c_int(T), c_int(H), c_int(rank), c_int(dk), c_int(window), c_float(scale),
                                       _p(ctx.err), _stream()), "latent_attention")
    return out


SSD_MIN_TOKENS = 32      # portions from this length on take the chunked state-space kernel (bfloat16 mode)
SSD_CHUNK = 64           # its chunk


def linear_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay_tok: Optional[torch.Tensor],
                      decay_head: Optional[torch.Tensor], q_scale: float, k_scale: float, state: torch.Tensor,
                      ctx, H: int, d: int, dv: int, heads_per_group: int = 1, dt_raw: Optional[torch.Tensor] = None,
                      dt_bias: Optional[torch.Tensor] = None, a_log: Optional[torch.Tensor] = None,
                      skip: Optional[torch.Tensor] = None, chunked: bool = False, wide_state: bool = False,
                      forget_lower: Optional[torch.Tensor] = None, forget_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """S <- diag(a_t) S + k_t v_t^T, o_t = S^T q_t per request and head over the step's tokens, the state
    [max_seqs, H, d, dv] float32 read and left in each request's slot.  q, k [T, H * d] and v [T, H * dv] are
    float32 views with one row stride; decay_tok [T, H * d] float32 (rows any stride) or decay_head [H].
    With `dt_raw` [T, H] (a float32 view, rows any stride), dt_bias and a_log [H]: the decay is one number per
    token and head, a = exp(-exp(a_log) dt) with dt = softplus(dt_raw + dt_bias), and v is scaled by dt.
    heads_per_group: neighbouring heads that share one head of q and k ([T, H / heads_per_group * d]).
    skip [H]: skip[h] * v is added to the output.  chunked (with dt_raw): portions of SSD_MIN_TOKENS tokens or more
    take the chunked tensor-core kernel, which rounds q, k and v to bfloat16 (a state of up to 128 rows).
    wide_state (with dt_raw): step sizes, decays and a step's updates are made in double and the state is rounded
    once, when it returns to its float32 slot.
    forget_lower [H * d] float32 (with forget_bias [H * d] or None): the keyless form.  k is None, decay_tok holds the
    forget gate's logits z, and the kernel makes a = l + (1 - l) sigmoid(z + bias), k = 1 - a and q = silu(q) itself.
    Returns o [T, H, dv] float32."""
    _dev(state, decay_head, dt_bias, a_log, skip, forget_lower, forget_bias)
    if forget_lower is not None:
        if k is not None or decay_tok is None or forget_lower.dtype != torch.float32 or forget_lower.numel() != H * d:
            raise KernelError("linear_recurrence: the keyless form takes the gate's logits as decay_tok and no keys")
    keyless = forget_lower is not None
    if dt_raw is not None and (dt_raw.dtype != torch.float32 or dt_raw.stride(1) != 1 or dt_bias is None or a_log is None):
        raise KernelError("linear_recurrence: step sizes are a float32 view with their bias and rates")
    T = q.shape[0]
    ld = q.stride(0)
    if (q.dtype != torch.float32 or v.dtype != torch.float32 or v.stride(0) != ld or q.stride(1) != 1
            or (not keyless and (k.dtype != torch.float32 or k.stride(0) != ld))
            or state.shape[1:] != (H, d, dv) or state.dtype != torch.float32):
        raise KernelError("linear_recurrence: shapes or dtypes do not fit")
    out = torch.empty((T, H, dv), dtype=torch.float32, device=q.device)
    max_len = 0
    if (chunked and dt_raw is not None and decay_tok is None and d <= 128 and ctx.max_q_len >= SSD_MIN_TOKENS
            and not os.environ.get("AI_ENGINE_B200_NO_CHUNKED_SCAN")):      # the switch is for measurement
        lib = library("state_space_chunked.cu")
        with region("state_space_chunked", _nb(out) + T * H * (2 * d // heads_per_group + dv) * 4,
                    2.0 * T * H * (SSD_CHUNK * (d + dv) / 2 + 2 * d * dv)):
            check(lib.aie_state_space_chunked(_p(q), _p(k), _p(v), c_int(ld), _p(dt_raw), c_int(dt_raw.stride(0)), _p(dt_bias),
                                              _p(a_log), _p(skip), _p(state), _p(out), _p(ctx.q_start), _p(ctx.q_len),
                                              _p(ctx.slots), c_int(ctx.R), c_int(H), c_int(d), c_int(dv),
                                              c_int(heads_per_group), c_int(state.shape[0]), c_int(SSD_MIN_TOKENS),
                                              _p(ctx.err), _stream()), "state_space_chunked")
        if int(ctx.h_q_len.min()) >= SSD_MIN_TOKENS:
            return out
        max_len = SSD_MIN_TOKENS - 1                # the shorter portions and single tokens of the same step
    lib = library("linear_recurrence.cu")
    with region("linear_recurrence", _nb(out) + T * H * (2 * d + dv) * 4 + 2 * ctx.R * H * d * dv * 4, 4.0 * T * H * d * dv):
        check(lib.aie_linear_recurrence(_p(q), _p(k), _p(v), c_int(ld), _p(decay_tok),
                                        c_int(decay_tok.stride(0) if decay_tok is not None else 0), _p(decay_head),
                                        c_float(q_scale), c_float(k_scale), _p(state), _p(out), _p(ctx.q_start),
                                        _p(ctx.q_len), _p(ctx.slots), c_int(T), c_int(ctx.R), c_int(H), c_int(d), c_int(dv),
                                        c_int(state.shape[0]), _p(ctx.err), c_int(heads_per_group), _p(dt_raw),
                                        c_int(dt_raw.stride(0) if dt_raw is not None else 0), _p(dt_bias), _p(a_log),
                                        _p(skip), c_int(max_len), c_int(1 if wide_state else 0), _p(forget_lower),
                                        _p(forget_bias), _stream()),
              "linear_recurrence")
    return out


def gather_rows(src: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    """out[r] = src[rows[r]], zeros where rows[r] < 0."""
    _dev(src, rows)
    out = torch.empty((rows.shape[0], src.shape[1]), dtype=src.dtype, device=src.device)
    lib = library("sequence_ops.cu")
    with region("gather_rows", 2 * _nb(out)):
        check(lib.aie_gather_rows(_p(src), _p(rows), _p(out), c_int(dtype_code(src)), c_int(rows.shape[0]),
                                  c_int(src.shape[1]), _stream()), "gather_rows")
    return out


def grouped_linear(x: torch.Tensor, w: torch.Tensor, tile_w: torch.Tensor, out_dtype: torch.dtype,
                   err: torch.Tensor, row_src: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rows grouped in tiles of EXPERT_TILE, tile i multiplied with the weight w[tile_w[i]] of the stack w [E, N, K]
    (tile_w[i] < 0: the tile is skipped, its output rows are undefined).  x [rows, K], or, with `row_src`
    [rows], the rows x[row_src[r]] (zeros for -1).  bfloat16 operands whose N is a multiple of 128 and K of 8
    take the tcgen05 kernel, everything else the float32 kernel on the CUDA cores."""
    E, N, K = w.shape
    rows = tile_w.shape[0] * EXPERT_TILE
    out = torch.empty((rows, N), dtype=out_dtype, device=x.device)
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and N % 128 == 0 and K % 8 == 0:
        xs = gather_rows(x, row_src) if row_src is not None else x
        _dev(xs, w, tile_w, err)
        lib = library("gemm_tc.cu")
        with region("gemm_tc_grouped", _nb(xs, w, out), 2.0 * rows * N * K):
            check(lib.aie_gemm_tc_grouped(_p(xs), _p(w), _p(out), c_int(dtype_code(out)), c_int(rows), c_int(N),
                                          c_int(K), c_int(N), c_int(EXPERT_TILE), c_int(E), _p(tile_w), _p(err),
                                          _stream()), "gemm_tc_grouped")
        return out
    return gemm_f32_ex(x, w, out, rows, N, K, K, N, w_bs=N * K, a_rows=row_src, tile_w=tile_w)


# ---------------------------------------------------------------------------
# parts of layers with a convolved projection, a state space, a router, bounded logits
def causal_conv(u: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor, ctx,
                out_dtype: torch.dtype, activation: Optional[str] = None, residual: bool = False,
                dup_from: int = 0, dup_n: int = 0) -> torch.Tensor:
    """y_t = (u_t +) bias + sum_j w[:, j] u_(t - taps + 1 + j) per channel over each request's tokens, then the
    activation (None | "silu").  u: a float32 view [T, C] with any row stride (a slice of a wider projection);
    w [C, taps], bias [C] or None, float32; state [max_seqs, taps - 1, C] float32: each request's last taps - 1
    inputs.  The last dup_n channels (from dup_from on) are written twice, the copy dup_n columns further on:
    the result is [T, C + dup_n]."""
    _dev(w, bias, state)
    T, C = u.shape
    taps = w.shape[1]
    if (u.dtype != torch.float32 or u.stride(1) != 1 or w.dtype != torch.float32 or state.dtype != torch.float32
            or (bias is not None and bias.dtype != torch.float32)):
        raise KernelError("causal_conv: inputs, taps, bias and state are float32")
    if w.shape[0] != C or state.shape[1:] != (max(taps - 1, 0), C) or (bias is not None and bias.shape != (C,)):
        raise KernelError("causal_conv: shapes do not fit")
    if activation not in (None, "silu"):
        raise KernelError(f"causal_conv: activation `{activation}` is not known (silu)")
    out = torch.empty((T, C + dup_n), dtype=out_dtype, device=u.device)
    lib = library("sequence_ops.cu")
    with region("causal_conv", T * C * 4 + _nb(out)):
        check(lib.aie_causal_conv(_p(u), c_int(u.stride(0)), _p(w), _p(bias), _p(state), _p(out), c_int(dtype_code(out)),
                                  c_int(out.stride(0)), _p(ctx.q_start), _p(ctx.q_len), _p(ctx.slots), _p(ctx.token_req),
                                  c_int(T), c_int(C), c_int(taps), c_int(1 if residual else 0),
                                  c_int(1 if activation == "silu" else 0), c_int(dup_from), c_int(dup_n),
                                  c_int(state.shape[0]), _p(ctx.err), _stream()), "causal_conv")
    return out


def gate_group_norm(y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, parts: int, eps: float,
                    out_dtype: torch.dtype) -> torch.Tensor:
    """g = y * silu(z); each of `parts` equal parts of a row is divided by its own root mean square; times weight.
    y [T, W] float32; z a float32 view [T, W] with any row stride; weight [W] float32."""
    _dev(y, weight)
    T, W = y.shape
    if (y.dtype != torch.float32 or z.dtype != torch.float32 or z.shape != (T, W) or z.stride(1) != 1
            or weight.dtype != torch.float32 or weight.shape != (W,) or parts < 1 or W % parts):
        raise KernelError("gate_group_norm: shapes or dtypes do not fit")
    out = torch.empty((T, W), dtype=out_dtype, device=y.device)
    lib = library("sequence_ops.cu")
    with region("gate_group_norm", 2 * _nb(y) + _nb(out)):
        check(lib.aie_gate_group_norm(_p(y), _p(z), c_int(z.stride(0)), _p(weight), _p(out), c_int(dtype_code(out)),
                                      c_int(T), c_int(W), c_int(parts), c_float(eps), _stream()), "gate_group_norm")
    return out


def route_topk(logits: torch.Tensor, correction: Optional[torch.Tensor], groups: int, keep: int, top: int,
               score: str = "softmax", group_top: int = 1, normalise: bool = False, weight_scale: float = 1.0):
    """A router's choice per token from float32 logits [T, E] (a view whose rows may be wider apart; overwritten by their softmax): the `top` outputs
    with the largest softmax + correction among the members of the `keep` groups (of `groups` equal groups of
    neighbours) whose best member is largest.  Returns (ids int32 [T, top], weights float32 [T, top]: the
    chosen outputs' softmax).  score "sigmoid": every output's score is its own sigmoid instead.  group_top n: a group
    counts as the sum of its n largest members.  normalise: the chosen weights are divided by their sum (+ 1e-20);
    weight_scale multiplies them."""
    _dev(correction)
    T, E = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or (correction is not None and (correction.dtype != torch.float32 or
                                                                    correction.shape != (E,))):
        raise KernelError("route_topk: float32 logits and correction")
    ids = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    scratch = torch.empty((T, E), dtype=torch.float32, device=logits.device)
    lib = library("sequence_ops.cu")
    with region("route_topk", 3 * _nb(scratch)):
        check(lib.aie_route_topk(_p(logits), c_int(logits.stride(0)), _p(scratch), _p(correction), c_int(T), c_int(E), c_int(groups), c_int(keep),
                                 c_int(top), _p(ids), _p(weights), c_int(1 if score == "sigmoid" else 0), c_int(group_top),
                                 c_int(1 if normalise else 0), c_float(weight_scale), _stream()), "route_topk")
    return ids, weights


def expert_combine_weighted(y: torch.Tensor, pair_row: torch.Tensor, weights: torch.Tensor, h: torch.Tensor,
                            shared: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = sum_s weights[t, s] * y[pair_row[t top + s]] (+ shared[t]), a pair marked -2 standing for h[t] itself;
    float32 [T, D].  y [rows, D] float32; weights [T, top] float32; h [T, D] in the compute dtype; shared float32
    [T, D] or [parts, T, D] (the unjoined parts of a split product, added here)."""
    _dev(y, pair_row, weights, h, shared)
    if shared is not None and (shared.dtype != torch.float32 or shared.shape[-2:] != h.shape):
        raise KernelError("expert_combine_weighted: the shared output is float32 [T, D] or [parts, T, D]")
    sh_parts, sh_stride = (0, 0) if shared is None else ((shared.shape[0], shared.stride(0)) if shared.dim() == 3 else (1, 0))
    T, top = weights.shape
    D = h.shape[1]
    if y.dtype != torch.float32 or weights.dtype != torch.float32 or y.shape[1] != D or pair_row.numel() != T * top:
        raise KernelError("expert_combine_weighted: shapes or dtypes do not fit")
    out = torch.empty((T, D), dtype=torch.float32, device=y.device)
    lib = library("sequence_ops.cu")
    with region("expert_combine", (top + 2) * T * D * 4):
        check(lib.aie_expert_combine_weighted(_p(y), _p(pair_row), _p(weights), c_int(top), _p(h), c_int(dtype_code(h)),
                                              _p(out), c_int(T), c_int(D), _p(shared), c_int(sh_parts),
                                              c_longlong(sh_stride), _stream()), "expert_combine_weighted")
    return out


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x <- cap * tanh(x / cap) in place (float32)."""
    _dev(x)
    if x.dtype != torch.float32:
        raise KernelError("softcap: float32 logits")
    lib = library("elementwise.cu")
    with region("softcap", 2 * _nb(x)):
        check(lib.aie_softcap(_p(x), c_longlong(x.numel()), c_float(cap), _stream()), "softcap")
    return x


def scaled_sum(a: torch.Tensor, sa: float, b: torch.Tensor, sb: float) -> torch.Tensor:
    """sa * a + sb * b in float32; a and b [T, D], or [parts, T, D] (the parts of a split product are added first)."""
    _dev(a, b)
    if a.dtype != torch.float32 or b.dtype != torch.float32 or a.shape[-2:] != b.shape[-2:]:
        raise KernelError("scaled_sum: float32 operands of one shape")
    out = torch.empty(a.shape[-2:], dtype=torch.float32, device=a.device)
    lib = library("elementwise.cu")
    with region("scaled_sum", _nb(a, b, out)):
        check(lib.aie_scaled_sum(_p(a), c_int(a.shape[0] if a.dim() == 3 else 1), c_float(sa), _p(b),
                                 c_int(b.shape[0] if b.dim() == 3 else 1), c_float(sb), _p(out),
                                 c_longlong(out.numel()), _stream()), "scaled_sum")
    return out


# ---------------------------------------------------------------------------
# parts of layers with a fixed position vector, a feed-forward without a gate, a stream mixed with an earlier one,
# attention with a sink behind a window, the delta rule
PLAIN_ACTIVATIONS = {"silu": 0, "relu": 1, "gelu_tanh": 2, "relu_squared": 3}


def activate(z: torch.Tensor, activation: str, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """act(z) element by element (silu, relu, gelu_tanh, relu_squared), computed in float32."""
    _dev(z)
    out = torch.empty(z.shape, dtype=out_dtype or z.dtype, device=z.device)
    lib = library("elementwise.cu")
    with region("activate", _nb(z, out)):
        check(lib.aie_activate(_p(z), c_int(dtype_code(z)), _p(out), c_int(dtype_code(out)), c_longlong(z.numel()),
                               c_int(PLAIN_ACTIVATIONS[activation]), _stream()), "activate")
    return out


def linear_activated(x: torch.Tensor, w: torch.Tensor, activation: str, err: Optional[torch.Tensor] = None) -> torch.Tensor:
    """act(x . w^T) in x's dtype for a feed-forward without a gate."""
    return activate(linear(x, w, x.dtype, err), activation)


def scale_(x: torch.Tensor, s: float) -> torch.Tensor:
    """x <- x * s in place (float32)."""
    _dev(x)
    if x.dtype != torch.float32:
        raise KernelError("scale_: float32 operand")
    lib = library("elementwise.cu")
    with region("scale", 2 * _nb(x)):
        check(lib.aie_scale(_p(x), c_longlong(x.numel()), c_float(s), _stream()), "scale")
    return x


def add_sinusoid(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> None:
    """x[t, 2i] += sin(p_t f_i), x[t, 2i + 1] += cos(p_t f_i) in place; x [T, D] float32, inv_freq [ceil(D / 2)]."""
    _dev(x, positions, inv_freq)
    T, D = x.shape
    if x.dtype != torch.float32 or inv_freq.dtype != torch.float32 or inv_freq.shape[0] != (D + 1) // 2:
        raise KernelError("add_sinusoid: a float32 stream and one frequency per pair of columns")
    lib = library("elementwise.cu")
    with region("add_sinusoid", 2 * _nb(x)):
        check(lib.aie_add_sinusoid(_p(x), _p(positions), _p(inv_freq), c_int(T), c_int(D), _stream()), "add_sinusoid")


def join_streams(x: torch.Tensor, delta: Optional[torch.Tensor], y: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """[x (+ delta, or the sum of its parts [parts, T, D]) | y] as rows [T, 2D] of `out_dtype`; x, y float32."""
    _dev(x, delta, y)
    T, D = x.shape
    if x.dtype != torch.float32 or y.dtype != torch.float32 or y.shape != x.shape:
        raise KernelError("join_streams: two float32 streams of one shape")
    parts, stride = 0, 0
    if delta is not None:
        parts, stride = (delta.shape[0], delta.stride(0)) if delta.dim() == 3 else (1, 0)
        if delta.shape[-2:] != x.shape:
            raise KernelError("join_streams: delta differs in shape from x")
    out = torch.empty((T, 2 * D), dtype=out_dtype, device=x.device)
    lib = library("elementwise.cu")
    with region("join_streams", _nb(x, delta, y, out)):
        check(lib.aie_join_streams(_p(x), _p(delta), c_int(dtype_code(delta) if delta is not None else 0), c_int(parts),
                                   c_longlong(stride), _p(y), _p(out), c_int(dtype_code(out)), c_int(T), c_int(D),
                                   _stream()), "join_streams")
    return out


def sink_attn_prepare(proj: torch.Tensor, bias: Optional[torch.Tensor], pages: torch.Tensor, ctx,
                      block_table: torch.Tensor, H: int, G: int, d: int, e: int, eps: float, write: bool = True):
    """From a step's fused projection [q (H d) | k (G d) | v (G e) | gate logits (H)] (float32 [T, >= that]):
    (q [T, H, d] in the cache's dtype with its bias added, gate [T, H] float32 = sigmoid of the logits); with
    `write`, each token's key (with bias) and its value (with bias, every head divided by its root mean square)
    go into its cache row [k | v].  pages [num_pages, G, P, d + e]; bias float32 [H d + G d + G e] or None."""
    _dev(proj, bias, pages, block_table)
    T, ld = proj.shape
    if (proj.dtype != torch.float32 or ld < H * d + G * (d + e) + H or pages.shape[1] != G or pages.shape[3] != d + e
            or (bias is not None and (bias.dtype != torch.float32 or bias.numel() != H * d + G * (d + e)))):
        raise KernelError("sink_attn_prepare: shapes or dtypes do not fit")
    q = torch.empty((T, H, d), dtype=pages.dtype, device=proj.device)
    gate = torch.empty((T, H), dtype=torch.float32, device=proj.device)
    lib = library("sink_attention.cu")
    with region("sink_attn_prepare", _nb(proj, q) + T * G * (d + e) * pages.element_size()):
        check(lib.aie_sink_attn_prepare(_p(proj), c_int(ld), _p(bias), _p(q), c_int(dtype_code(q)), _p(pages),
                                        c_int(dtype_code(pages)), _p(gate), _p(ctx.positions), _p(ctx.token_req),
                                        _p(block_table), c_int(block_table.shape[1]), c_int(pages.shape[0]),
                                        c_int(pages.shape[2]), c_int(T), c_int(H), c_int(G), c_int(d), c_int(e),
                                        c_float(eps), c_int(1 if write else 0), _p(ctx.err), _stream()),
              "sink_attn_prepare")
    return q, gate


SINK_FAST_SIZES = (32, 64, 128)      # key and value sizes of the tensor-core kernels of sink_attention


def sink_attention(q: torch.Tensor, pages: torch.Tensor, gate: Optional[torch.Tensor], temp: Optional[torch.Tensor],
                   slope: Optional[torch.Tensor], sink: Optional[torch.Tensor], ctx, work, block_table: torch.Tensor,
                   e: int, scale: float, window: int, keep_first: int) -> torch.Tensor:
    """Attention of a step's query tokens over cache rows [k (d) | v (e)]:
    s(i, j) = (q_i . k_j) * scale * temp[h] - slope[h] * (i - j) over the keys j <= i with i - j < window or
    j < keep_first (window 0: all); softmax whose denominator also holds exp(sink[h]); times gate[i, h].
    q [T, H, d]; gate [T, H], temp, slope, sink [H] float32 or None.  Returns [T, H, e] in q's dtype.
    bfloat16 with key and value sizes of 32, 64 or 128: lone tokens take the split-KV kernel, portions of prompts
    the tiled tensor-core kernel (`work`: the attention work lists); everything else takes the plain kernel."""
    _dev(q, pages, gate, temp, slope, sink, block_table)
    T, H, d = q.shape
    G = pages.shape[1]
    if pages.shape[3] != d + e or H % G or pages.dtype != q.dtype:
        raise KernelError("sink_attention: shapes or dtypes do not fit")
    out = torch.empty((T, H, e), dtype=q.dtype, device=q.device)
    cost = (0.0, 0.0)
    if _profiling() and hasattr(ctx, "h_q_len"):
        ql, cl = ctx.h_q_len.astype(float), ctx.h_ctx_len.astype(float)
        seen = cl + (ql + 1) / 2
        if window > 0:
            seen = seen.clip(max=float(window + keep_first))
        rows = (cl + ql).clip(max=float(window + keep_first) + ql) if window > 0 else cl + ql
        cost = (float(rows.sum()) * G * (d + e) * pages.element_size() + _nb(q, out),
                2.0 * float((ql * seen).sum()) * H * (d + e))
    if q.dtype == torch.bfloat16 and d in SINK_FAST_SIZES and e in SINK_FAST_SIZES:
        fast = library("sink_attention_tc.cu")
        common = (_p(block_table), c_int(block_table.shape[1]), c_int(pages.shape[0]), c_int(pages.shape[2]),
                  c_int(H), c_int(G), c_int(d), c_int(e), c_int(window), c_int(keep_first), c_float(scale))
        if work.n_decode:
            n = work.n_decode
            keys = work.max_decode_len if window <= 0 else min(window + keep_first, work.max_decode_len)
            S = min(decode_splits(n, G, H // G, keys), 64)
            part_o = part_lse = None
            if S > 1:
                part_o = torch.empty((n, H, S, e), dtype=torch.float32, device=q.device)
                part_lse = torch.empty((n, H, S), dtype=torch.float32, device=q.device)
            share = float(n) / T
            with region("sink_attention_decode", cost[0] * share, cost[1] * share):
                check(fast.aie_sink_attention_decode(_p(q), _p(pages), _p(out), _p(part_o), _p(part_lse), _p(gate),
                                                     _p(temp), _p(slope), _p(sink), _p(work.decode_tokens), c_int(n),
                                                     _p(ctx.positions), _p(ctx.token_req), *common, c_int(S),
                                                     _p(ctx.err), _stream()), "sink_attention_decode")
        if work.n_decode < ctx.R:
            tiles = work.prefill_tiles
            share = 1.0 - float(work.n_decode) / T
            with region("sink_attention_prefill", cost[0] * share, cost[1] * share):
                check(fast.aie_sink_attention_prefill(_p(q), _p(pages), _p(out), _p(gate), _p(temp), _p(slope), _p(sink),
                                                      _p(tiles), c_int(tiles.shape[0]), _p(ctx.q_start), _p(ctx.q_len),
                                                      _p(ctx.ctx_len), *common, _p(ctx.err), _stream()),
                      "sink_attention_prefill")
        return out
    lib = library("sink_attention.cu")
    with region("sink_attention_plain", *cost):
        check(lib.aie_sink_attention_plain(_p(q), _p(pages), _p(out), c_int(dtype_code(q)), _p(gate), _p(temp), _p(slope),
                                           _p(sink), _p(ctx.positions), _p(ctx.token_req), _p(block_table),
                                           c_int(block_table.shape[1]), c_int(pages.shape[0]), c_int(pages.shape[2]),
                                           c_int(T), c_int(H), c_int(G), c_int(d), c_int(e), c_int(window),
                                           c_int(keep_first), c_float(scale), _p(None), _p(ctx.err), _stream()),
              "sink_attention_plain")
    return out


DELTA_MIN_TOKENS = 32    # portions from this length on take the chunked delta-rule kernel (bfloat16 mode)
DELTA_CHUNK = 64         # its chunk


def delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, b_raw: torch.Tensor, a_raw: torch.Tensor,
               a_log: torch.Tensor, dt_bias: torch.Tensor, q_scale: float, unit_eps: float, state: torch.Tensor, ctx,
               H: int, G: int, d: int, e: int, chunked: bool = False) -> torch.Tensor:
    """The gated delta rule over a step's tokens, the state [max_seqs, H, d, e] float32 read and left in each
    request's slot:  q, k made unit vectors per head (x / sqrt(|x|^2 + unit_eps), q times q_scale);
    beta = sigmoid(b_raw); g = exp(-exp(a_log) softplus(a_raw + dt_bias));  S <- g S;  u = beta (v - S^T k);
    S <- S + k u^T;  o = S^T q.  q, k [T, G d] and v [T, H e] are float32 views with one row stride; b_raw, a_raw
    [T, H] float32 views (rows any stride); head h reads q/k head h / (H / G).  chunked: portions of
    DELTA_MIN_TOKENS tokens or more take the chunked tensor-core kernel, whose products see 16 bits of mantissa
    (a state of up to 128 rows); everything else, and all of a float32 engine, goes token by token in float32.
    Returns o [T, H, e] float32."""
    _dev(a_log, dt_bias, state)
    T, ld = q.shape[0], q.stride(0)
    if (q.dtype != torch.float32 or k.dtype != torch.float32 or v.dtype != torch.float32 or k.stride(0) != ld
            or v.stride(0) != ld or q.stride(1) != 1 or k.stride(1) != 1 or v.stride(1) != 1
            or b_raw.dtype != torch.float32 or a_raw.dtype != torch.float32 or b_raw.stride(1) != 1 or a_raw.stride(1) != 1
            or state.shape[1:] != (H, d, e) or state.dtype != torch.float32 or H % G or d > 256):
        raise KernelError("delta_rule: shapes or dtypes do not fit")
    out = torch.empty((T, H, e), dtype=torch.float32, device=q.device)
    max_len = 0
    if (chunked and d <= 128 and ctx.max_q_len >= DELTA_MIN_TOKENS
            and not os.environ.get("AI_ENGINE_B200_NO_CHUNKED_SCAN")):      # the switch is for measurement
        lib = library("delta_rule_chunked.cu")
        Q = DELTA_CHUNK
        with region("delta_rule_chunked", _nb(out) + T * (2 * G * d + H * e) * 4 + 2 * ctx.R * H * d * e * 4,
                    2.0 * T * H * (Q * d + Q * e + 3 * d * e)):
            check(lib.aie_delta_rule_chunked(_p(q), _p(k), _p(v), c_int(ld), _p(b_raw), c_int(b_raw.stride(0)), _p(a_raw),
                                             c_int(a_raw.stride(0)), _p(a_log), _p(dt_bias), c_float(q_scale),
                                             c_float(unit_eps), _p(state), _p(out), _p(ctx.q_start), _p(ctx.q_len),
                                             _p(ctx.slots), _p(ctx.live), c_int(ctx.R), c_int(H), c_int(G), c_int(d),
                                             c_int(e), c_int(state.shape[0]), c_int(DELTA_MIN_TOKENS), _p(ctx.err),
                                             _stream()), "delta_rule_chunked")
        if int(ctx.h_q_len.min()) >= DELTA_MIN_TOKENS:
            return out
        max_len = DELTA_MIN_TOKENS - 1              # the shorter portions and single tokens of the same step
    lib = library("delta_rule.cu")
    with region("delta_rule", _nb(out) + T * (2 * G * d + H * e) * 4 + 2 * ctx.R * H * d * e * 4, 6.0 * T * H * d * e):
        check(lib.aie_delta_rule(_p(q), _p(k), _p(v), c_int(ld), _p(b_raw), c_int(b_raw.stride(0)), _p(a_raw),
                                 c_int(a_raw.stride(0)), _p(a_log), _p(dt_bias), c_float(q_scale), c_float(unit_eps),
                                 _p(state), _p(out), _p(ctx.q_start), _p(ctx.q_len), _p(ctx.slots), _p(ctx.live),
                                 c_int(ctx.R), c_int(H), c_int(G), c_int(d), c_int(e), c_int(state.shape[0]),
                                 c_int(max_len), _p(ctx.err), _stream()), "delta_rule")
    return out


# ---------------------------------------------------------------------------
# parts of layers whose sublayers run side by side behind a norm without statistics, attention with normed and
# rotated heads whose values are mixed across layers, gates on attention outputs
def add_dyt(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, bias: torch.Tensor, alpha: torch.Tensor,
            out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None, write_back: bool = True) -> torch.Tensor:
    """s = x (+ delta, or the sum of its parts [parts, T, D]); out = tanh(alpha s) * weight + bias, element by element
    in float32.  x is the float32 residual stream and receives s when `write_back`; `rows` picks rows; weight, bias
    [D] and alpha [1] are float32 on the device."""
    _dev(x, delta, weight, bias, alpha, rows)
    D = x.shape[-1]
    if x.dtype != torch.float32 or any(t.dtype != torch.float32 for t in (weight, bias, alpha)):
        raise KernelError("add_dyt: the stream and the norm's tensors are float32")
    if weight.shape != (D,) or bias.shape != (D,) or alpha.numel() != 1:
        raise KernelError("add_dyt: weight and bias [D], alpha one number")
    parts, stride = 0, 0
    if delta is not None:
        parts, stride = (delta.shape[0], delta.stride(0)) if delta.dim() == 3 else (1, 0)
        if delta.shape[-2:] != x.shape:
            raise KernelError("add_dyt: delta differs in shape from x")
    n = x.shape[0] if rows is None else rows.shape[0]
    out = torch.empty((n, D), dtype=out_dtype, device=x.device)
    stored = write_back and rows is None and delta is not None
    lib = library("elementwise.cu")
    with region("add_dyt", n * D * 4 * (2 if stored else 1) + (_nb(delta) if rows is None else 0) + _nb(out)):
        check(lib.aie_add_dyt(_p(x), _p(delta), c_int(dtype_code(delta) if delta is not None else 0), c_int(parts),
                              c_longlong(stride), _p(weight), _p(bias), _p(alpha), _p(out), c_int(dtype_code(out)), _p(rows),
                              c_int(n), c_int(D), c_int(1 if stored else 0), _stream()), "add_dyt")
    return out


def sigmoid_gate_mul_(a: torch.Tensor, g: torch.Tensor, group: int = 1) -> torch.Tensor:
    """a[t, n] <- a[t, n] * sigmoid(g[t, n / group]) in place.  a [T, N] (float32 or bfloat16); g a float32 view
    [T, N / group] with any row stride.  group 1: a gate per element; group = a head's width: a gate per head."""
    _dev(a)
    T, N = a.shape
    if g.dtype != torch.float32 or g.stride(1) != 1 or N % group or g.shape != (T, N // group):
        raise KernelError("sigmoid_gate_mul: the gate's logits are a float32 view [T, N / group]")
    lib = library("elementwise.cu")
    with region("sigmoid_gate_mul", 2 * _nb(a) + T * (N // group) * 4):
        check(lib.aie_sigmoid_gate_mul(_p(a), c_int(dtype_code(a)), _p(g), c_int(g.stride(0)), c_int(T), c_int(N), c_int(group),
                                       _stream()), "sigmoid_gate_mul")
    return a


def add_bias_(y: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """y[..., n] += bias[n] in place; y float32 [T, N], or [parts, T, N] (the bias joins the first part)."""
    _dev(y, bias)
    N = y.shape[-1]
    if y.dtype != torch.float32 or bias.dtype != torch.float32 or bias.shape != (N,):
        raise KernelError("add_bias: float32 operands, one bias per column")
    first = y[0] if y.dim() == 3 else y
    lib = library("elementwise.cu")
    with region("add_bias", 2 * _nb(first)):
        check(lib.aie_add_bias(_p(first), _p(bias), c_int(first.shape[0]), c_int(N), _stream()), "add_bias")
    return y


def _parts_of(t: Optional[torch.Tensor], shape):
    if t is None:
        return 0, 0
    if t.dtype != torch.float32 or t.shape[-2:] != shape:
        raise KernelError("a branch output is float32 [T, D] or [parts, T, D]")
    return (t.shape[0], t.stride(0)) if t.dim() == 3 else (1, 0)


def parallel_residual(x: torch.Tensor, a: torch.Tensor, b: Optional[torch.Tensor], mult: float,
                      history: Optional[torch.Tensor] = None, coef: Optional[torch.Tensor] = None, depth: int = 0,
                      norm_ahead=None, out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """X = x + mult * (a + b) for two branches that read the same input (float32 [T, D] or the unjoined parts
    [parts, T, D] of a split product; b may be None).  With `coef` (float32 [>= depth + 1]) and `history`
    [levels, T, D]: history[depth] = X and x = sum_{j <= depth} coef[j] history[j]; otherwise x = X.  In place.
    norm_ahead = (weight, bias, alpha) of a norm without statistics: also returns tanh(alpha x) weight + bias of the
    new stream in `out_dtype`, so that whoever norms the stream next need not read it again."""
    _dev(x, a, b, history, coef)
    if x.dtype != torch.float32:
        raise KernelError("parallel_residual: the stream is float32")
    pa, sa = _parts_of(a, x.shape)
    pb, sb = _parts_of(b, x.shape)
    if coef is not None and (history is None or history.shape[1:] != x.shape or depth >= history.shape[0]
                             or coef.shape[0] < depth + 1 or coef.dtype != torch.float32):
        raise KernelError("parallel_residual: history and weights do not fit")
    normed = None
    w = nb = al = None
    if norm_ahead is not None:
        w, nb, al = norm_ahead
        normed = torch.empty(x.shape, dtype=out_dtype or torch.float32, device=x.device)
    lib = library("sequence_ops.cu")
    with region("parallel_residual", ((depth + 3) if coef is not None else 2) * _nb(x) + _nb(a, b, normed)):
        check(lib.aie_depth_average2(_p(x), _p(a), c_int(pa), c_longlong(sa), _p(b), c_int(pb), c_longlong(sb), c_float(mult),
                                     _p(history), _p(coef), c_int(depth), c_longlong(x.numel()), _p(w), _p(nb), _p(al),
                                     _p(normed), c_int(dtype_code(normed) if normed is not None else 0),
                                     c_int(x.shape[-1]), _stream()), "parallel_residual")
    return normed


def normed_attn_prepare(proj: torch.Tensor, bias: Optional[torch.Tensor], q_weight: Optional[torch.Tensor],
                        k_weight: Optional[torch.Tensor], eps: float, inv_freq: Optional[torch.Tensor], rot_dims: int,
                        halves: bool, pages: torch.Tensor, ctx, block_table: torch.Tensor, H: int, G: int, d: int, e: int,
                        mix_from: Optional[torch.Tensor] = None, mix_lambda: Optional[torch.Tensor] = None,
                        keep_values: bool = False, write: bool = True):
    """From a step's fused projection whose first columns are [q (H d) | k (G d) | v (G e)] (float32 [T, >= that]):
    biases added; all of q divided by its root mean square over the H d elements, times q_weight (k likewise; None: no
    norm); the first rot_dims elements of every head of q and k rotated by the token's position (pairs of neighbours,
    or halves); v <- (1 - lambda) v + lambda mix_from[t] when mix_from [T, G e] float32 is given (lambda one float on
    the device).  q [T, H, d] in the cache's dtype is returned; with `write`, the token's cache row [k | v] is
    written.  keep_values: the values as they are cached are also returned in float32 [T, G e].
    pages [num_pages, G, P, d + e]."""
    _dev(proj, bias, q_weight, k_weight, inv_freq, pages, block_table, mix_from, mix_lambda)
    T, ld = proj.shape
    n = H * d + G * (d + e)
    if (proj.dtype != torch.float32 or ld < n or pages.shape[1] != G or pages.shape[3] != d + e
            or (bias is not None and (bias.dtype != torch.float32 or bias.numel() != n))
            or (q_weight is not None and (k_weight is None or q_weight.numel() != H * d or k_weight.numel() != G * d))
            or (mix_from is not None and (mix_from.dtype != torch.float32 or mix_from.shape != (T, G * e) or mix_lambda is None))):
        raise KernelError("normed_attn_prepare: shapes or dtypes do not fit")
    q = torch.empty((T, H, d), dtype=pages.dtype, device=proj.device)
    kept = torch.empty((T, G * e), dtype=torch.float32, device=proj.device) if keep_values else None
    lib = library("sink_attention.cu")
    with region("normed_attn_prepare", T * n * 4 + _nb(q, kept, mix_from) + T * G * (d + e) * pages.element_size()):
        check(lib.aie_normed_attn_prepare(_p(proj), c_int(ld), _p(bias), _p(q_weight), _p(k_weight), c_float(eps),
                                          _p(inv_freq), c_int(rot_dims), c_int(1 if halves else 0), _p(mix_from),
                                          _p(mix_lambda), _p(kept), _p(q), _p(pages), c_int(dtype_code(pages)),
                                          _p(ctx.positions), _p(ctx.token_req), _p(block_table), c_int(block_table.shape[1]),
                                          c_int(pages.shape[0]), c_int(pages.shape[2]), c_int(T), c_int(H), c_int(G), c_int(d),
                                          c_int(e), c_int(1 if write else 0), _p(ctx.err), _stream()), "normed_attn_prepare")
    return q, kept


def slice_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """out[t] = x[t] / sqrt(mean(x[t]^2) + eps) * weight for a float32 view x [T, n] with any row stride (a slice of
    a wider projection); weight [n] float32."""
    _dev(weight)
    T, n = x.shape
    if x.dtype != torch.float32 or x.stride(1) != 1 or weight.dtype != torch.float32 or weight.shape != (n,):
        raise KernelError("slice_rmsnorm: a float32 view and one float32 weight per column")
    out = torch.empty((T, n), dtype=out_dtype, device=x.device)
    lib = library("sequence_ops.cu")
    with region("slice_rmsnorm", T * n * 4 + _nb(out)):
        check(lib.aie_slice_rmsnorm(_p(x), c_int(x.stride(0)), _p(weight), _p(out), c_int(dtype_code(out)), c_int(T), c_int(n),
                                    c_float(eps), _stream()), "slice_rmsnorm")
    return out
