// Memory-bound row kernels: embedding gather, residual add fused with RMSNorm,
// SiLU(gate) * up, dtype casts.  The residual stream is float32 in both compute
// dtypes; statistics and scaling are float32.
#include "common.cuh"

// ---------------------------------------------------------------------------
// x[t, :] = float(E[ids[t], :])        (crates/ai-engine-runtime/src/arch/embedding.rs:14-20)
// ---------------------------------------------------------------------------
template <typename W>
__global__ void embed_gather_kernel(const int* __restrict__ ids, const W* __restrict__ table,
                                    float* __restrict__ x, int D, int vocab, unsigned* err) {
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(err, AIE_DEV_TOKEN_OOB);
        for (int i = threadIdx.x; i < D; i += blockDim.x) x[(size_t)t * D + i] = 0.f;
        return;
    }
    const W* row = table + (size_t)id * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) x[(size_t)t * D + i] = to_f32<W>(row[i]);
}

// bf16 table, D a multiple of 8: 16-byte loads, two float4 stores per thread
__global__ void embed_gather_vec_kernel(const int* __restrict__ ids, const bf16* __restrict__ table,
                                        float* __restrict__ x, int D, int vocab, unsigned* err) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    if (!ok && threadIdx.x == 0) atomicOr(err, AIE_DEV_TOKEN_OOB);
    const uint4* row = reinterpret_cast<const uint4*>(table + (size_t)(ok ? id : 0) * D);
    float4* dst = reinterpret_cast<float4*>(x + (size_t)t * D);
    for (int i = threadIdx.x; i < D / 8; i += blockDim.x) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
        if (ok) {
            const uint4 raw = row[i];
            const bf16* e = reinterpret_cast<const bf16*>(&raw);
            a = make_float4(__bfloat162float(e[0]), __bfloat162float(e[1]), __bfloat162float(e[2]), __bfloat162float(e[3]));
            b = make_float4(__bfloat162float(e[4]), __bfloat162float(e[5]), __bfloat162float(e[6]), __bfloat162float(e[7]));
        }
        dst[2 * i] = a;
        dst[2 * i + 1] = b;
    }
}

extern "C" int aie_embed_gather(const int* ids, const void* table, int table_dtype, float* x,
                                int T, int D, int vocab, unsigned* err, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (table_dtype == AIE_F32)
        embed_gather_kernel<float><<<T, 256, 0, stream>>>(ids, (const float*)table, x, D, vocab, err);
    else if (table_dtype == AIE_BF16 && D % 8 == 0)
        launch_pdl(embed_gather_vec_kernel, dim3(T), dim3(D >= 4096 ? 512 : 128), 0, stream, ids, (const bf16*)table, x, D, vocab, err);
    else if (table_dtype == AIE_BF16)
        embed_gather_kernel<bf16><<<T, 256, 0, stream>>>(ids, (const bf16*)table, x, D, vocab, err);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}

// ids[t] = last[src[t]] where src[t] >= 0: a token that the previous step sampled and that the host
// has not read yet is taken from the device buffer the sampler left it in (no counterpart in the
// reference, whose loop reads every token back before the next step: crates/ai-engine-candle/src/paged/engine.rs:150-170)
__global__ void take_sampled_ids_kernel(int* __restrict__ ids, const int* __restrict__ src,
                                        const int* __restrict__ last, int T, int n_last, unsigned* err) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    const int k = src[t];
    if (k < 0) return;
    if (k >= n_last) {
        atomicOr(err, AIE_DEV_TOKEN_OOB);
        return;
    }
    ids[t] = last[k];
}

extern "C" int aie_take_sampled_ids(int* ids, const int* src, const int* last, int T, int n_last, unsigned* err,
                                    cudaStream_t stream) {
    if (T <= 0) return 0;
    take_sampled_ids_kernel<<<(T + 127) / 128, 128, 0, stream>>>(ids, src, last, T, n_last, err);
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// Residual add + RMSNorm (crates/ai-engine-runtime/src/arch/rmsnorm.rs:29-42):
//   s = x[row] (+ delta[row], or the sum of `parts` deltas `part_stride` elements apart);  ms = mean(s^2);  r = 1/sqrt(ms + eps);
//   out[i] = (s * r) * w          with eps inside the root and the weight last.
// `rows` (optional) picks input rows; `write_back` stores s into x.
// ---------------------------------------------------------------------------
template <typename A, typename W, typename O>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const A* __restrict__ delta,
                                   const W* __restrict__ w, O* __restrict__ out,
                                   const int* __restrict__ rows, int D, float eps, int write_back,
                                   int parts, size_t part_stride) {
    extern __shared__ float srow[];   // D floats + 32
    float* red = srow + D;
    const int o = blockIdx.x;
    const size_t r = rows ? (size_t)rows[o] : (size_t)o;
    float* xr = x + r * D;
    float ss = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float s = xr[i];
        if (delta)
            for (int p = 0; p < parts; ++p) s += to_f32<A>(delta[p * part_stride + r * D + i]);
        srow[i] = s;
        ss += s * s;
    }
    ss = block_sum(ss, red);
    const float ms = ss / (float)D;
    const float rinv = 1.0f / sqrtf(ms + eps);
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float s = srow[i];
        if (write_back) xr[i] = s;
        out[(size_t)o * D + i] = from_f32<O>((s * rinv) * to_f32<W>(w[i]));
    }
}

// Fast path: D a multiple of 4 and at most 4 * 1024: the whole row lives in registers
// (one float4 per thread), read once and written once.  Same arithmetic and the same
// block reduction as the general kernel.
template <typename A, typename W, typename O>
__global__ void __launch_bounds__(1024)
add_rmsnorm_row_kernel(float* __restrict__ x, const A* __restrict__ delta, const W* __restrict__ w,
                       O* __restrict__ out, const int* __restrict__ rows, int D, float eps, int write_back,
                       int parts, size_t part_stride) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const int o = blockIdx.x;
    const size_t r = rows ? (size_t)rows[o] : (size_t)o;
    const int i = threadIdx.x;
    const bool on = i < D / 4;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    if (on) {
        s = reinterpret_cast<const float4*>(x + r * D)[i];
        if (delta) {
            // parts of a split product, added in order; four loads are in flight at a time
            const A* dp = delta + r * D + 4 * i;
            int p = 0;
            for (; p + 4 <= parts; p += 4) {
                float4 dl[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) dl[u] = load4<A>(dp + (size_t)(p + u) * part_stride);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    s.x += dl[u].x;
                    s.y += dl[u].y;
                    s.z += dl[u].z;
                    s.w += dl[u].w;
                }
            }
            for (; p < parts; ++p) {
                const float4 dl = load4<A>(dp + (size_t)p * part_stride);
                s.x += dl.x;
                s.y += dl.y;
                s.z += dl.z;
                s.w += dl.w;
            }
        }
    }
    float ss = s.x * s.x;
    ss += s.y * s.y;
    ss += s.z * s.z;
    ss += s.w * s.w;
    ss = block_sum(ss, red);
    const float rinv = 1.0f / sqrtf(ss / (float)D + eps);
    if (on) {
        if (write_back) reinterpret_cast<float4*>(x + r * D)[i] = s;
        const float4 wv = load4<W>(w + 4 * i);
        store4<O>(out + (size_t)o * D + 4 * i,
                  make_float4((s.x * rinv) * wv.x, (s.y * rinv) * wv.y, (s.z * rinv) * wv.z, (s.w * rinv) * wv.w));
    }
}

// Many rows (portions of prompts, bfloat16 out): a quarter of the threads per row, four float4 each, all loads
// issued before the first use, so that eight blocks sit on an SM and keep 128 KB of loads in flight (with a
// thread per float4 two blocks of 1,024 threads fit, and the memory system idles through their reductions).
template <typename A, typename W, typename O>
__global__ void __launch_bounds__(256)
add_rmsnorm_row4_kernel(float* __restrict__ x, const A* __restrict__ delta, const W* __restrict__ w,
                        O* __restrict__ out, const int* __restrict__ rows, int D, float eps, int write_back) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const int o = blockIdx.x;
    const size_t r = rows ? (size_t)rows[o] : (size_t)o;
    const int i = threadIdx.x, nt = blockDim.x;       // D == 16 * nt
    float4 s[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) s[k] = reinterpret_cast<const float4*>(x + r * D)[i + k * nt];
    if (delta) {
        float4 dl[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) dl[k] = load4<A>(delta + r * D + 4 * (i + k * nt));
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            s[k].x += dl[k].x;
            s[k].y += dl[k].y;
            s[k].z += dl[k].z;
            s[k].w += dl[k].w;
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        ss += s[k].x * s[k].x;
        ss += s[k].y * s[k].y;
        ss += s[k].z * s[k].z;
        ss += s[k].w * s[k].w;
    }
    ss = block_sum(ss, red);
    const float rinv = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (write_back) reinterpret_cast<float4*>(x + r * D)[i + k * nt] = s[k];
        const float4 wv = load4<W>(w + 4 * (i + k * nt));
        store4<O>(out + (size_t)o * D + 4 * (i + k * nt),
                  make_float4((s[k].x * rinv) * wv.x, (s[k].y * rinv) * wv.y, (s[k].z * rinv) * wv.z, (s[k].w * rinv) * wv.w));
    }
}

template <typename A, typename W>
static int launch_rmsnorm_o(float* x, const void* delta, const void* w, void* out, int out_dtype,
                            const int* rows, int n, int D, float eps, int write_back, int parts,
                            size_t part_stride, cudaStream_t stream) {
    if (n >= 256 && parts == 1 && out_dtype == AIE_BF16 && D % 512 == 0 && D <= 4096) {
        launch_pdl(add_rmsnorm_row4_kernel<A, W, bf16>, dim3(n), dim3(D / 16), 0, stream, x, (const A*)delta, (const W*)w,
                   (bf16*)out, rows, D, eps, write_back);
        AIE_LAUNCH_CHECK();
    }
    if (D % 4 == 0 && D <= 4096) {
        const int threads = ((D / 4) + 31) / 32 * 32;
        if (out_dtype == AIE_F32)
            launch_pdl(add_rmsnorm_row_kernel<A, W, float>, dim3(n), dim3(threads), 0, stream, x, (const A*)delta, (const W*)w, (float*)out, rows, D, eps, write_back, parts, part_stride);
        else if (out_dtype == AIE_BF16)
            launch_pdl(add_rmsnorm_row_kernel<A, W, bf16>, dim3(n), dim3(threads), 0, stream, x, (const A*)delta, (const W*)w, (bf16*)out, rows, D, eps, write_back, parts, part_stride);
        else
            return AIE_BAD_ARG;
        AIE_LAUNCH_CHECK();
    }
    const size_t smem = (size_t)(D + 32) * sizeof(float);
    if (smem > 200 * 1024) return AIE_UNSUPPORTED;
    const int threads = D >= 1024 ? 512 : 256;
    if (out_dtype == AIE_F32) {
        auto k = add_rmsnorm_kernel<A, W, float>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        k<<<n, threads, smem, stream>>>(x, (const A*)delta, (const W*)w, (float*)out, rows, D, eps, write_back, parts, part_stride);
    } else if (out_dtype == AIE_BF16) {
        auto k = add_rmsnorm_kernel<A, W, bf16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        k<<<n, threads, smem, stream>>>(x, (const A*)delta, (const W*)w, (bf16*)out, rows, D, eps, write_back, parts, part_stride);
    } else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}

extern "C" int aie_add_rmsnorm(float* x, const void* delta, int delta_dtype, const void* w,
                               int w_dtype, void* out, int out_dtype, const int* rows, int n, int D,
                               float eps, int write_back, int parts, long long part_stride,
                               cudaStream_t stream) {
    if (n <= 0) return 0;
    if (delta == nullptr) delta_dtype = AIE_F32;
    if (parts < 1) return AIE_BAD_ARG;
#define GO(A, W) return launch_rmsnorm_o<A, W>(x, delta, w, out, out_dtype, rows, n, D, eps, write_back, parts, (size_t)part_stride, stream)
    if (delta_dtype == AIE_F32 && w_dtype == AIE_F32) GO(float, float);
    if (delta_dtype == AIE_F32 && w_dtype == AIE_BF16) GO(float, bf16);
    if (delta_dtype == AIE_BF16 && w_dtype == AIE_F32) GO(bf16, float);
    if (delta_dtype == AIE_BF16 && w_dtype == AIE_BF16) GO(bf16, bf16);
#undef GO
    return AIE_BAD_ARG;
}

// ---------------------------------------------------------------------------
// a[t, f] = silu(gate) * up   (crates/ai-engine-runtime/src/arch/ffn.rs:50-54), silu(z) = z * sigmoid(z)
// in float32.  block == 0: gu[t] = [gate (F) | up (F)].  block > 0: gu[t] is in groups of
// 2 * block columns, `block` gate columns followed by their `block` up columns.
// ---------------------------------------------------------------------------
// the activation of a gated unit: 0 silu, 1 relu, 2 gelu (tanh form)
__device__ __forceinline__ float glu_act(float g, int act) {
    if (act == 1) return fmaxf(g, 0.f);
    if (act == 2) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    return g * (1.0f / (1.0f + expf(-g)));
}

template <typename A>
__global__ void silu_mul_kernel(const A* __restrict__ gu, A* __restrict__ a, int F, int block, size_t total, int act) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const size_t t = i / F, f = i % F;
        const size_t gc = block ? (f / block) * 2 * block + f % block : f;
        const size_t uc = block ? gc + block : F + f;
        const float g = to_f32<A>(gu[t * 2 * F + gc]);
        const float u = to_f32<A>(gu[t * 2 * F + uc]);
        a[i] = from_f32<A>(glu_act(g, act) * u);
    }
}

// Eight outputs per thread with 16-byte accesses (bfloat16) when F and the group size are
// multiples of 8.
__global__ void silu_mul_vec8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ a, int F, int block,
                                     size_t total8, int act) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const unsigned F8 = (unsigned)(F / 8);
    for (; i < total8; i += stride) {
        const size_t t = i / F8;
        const unsigned f = (unsigned)(i - t * F8) * 8u;
        const unsigned gc = block ? (f / (unsigned)block) * 2u * (unsigned)block + f % (unsigned)block : f;
        const unsigned uc = block ? gc + (unsigned)block : (unsigned)F + f;
        const uint4 gr = *reinterpret_cast<const uint4*>(gu + t * 2 * F + gc);
        const uint4 ur = *reinterpret_cast<const uint4*>(gu + t * 2 * F + uc);
        const bf16* ge = reinterpret_cast<const bf16*>(&gr);
        const bf16* ue = reinterpret_cast<const bf16*>(&ur);
        uint4 o;
        bf16* oe = reinterpret_cast<bf16*>(&o);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            // sigmoid by ex2.approx and rcp.approx (relative error about 1e-6, far below the bf16 rounding of
            // the result): with expf and a division the kernel was bound by instruction issue, not by memory
            const float g = __bfloat162float(ge[j]), u = __bfloat162float(ue[j]);
            if (act) {
                oe[j] = __float2bfloat16_rn(glu_act(g, act) * u);
                continue;
            }
            float e, r;
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(g * -1.4426950408889634f));
            asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
            oe[j] = __float2bfloat16_rn((g * r) * u);
        }
        *reinterpret_cast<uint4*>(a + t * F + f) = o;
    }
}

extern "C" int aie_silu_mul(const void* gu, void* a, int dtype, int T, int F, int block, int act, cudaStream_t stream) {
    if (block < 0 || (block && F % block) || act < 0 || act > 2) return AIE_BAD_ARG;
    if (T <= 0) return 0;
    const size_t total = (size_t)T * F;
    int blocks = (int)((total + 255) / 256);
    if (blocks > aie_sm_count() * 16) blocks = aie_sm_count() * 16;
    if (dtype == AIE_BF16 && F % 8 == 0 && block % 8 == 0 && !((size_t)gu & 15) && !((size_t)a & 15)) {
        const size_t total8 = total / 8;
        int b8 = (int)((total8 + 255) / 256);
        if (b8 > aie_sm_count() * 16) b8 = aie_sm_count() * 16;
        launch_pdl(silu_mul_vec8_kernel, dim3(b8), dim3(256), 0, stream, (const bf16*)gu, (bf16*)a, F, block, total8, act);
        AIE_LAUNCH_CHECK();
    }
    if (dtype == AIE_F32)
        launch_pdl(silu_mul_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)gu, (float*)a, F, block, total, act);
    else if (dtype == AIE_BF16)
        launch_pdl(silu_mul_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)gu, (bf16*)a, F, block, total, act);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// casts between float32 and bfloat16 (a 32-bit weight under bf16 activations)
// ---------------------------------------------------------------------------
template <typename I, typename O>
__global__ void cast_kernel(const I* __restrict__ in, O* __restrict__ out, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) out[i] = from_f32<O>(to_f32<I>(in[i]));
}

extern "C" int aie_cast(const void* in, int in_dtype, void* out, int out_dtype, long long n,
                        cudaStream_t stream) {
    if (n <= 0) return 0;
    int blocks = (int)((n + 255) / 256);
    if (blocks > aie_sm_count() * 16) blocks = aie_sm_count() * 16;
    if (in_dtype == AIE_F32 && out_dtype == AIE_BF16)
        cast_kernel<float, bf16><<<blocks, 256, 0, stream>>>((const float*)in, (bf16*)out, (size_t)n);
    else if (in_dtype == AIE_BF16 && out_dtype == AIE_F32)
        cast_kernel<bf16, float><<<blocks, 256, 0, stream>>>((const bf16*)in, (float*)out, (size_t)n);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// x <- cap * tanh(x / cap), float32, in place (logits kept within +-cap)
// ---------------------------------------------------------------------------
__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap, float inv_cap) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) x[i] = cap * tanhf(x[i] * inv_cap);
}

extern "C" int aie_softcap(float* x, long long n, float cap, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!(cap > 0.f)) return AIE_BAD_ARG;
    int blocks = (int)((n + 255) / 256);
    if (blocks > aie_sm_count() * 16) blocks = aie_sm_count() * 16;
    softcap_kernel<<<blocks, 256, 0, stream>>>(x, (size_t)n, cap, 1.0f / cap);
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// out = sa * a + sb * b, float32 (two branches that read the same input, each with its weight); a and b may be
// [parts, n]: the unjoined parts of a split product, added in order before the scaling
// ---------------------------------------------------------------------------
__global__ void scaled_sum_kernel(const float* __restrict__ a, int pa, float sa, const float* __restrict__ b, int pb,
                                  float sb, float* __restrict__ out, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        float x = a[i], y = b[i];
        for (int p = 1; p < pa; ++p) x += a[(size_t)p * n + i];
        for (int p = 1; p < pb; ++p) y += b[(size_t)p * n + i];
        out[i] = fmaf(sb, y, sa * x);
    }
}

extern "C" int aie_scaled_sum(const float* a, int pa, float sa, const float* b, int pb, float sb, float* out,
                              long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (pa < 1 || pb < 1) return AIE_BAD_ARG;
    int blocks = (int)((n + 255) / 256);
    if (blocks > aie_sm_count() * 16) blocks = aie_sm_count() * 16;
    scaled_sum_kernel<<<blocks, 256, 0, stream>>>(a, pa, sa, b, pb, sb, out, (size_t)n);
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// out = act(z) element by element for a feed-forward without a gate.  act: 0 silu, 1 relu, 2 gelu (tanh form),
// 3 the square of relu.  Computed in float32, rounded once.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float plain_act(float z, int act) {
    if (act == 1) return fmaxf(z, 0.f);
    if (act == 3) {
        const float r = fmaxf(z, 0.f);
        return r * r;
    }
    if (act == 2) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    return z / (1.f + expf(-z));
}

template <typename I, typename O>
__global__ void activate_kernel(const I* __restrict__ z, O* __restrict__ out, size_t n, int act) {
    size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    const size_t stride = (size_t)gridDim.x * blockDim.x * 4;
    for (; i + 3 < n; i += stride) {
        float4 v = load4<I>(z + i);
        v.x = plain_act(v.x, act); v.y = plain_act(v.y, act); v.z = plain_act(v.z, act); v.w = plain_act(v.w, act);
        store4<O>(out + i, v);
    }
    if (i < n)                                       // the last one to three elements
        for (size_t j = i; j < n; ++j) out[j] = from_f32<O>(plain_act(to_f32<I>(z[j]), act));
}

extern "C" int aie_activate(const void* z, int in_dtype, void* out, int out_dtype, long long n, int act,
                            cudaStream_t stream) {
    if (n <= 0) return 0;
    if (act < 0 || act > 3) return AIE_BAD_ARG;
    int blocks = (int)((n / 4 + 256) / 256);
    if (blocks > aie_sm_count() * 16) blocks = aie_sm_count() * 16;
    if (in_dtype == AIE_F32 && out_dtype == AIE_F32)
        activate_kernel<float, float><<<blocks, 256, 0, stream>>>((const float*)z, (float*)out, (size_t)n, act);
    else if (in_dtype == AIE_F32 && out_dtype == AIE_BF16)
        activate_kernel<float, bf16><<<blocks, 256, 0, stream>>>((const float*)z, (bf16*)out, (size_t)n, act);
    else if (in_dtype == AIE_BF16 && out_dtype == AIE_BF16)
        activate_kernel<bf16, bf16><<<blocks, 256, 0, stream>>>((const bf16*)z, (bf16*)out, (size_t)n, act);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// x <- x * s, float32, in place (logits with a constant factor)
// ---------------------------------------------------------------------------
__global__ void scale_kernel(float* __restrict__ x, size_t n, float s) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) x[i] *= s;
}

extern "C" int aie_scale(float* x, long long n, float s, cudaStream_t stream) {
    if (n <= 0) return 0;
    int blocks = (int)((n + 255) / 256);
    if (blocks > aie_sm_count() * 16) blocks = aie_sm_count() * 16;
    scale_kernel<<<blocks, 256, 0, stream>>>(x, (size_t)n, s);
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// Sinusoidal position vectors added to the float32 stream: x[t, 2i] += sin(p_t f_i), x[t, 2i + 1] += cos(p_t f_i),
// the angle float(p) * f_i in float32.  inv_freq holds ceil(D / 2) frequencies.
// ---------------------------------------------------------------------------
__global__ void add_sinusoid_kernel(float* __restrict__ x, const int* __restrict__ positions,
                                    const float* __restrict__ inv_freq, int D, int pairs) {
    const int t = blockIdx.x;
    const float p = (float)positions[t];
    float* row = x + (size_t)t * D;
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        float s, c;
        sincosf(p * inv_freq[i], &s, &c);
        row[2 * i] += s;
        if (2 * i + 1 < D) row[2 * i + 1] += c;
    }
}

extern "C" int aie_add_sinusoid(float* x, const int* positions, const float* inv_freq, int T, int D,
                                cudaStream_t stream) {
    if (T <= 0 || D <= 0) return 0;
    add_sinusoid_kernel<<<T, 128, 0, stream>>>(x, positions, inv_freq, D, (D + 1) / 2);
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// Two float32 streams side by side as one row of the compute dtype: out[t] = [x[t] (+ delta[t], or the sum of
// its parts) | y[t]], the input of a projection that mixes the running stream with an earlier one.
// ---------------------------------------------------------------------------
template <typename A, typename O>
__global__ void join_streams_kernel(const float* __restrict__ x, const A* __restrict__ delta, int parts,
                                    size_t part_stride, const float* __restrict__ y, O* __restrict__ out, int D,
                                    size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        const size_t t = i / D, c = i - t * D;
        float s = x[i];
        if (delta != nullptr)
            for (int p = 0; p < parts; ++p) s += to_f32<A>(delta[(size_t)p * part_stride + i]);
        out[t * 2 * D + c] = from_f32<O>(s);
        out[t * 2 * D + D + c] = from_f32<O>(y[i]);
    }
}

extern "C" int aie_join_streams(const float* x, const void* delta, int delta_dtype, int parts, long long part_stride,
                                const float* y, void* out, int out_dtype, int T, int D, cudaStream_t stream) {
    if (T <= 0 || D <= 0) return 0;
    const size_t n = (size_t)T * D;
    int blocks = (int)((n + 255) / 256);
    if (blocks > aie_sm_count() * 16) blocks = aie_sm_count() * 16;
#define AIE_JS(A, O)                                                                                         \
    join_streams_kernel<A, O><<<blocks, 256, 0, stream>>>(x, (const A*)delta, parts, (size_t)part_stride, y, \
                                                          (O*)out, D, n)
    const bool dbf = delta != nullptr && delta_dtype == AIE_BF16;
    if (out_dtype == AIE_F32) { if (dbf) AIE_JS(bf16, float); else AIE_JS(float, float); }
    else if (out_dtype == AIE_BF16) { if (dbf) AIE_JS(bf16, bf16); else AIE_JS(float, bf16); }
    else return AIE_BAD_ARG;
#undef AIE_JS
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// Dynamic Tanh, a norm without statistics: s = x[row] (+ delta, or the sum of `parts` deltas);
//   out = tanh(alpha * s) * w + b          element by element, float32, rounded once.
// alpha is read from the device (one float).  `rows` (optional) picks input rows; `write_back` stores s into x.
// ---------------------------------------------------------------------------
template <typename A, typename O>
__global__ void add_dyt_kernel(float* __restrict__ x, const A* __restrict__ delta, int parts, size_t part_stride,
                               const float* __restrict__ w, const float* __restrict__ b, const float* __restrict__ alpha,
                               O* __restrict__ out, const int* __restrict__ rows, int D, int write_back, size_t n) {
    const float al = alpha[0];
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        const size_t o = i / D;
        const int c = (int)(i - o * D);
        const size_t at = (rows ? (size_t)rows[o] : o) * D + c;
        float s = x[at];
        if (delta) {
            for (int p = 0; p < parts; ++p) s += to_f32<A>(delta[p * part_stride + at]);
            if (write_back) x[at] = s;
        }
        out[i] = from_f32<O>(fmaf(tanhf(al * s), w[c], b[c]));
    }
}

// four neighbouring elements a thread: D a multiple of 4, no row pick, 16-byte aligned pointers and part strides
template <typename A, typename O>
__global__ void add_dyt_vec4_kernel(float* __restrict__ x, const A* __restrict__ delta, int parts, size_t part_stride,
                                    const float* __restrict__ w, const float* __restrict__ b, const float* __restrict__ alpha,
                                    O* __restrict__ out, int D, int write_back, size_t n) {
    const float al = alpha[0];
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    float4 s = *reinterpret_cast<const float4*>(x + i);
    if (delta) {
        for (int p = 0; p < parts; ++p) {
            const float4 t = load4<A>(delta + p * part_stride + i);
            s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
        }
        if (write_back) *reinterpret_cast<float4*>(x + i) = s;
    }
    const int c = (int)(i % D);
    const float4 wv = *reinterpret_cast<const float4*>(w + c), bv = *reinterpret_cast<const float4*>(b + c);
    store4<O>(out + i, make_float4(fmaf(tanhf(al * s.x), wv.x, bv.x), fmaf(tanhf(al * s.y), wv.y, bv.y),
                                   fmaf(tanhf(al * s.z), wv.z, bv.z), fmaf(tanhf(al * s.w), wv.w, bv.w)));
}

extern "C" int aie_add_dyt(float* x, const void* delta, int delta_dtype, int parts, long long part_stride, const float* w,
                           const float* b, const float* alpha, void* out, int out_dtype, const int* rows, int n_rows, int D,
                           int write_back, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (D <= 0 || (delta && parts < 1)) return AIE_BAD_ARG;
    const size_t n = (size_t)n_rows * D;
    int blocks = (int)((n + 255) / 256);
    if (blocks > aie_sm_count() * 16) blocks = aie_sm_count() * 16;
    const bool dbf = delta && delta_dtype == AIE_BF16;
    const bool vec = !rows && D % 4 == 0 && !((size_t)x & 15) && !((size_t)w & 15) && !((size_t)b & 15) && !((size_t)out & 15) &&
                     (!delta || (part_stride % 8 == 0 && !((size_t)delta & 15)));
    const unsigned vblocks = (unsigned)((n / 4 + 255) / 256);
#define GO(A, O)                                                                                                      \
    do {                                                                                                              \
        if (vec)                                                                                                      \
            add_dyt_vec4_kernel<A, O><<<vblocks, 256, 0, stream>>>(x, (const A*)delta, parts, (size_t)part_stride, w, b, alpha, \
                                                                  (O*)out, D, write_back, n);                          \
        else                                                                                                          \
            add_dyt_kernel<A, O><<<blocks, 256, 0, stream>>>(x, (const A*)delta, parts, (size_t)part_stride, w, b, alpha,     \
                                                             (O*)out, rows, D, write_back, n);                        \
    } while (0)
    if (out_dtype == AIE_F32) { if (dbf) GO(bf16, float); else GO(float, float); }
    else if (out_dtype == AIE_BF16) { if (dbf) GO(bf16, bf16); else GO(float, bf16); }
    else return AIE_BAD_ARG;
#undef GO
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// a[t, n] <- a[t, n] * sigmoid(g[t, n / group])   in place; g float32 with rows `ldg` floats apart (a slice of a
// wider projection).  group 1: a gate per element; group = a head's width: a gate per head.
// ---------------------------------------------------------------------------
template <typename A>
__global__ void sigmoid_gate_mul_kernel(A* __restrict__ a, const float* __restrict__ g, int ldg, int N, int group, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        const size_t t = i / N;
        const int c = (int)(i - t * N);
        const float z = g[t * ldg + c / group];
        a[i] = from_f32<A>(to_f32<A>(a[i]) * (1.0f / (1.0f + expf(-z))));
    }
}

// four neighbouring elements a thread: N a multiple of 4; a group is one element or a multiple of four
template <typename A>
__global__ void sigmoid_gate_mul_vec4_kernel(A* __restrict__ a, const float* __restrict__ g, int ldg, int N, int group, size_t n) {
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    const size_t t = i / N;
    const int c = (int)(i - t * N);
    float4 z;
    if (group == 1) {
        const float* gp = g + t * ldg + c;
        z = make_float4(gp[0], gp[1], gp[2], gp[3]);
    } else {
        const float zz = g[t * ldg + c / group];
        z = make_float4(zz, zz, zz, zz);
    }
    float4 v = load4<A>(a + i);
    v.x *= 1.0f / (1.0f + expf(-z.x));
    v.y *= 1.0f / (1.0f + expf(-z.y));
    v.z *= 1.0f / (1.0f + expf(-z.z));
    v.w *= 1.0f / (1.0f + expf(-z.w));
    store4<A>(a + i, v);
}

extern "C" int aie_sigmoid_gate_mul(void* a, int dtype, const float* g, int ldg, int T, int N, int group, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (N <= 0 || group <= 0 || N % group) return AIE_BAD_ARG;
    const size_t n = (size_t)T * N;
    int blocks = (int)((n + 255) / 256);
    if (blocks > aie_sm_count() * 16) blocks = aie_sm_count() * 16;
    const bool vec = N % 4 == 0 && (group == 1 || group % 4 == 0) && !((size_t)a & 15);
    const unsigned vblocks = (unsigned)((n / 4 + 255) / 256);
    if (dtype == AIE_F32) {
        if (vec) sigmoid_gate_mul_vec4_kernel<float><<<vblocks, 256, 0, stream>>>((float*)a, g, ldg, N, group, n);
        else sigmoid_gate_mul_kernel<float><<<blocks, 256, 0, stream>>>((float*)a, g, ldg, N, group, n);
    } else if (dtype == AIE_BF16) {
        if (vec) sigmoid_gate_mul_vec4_kernel<bf16><<<vblocks, 256, 0, stream>>>((bf16*)a, g, ldg, N, group, n);
        else sigmoid_gate_mul_kernel<bf16><<<blocks, 256, 0, stream>>>((bf16*)a, g, ldg, N, group, n);
    } else return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}

// y[t, n] += bias[n] in place, float32 (a projection's bias, added to the first of its unjoined parts)
__global__ void add_bias_kernel(float* __restrict__ y, const float* __restrict__ bias, int N, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) y[i] += bias[i % N];
}

extern "C" int aie_add_bias(float* y, const float* bias, int T, int N, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (N <= 0) return AIE_BAD_ARG;
    const size_t n = (size_t)T * N;
    int blocks = (int)((n + 255) / 256);
    if (blocks > aie_sm_count() * 16) blocks = aie_sm_count() * 16;
    add_bias_kernel<<<blocks, 256, 0, stream>>>(y, bias, N, n);
    AIE_LAUNCH_CHECK();
}
