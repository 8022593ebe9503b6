// Row kernels of layers that carry more than a residual stream: a short causal convolution over time with
// its per-request tail, the weighted average over the streams of all earlier layers, activations that
// normalise over the feed-forward width or clamp their operands, a per-head norm with an output gate,
// per-channel decays from logits, and the bookkeeping of a mixture of experts whose experts are chosen
// by a table (rows grouped by expert, outputs summed per token).  Statistics, decays and sums are float32.
#include "common.cuh"

// ---------------------------------------------------------------------------
// out[t] = h[t] + sum_j w[:, j] * h[t - (taps-1) + j]      (per channel, zeros before the sequence's start)
// The inputs of the taps-1 tokens before a portion are the request's tail `state[slot]` [taps-1, D], oldest
// first.  Only the block of a request's first token of the step reads the tail: it computes the (at most
// taps-1) tokens that need it and then stores the new tail, so no other block races with the update.
// ---------------------------------------------------------------------------
template <typename O>
__global__ void short_conv_kernel(const float* __restrict__ h, const float* __restrict__ w, float* __restrict__ state,
                                  O* __restrict__ out, const int* __restrict__ q_start, const int* __restrict__ q_len,
                                  const int* __restrict__ slots, const int* __restrict__ token_req, int D, int taps,
                                  int max_slots, unsigned* err) {
    const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= D) return;
    const int r = token_req[t];
    const int a = q_start[r], n = q_len[r], i = t - a, slot = slots[r];
    const int Hh = taps - 1;
    const float* wc = w + (size_t)c * taps;
    if (i >= Hh) {
        float acc = h[(size_t)t * D + c];
        for (int j = 0; j < taps; ++j) acc = fmaf(wc[j], h[(size_t)(t - Hh + j) * D + c], acc);
        out[(size_t)t * D + c] = from_f32<O>(acc);
        return;
    }
    if (i != 0) return;
    if (slot < 0 || slot >= max_slots) {
        if (threadIdx.x == 0) atomicOr(err, AIE_DEV_SLOT_OOB);
        return;
    }
    float* st = state + (size_t)slot * Hh * D + c;          // st[k * D]: input at local index k - Hh
    const int first = min(n, Hh);
    for (int ii = 0; ii < first; ++ii) {
        float acc = h[(size_t)(a + ii) * D + c];
        for (int j = 0; j < taps; ++j) {
            const int src = ii - Hh + j;
            const float x = src >= 0 ? h[(size_t)(a + src) * D + c] : st[(size_t)(src + Hh) * D];
            acc = fmaf(wc[j], x, acc);
        }
        out[(size_t)(a + ii) * D + c] = from_f32<O>(acc);
    }
    for (int k = 0; k < Hh; ++k) {                          // ascending: entry n + k > k is still the old one
        const int src = n - Hh + k;
        st[(size_t)k * D] = src >= 0 ? h[(size_t)(a + src) * D + c] : st[(size_t)(n + k) * D];
    }
}

// The same for widths that are multiples of 4: a thread owns four neighbouring channels (16-byte loads).
template <typename O>
__global__ void short_conv4_kernel(const float* __restrict__ h, const float* __restrict__ w, float* __restrict__ state,
                                   O* __restrict__ out, const int* __restrict__ q_start, const int* __restrict__ q_len,
                                   const int* __restrict__ slots, const int* __restrict__ token_req, int D, int taps,
                                   int max_slots, unsigned* err) {
    const int t = blockIdx.x, c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (c >= D) return;
    const int r = token_req[t];
    const int a = q_start[r], n = q_len[r], i = t - a, slot = slots[r];
    const int Hh = taps - 1;
    const float* wc = w + (size_t)c * taps;                 // channel c + e: wc[e * taps + j]
    if (i >= Hh) {
        float4 acc = *reinterpret_cast<const float4*>(h + (size_t)t * D + c);
        for (int j = 0; j < taps; ++j) {
            const float4 x = *reinterpret_cast<const float4*>(h + (size_t)(t - Hh + j) * D + c);
            acc.x = fmaf(wc[j], x.x, acc.x);
            acc.y = fmaf(wc[taps + j], x.y, acc.y);
            acc.z = fmaf(wc[2 * taps + j], x.z, acc.z);
            acc.w = fmaf(wc[3 * taps + j], x.w, acc.w);
        }
        store4<O>(out + (size_t)t * D + c, acc);
        return;
    }
    if (i != 0) return;
    if (slot < 0 || slot >= max_slots) {
        if (threadIdx.x == 0) atomicOr(err, AIE_DEV_SLOT_OOB);
        return;
    }
    float* st = state + (size_t)slot * Hh * D + c;
    const int first = min(n, Hh);
    for (int ii = 0; ii < first; ++ii) {
        float4 acc = *reinterpret_cast<const float4*>(h + (size_t)(a + ii) * D + c);
        for (int j = 0; j < taps; ++j) {
            const int src = ii - Hh + j;
            const float4 x = src >= 0 ? *reinterpret_cast<const float4*>(h + (size_t)(a + src) * D + c)
                                      : *reinterpret_cast<const float4*>(st + (size_t)(src + Hh) * D);
            acc.x = fmaf(wc[j], x.x, acc.x);
            acc.y = fmaf(wc[taps + j], x.y, acc.y);
            acc.z = fmaf(wc[2 * taps + j], x.z, acc.z);
            acc.w = fmaf(wc[3 * taps + j], x.w, acc.w);
        }
        store4<O>(out + (size_t)(a + ii) * D + c, acc);
    }
    for (int k = 0; k < Hh; ++k) {
        const int src = n - Hh + k;
        *reinterpret_cast<float4*>(st + (size_t)k * D) =
            src >= 0 ? *reinterpret_cast<const float4*>(h + (size_t)(a + src) * D + c)
                     : *reinterpret_cast<const float4*>(st + (size_t)(n + k) * D);
    }
}

extern "C" int aie_short_conv(const float* h, const float* w, float* state, void* out, int out_dtype, const int* q_start,
                              const int* q_len, const int* slots, const int* token_req, int T, int D, int taps,
                              int max_slots, unsigned* err, cudaStream_t st) {
    if (T <= 0) return 0;
    if (D <= 0 || taps < 1) return AIE_BAD_ARG;
    if (D % 4 == 0 && !((size_t)h & 15) && !((size_t)state & 15) && !((size_t)out & 15)) {
        const int threads = 64;
        dim3 grid4(T, (D / 4 + threads - 1) / threads);
        if (out_dtype == AIE_F32)
            short_conv4_kernel<float><<<grid4, threads, 0, st>>>(h, w, state, (float*)out, q_start, q_len, slots, token_req, D, taps, max_slots, err);
        else if (out_dtype == AIE_BF16)
            short_conv4_kernel<bf16><<<grid4, threads, 0, st>>>(h, w, state, (bf16*)out, q_start, q_len, slots, token_req, D, taps, max_slots, err);
        else
            return AIE_BAD_ARG;
        AIE_LAUNCH_CHECK();
    }
    dim3 grid(T, (D + 255) / 256);
    if (grid.y > 65535) return AIE_UNSUPPORTED;
    if (out_dtype == AIE_F32)
        short_conv_kernel<float><<<grid, 256, 0, st>>>(h, w, state, (float*)out, q_start, q_len, slots, token_req, D, taps, max_slots, err);
    else if (out_dtype == AIE_BF16)
        short_conv_kernel<bf16><<<grid, 256, 0, st>>>(h, w, state, (bf16*)out, q_start, q_len, slots, token_req, D, taps, max_slots, err);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// The stream that leaves layer i is a weighted sum of the streams all layers so far produced:
//   X = x (+ delta parts);  history[depth] = X;  x = sum_{j <= depth} coef[j] * history[j]
// history: [levels, n] float32 with n = T * D; x: [n] float32, rewritten in place.
// ---------------------------------------------------------------------------
template <typename A>
__global__ void depth_average_kernel(float* __restrict__ x, const A* __restrict__ delta, int parts, size_t part_stride,
                                     float* __restrict__ history, const float* __restrict__ coef, int depth, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float s = x[i];
    for (int p = 0; p < parts; ++p) s += to_f32<A>(delta[p * part_stride + i]);
    history[(size_t)depth * n + i] = s;
    float acc = 0.f;
    for (int j = 0; j < depth; ++j) acc = fmaf(coef[j], history[(size_t)j * n + i], acc);
    x[i] = fmaf(coef[depth], s, acc);
}

// Two branches that read the same input, added to the stream with one multiplier:
//   X = x + mult * (sum of a's parts + sum of b's parts), then as above.  a and b are float32; b may be absent.
// With norm_w: also out = tanh(alpha x) w + b_n of the averaged stream (the next layer's input norm, when that is a
// norm without statistics), so the stream is not read again.
template <typename O>
__global__ void depth_average2_kernel(float* __restrict__ x, const float* __restrict__ a, int pa, size_t sa,
                                      const float* __restrict__ b, int pb, size_t sb, float mult,
                                      float* __restrict__ history, const float* __restrict__ coef, int depth, size_t n,
                                      const float* __restrict__ norm_w, const float* __restrict__ norm_b,
                                      const float* __restrict__ norm_alpha, O* __restrict__ normed, int D) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float d = 0.f;
    for (int p = 0; p < pa; ++p) d += a[p * sa + i];
    float e = 0.f;
    for (int p = 0; p < pb; ++p) e += b[p * sb + i];
    const float s = fmaf(mult, d + e, x[i]);
    float y = s;
    if (coef) {
        history[(size_t)depth * n + i] = s;
        float acc = 0.f;
        for (int j = 0; j < depth; ++j) acc = fmaf(coef[j], history[(size_t)j * n + i], acc);
        y = fmaf(coef[depth], s, acc);
    }
    x[i] = y;
    if (norm_w) {
        const int c = (int)(i % D);
        normed[i] = from_f32<O>(fmaf(tanhf(norm_alpha[0] * y), norm_w[c], norm_b[c]));
    }
}

extern "C" int aie_depth_average(float* x, const void* delta, int delta_dtype, int parts, long long part_stride,
                                 float* history, const float* coef, int depth, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    if (depth < 0) return AIE_BAD_ARG;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (!delta) parts = 0;
    if (delta_dtype == AIE_BF16 && delta)
        depth_average_kernel<bf16><<<blocks, 256, 0, st>>>(x, (const bf16*)delta, parts, (size_t)part_stride, history, coef, depth, (size_t)n);
    else
        depth_average_kernel<float><<<blocks, 256, 0, st>>>(x, (const float*)delta, parts, (size_t)part_stride, history, coef, depth, (size_t)n);
    AIE_LAUNCH_CHECK();
}

// The same, four neighbouring elements a thread (16-byte loads and stores): n and D multiples of 4, every pointer and
// every part's stride 16-byte aligned.
template <typename O>
__global__ void depth_average2_vec4_kernel(float* __restrict__ x, const float* __restrict__ a, int pa, size_t sa,
                                           const float* __restrict__ b, int pb, size_t sb, float mult,
                                           float* __restrict__ history, const float* __restrict__ coef, int depth, size_t n,
                                           const float* __restrict__ norm_w, const float* __restrict__ norm_b,
                                           const float* __restrict__ norm_alpha, O* __restrict__ normed, int D) {
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    float4 d = make_float4(0.f, 0.f, 0.f, 0.f), e = d;
    for (int p = 0; p < pa; ++p) {
        const float4 t = *reinterpret_cast<const float4*>(a + p * sa + i);
        d.x += t.x; d.y += t.y; d.z += t.z; d.w += t.w;
    }
    for (int p = 0; p < pb; ++p) {
        const float4 t = *reinterpret_cast<const float4*>(b + p * sb + i);
        e.x += t.x; e.y += t.y; e.z += t.z; e.w += t.w;
    }
    const float4 xv = *reinterpret_cast<const float4*>(x + i);
    const float4 s = make_float4(fmaf(mult, d.x + e.x, xv.x), fmaf(mult, d.y + e.y, xv.y), fmaf(mult, d.z + e.z, xv.z),
                                 fmaf(mult, d.w + e.w, xv.w));
    float4 y = s;
    if (coef) {
        *reinterpret_cast<float4*>(history + (size_t)depth * n + i) = s;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < depth; ++j) {
            const float c = coef[j];
            const float4 hv = *reinterpret_cast<const float4*>(history + (size_t)j * n + i);
            acc.x = fmaf(c, hv.x, acc.x); acc.y = fmaf(c, hv.y, acc.y); acc.z = fmaf(c, hv.z, acc.z); acc.w = fmaf(c, hv.w, acc.w);
        }
        const float c = coef[depth];
        y = make_float4(fmaf(c, s.x, acc.x), fmaf(c, s.y, acc.y), fmaf(c, s.z, acc.z), fmaf(c, s.w, acc.w));
    }
    *reinterpret_cast<float4*>(x + i) = y;
    if (norm_w) {
        const int c = (int)(i % D);
        const float al = norm_alpha[0];
        const float4 w = *reinterpret_cast<const float4*>(norm_w + c), bb = *reinterpret_cast<const float4*>(norm_b + c);
        store4<O>(normed + i, make_float4(fmaf(tanhf(al * y.x), w.x, bb.x), fmaf(tanhf(al * y.y), w.y, bb.y),
                                          fmaf(tanhf(al * y.z), w.z, bb.z), fmaf(tanhf(al * y.w), w.w, bb.w)));
    }
}

// coef null: no averaging (x <- X).  norm_w null: no norm is made.
extern "C" int aie_depth_average2(float* x, const float* a, int pa, long long sa, const float* b, int pb, long long sb,
                                  float mult, float* history, const float* coef, int depth, long long n,
                                  const float* norm_w, const float* norm_b, const float* norm_alpha, void* normed,
                                  int normed_dtype, int D, cudaStream_t st) {
    if (n <= 0) return 0;
    if (depth < 0 || !a || pa < 1 || (coef && !history) || (norm_w && (!norm_b || !norm_alpha || !normed || D <= 0)))
        return AIE_BAD_ARG;
    if (!b) pb = 0;
    const bool bf = norm_w && normed_dtype == AIE_BF16;
    auto al16 = [](const void* p) { return ((size_t)p & 15) == 0; };
    const bool vec = n % 4 == 0 && (!norm_w || D % 4 == 0) && al16(x) && al16(a) && sa % 4 == 0 && (!pb || (al16(b) && sb % 4 == 0)) &&
                     (!coef || al16(history)) && (!norm_w || (al16(norm_w) && al16(norm_b) && al16(normed)));
#define GO(KERN, O, BLOCKS)                                                                                            \
    KERN<O><<<BLOCKS, 256, 0, st>>>(x, a, pa, (size_t)sa, b, pb, (size_t)sb, mult, history, coef, depth, (size_t)n, norm_w,  \
                                    norm_b, norm_alpha, (O*)normed, D > 0 ? D : 1)
    if (vec) {
        const unsigned blocks = (unsigned)((n / 4 + 255) / 256);
        if (bf) GO(depth_average2_vec4_kernel, bf16, blocks);
        else GO(depth_average2_vec4_kernel, float, blocks);
    } else {
        const unsigned blocks = (unsigned)((n + 255) / 256);
        if (bf) GO(depth_average2_kernel, bf16, blocks);
        else GO(depth_average2_kernel, float, blocks);
    }
#undef GO
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// A polynomial of normalised powers over the feed-forward width F, per token:
//   out = a N(z) + b N(z^2) + c N(z^3) + e,   N(y) = y / sqrt(mean(y^2) + eps)
// ---------------------------------------------------------------------------
template <typename O>
__global__ void polynorm_kernel(const float* __restrict__ z, const float* __restrict__ coef, O* __restrict__ out, int F,
                                float eps) {
    __shared__ float red[32];
    const float* zr = z + (size_t)blockIdx.x * F;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const float v = zr[i], v2 = v * v, v3 = v2 * v;
        s2 += v2;
        s4 += v2 * v2;
        s6 += v3 * v3;
    }
    s2 = block_sum(s2, red);
    s4 = block_sum(s4, red);
    s6 = block_sum(s6, red);
    const float r1 = 1.0f / sqrtf(s2 / (float)F + eps), r2 = 1.0f / sqrtf(s4 / (float)F + eps),
                r3 = 1.0f / sqrtf(s6 / (float)F + eps);
    const float a = coef[0] * r1, b = coef[1] * r2, c = coef[2] * r3, e = coef[3];
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const float v = zr[i], v2 = v * v;
        out[(size_t)blockIdx.x * F + i] = from_f32<O>(a * v + b * v2 + c * (v2 * v) + e);
    }
}

extern "C" int aie_polynorm(const float* z, const float* coef, void* out, int out_dtype, int T, int F, float eps,
                            cudaStream_t st) {
    if (T <= 0) return 0;
    if (F <= 0) return AIE_BAD_ARG;
    const int threads = F >= 2048 ? 512 : 256;
    if (out_dtype == AIE_F32)
        polynorm_kernel<float><<<T, threads, 0, st>>>(z, coef, (float*)out, F, eps);
    else if (out_dtype == AIE_BF16)
        polynorm_kernel<bf16><<<T, threads, 0, st>>>(z, coef, (bf16*)out, F, eps);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// Per (token, head): y = o / sqrt(mean(o^2) + eps) (* w) (* silu(g)).  o [T, H, dv] float32; g has rows of
// `ldg` floats (a slice of a wider projection) or is null (no gate); w [dv] or null.  One warp per (token, head).
// ---------------------------------------------------------------------------
template <typename O>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ g, int ldg,
                                      const float* __restrict__ w, O* __restrict__ out, int TH, int H, int dv, float eps) {
    const int wi = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (wi >= TH) return;
    const int t = wi / H, hh = wi % H;
    const float* orow = o + (size_t)wi * dv;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) ss += orow[i] * orow[i];
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)dv + eps);
    const float* grow = g ? g + (size_t)t * ldg + (size_t)hh * dv : nullptr;
    for (int i = lane; i < dv; i += 32) {
        float y = orow[i] * r;
        if (w) y *= w[i];
        if (grow) {
            const float gv = grow[i];
            y *= gv / (1.0f + expf(-gv));
        }
        out[(size_t)wi * dv + i] = from_f32<O>(y);
    }
}

extern "C" int aie_head_norm_gate(const float* o, const float* g, int ldg, const float* w, void* out, int out_dtype, int T,
                                  int H, int dv, float eps, cudaStream_t st) {
    if (T <= 0) return 0;
    if (H <= 0 || dv <= 0) return AIE_BAD_ARG;
    const long long warps = (long long)T * H;
    const unsigned blocks = (unsigned)((warps + 3) / 4);
    if (out_dtype == AIE_F32)
        head_norm_gate_kernel<float><<<blocks, 128, 0, st>>>(o, g, ldg, w, (float*)out, (int)warps, H, dv, eps);
    else if (out_dtype == AIE_BF16)
        head_norm_gate_kernel<bf16><<<blocks, 128, 0, st>>>(o, g, ldg, w, (bf16*)out, (int)warps, H, dv, eps);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// A gated unit whose operands are clamped: g = min(gate, limit), u = clamp(up, -limit, limit),
//   y = g * sigmoid(alpha g) * (u + shift).   gu rows of `ld` floats: gate in [0, F), up in [F, 2F).
// ---------------------------------------------------------------------------
template <typename O>
__global__ void clamped_glu_kernel(const float* __restrict__ gu, int ld, O* __restrict__ out, long long n, int F,
                                   float limit, float alpha, float shift) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long t = i / F;
    const int f = (int)(i % F);
    const float g = fminf(gu[t * ld + f], limit);
    const float u = fminf(fmaxf(gu[t * ld + F + f], -limit), limit);
    out[i] = from_f32<O>(g / (1.0f + expf(-alpha * g)) * (u + shift));
}

extern "C" int aie_clamped_glu(const float* gu, int ld, void* out, int out_dtype, long long T, int F, float limit,
                               float alpha, float shift, cudaStream_t st) {
    if (T <= 0) return 0;
    if (F <= 0) return AIE_BAD_ARG;
    const long long n = T * F;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (out_dtype == AIE_F32)
        clamped_glu_kernel<float><<<blocks, 256, 0, st>>>(gu, ld, (float*)out, n, F, limit, alpha, shift);
    else if (out_dtype == AIE_BF16)
        clamped_glu_kernel<bf16><<<blocks, 256, 0, st>>>(gu, ld, (bf16*)out, n, F, limit, alpha, shift);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// decay = sigmoid(z + bias)^(1 / tau) = exp(log_sigmoid(z + bias) / tau), float32 throughout.
// ---------------------------------------------------------------------------
__global__ void gated_decay_kernel(const float* __restrict__ z, const float* __restrict__ bias, float* __restrict__ out,
                                   long long n, int N, float inv_tau) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = z[i] + (bias ? bias[i % N] : 0.f);
    const float ls = fminf(v, 0.f) - log1pf(expf(-fabsf(v)));      // log(sigmoid(v)), stable on both sides
    out[i] = expf(ls * inv_tau);
}

extern "C" int aie_gated_decay(const float* z, const float* bias, float* out, long long T, int N, float tau,
                               cudaStream_t st) {
    if (T <= 0) return 0;
    if (N <= 0 || !(tau > 0.f)) return AIE_BAD_ARG;
    const long long n = T * N;
    gated_decay_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(z, bias, out, n, N, 1.0f / tau);
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// Experts chosen by a table of the token's id: pair p = (token t, choice s) goes to expert table[id[t], s]
// (ids null: the table has a row per token of the step, as a router leaves it).  Experts E .. E + ident - 1 are
// accepted but get no row: they stand for experts without weights, and their pairs are marked with -2.
// One block groups the pairs by expert into tiles of `tile` rows (each expert's rows padded up to whole tiles):
//   row_token[row]  = token of the row, -1 for padding         [n_tiles * tile]
//   pair_row[p]     = row of pair p (-1: bad token id or expert)  [T * top]
//   tile_expert[i]  = expert of tile i, -1 for unused tiles     [n_tiles], n_tiles >= ceil(T top / tile) + E
// Which row of its expert's range a pair gets depends on timing; no result depends on it, since every row
// of the grouped products is computed for itself.
// ---------------------------------------------------------------------------
__global__ void expert_plan_kernel(const int* __restrict__ ids, const int* __restrict__ table, int T, int V, int top,
                                   int E, int ident, int tile, int n_tiles, int* __restrict__ row_token, int* __restrict__ pair_row,
                                   int* __restrict__ tile_expert, unsigned* err) {
    extern __shared__ int sh[];
    int* count = sh;            // [E]
    int* start = sh + E;        // [E]
    int* cursor = sh + 2 * E;   // [E]
    const int tid = threadIdx.x, P = T * top;
    for (int e = tid; e < E; e += blockDim.x) count[e] = cursor[e] = 0;
    for (int i = tid; i < n_tiles * tile; i += blockDim.x) row_token[i] = -1;
    for (int i = tid; i < n_tiles; i += blockDim.x) tile_expert[i] = -1;
    __syncthreads();
    for (int p = tid; p < P; p += blockDim.x) {
        const int id = ids ? ids[p / top] : p / top;
        int e = -1;
        if (id >= 0 && id < V) e = table[(size_t)id * top + p % top];
        if (e >= E && e < E + ident) continue;
        if (e < 0 || e >= E) {
            atomicOr(err, AIE_DEV_TOKEN_OOB);
            continue;
        }
        atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (tid == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) {
            start[e] = at * tile;
            const int nt = (count[e] + tile - 1) / tile;
            for (int i = 0; i < nt && at + i < n_tiles; ++i) tile_expert[at + i] = e;
            at += nt;
        }
    }
    __syncthreads();
    for (int p = tid; p < P; p += blockDim.x) {
        const int id = ids ? ids[p / top] : p / top;
        int e = -1;
        if (id >= 0 && id < V) e = table[(size_t)id * top + p % top];
        if (e < 0 || e >= E) {
            pair_row[p] = (e >= E && e < E + ident) ? -2 : -1;
            continue;
        }
        const int row = start[e] + atomicAdd(&cursor[e], 1);
        pair_row[p] = row;
        if (row < n_tiles * tile) row_token[row] = p / top;
    }
}

extern "C" int aie_expert_plan(const int* ids, const int* table, int T, int V, int top, int E, int ident, int tile, int n_tiles,
                               int* row_token, int* pair_row, int* tile_expert, unsigned* err, cudaStream_t st) {
    if (T <= 0) return 0;
    if (top <= 0 || E <= 0 || tile <= 0 || (long long)n_tiles * tile < (long long)T * top) return AIE_BAD_ARG;
    if ((size_t)3 * E * sizeof(int) > 40000) return AIE_UNSUPPORTED;
    expert_plan_kernel<<<1, 1024, 3 * E * sizeof(int), st>>>(ids, table, T, V, top, E, ident, tile, n_tiles, row_token, pair_row,
                                                              tile_expert, err);
    AIE_LAUNCH_CHECK();
}

// out[t] = w * sum_s y[pair_row[t top + s]]  (+ shared[t] * sigmoid(gate[t]))        float32
__global__ void expert_combine_kernel(const float* __restrict__ y, const int* __restrict__ pair_row, int top, float w,
                                      const float* __restrict__ shared, const float* __restrict__ gate, int ld_gate,
                                      float* __restrict__ out, int D) {
    const int t = blockIdx.x;
    float sg = 0.f;
    if (shared) sg = 1.0f / (1.0f + expf(-gate[(size_t)t * ld_gate]));
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < top; ++s) {
            const int row = pair_row[(size_t)t * top + s];
            if (row >= 0) acc = fmaf(w, y[(size_t)row * D + c], acc);
        }
        if (shared) acc = fmaf(shared[(size_t)t * D + c], sg, acc);
        out[(size_t)t * D + c] = acc;
    }
}

extern "C" int aie_expert_combine(const float* y, const int* pair_row, int top, float w, const float* shared,
                                  const float* gate, int ld_gate, float* out, int T, int D, cudaStream_t st) {
    if (T <= 0) return 0;
    if (D <= 0 || top <= 0) return AIE_BAD_ARG;
    expert_combine_kernel<<<T, 256, 0, st>>>(y, pair_row, top, w, shared, gate, ld_gate, out, D);
    AIE_LAUNCH_CHECK();
}

// out[r] = src[rows[r]] (zeros where rows[r] < 0): the step's rows in the order of a grouping
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ src, const int* __restrict__ rows, T* __restrict__ out, int D) {
    const int r = blockIdx.x, s = rows[r];
    for (int c = threadIdx.x; c < D; c += blockDim.x)
        out[(size_t)r * D + c] = s >= 0 ? src[(size_t)s * D + c] : from_f32<T>(0.f);
}

extern "C" int aie_gather_rows(const void* src, const int* rows, void* out, int dtype, int n, int D, cudaStream_t st) {
    if (n <= 0) return 0;
    if (D <= 0) return AIE_BAD_ARG;
    if (dtype == AIE_F32)
        gather_rows_kernel<float><<<n, 256, 0, st>>>((const float*)src, rows, (float*)out, D);
    else if (dtype == AIE_BF16)
        gather_rows_kernel<bf16><<<n, 256, 0, st>>>((const bf16*)src, rows, (bf16*)out, D);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// A causal convolution over time on a slice of a wider projection, per channel:
//   y[t, c] = (residual ? u[t, c] : 0) + bias[c] + sum_j w[c, j] * u[t - (taps-1) + j, c],   then act (0: none, 1: silu)
// u rows are ld_in floats apart, out rows ld_out elements.  Channels [dup_from, dup_from + dup_n) are written a
// second time dup_n columns further on (keys that are also values).  The inputs of the taps-1 tokens before a
// portion are the request's tail `state[slot]` [taps-1, C]; as in short_conv only the block of a request's first
// token of the step reads and replaces it.
// ---------------------------------------------------------------------------
template <typename O>
__global__ void causal_conv_kernel(const float* __restrict__ u, int ld_in, const float* __restrict__ w,
                                   const float* __restrict__ bias, float* __restrict__ state, O* __restrict__ out,
                                   int ld_out, const int* __restrict__ q_start, const int* __restrict__ q_len,
                                   const int* __restrict__ slots, const int* __restrict__ token_req, int C, int taps,
                                   int residual, int act, int dup_from, int dup_n, int max_slots, unsigned* err) {
    const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int r = token_req[t];
    const int a = q_start[r], n = q_len[r], i = t - a, slot = slots[r];
    const int Hh = taps - 1;
    const float* wc = w + (size_t)c * taps;
    const float b = bias ? bias[c] : 0.f;
    const bool dup = c >= dup_from && c < dup_from + dup_n;
    if (i >= Hh) {
        float acc = residual ? u[(size_t)t * ld_in + c] + b : b;
        for (int j = 0; j < taps; ++j) acc = fmaf(wc[j], u[(size_t)(t - Hh + j) * ld_in + c], acc);
        if (act == 1) acc = acc / (1.0f + expf(-acc));
        out[(size_t)t * ld_out + c] = from_f32<O>(acc);
        if (dup) out[(size_t)t * ld_out + c + dup_n] = from_f32<O>(acc);
        return;
    }
    if (i != 0) return;
    if (slot < 0 || slot >= max_slots) {
        if (threadIdx.x == 0) atomicOr(err, AIE_DEV_SLOT_OOB);
        return;
    }
    float* st = state + (size_t)slot * Hh * C + c;          // st[k * C]: input at local index k - Hh
    const int first = min(n, Hh);
    for (int ii = 0; ii < first; ++ii) {
        float acc = residual ? u[(size_t)(a + ii) * ld_in + c] + b : b;
        for (int j = 0; j < taps; ++j) {
            const int src = ii - Hh + j;
            const float x = src >= 0 ? u[(size_t)(a + src) * ld_in + c] : st[(size_t)(src + Hh) * C];
            acc = fmaf(wc[j], x, acc);
        }
        if (act == 1) acc = acc / (1.0f + expf(-acc));
        out[(size_t)(a + ii) * ld_out + c] = from_f32<O>(acc);
        if (dup) out[(size_t)(a + ii) * ld_out + c + dup_n] = from_f32<O>(acc);
    }
    for (int k = 0; k < Hh; ++k) {                          // ascending: entry n + k > k is still the old one
        const int src = n - Hh + k;
        st[(size_t)k * C] = src >= 0 ? u[(size_t)(a + src) * ld_in + c] : st[(size_t)(n + k) * C];
    }
}

// The same for channel counts, row strides and copied ranges that are multiples of 4: a thread owns four neighbouring
// channels (16-byte loads and stores).
template <typename O>
__global__ void causal_conv4_kernel(const float* __restrict__ u, int ld_in, const float* __restrict__ w,
                                    const float* __restrict__ bias, float* __restrict__ state, O* __restrict__ out,
                                    int ld_out, const int* __restrict__ q_start, const int* __restrict__ q_len,
                                    const int* __restrict__ slots, const int* __restrict__ token_req, int C, int taps,
                                    int residual, int act, int dup_from, int dup_n, int max_slots, unsigned* err) {
    const int t = blockIdx.x, c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (c >= C) return;
    const int r = token_req[t];
    const int a = q_start[r], n = q_len[r], i = t - a, slot = slots[r];
    const int Hh = taps - 1;
    const float* wc = w + (size_t)c * taps;                 // channel c + e: wc[e * taps + j]
    const float4 b = bias ? *reinterpret_cast<const float4*>(bias + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    const bool dup = c >= dup_from && c < dup_from + dup_n;
    float* st = state + (size_t)slot * Hh * C + c;          // st[k * C]: input at local index k - Hh
    if (i < Hh && (slot < 0 || slot >= max_slots)) {
        if (threadIdx.x == 0 && i == 0) atomicOr(err, AIE_DEV_SLOT_OOB);
        return;
    }
    if (i >= Hh || i == 0) {
        const int first = i >= Hh ? 1 : min(n, Hh);         // the request's first block also serves the tokens that need the tail
        for (int ii = 0; ii < first; ++ii) {
            const int li = i + ii;                          // index of the token among the request's tokens of this step
            float4 acc = b;
            if (residual) {
                const float4 x = *reinterpret_cast<const float4*>(u + (size_t)(a + li) * ld_in + c);
                acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
            }
            for (int j = 0; j < taps; ++j) {
                const int src = li - Hh + j;
                const float4 x = src >= 0 ? *reinterpret_cast<const float4*>(u + (size_t)(a + src) * ld_in + c)
                                          : *reinterpret_cast<const float4*>(st + (size_t)(src + Hh) * C);
                acc.x = fmaf(wc[j], x.x, acc.x);
                acc.y = fmaf(wc[taps + j], x.y, acc.y);
                acc.z = fmaf(wc[2 * taps + j], x.z, acc.z);
                acc.w = fmaf(wc[3 * taps + j], x.w, acc.w);
            }
            if (act == 1) {
                acc.x = acc.x / (1.0f + expf(-acc.x));
                acc.y = acc.y / (1.0f + expf(-acc.y));
                acc.z = acc.z / (1.0f + expf(-acc.z));
                acc.w = acc.w / (1.0f + expf(-acc.w));
            }
            store4<O>(out + (size_t)(a + li) * ld_out + c, acc);
            if (dup) store4<O>(out + (size_t)(a + li) * ld_out + c + dup_n, acc);
        }
    }
    if (i != 0) return;
    for (int k = 0; k < Hh; ++k) {                          // ascending: entry n + k > k is still the old one
        const int src = n - Hh + k;
        *reinterpret_cast<float4*>(st + (size_t)k * C) =
            src >= 0 ? *reinterpret_cast<const float4*>(u + (size_t)(a + src) * ld_in + c)
                     : *reinterpret_cast<const float4*>(st + (size_t)(n + k) * C);
    }
}

extern "C" int aie_causal_conv(const float* u, int ld_in, const float* w, const float* bias, float* state, void* out,
                               int out_dtype, int ld_out, const int* q_start, const int* q_len, const int* slots,
                               const int* token_req, int T, int C, int taps, int residual, int act, int dup_from,
                               int dup_n, int max_slots, unsigned* err, cudaStream_t st) {
    if (T <= 0) return 0;
    if (C <= 0 || taps < 1 || act < 0 || act > 1 || dup_n < 0 || (dup_n && (dup_from < 0 || dup_from + dup_n != C)))
        return AIE_BAD_ARG;
    const int esz = out_dtype == AIE_F32 ? 4 : 2;
    if (C % 4 == 0 && ld_in % 4 == 0 && ld_out % 4 == 0 && dup_from % 4 == 0 && dup_n % 4 == 0 && !((size_t)u & 15) &&
        !((size_t)state & 15) && !((size_t)out & (4 * esz - 1)) && (!bias || !((size_t)bias & 15)) &&
        (out_dtype == AIE_F32 || out_dtype == AIE_BF16)) {
        const int threads4 = 64;
        dim3 grid4(T, (C / 4 + threads4 - 1) / threads4);
        if (out_dtype == AIE_F32)
            causal_conv4_kernel<float><<<grid4, threads4, 0, st>>>(u, ld_in, w, bias, state, (float*)out, ld_out, q_start, q_len, slots, token_req, C, taps, residual, act, dup_from, dup_n, max_slots, err);
        else
            causal_conv4_kernel<bf16><<<grid4, threads4, 0, st>>>(u, ld_in, w, bias, state, (bf16*)out, ld_out, q_start, q_len, slots, token_req, C, taps, residual, act, dup_from, dup_n, max_slots, err);
        AIE_LAUNCH_CHECK();
    }
    const int threads = C >= 256 ? 256 : 128;
    dim3 grid(T, (C + threads - 1) / threads);
    if (grid.y > 65535) return AIE_UNSUPPORTED;
    if (out_dtype == AIE_F32)
        causal_conv_kernel<float><<<grid, threads, 0, st>>>(u, ld_in, w, bias, state, (float*)out, ld_out, q_start, q_len, slots, token_req, C, taps, residual, act, dup_from, dup_n, max_slots, err);
    else if (out_dtype == AIE_BF16)
        causal_conv_kernel<bf16><<<grid, threads, 0, st>>>(u, ld_in, w, bias, state, (bf16*)out, ld_out, q_start, q_len, slots, token_req, C, taps, residual, act, dup_from, dup_n, max_slots, err);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// Gate, then norm in equal parts of the width: g = y * silu(z); out = g / sqrt(mean_part(g^2) + eps) * w.
// y [T, W] float32; z rows of ldz floats (a slice of a wider projection); w [W]; `parts` equal parts of W,
// each divided by its own root mean square.  One block per (token, part).
// ---------------------------------------------------------------------------
template <typename O>
__global__ void gate_group_norm_kernel(const float* __restrict__ y, const float* __restrict__ z, int ldz,
                                       const float* __restrict__ w, O* __restrict__ out, int W, int parts, float eps) {
    __shared__ float red[32];
    const int t = blockIdx.x / parts, p = blockIdx.x % parts, n = W / parts;
    const float* yr = y + (size_t)t * W + (size_t)p * n;
    const float* zr = z + (size_t)t * ldz + (size_t)p * n;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float zv = zr[i], g = yr[i] * (zv / (1.0f + expf(-zv)));
        ss = fmaf(g, g, ss);
    }
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float zv = zr[i], g = yr[i] * (zv / (1.0f + expf(-zv)));
        out[(size_t)t * W + (size_t)p * n + i] = from_f32<O>(g * r * w[(size_t)p * n + i]);
    }
}

extern "C" int aie_gate_group_norm(const float* y, const float* z, int ldz, const float* w, void* out, int out_dtype,
                                   int T, int W, int parts, float eps, cudaStream_t st) {
    if (T <= 0) return 0;
    if (W <= 0 || parts <= 0 || W % parts) return AIE_BAD_ARG;
    const int n = W / parts, threads = n >= 1024 ? 256 : (n >= 256 ? 128 : 64);
    const long long blocks = (long long)T * parts;
    if (blocks > 0x7fffffffLL) return AIE_UNSUPPORTED;
    if (out_dtype == AIE_F32)
        gate_group_norm_kernel<float><<<(unsigned)blocks, threads, 0, st>>>(y, z, ldz, w, (float*)out, W, parts, eps);
    else if (out_dtype == AIE_BF16)
        gate_group_norm_kernel<bf16><<<(unsigned)blocks, threads, 0, st>>>(y, z, ldz, w, (bf16*)out, W, parts, eps);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// A router's choice, per token, float32: s = softmax(z) over the E outputs; the choice is made on s + correction;
// the outputs form `groups` equal groups of neighbours, a group counts as its best member, and only members of the
// `keep` best groups can be chosen (the others count as minus infinity); the `top` largest are taken, and their
// weights are their s.  z [T, E] (rows ld floats apart) is replaced by s; scratch [T, E]; ids, weights [T, top].
// Variants: sigmoid != 0: s = sigmoid(z) per output instead of the softmax; group_top n > 1: a group counts as the sum
// of its n largest members; normalise != 0: the chosen weights are divided by their sum (+ 1e-20); all weights are
// multiplied by weight_scale.  One thread per token.
// ---------------------------------------------------------------------------
__global__ void route_topk_kernel(float* __restrict__ z, int ld, float* __restrict__ scratch, const float* __restrict__ corr,
                                  int T, int E, int groups, int keep, int top, int* __restrict__ ids,
                                  float* __restrict__ weights, int sigmoid, int group_top, int normalise,
                                  float weight_scale) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    float* s = z + (size_t)t * ld;
    float* c = scratch + (size_t)t * E;
    if (sigmoid) {
        for (int e = 0; e < E; ++e) {
            s[e] = 1.0f / (1.0f + expf(-s[e]));
            c[e] = s[e] + (corr ? corr[e] : 0.f);
        }
    } else {
        float m = -INFINITY;
        for (int e = 0; e < E; ++e) m = fmaxf(m, s[e]);
        float sum = 0.f;
        for (int e = 0; e < E; ++e) {
            const float v = expf(s[e] - m);
            s[e] = v;
            sum += v;
        }
        for (int e = 0; e < E; ++e) {
            s[e] = s[e] / sum;
            c[e] = s[e] + (corr ? corr[e] : 0.f);
        }
    }
    const int per = E / groups;
    if (keep < groups) {
        unsigned long long kept = 0ull;                     // groups <= 64 (checked by the launcher)
        for (int k = 0; k < keep; ++k) {
            int bg = -1;
            float bv = -INFINITY;
            for (int g = 0; g < groups; ++g) {
                if (kept >> g & 1ull) continue;
                float gv = -INFINITY;
                if (group_top <= 1) {
                    for (int e = g * per; e < (g + 1) * per; ++e) gv = fmaxf(gv, c[e]);
                } else {                                    // the sum of the group's group_top largest members
                    gv = 0.f;
                    float bound = INFINITY;                 // members are taken in descending order; ties by index
                    int bound_e = -1;
                    for (int n = 0; n < group_top && n < per; ++n) {
                        float best = -INFINITY;
                        int best_e = -1;
                        for (int e = g * per; e < (g + 1) * per; ++e) {
                            const bool below = c[e] < bound || (c[e] == bound && e > bound_e);
                            if (below && (best_e < 0 || c[e] > best)) {
                                best = c[e];
                                best_e = e;
                            }
                        }
                        if (best_e < 0) break;
                        gv += best;
                        bound = best;
                        bound_e = best_e;
                    }
                }
                if (bg < 0 || gv > bv) {
                    bg = g;
                    bv = gv;
                }
            }
            if (bg >= 0) kept |= 1ull << bg;
        }
        for (int g = 0; g < groups; ++g)
            if (!(kept >> g & 1ull))
                for (int e = g * per; e < (g + 1) * per; ++e) c[e] = -INFINITY;
    }
    for (int k = 0; k < top; ++k) {
        int be = -1;
        float bv = -INFINITY;
        for (int e = 0; e < E; ++e)
            if (c[e] > bv) {
                be = e;
                bv = c[e];
            }
        ids[(size_t)t * top + k] = be;
        weights[(size_t)t * top + k] = be >= 0 ? s[be] : 0.f;
        if (be >= 0) c[be] = -INFINITY;
    }
    float div = 1.f;
    if (normalise) {
        float sum = 0.f;
        for (int k = 0; k < top; ++k) sum += weights[(size_t)t * top + k];
        div = sum + 1e-20f;
    }
    if (normalise || weight_scale != 1.f)
        for (int k = 0; k < top; ++k) weights[(size_t)t * top + k] = weights[(size_t)t * top + k] / div * weight_scale;
}

extern "C" int aie_route_topk(float* z, int ld, float* scratch, const float* corr, int T, int E, int groups, int keep, int top,
                              int* ids, float* weights, int sigmoid, int group_top, int normalise, float weight_scale,
                              cudaStream_t st) {
    if (T <= 0) return 0;
    if (E <= 0 || ld < E || groups <= 0 || E % groups || keep <= 0 || keep > groups || top <= 0 || top > E / groups * keep)
        return AIE_BAD_ARG;
    if (groups > 64) return AIE_UNSUPPORTED;
    route_topk_kernel<<<(T + 63) / 64, 64, 0, st>>>(z, ld, scratch, corr, T, E, groups, keep, top, ids, weights, sigmoid,
                                                    group_top, normalise, weight_scale);
    AIE_LAUNCH_CHECK();
}

// out[t] = sum_s weight[t, s] * (row >= 0 ? y[row] : row == -2 ? h[t] : 0),  row = pair_row[t top + s]      float32
// (a pair marked -2 belongs to an expert that hands its input on unchanged); with `shared` (float32 [parts, T, D], the
// parts shared_stride floats apart): the sum of its parts is added, an expert that every token uses
template <typename A>
__global__ void expert_combine_weighted_kernel(const float* __restrict__ y, const int* __restrict__ pair_row,
                                               const float* __restrict__ weight, int top, const A* __restrict__ h,
                                               float* __restrict__ out, int D, const float* __restrict__ shared,
                                               int shared_parts, size_t shared_stride) {
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < top; ++s) {
            const int row = pair_row[(size_t)t * top + s];
            const float w = weight[(size_t)t * top + s];
            if (row >= 0) acc = fmaf(w, y[(size_t)row * D + c], acc);
            else if (row == -2) acc = fmaf(w, to_f32<A>(h[(size_t)t * D + c]), acc);
        }
        if (shared) {
            float sh = 0.f;
            for (int p = 0; p < shared_parts; ++p) sh += shared[p * shared_stride + (size_t)t * D + c];
            acc += sh;
        }
        out[(size_t)t * D + c] = acc;
    }
}

extern "C" int aie_expert_combine_weighted(const float* y, const int* pair_row, const float* weight, int top,
                                           const void* h, int h_dtype, float* out, int T, int D, const float* shared,
                                           int shared_parts, long long shared_stride, cudaStream_t st) {
    if (T <= 0) return 0;
    if (D <= 0 || top <= 0) return AIE_BAD_ARG;
    const int threads = D >= 1024 ? 256 : 128;
    if (h_dtype == AIE_BF16)
        expert_combine_weighted_kernel<bf16><<<T, threads, 0, st>>>(y, pair_row, weight, top, (const bf16*)h, out, D, shared, shared_parts, (size_t)shared_stride);
    else
        expert_combine_weighted_kernel<float><<<T, threads, 0, st>>>(y, pair_row, weight, top, (const float*)h, out, D, shared, shared_parts, (size_t)shared_stride);
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// RMS norm of a slice of a wider projection: out[t, :] = x[t, :n] / sqrt(mean(x[t, :n]^2) + eps) * w, rows of x
// `ld` floats apart, float32 statistics.  One block per token.
// ---------------------------------------------------------------------------
template <typename O>
__global__ void slice_rmsnorm_kernel(const float* __restrict__ x, int ld, const float* __restrict__ w, O* __restrict__ out,
                                     int n, float eps) {
    __shared__ float red[32];
    const float* row = x + (size_t)blockIdx.x * ld;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss += row[i] * row[i];
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) out[(size_t)blockIdx.x * n + i] = from_f32<O>((row[i] * r) * w[i]);
}

extern "C" int aie_slice_rmsnorm(const float* x, int ld, const float* w, void* out, int out_dtype, int T, int n, float eps,
                                 cudaStream_t st) {
    if (T <= 0) return 0;
    if (n <= 0 || ld < n) return AIE_BAD_ARG;
    const int threads = n >= 1024 ? 256 : 128;
    if (out_dtype == AIE_F32) slice_rmsnorm_kernel<float><<<T, threads, 0, st>>>(x, ld, w, (float*)out, n, eps);
    else if (out_dtype == AIE_BF16) slice_rmsnorm_kernel<bf16><<<T, threads, 0, st>>>(x, ld, w, (bf16*)out, n, eps);
    else return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}
