// Softmax attention with a distance bias, a window that keeps the first tokens, a sink and a gate per head,
// over a paged cache of one plane whose rows hold a key (d elements) and behind it a value (e elements).
//
//   s(i, j) = (q_i . k_j) * scale * temp[h] - slope[h] * (i - j)
//   i reads j  iff  j <= i and (window <= 0 or i - j < window or j < keep_first)
//   out_i = gate[i, h] * sum_j exp(s(i, j)) v_j / (exp(sink[h]) + sum_j exp(s(i, j)))
//
// The sink is a term of the denominator that has no key and no value.  Scores, weights and sums are float32.
//
//   sink_attn_prepare    from a step's fused projection [q | k | v | gate logits] (float32): adds the biases,
//                        writes q in the compute dtype, divides each head's value by its root mean square
//                        (no weight) and writes key and value into the token's cache row, gate = sigmoid.
//   normed_attn_prepare  for a layer that norms and rotates instead: from a fused projection whose first columns are
//                        [q | k | v] it adds the biases, divides all of q (and all of k) by its root mean square
//                        over the whole projection, times a weight per element, rotates the first rot_dims
//                        elements of every head (neighbouring pairs, or halves), mixes the value with another
//                        layer's value of the same token, and writes q and the cache row [k | v].
//   sink_attention_plain one block per (query token, head), any sizes up to 256; keys are walked in chunks of
//                        128 that start at multiples of 128 of the absolute key position, so the order of
//                        every addition depends on the query's position only.
#include "common.cuh"

#define SA_CHUNK 128

template <typename A, typename C>
__global__ void __launch_bounds__(256)
sink_attn_prepare_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ bias, A* __restrict__ q_out,
                         C* __restrict__ pages, float* __restrict__ gate_out, const int* __restrict__ positions,
                         const int* __restrict__ token_req, const int* __restrict__ block_table, int bt_width,
                         int num_pages, int P, int H, int G, int d, int e, float eps, int write, unsigned* err) {
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    const float* row = proj + (size_t)t * ld;
    const int nq = H * d, nk = G * d, nv = G * e;
    for (int c = tid; c < nq; c += blockDim.x)
        q_out[(size_t)t * nq + c] = from_f32<A>(row[c] + (bias ? bias[c] : 0.f));
    for (int h = tid; h < H; h += blockDim.x)
        gate_out[(size_t)t * H + h] = 1.f / (1.f + expf(-row[nq + nk + nv + h]));
    if (!write) return;
    const int pos = positions[t], r = token_req[t];
    const int pidx = pos / P;
    const int page = pidx < bt_width ? block_table[(size_t)r * bt_width + pidx] : -1;
    if (page < 0 || page >= num_pages) {
        if (tid == 0) atomicOr(err, AIE_DEV_PAGE_OOB);
        return;
    }
    const int w = d + e;
    for (int g = warp; g < G; g += nw) {          // a warp per key/value head
        C* dst = pages + (((size_t)page * G + g) * P + (pos % P)) * w;
        for (int c = lane; c < d; c += 32)
            dst[c] = from_f32<C>(row[nq + g * d + c] + (bias ? bias[nq + g * d + c] : 0.f));
        float ss = 0.f;
        for (int c = lane; c < e; c += 32) {
            const float v = row[nq + nk + g * e + c] + (bias ? bias[nq + nk + g * e + c] : 0.f);
            ss += v * v;
        }
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)e + eps);
        for (int c = lane; c < e; c += 32) {
            const float v = row[nq + nk + g * e + c] + (bias ? bias[nq + nk + g * e + c] : 0.f);
            dst[d + c] = from_f32<C>(v * inv);
        }
    }
}

extern "C" int aie_sink_attn_prepare(const float* proj, int ld, const float* bias, void* q_out, int q_dtype, void* pages,
                                     int cache_dtype, float* gate_out, const int* positions, const int* token_req,
                                     const int* block_table, int bt_width, int num_pages, int P, int T, int H, int G,
                                     int d, int e, float eps, int write, unsigned* err, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || d <= 0 || e <= 0 || q_dtype != cache_dtype) return AIE_BAD_ARG;
#define AIE_SAP(A)                                                                                                    \
    sink_attn_prepare_kernel<A, A><<<T, 256, 0, stream>>>(proj, ld, bias, (A*)q_out, (A*)pages, gate_out, positions,    \
                                                         token_req, block_table, bt_width, num_pages, P, H, G, d, e,  \
                                                         eps, write, err)
    if (q_dtype == AIE_F32) AIE_SAP(float);
    else if (q_dtype == AIE_BF16) AIE_SAP(bf16);
    else return AIE_BAD_ARG;
#undef AIE_SAP
    AIE_LAUNCH_CHECK();
}

// The two elements of pair j (of rot_dims / 2) of a head that starts at x, turned by `pos`: neighbours (2j, 2j + 1) or,
// with `halves`, (j, j + rot_dims / 2).  One sincosf a pair.
__device__ __forceinline__ void head_pair_rotated(const float* x, int j, int rot_dims, int halves, int pos,
                                                  const float* __restrict__ inv_freq, int* ia, int* ib, float* ya,
                                                  float* yb) {
    const int a = halves ? j : 2 * j, b = halves ? j + (rot_dims >> 1) : 2 * j + 1;
    float sn, cs;
    sincosf((float)pos * inv_freq[j], &sn, &cs);
    *ia = a;
    *ib = b;
    *ya = x[a] * cs - x[b] * sn;
    *yb = x[b] * cs + x[a] * sn;
}

// proj [T, >= H d + G d + G e] float32; bias [H d + G d + G e] or null; q_w [H d], k_w [G d] float32 or null (no norm).
// mix_from [T, G e] float32 with lambda (one float on the device): v <- (1 - lambda) v + lambda mix_from[t].
// v_keep [T, G e]: receives v as it is cached, in float32 (for the layers that mix with it).
template <typename A>
__global__ void __launch_bounds__(256)
normed_attn_prepare_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ bias,
                           const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                           const float* __restrict__ inv_freq, int rot_dims, int halves,
                           const float* __restrict__ mix_from, const float* __restrict__ lambda,
                           float* __restrict__ v_keep, A* __restrict__ q_out, A* __restrict__ pages,
                           const int* __restrict__ positions, const int* __restrict__ token_req,
                           const int* __restrict__ block_table, int bt_width, int num_pages, int P, int H, int G, int d,
                           int e, int write, unsigned* err) {
    extern __shared__ __align__(16) float np_sm[];     // q (H d) | k (G d) | 32
    const int t = blockIdx.x, tid = threadIdx.x;
    const int nq = H * d, nk = G * d, nv = G * e;
    float* qs = np_sm;
    float* ks = qs + nq;
    float* red = ks + nk;
    const float* row = proj + (size_t)t * ld;
    float ssq = 0.f, ssk = 0.f;
    for (int c = tid; c < nq; c += blockDim.x) {
        const float x = row[c] + (bias ? bias[c] : 0.f);
        qs[c] = x;
        ssq += x * x;
    }
    for (int c = tid; c < nk; c += blockDim.x) {
        const float x = row[nq + c] + (bias ? bias[nq + c] : 0.f);
        ks[c] = x;
        ssk += x * x;
    }
    ssq = block_sum(ssq, red);
    ssk = block_sum(ssk, red);
    if (q_w) {
        const float rq = 1.0f / sqrtf(ssq / (float)nq + eps), rk = 1.0f / sqrtf(ssk / (float)nk + eps);
        for (int c = tid; c < nq; c += blockDim.x) qs[c] = (qs[c] * rq) * q_w[c];
        for (int c = tid; c < nk; c += blockDim.x) ks[c] = (ks[c] * rk) * k_w[c];
    }
    __syncthreads();
    const int pos = positions[t];
    const int half = rot_dims >> 1, rest = d - rot_dims;
    for (int p = tid; p < H * half; p += blockDim.x) {            // a thread a pair
        const int hh = p / half, j = p - hh * half;
        int ia, ib;
        float ya, yb;
        head_pair_rotated(qs + hh * d, j, rot_dims, halves, pos, inv_freq, &ia, &ib, &ya, &yb);
        q_out[(size_t)t * nq + hh * d + ia] = from_f32<A>(ya);
        q_out[(size_t)t * nq + hh * d + ib] = from_f32<A>(yb);
    }
    for (int p = tid; p < H * rest; p += blockDim.x) {            // what the rotation leaves as it is
        const int c = (p / rest) * d + rot_dims + p % rest;
        q_out[(size_t)t * nq + c] = from_f32<A>(qs[c]);
    }
    const int pidx = pos / P;
    const int page = (pos >= 0 && pidx < bt_width) ? block_table[(size_t)token_req[t] * bt_width + pidx] : -1;
    const bool page_ok = page >= 0 && page < num_pages;
    if (write && !page_ok && tid == 0) atomicOr(err, AIE_DEV_PAGE_OOB);
    const int w = d + e;
    A* base = pages + ((size_t)(page_ok ? page : 0) * G * P + (pos % P)) * w;
    if (write && page_ok) {
        for (int p = tid; p < G * half; p += blockDim.x) {
            const int g = p / half, j = p - g * half;
            int ia, ib;
            float ya, yb;
            head_pair_rotated(ks + g * d, j, rot_dims, halves, pos, inv_freq, &ia, &ib, &ya, &yb);
            base[(size_t)g * P * w + ia] = from_f32<A>(ya);
            base[(size_t)g * P * w + ib] = from_f32<A>(yb);
        }
        for (int p = tid; p < G * rest; p += blockDim.x) {
            const int g = p / rest, i = rot_dims + p % rest;
            base[(size_t)g * P * w + i] = from_f32<A>(ks[g * d + i]);
        }
    }
    const float lam = mix_from ? lambda[0] : 0.f;
    for (int c = tid; c < nv; c += blockDim.x) {
        float v = row[nq + nk + c] + (bias ? bias[nq + nk + c] : 0.f);
        if (mix_from) v = (1.0f - lam) * v + lam * mix_from[(size_t)t * nv + c];
        if (v_keep) v_keep[(size_t)t * nv + c] = v;
        if (write && page_ok) {
            const int g = c / e;
            base[(size_t)g * P * w + d + (c - g * e)] = from_f32<A>(v);
        }
    }
}

extern "C" int aie_normed_attn_prepare(const float* proj, int ld, const float* bias, const float* q_w, const float* k_w,
                                       float eps, const float* inv_freq, int rot_dims, int halves, const float* mix_from,
                                       const float* lambda, float* v_keep, void* q_out, void* pages, int dtype,
                                       const int* positions, const int* token_req, const int* block_table, int bt_width,
                                       int num_pages, int P, int T, int H, int G, int d, int e, int write, unsigned* err,
                                       cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || d <= 0 || e <= 0 || rot_dims < 0 || rot_dims > d || rot_dims % 2 ||
        (mix_from && !lambda) || (q_w && !k_w) || (rot_dims > 0 && !inv_freq))
        return AIE_BAD_ARG;
    const size_t smem = ((size_t)(H + G) * d + 32) * sizeof(float);
    if (smem > 48 * 1024) return AIE_UNSUPPORTED;
#define AIE_NAP(A)                                                                                                    \
    normed_attn_prepare_kernel<A><<<T, 256, smem, stream>>>(proj, ld, bias, q_w, k_w, eps, inv_freq, rot_dims, halves, \
                                                           mix_from, lambda, v_keep, (A*)q_out, (A*)pages, positions, \
                                                           token_req, block_table, bt_width, num_pages, P, H, G, d, e, \
                                                           write, err)
    if (dtype == AIE_F32) AIE_NAP(float);
    else if (dtype == AIE_BF16) AIE_NAP(bf16);
    else return AIE_BAD_ARG;
#undef AIE_NAP
    AIE_LAUNCH_CHECK();
}

template <typename A, typename C>
__global__ void __launch_bounds__(SA_CHUNK)
sink_attention_plain_kernel(const A* __restrict__ q, const C* __restrict__ pages, A* __restrict__ out,
                            const float* __restrict__ gate, const float* __restrict__ temp,
                            const float* __restrict__ slope, const float* __restrict__ sink,
                            const int* __restrict__ positions, const int* __restrict__ token_req,
                            const int* __restrict__ block_table, int bt_width, int num_pages, int P, int H, int G,
                            int d, int e, int window, int keep_first, float scale,
                            const int* __restrict__ token_list, unsigned* err) {
    extern __shared__ __align__(16) float sm[];
    float* q_s = sm;                                  // d (rounded up to even)
    float* p_s = q_s + ((d + 1) & ~1);                // CHUNK
    float* red = p_s + SA_CHUNK;                      // 32
    long long* off_s = (long long*)(red + 32);        // CHUNK

    const int t = token_list ? token_list[blockIdx.x] : blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int pos = positions[t];
    const int row = token_req[t];
    const int g = h / (H / G);
    const int w = d + e;
    const float qs = scale * (temp ? temp[h] : 1.f), sl = slope ? slope[h] : 0.f;
    for (int c = tid; c < d; c += blockDim.x) q_s[c] = to_f32<A>(q[((size_t)t * H + h) * d + c]);
    __syncthreads();

    int lo = 0;
    if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
    const int kept = min(keep_first, lo);              // keys [0, kept) are read although the window has passed them
    // the sink opens the running softmax: a weight exp(sink - m) = 1 at m = sink, with no value
    float m = sink ? sink[h] : -INFINITY, l = sink ? 1.f : 0.f;
    float acc0 = 0.f, acc1 = 0.f;                      // value elements tid and tid + 128 (e <= 256)

    const int first_b = (lo / SA_CHUNK) * SA_CHUNK;    // chunk of the window's first key
    for (int c0 = 0; c0 <= pos; c0 += SA_CHUNK) {
        if (c0 >= kept && c0 < first_b) {              // between the kept keys and the window: nothing to read
            c0 = first_b - SA_CHUNK;
            continue;
        }
        const int kp = c0 + tid;
        const bool valid = kp <= pos && (kp >= lo || kp < kept);
        float s = -INFINITY;
        long long off = -1;
        if (valid) {
            const int pidx = kp / P;
            const int page = pidx < bt_width ? block_table[(size_t)row * bt_width + pidx] : -1;
            if (page < 0 || page >= num_pages) {
                atomicOr(err, AIE_DEV_PAGE_OOB);
            } else {
                off = (((long long)page * G + g) * P + (kp % P)) * w;
                const C* kr = pages + off;
                float dot = 0.f;
                for (int c = 0; c < d; ++c) dot += q_s[c] * to_f32<C>(kr[c]);
                s = dot * qs - sl * (float)(pos - kp);
            }
        }
        off_s[tid] = off;
        const float cmax = block_max(s, red);
        const float m_new = fmaxf(m, cmax);
        const float p = (off >= 0) ? expf(s - m_new) : 0.f;
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        p_s[tid] = p;
        const float csum = block_sum(p, red);          // has __syncthreads inside: p_s, off_s visible
        l = l * corr + csum;
        m = m_new;
        acc0 *= corr;
        acc1 *= corr;
        const int n = min(SA_CHUNK, pos - c0 + 1);
        for (int j = 0; j < n; ++j) {
            const long long o = off_s[j];
            if (o < 0) continue;
            const float pj = p_s[j];
            if (tid < e) acc0 += pj * to_f32<C>(pages[o + d + tid]);
            if (tid + SA_CHUNK < e) acc1 += pj * to_f32<C>(pages[o + d + tid + SA_CHUNK]);
        }
        __syncthreads();
    }
    const float inv = (l > 0.f ? 1.0f / l : 0.f) * (gate ? gate[(size_t)t * H + h] : 1.f);
    A* o = out + ((size_t)t * H + h) * e;
    if (tid < e) o[tid] = from_f32<A>(acc0 * inv);
    if (tid + SA_CHUNK < e) o[tid + SA_CHUNK] = from_f32<A>(acc1 * inv);
}

extern "C" int aie_sink_attention_plain(const void* q, const void* pages, void* out, int dtype, const float* gate,
                                        const float* temp, const float* slope, const float* sink, const int* positions,
                                        const int* token_req, const int* block_table, int bt_width, int num_pages,
                                        int P, int T, int H, int G, int d, int e, int window, int keep_first,
                                        float scale, const int* token_list, unsigned* err, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0 || d > 2 * SA_CHUNK || e <= 0 || e > 2 * SA_CHUNK || G <= 0 || H % G || H > 65535) return AIE_UNSUPPORTED;
    const size_t smem = (size_t)(((d + 1) & ~1) + SA_CHUNK + 32) * sizeof(float) + SA_CHUNK * sizeof(long long);
    dim3 grid(T, H);
#define AIE_SA(A)                                                                                                      \
    sink_attention_plain_kernel<A, A><<<grid, SA_CHUNK, smem, stream>>>(                                               \
        (const A*)q, (const A*)pages, (A*)out, gate, temp, slope, sink, positions, token_req, block_table, bt_width,   \
        num_pages, P, H, G, d, e, window, keep_first, scale, token_list, err)
    if (dtype == AIE_F32) AIE_SA(float);
    else if (dtype == AIE_BF16) AIE_SA(bf16);
    else return AIE_BAD_ARG;
#undef AIE_SA
    AIE_LAUNCH_CHECK();
}
