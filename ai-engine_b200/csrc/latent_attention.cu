// Attention over a compressed cache: per token the cache holds one latent vector c [rank] (shared by all
// heads, normalised) and one rotated key part kr [rot] (shared by all heads), together one row of
// dk = rank + rot elements.  A head's key is [W_uk c | kr] and its value W_uv c; with the up-projections
// folded into the query (qa = W_uk^T q_plain) and applied to the output (o = W_uv (sum_j p_j c_j)) the
// kernel reads the cache rows as they are: score_j = (qa . c_j + q_rot . kr_j) * scale, one "kv head" for all
// query heads.
//
// latent_prepare: from the fused projection [q heads | c | kr] of the step's tokens it writes the plain
//   query parts (compute dtype, for the folding product), the rotated query parts (float32), and the
//   normalised c and rotated kr into the token's cache row.  The rotation pairs element 2i with 2i+1 over the
//   first `rot_dims` elements of the rot-wide part (or, with `halves`, element i with i + rot_dims / 2); the
//   angle is float(position) * inv_freq[i] in float32.  The latent and the key part may come from a projection
//   of their own (`kv`, rows ld_kv floats apart) when the queries are made by a second product.
// latent_attention: one block per (token, head); keys in chunks of 128 that start at multiples of 128 of the
//   absolute key position with a running maximum and sum, so a row's additions depend on its position only.
#include "common.cuh"

#define LAT_CHUNK 128

// element i of a rot-wide vector x after the rotation by `pos`
__device__ __forceinline__ float latent_rotated(const float* x, int i, int half, int halves, int pos,
                                                const float* __restrict__ inv_freq) {
    if (i >= 2 * half) return x[i];
    float sn, cs;
    if (halves) {
        const int j = i < half ? i : i - half;
        sincosf((float)pos * inv_freq[j], &sn, &cs);
        return i < half ? x[i] * cs - x[i + half] * sn : x[i] * cs + x[j] * sn;
    }
    sincosf((float)pos * inv_freq[i >> 1], &sn, &cs);
    return (i & 1) ? x[i] * cs + x[i - 1] * sn : x[i] * cs - x[i + 1] * sn;
}

template <typename A, typename C>
__global__ void latent_prepare_kernel(const float* __restrict__ proj, int ld, int H, int d, int rot, int rank,
                                      int rot_dims, int has_kv, const float* __restrict__ c_weight, float eps,
                                      const float* __restrict__ inv_freq, A* __restrict__ q_plain,
                                      float* __restrict__ q_full, C* __restrict__ pages,
                                      const int* __restrict__ positions, const int* __restrict__ token_req,
                                      const int* __restrict__ block_table, int bt_width, int num_pages, int P,
                                      unsigned* err, const float* __restrict__ kv, int ld_kv, int halves) {
    __shared__ float red[32];
    const int t = blockIdx.x, tid = threadIdx.x;
    const float* row = proj + (size_t)t * ld;
    const int pos = positions[t];
    const int dq = d + rot, dk = rank + rot, half = rot_dims / 2;
    // queries: the plain part as it is, the rotated part turned by the position
    for (int e = tid; e < H * d; e += blockDim.x) {
        const int hh = e / d, i = e % d;
        q_plain[((size_t)t * H + hh) * d + i] = from_f32<A>(row[hh * dq + i]);
    }
    for (int e = tid; e < H * rot; e += blockDim.x) {
        const int hh = e / rot, i = e % rot;
        const float* qr = row + hh * dq + d;
        q_full[((size_t)t * H + hh) * dk + rank + i] = latent_rotated(qr, i, half, halves, pos, inv_freq);
    }
    if (!has_kv) return;
    const float* z = kv ? kv + (size_t)t * ld_kv : row + H * dq;
    float ss = 0.f;
    for (int i = tid; i < rank; i += blockDim.x) ss += z[i] * z[i];
    ss = block_sum(ss, red);
    const float rinv = 1.0f / sqrtf(ss / (float)rank + eps);
    const int pidx = pos / P;
    const int page = (pos >= 0 && pidx < bt_width) ? block_table[(size_t)token_req[t] * bt_width + pidx] : -1;
    if (page < 0 || page >= num_pages) {
        if (tid == 0) atomicOr(err, AIE_DEV_PAGE_OOB);
        return;
    }
    C* dst = pages + ((size_t)page * P + (pos - pidx * P)) * dk;
    for (int i = tid; i < rank; i += blockDim.x) dst[i] = from_f32<C>((z[i] * rinv) * c_weight[i]);
    const float* kr = z + rank;
    for (int i = tid; i < rot; i += blockDim.x) dst[rank + i] = from_f32<C>(latent_rotated(kr, i, half, halves, pos, inv_freq));
}

extern "C" int aie_latent_prepare(const float* proj, int ld, int T, int H, int d, int rot, int rank, int rot_dims,
                                  int has_kv, const float* c_weight, float eps, const float* inv_freq, void* q_plain,
                                  int q_dtype, float* q_full, void* pages, int cache_dtype, const int* positions,
                                  const int* token_req, const int* block_table, int bt_width, int num_pages, int P,
                                  unsigned* err, const float* kv, int ld_kv, int halves, cudaStream_t st) {
    if (T <= 0) return 0;
    if (rot_dims % 2 || rot_dims > rot || H <= 0 || d < 0 || rank <= 0) return AIE_BAD_ARG;
#define GO(A, C)                                                                                                      \
    latent_prepare_kernel<A, C><<<T, 128, 0, st>>>(proj, ld, H, d, rot, rank, rot_dims, has_kv, c_weight, eps, inv_freq, \
                                                   (A*)q_plain, q_full, (C*)pages, positions, token_req, block_table,  \
                                                   bt_width, num_pages, P, err, kv, ld_kv, halves)
    if (q_dtype == AIE_F32 && cache_dtype == AIE_F32) GO(float, float);
    else if (q_dtype == AIE_BF16 && cache_dtype == AIE_BF16) GO(bf16, bf16);
    else if (q_dtype == AIE_BF16 && cache_dtype == AIE_F32) GO(bf16, float);
    else if (q_dtype == AIE_F32 && cache_dtype == AIE_BF16) GO(float, bf16);
    else return AIE_BAD_ARG;
#undef GO
    AIE_LAUNCH_CHECK();
}

// q_full [T, H, dk] float32 (folded plain part | rotated part); pages [num_pages, P, dk]; out [T, H, rank].
template <typename C, typename O, int NACC>
__global__ void __launch_bounds__(LAT_CHUNK)
latent_attention_kernel(const float* __restrict__ q_full, const C* __restrict__ pages, O* __restrict__ out,
                        const int* __restrict__ positions, const int* __restrict__ token_req,
                        const int* __restrict__ block_table, int bt_width, int num_pages, int P, int H, int rank,
                        int dk, int window, float scale, unsigned* err) {
    extern __shared__ __align__(16) float sm[];
    float* q_s = sm;                                   // dk (rounded up to even)
    float* p_s = q_s + ((dk + 1) & ~1);                // CHUNK
    float* red = p_s + LAT_CHUNK;                      // 32
    long long* off_s = (long long*)(red + 32);         // CHUNK

    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int pos = positions[t], row = token_req[t];
    for (int e = tid; e < dk; e += blockDim.x) q_s[e] = q_full[((size_t)t * H + h) * dk + e];
    __syncthreads();

    int lo = 0;
    if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
    float m = -INFINITY, l = 0.f;
    float acc[NACC];
#pragma unroll
    for (int a = 0; a < NACC; ++a) acc[a] = 0.f;

    for (int c0 = (lo / LAT_CHUNK) * LAT_CHUNK; c0 <= pos; c0 += LAT_CHUNK) {
        const int kp = c0 + tid;
        const bool valid = kp >= lo && kp <= pos;
        float s = -INFINITY;
        long long off = -1;
        if (valid) {
            const int pidx = kp / P;
            const int page = pidx < bt_width ? block_table[(size_t)row * bt_width + pidx] : -1;
            if (page < 0 || page >= num_pages) {
                atomicOr(err, AIE_DEV_PAGE_OOB);
            } else {
                off = ((long long)page * P + (kp % P)) * dk;
                const C* kr = pages + off;
                float dot = 0.f;
                for (int e = 0; e < dk; ++e) dot = fmaf(q_s[e], to_f32<C>(kr[e]), dot);
                s = dot * scale;
            }
        }
        off_s[tid] = off;
        const float cmax = block_max(s, red);
        const float m_new = fmaxf(m, cmax);
        const float p = (off >= 0) ? expf(s - m_new) : 0.f;
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        p_s[tid] = p;
        const float csum = block_sum(p, red);
        l = l * corr + csum;
        m = m_new;
#pragma unroll
        for (int a = 0; a < NACC; ++a) acc[a] *= corr;
        const int n = min(LAT_CHUNK, pos - c0 + 1);
        for (int j = 0; j < n; ++j) {
            const long long o = off_s[j];
            if (o < 0) continue;
            const float pj = p_s[j];
#pragma unroll
            for (int a = 0; a < NACC; ++a)
                if (tid + a * LAT_CHUNK < rank) acc[a] = fmaf(pj, to_f32<C>(pages[o + tid + a * LAT_CHUNK]), acc[a]);
        }
        __syncthreads();
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    O* o = out + ((size_t)t * H + h) * rank;
#pragma unroll
    for (int a = 0; a < NACC; ++a)
        if (tid + a * LAT_CHUNK < rank) o[tid + a * LAT_CHUNK] = from_f32<O>(acc[a] * inv);
}

template <typename C, typename O>
static int latent_go(const float* q_full, const void* pages, void* out, const int* positions, const int* token_req,
                     const int* block_table, int bt_width, int num_pages, int P, int T, int H, int rank, int dk,
                     int window, float scale, unsigned* err, cudaStream_t st) {
    const size_t smem = (size_t)(((dk + 1) & ~1) + LAT_CHUNK + 32) * sizeof(float) + LAT_CHUNK * sizeof(long long);
    dim3 grid(T, H);
#define GO(N)                                                                                                        \
    latent_attention_kernel<C, O, N><<<grid, LAT_CHUNK, smem, st>>>(q_full, (const C*)pages, (O*)out, positions,     \
                                                                    token_req, block_table, bt_width, num_pages, P, \
                                                                    H, rank, dk, window, scale, err)
    if (rank <= LAT_CHUNK) GO(1);
    else if (rank <= 2 * LAT_CHUNK) GO(2);
    else if (rank <= 4 * LAT_CHUNK) GO(4);
    else GO(8);
#undef GO
    AIE_LAUNCH_CHECK();
}

extern "C" int aie_latent_attention(const float* q_full, const void* pages, int cache_dtype, void* out, int out_dtype,
                                    const int* positions, const int* token_req, const int* block_table, int bt_width,
                                    int num_pages, int P, int T, int H, int rank, int dk, int window, float scale,
                                    unsigned* err, cudaStream_t st) {
    if (T <= 0) return 0;
    if (rank <= 0 || dk < rank || H <= 0 || H > 65535) return AIE_BAD_ARG;
    if (rank > 8 * LAT_CHUNK || dk > 8192) return AIE_UNSUPPORTED;
    if (cache_dtype == AIE_F32 && out_dtype == AIE_F32)
        return latent_go<float, float>(q_full, pages, out, positions, token_req, block_table, bt_width, num_pages, P, T, H, rank, dk, window, scale, err, st);
    if (cache_dtype == AIE_BF16 && out_dtype == AIE_BF16)
        return latent_go<bf16, bf16>(q_full, pages, out, positions, token_req, block_table, bt_width, num_pages, P, T, H, rank, dk, window, scale, err, st);
    if (cache_dtype == AIE_BF16 && out_dtype == AIE_F32)
        return latent_go<bf16, float>(q_full, pages, out, positions, token_req, block_table, bt_width, num_pages, P, T, H, rank, dk, window, scale, err, st);
    return AIE_BAD_ARG;
}
