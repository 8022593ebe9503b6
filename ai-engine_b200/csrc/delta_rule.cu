// The gated delta rule, token by token: per request and head a matrix state S [d, e] (float32, in the
// request's slot) is decayed, corrected towards the token's value along its key, and read with its query:
//
//   q_t, k_t  <-  q_t / sqrt(|q_t|^2 + unit_eps) * q_scale,   k_t / sqrt(|k_t|^2 + unit_eps)
//   beta_t = sigmoid(b_t);   g_t = exp(-exp(a_log[h]) * softplus(a_t + dt_bias[h]))
//   S <- g_t S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
//
// With a = S^T k and b = S^T q taken on the state before the token, u = beta (v - g a) and
// o = g b + (k . q) u, so one pass over the state gives both sums and the update follows at once.
//
// One block per (request, head, 32 value columns): the columns of S are independent of one another.  A column
// is held by eight neighbouring lanes of a warp, each with every eighth row in registers; the sums over rows
// are joined by shuffles.  Sixteen tokens at a time are staged in shared memory, where a warp per token makes
// the unit vectors and k . q.  The order of all additions is fixed by this layout, so a token's output does not
// depend on how its request's tokens were cut into steps or on what else runs in the step.
#include "common.cuh"

#define DR_COLS 32       // value columns a block
#define DR_LANES 8       // lanes a column
#define DR_TOKENS 16     // tokens staged at a time
#define DR_THREADS (DR_COLS * DR_LANES)

template <int RPT>
__global__ void __launch_bounds__(DR_THREADS)
delta_rule_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, int ld,
                  const float* __restrict__ b_raw, int ldb, const float* __restrict__ a_raw, int lda,
                  const float* __restrict__ a_log, const float* __restrict__ dt_bias, float q_scale, float unit_eps,
                  float* __restrict__ state, float* __restrict__ out, const int* __restrict__ q_start,
                  const int* __restrict__ q_len, const int* __restrict__ slots, const int* __restrict__ live,
                  int H, int G, int d, int e, int max_seqs, int max_len, unsigned* err) {
    extern __shared__ __align__(16) float sm[];
    float* k_s = sm;                                   // [TOKENS][d]
    float* q_s = k_s + DR_TOKENS * d;                  // [TOKENS][d]
    float* v_s = q_s + DR_TOKENS * d;                  // [TOKENS][COLS]
    float* g_s = v_s + DR_TOKENS * DR_COLS;            // [TOKENS] decay
    float* be_s = g_s + DR_TOKENS;                     // [TOKENS] beta
    float* kq_s = be_s + DR_TOKENS;                    // [TOKENS] k . q

    const int r = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * DR_COLS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rl = lane & (DR_LANES - 1);              // which rows: rl, rl + 8, ...
    const int col = c0 + warp * (32 / DR_LANES) + (lane >> 3);
    const bool has_col = col < e;
    const int slot = slots[r];
    if (slot < 0 || slot >= max_seqs) {
        if (tid == 0) atomicOr(err, AIE_DEV_SLOT_OOB);
        return;
    }
    const int t0 = q_start[r], n = q_len[r];
    if (max_len > 0 && n > max_len) return;            // longer portions went to the chunked kernel
    const int kh = h / (H / G);
    float* S = state + ((size_t)slot * H + h) * d * e;
    float s[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int row = rl + DR_LANES * i;
        s[i] = (has_col && row < d) ? S[(size_t)row * e + col] : 0.f;
    }
    const float rate = expf(a_log[h]), bias = dt_bias[h];

    for (int base = 0; base < n; base += DR_TOKENS) {
        const int m = min(DR_TOKENS, n - base);
        __syncthreads();                               // the tokens staged before have been used
        for (int i = tid; i < m * d; i += DR_THREADS) {
            const int j = i / d, c = i - j * d;
            const size_t at = (size_t)(t0 + base + j) * ld + kh * d + c;
            k_s[j * d + c] = k[at];
            q_s[j * d + c] = q[at];
        }
        for (int i = tid; i < m * DR_COLS; i += DR_THREADS) {
            const int j = i / DR_COLS, c = i - j * DR_COLS;
            v_s[i] = (c0 + c < e) ? v[(size_t)(t0 + base + j) * ld + h * e + c0 + c] : 0.f;
        }
        if (tid < m) {
            const float x = a_raw[(size_t)(t0 + base + tid) * lda + h] + bias;
            const float sp = x > 20.f ? x : log1pf(expf(x));
            g_s[tid] = expf(-rate * sp);
            be_s[tid] = 1.f / (1.f + expf(-b_raw[(size_t)(t0 + base + tid) * ldb + h]));
        }
        __syncthreads();
        for (int j = warp; j < m; j += DR_THREADS / 32) {       // a warp per token: unit vectors and k . q
            float kk = 0.f, qq = 0.f;
            for (int c = lane; c < d; c += 32) {
                const float a = k_s[j * d + c], b = q_s[j * d + c];
                kk += a * a;
                qq += b * b;
            }
            kk = warp_sum(kk);
            qq = warp_sum(qq);
            const float ik = rsqrtf(kk + unit_eps), iq = rsqrtf(qq + unit_eps) * q_scale;
            float kq = 0.f;
            for (int c = lane; c < d; c += 32) {
                const float a = k_s[j * d + c] * ik, b = q_s[j * d + c] * iq;
                k_s[j * d + c] = a;
                q_s[j * d + c] = b;
                kq += a * b;
            }
            kq = warp_sum(kq);
            if (lane == 0) kq_s[j] = kq;
        }
        __syncthreads();
        for (int j = 0; j < m; ++j) {
            const float* kj = k_s + j * d;
            const float* qj = q_s + j * d;
            float a = 0.f, b = 0.f;
#pragma unroll
            for (int i = 0; i < RPT; ++i) {
                const int row = rl + DR_LANES * i;
                if (row < d) {
                    a += s[i] * kj[row];
                    b += s[i] * qj[row];
                }
            }
#pragma unroll
            for (int o = DR_LANES / 2; o > 0; o >>= 1) {
                a += __shfl_xor_sync(0xffffffffu, a, o);
                b += __shfl_xor_sync(0xffffffffu, b, o);
            }
            const float g = g_s[j];
            const float u = be_s[j] * (v_s[j * DR_COLS + (col - c0)] - g * a);
#pragma unroll
            for (int i = 0; i < RPT; ++i) {
                const int row = rl + DR_LANES * i;
                if (row < d) s[i] = g * s[i] + kj[row] * u;
            }
            if (rl == 0 && has_col) out[((size_t)(t0 + base + j) * H + h) * e + col] = g * b + kq_s[j] * u;
        }
    }
    if (has_col && (live == nullptr || live[r] != 0)) {
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
            const int row = rl + DR_LANES * i;
            if (row < d) S[(size_t)row * e + col] = s[i];
        }
    }
}

extern "C" int aie_delta_rule(const float* q, const float* k, const float* v, int ld, const float* b_raw, int ldb,
                              const float* a_raw, int lda, const float* a_log, const float* dt_bias, float q_scale,
                              float unit_eps, float* state, float* out, const int* q_start, const int* q_len,
                              const int* slots, const int* live, int R, int H, int G, int d, int e, int max_seqs,
                              int max_len, unsigned* err, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || d <= 0 || d > 256 || e <= 0 || H > 65535) return AIE_UNSUPPORTED;
    const size_t smem = (size_t)(2 * DR_TOKENS * d + DR_TOKENS * DR_COLS + 3 * DR_TOKENS) * sizeof(float);
    dim3 grid(R, H, (e + DR_COLS - 1) / DR_COLS);
#define AIE_DR(RPT)                                                                                                \
    delta_rule_kernel<RPT><<<grid, DR_THREADS, smem, stream>>>(q, k, v, ld, b_raw, ldb, a_raw, lda, a_log, dt_bias, \
                                                               q_scale, unit_eps, state, out, q_start, q_len, slots, \
                                                               live, H, G, d, e, max_seqs, max_len, err)
    if (d <= 32) AIE_DR(4);
    else if (d <= 64) AIE_DR(8);
    else if (d <= 128) AIE_DR(16);
    else AIE_DR(32);
#undef AIE_DR
    AIE_LAUNCH_CHECK();
}
