// The gated delta rule of a prompt portion in chunks, on tensor cores.  Token by token,
//     S_t = g_t S_(t-1) + k_t u_t^T,   u_t = beta_t (v_t - g_t S_(t-1)^T k_t),   o_t = S_t^T q_t     (S: [d, e], float32)
// is a chain of dependent rank-1 updates.  Over a chunk of Q tokens that starts from S_0, with the running sums
// l_t = sum_{s <= t} log g_s, the corrections u of all its tokens solve one lower-triangular system:
//     (I + A) U = beta * (V - diag(exp(l_t)) K S_0),     A[t, s] = beta_t exp(l_t - l_s) (k_t . k_s)   for s < t
//     O = diag(exp(l_t)) Q S_0 + P U,                    P[t, s] = exp(l_t - l_s) (q_t . k_s)          for s <= t
//     S_Q = exp(l_Q) S_0 + K^T (w * U),                  w_s = exp(l_Q - l_s)
// The system is solved in blocks of 16 rows: the diagonal blocks of I + A are inverted in float32 (16 steps of forward
// substitution, a thread per column), a block's right-hand side first loses what the blocks before it contribute (a
// product), then meets the inverse (a small float32 product).
// One CTA owns a (request, head, 64 or 32 value columns) and walks the request's chunks in order with the state in
// shared memory, so a portion continues where the last step stopped and no result depends on the batch.  The unit
// vectors q and k, A, P, U and the state enter the tensor cores as pairs of bfloat16 values, the rounded value and the
// rounded rest (16 bits of mantissa), in three products hi hi + hi lo + lo hi; sums, decays, beta and the solve are
// float32.  Exponents are never positive: nothing can overflow.
#include <mma.h>

#include "common.cuh"

using namespace nvcuda;

#define DC_Q 64
#define DC_THREADS 512
#define DC_WARPS 16
#define DC_PAD 8         // bfloat16 elements (16 bytes) behind every row in shared memory
#define DC_PADF 4        // the same 16 bytes behind float32 rows

typedef wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> FragA;
typedef wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::col_major> FragAT;
typedef wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::row_major> FragB;
typedef wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::col_major> FragBT;
typedef wmma::fragment<wmma::accumulator, 16, 16, 16, float> FragC;

__device__ __forceinline__ void dc_split(float v, bf16* hi, bf16* lo) {
    const bf16 h = __float2bfloat16_rn(v);
    *hi = h;
    *lo = __float2bfloat16_rn(v - __bfloat162float(h));
}

// acc += (aH + aL) (bH + bL) without the lo lo term, over `steps` tiles of 16 along the inner dimension.  The three
// products have an accumulator each, so that a warp has three independent chains of tensor-core instructions in flight.
template <class FA, class FB>
__device__ __forceinline__ void dc_mma3(FragC& acc, const bf16* aH, const bf16* aL, int lda, int a_step, const bf16* bH,
                                        const bf16* bL, int ldb, int b_step, int steps) {
    FragC hl, lh;
    wmma::fill_fragment(hl, 0.f);
    wmma::fill_fragment(lh, 0.f);
    for (int k = 0; k < steps; ++k) {
        FA ah, al;
        FB bh, bl;
        wmma::load_matrix_sync(ah, aH + (size_t)k * a_step, lda);
        wmma::load_matrix_sync(bh, bH + (size_t)k * b_step, ldb);
        wmma::load_matrix_sync(bl, bL + (size_t)k * b_step, ldb);
        wmma::load_matrix_sync(al, aL + (size_t)k * a_step, lda);
        wmma::mma_sync(acc, ah, bh, acc);
        wmma::mma_sync(hl, ah, bl, hl);
        wmma::mma_sync(lh, al, bh, lh);
    }
    for (int x = 0; x < acc.num_elements; ++x) acc.x[x] += hl.x[x] + lh.x[x];
}

// which tile of the ten on and below the diagonal of a 4 x 4 grid
__device__ __forceinline__ void dc_lower_tile(int tile, int* ti, int* tj) {
    const int i = tile < 1 ? 0 : (tile < 3 ? 1 : (tile < 6 ? 2 : 3));
    *ti = i;
    *tj = tile - i * (i + 1) / 2;
}

// NP: the state's rows padded to a multiple of 32 (zero rows and columns change nothing); DV: value columns a CTA
template <int NP, int DV>
__global__ void __launch_bounds__(DC_THREADS)
delta_rule_chunked_kernel(const float* __restrict__ qg, const float* __restrict__ kg, const float* __restrict__ vg, int ld,
                          const float* __restrict__ b_raw, int ldb, const float* __restrict__ a_raw, int lda,
                          const float* __restrict__ a_log, const float* __restrict__ dt_bias, float q_scale, float unit_eps,
                          float* __restrict__ state, float* __restrict__ out, const int* __restrict__ q_start,
                          const int* __restrict__ q_len, const int* __restrict__ slots, const int* __restrict__ live, int H,
                          int G, int d, int e, int col_blocks, int max_slots, int min_len, int vec4, unsigned* err) {
    extern __shared__ __align__(128) unsigned char dc_sm[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cb = blockIdx.x % col_blocks, h = (blockIdx.x / col_blocks) % H, r = blockIdx.x / (col_blocks * H);
    const int n_tok = q_len[r];
    if (n_tok < min_len) return;                       // short portions and single tokens take the token-by-token kernel
    const int slot = slots[r];
    if (slot < 0 || slot >= max_slots) {
        if (tid == 0) atomicOr(err, AIE_DEV_SLOT_OOB);
        return;
    }
    constexpr int LN = NP + DC_PAD, LD = DV + DC_PAD, LQ = DC_Q + DC_PAD;      // row strides, bfloat16 buffers
    constexpr int FY = DC_Q + DC_PADF, FD = DV + DC_PADF;                      // ... float32 buffers
    constexpr int DT = DV / 16;                                                // column tiles of a CTA
    bf16* KH = reinterpret_cast<bf16*>(dc_sm);                    // [Q][NP] unit keys
    bf16* KL = KH + DC_Q * LN;
    bf16* QH = KL + DC_Q * LN;                                    // [Q][NP] unit queries, scaled
    bf16* QL = QH + DC_Q * LN;
    bf16* SH = QL + DC_Q * LN;                                    // [NP][DV] the state
    bf16* SL = SH + NP * LD;
    bf16* NH = SL + NP * LD;                                      // [Q][Q] -A
    bf16* NL = NH + DC_Q * LQ;
    bf16* PH = NL + DC_Q * LQ;                                    // [Q][Q] P
    bf16* PL = PH + DC_Q * LQ;
    bf16* UH = PL + DC_Q * LQ;                                    // [Q][DV] U
    bf16* UL = UH + DC_Q * LD;
    bf16* WH = UL + DC_Q * LD;                                    // [Q][DV] w * U
    bf16* WL = WH + DC_Q * LD;
    float* G1 = reinterpret_cast<float*>(WL + DC_Q * LD);         // [Q][Q] K K^T
    float* G2 = G1 + DC_Q * FY;                                   // [Q][Q] Q K^T
    float* R1 = G2 + DC_Q * FY;                                   // [Q][DV] K S_0, then the right-hand side
    float* R2 = R1 + DC_Q * FD;                                   // [Q][DV] Q S_0, then O
    float* Sf = R2 + DC_Q * FD;                                   // [NP][DV]
    float* Ad = Sf + NP * FD;                                     // [4][16][16] diagonal blocks of A
    float* Md = Ad + 4 * 256;                                     // [4][16][16] inverses of I + those
    float* la = Md + 4 * 256;                                     // [Q] running sums of log decays
    float* be = la + DC_Q;                                        // [Q] beta
    float* ela = be + DC_Q;                                       // [Q] exp(l_t)
    float* wv = ela + DC_Q;                                       // [Q] w_s = exp(l_Q - l_s)

    const int hq = h / (H / G), col0 = cb * DV, a0 = q_start[r];
    const float rate = expf(a_log[h]), bias = dt_bias[h];
    float* sp = state + ((size_t)slot * H + h) * d * e;
    for (int i = tid; i < NP * DV; i += DC_THREADS) {
        const int n = i / DV, j = i % DV;
        const float v = (n < d && col0 + j < e) ? sp[(size_t)n * e + col0 + j] : 0.f;
        Sf[n * FD + j] = v;
        dc_split(v, SH + n * LD + j, SL + n * LD + j);
    }
    for (int t0 = 0; t0 < n_tok; t0 += DC_Q) {
        const int nt = min(DC_Q, n_tok - t0);
        __syncthreads();                               // the last chunk is done with; the state's halves are written
        // a warp makes the unit vectors of four rows; all its loads are in flight before the first sum
        constexpr int PER = NP / 32, ROWS = DC_Q / DC_WARPS;
        constexpr int PERX = DC_Q * DV / DC_THREADS;
        float vv[PERX];                                // the chunk's values stay in registers until they are needed
        {
            // a lane holds channels lane + 32 c; where a row of 128 channels can be read 16 bytes at a time, 4 lane + c
            float kv[ROWS][PER], qv[ROWS][PER];
            const bool wide = PER == 4 && vec4;
            if (wide) {
#pragma unroll
                for (int rr = 0; rr < ROWS; ++rr) {
                    const int t = warp + rr * DC_WARPS, n = 4 * lane;
                    const bool ok = t < nt && n < d;               // d is a multiple of 4 here
                    const size_t at = (size_t)(a0 + t0 + t) * ld + (size_t)hq * d + n;
                    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
                    const float4 kx = ok ? *reinterpret_cast<const float4*>(kg + at) : z;
                    const float4 qx = ok ? *reinterpret_cast<const float4*>(qg + at) : z;
                    kv[rr][0] = kx.x, kv[rr][1 % PER] = kx.y, kv[rr][2 % PER] = kx.z, kv[rr][3 % PER] = kx.w;
                    qv[rr][0] = qx.x, qv[rr][1 % PER] = qx.y, qv[rr][2 % PER] = qx.z, qv[rr][3 % PER] = qx.w;
                }
            } else {
#pragma unroll
                for (int rr = 0; rr < ROWS; ++rr) {
                    const int t = warp + rr * DC_WARPS;
#pragma unroll
                    for (int c = 0; c < PER; ++c) {
                        const int n = lane + 32 * c;
                        const bool ok = t < nt && n < d;
                        const size_t at = (size_t)(a0 + t0 + t) * ld + (size_t)hq * d + n;
                        kv[rr][c] = ok ? kg[at] : 0.f;
                        qv[rr][c] = ok ? qg[at] : 0.f;
                    }
                }
            }
#pragma unroll
            for (int it = 0; it < PERX; ++it) {
                const int i = tid + it * DC_THREADS, t = i / DV, j = i % DV;
                vv[it] = (t < nt && col0 + j < e) ? vg[(size_t)(a0 + t0 + t) * ld + (size_t)h * e + col0 + j] : 0.f;
            }
            if (tid < DC_Q) {
                float lg = 0.f, b = 0.f;               // a token behind the portion's end: no decay, no correction
                if (tid < nt) {
                    const float x = a_raw[(size_t)(a0 + t0 + tid) * lda + h] + bias;
                    lg = -rate * (x > 20.f ? x : log1pf(expf(x)));
                    b = 1.f / (1.f + expf(-b_raw[(size_t)(a0 + t0 + tid) * ldb + h]));
                }
                wv[tid] = lg;
                be[tid] = b;
            }
#pragma unroll
            for (int rr = 0; rr < ROWS; ++rr) {
                const int t = warp + rr * DC_WARPS;
                float kk = 0.f, qq = 0.f;
#pragma unroll
                for (int c = 0; c < PER; ++c) {
                    kk += kv[rr][c] * kv[rr][c];
                    qq += qv[rr][c] * qv[rr][c];
                }
                kk = warp_sum(kk);
                qq = warp_sum(qq);
                const float ik = rsqrtf(kk + unit_eps), iq = rsqrtf(qq + unit_eps) * q_scale;
#pragma unroll
                for (int c = 0; c < PER; ++c) {
                    const int n = wide ? 4 * lane + c : lane + 32 * c;
                    dc_split(kv[rr][c] * ik, KH + t * LN + n, KL + t * LN + n);
                    dc_split(qv[rr][c] * iq, QH + t * LN + n, QL + t * LN + n);
                }
            }
        }
        __syncthreads();
        if (warp == 0) {                               // running sums of the 64 log decays: a scan over pairs
            const float v0 = wv[2 * lane], v1 = wv[2 * lane + 1];
            float run = v0 + v1;
            for (int o = 1; o < 32; o <<= 1) {
                const float up = __shfl_up_sync(0xffffffffu, run, o);
                if (lane >= o) run += up;
            }
            const float end = __shfl_sync(0xffffffffu, run, 31);
            la[2 * lane] = run - v1;
            la[2 * lane + 1] = run;
            ela[2 * lane] = expf(run - v1);
            ela[2 * lane + 1] = expf(run);
            __syncwarp();
            wv[2 * lane] = expf(end - (run - v1));
            wv[2 * lane + 1] = expf(end - run);
        }
        // K K^T and Q K^T, the tiles on and below the diagonal; K S_0 and Q S_0
        for (int job = warp; job < 20 + 8 * DT; job += DC_WARPS) {
            FragC acc;
            wmma::fill_fragment(acc, 0.f);
            if (job < 20) {
                int ti, tj;
                dc_lower_tile(job < 10 ? job : job - 10, &ti, &tj);
                const bf16* aH = (job < 10 ? KH : QH) + ti * 16 * LN;
                const bf16* aL = (job < 10 ? KL : QL) + ti * 16 * LN;
                dc_mma3<FragA, FragBT>(acc, aH, aL, LN, 16, KH + tj * 16 * LN, KL + tj * 16 * LN, LN, 16, NP / 16);
                wmma::store_matrix_sync((job < 10 ? G1 : G2) + ti * 16 * FY + tj * 16, acc, FY, wmma::mem_row_major);
            } else {
                const int jb = job - 20, which = jb / (4 * DT), ti = (jb / DT) % 4, tj = jb % DT;
                dc_mma3<FragA, FragB>(acc, (which ? QH : KH) + ti * 16 * LN, (which ? QL : KL) + ti * 16 * LN, LN, 16,
                                      SH + tj * 16, SL + tj * 16, LD, 16 * LD, NP / 16);
                wmma::store_matrix_sync((which ? R2 : R1) + ti * 16 * FD + tj * 16, acc, FD, wmma::mem_row_major);
            }
        }
        __syncthreads();
        // -A and P on and below the diagonal, tile by tile and two neighbours a thread (the tiles above are never read)
        for (int i = tid; i < 10 * 128; i += DC_THREADS) {
            int ti, tj;
            dc_lower_tile(i >> 7, &ti, &tj);
            const int pr = i & 127, tl = pr >> 3, sl = (pr & 7) * 2, t = ti * 16 + tl, s = tj * 16 + sl;
            const float lt = la[t], bt = be[t];
            const float2 ls = *reinterpret_cast<const float2*>(la + s);
            const float2 g1 = *reinterpret_cast<const float2*>(G1 + t * FY + s);
            const float2 g2 = *reinterpret_cast<const float2*>(G2 + t * FY + s);
            const float d0 = __expf(lt - ls.x), d1 = __expf(lt - ls.y);
            const float a0v = s < t ? bt * d0 * g1.x : 0.f, a1v = s + 1 < t ? bt * d1 * g1.y : 0.f;
            const float p0 = s <= t ? d0 * g2.x : 0.f, p1 = s + 1 <= t ? d1 * g2.y : 0.f;
            __nv_bfloat162 hi, lo;
            dc_split(-a0v, &hi.x, &lo.x);
            dc_split(-a1v, &hi.y, &lo.y);
            *reinterpret_cast<__nv_bfloat162*>(NH + t * LQ + s) = hi;
            *reinterpret_cast<__nv_bfloat162*>(NL + t * LQ + s) = lo;
            dc_split(p0, &hi.x, &lo.x);
            dc_split(p1, &hi.y, &lo.y);
            *reinterpret_cast<__nv_bfloat162*>(PH + t * LQ + s) = hi;
            *reinterpret_cast<__nv_bfloat162*>(PL + t * LQ + s) = lo;
            if (ti == tj) *reinterpret_cast<float2*>(Ad + ti * 256 + tl * 16 + sl) = make_float2(a0v, a1v);
        }
        // the right-hand side beta (V - exp(l_t) K S_0), and the part of O that comes from the old state
#pragma unroll
        for (int it = 0; it < PERX; ++it) {
            const int i = tid + it * DC_THREADS, t = i / DV, j = i % DV;
            R1[t * FD + j] = be[t] * (vv[it] - ela[t] * R1[t * FD + j]);
            R2[t * FD + j] *= ela[t];
        }
        __syncthreads();
        // the inverses of the diagonal blocks of I + A: a thread per column, forward substitution in registers
        if (tid < 64) {
            const int blk = tid >> 4, c = tid & 15;
            const float* A = Ad + blk * 256;
            float m[16];
#pragma unroll
            for (int t = 0; t < 16; ++t) {
                float acc0 = t == c ? 1.f : 0.f, acc1 = 0.f;
#pragma unroll
                for (int s = 0; s + 1 < t; s += 2) {
                    acc0 -= A[t * 16 + s] * m[s];
                    acc1 -= A[t * 16 + s + 1] * m[s + 1];
                }
                if (t & 1) acc0 -= A[t * 16 + t - 1] * m[t - 1];
                m[t] = acc0 + acc1;
                Md[blk * 256 + t * 16 + c] = m[t];
            }
        }
        __syncthreads();
        // (I + A) U = right-hand side, 16 rows at a time
        for (int bi = 0; bi < 4; ++bi) {
            if (bi > 0) {
                if (warp < DT) {                       // what the blocks before contribute leaves the right-hand side
                    FragC acc;
                    wmma::load_matrix_sync(acc, R1 + bi * 16 * FD + warp * 16, FD, wmma::mem_row_major);
                    dc_mma3<FragA, FragB>(acc, NH + bi * 16 * LQ, NL + bi * 16 * LQ, LQ, 16, UH + warp * 16, UL + warp * 16,
                                          LD, 16 * LD, bi);
                    wmma::store_matrix_sync(R1 + bi * 16 * FD + warp * 16, acc, FD, wmma::mem_row_major);
                }
                __syncthreads();
            }
#pragma unroll
            for (int o = tid; o < 16 * DV; o += DC_THREADS) {
                const int tl = o / DV, j = o % DV, t = bi * 16 + tl;
                const float* mrow = Md + bi * 256 + tl * 16;
                float u0 = 0.f, u1 = 0.f;
#pragma unroll
                for (int s = 0; s < 16; s += 2) {      // zeros above the diagonal
                    u0 = fmaf(mrow[s], R1[(bi * 16 + s) * FD + j], u0);
                    u1 = fmaf(mrow[s + 1], R1[(bi * 16 + s + 1) * FD + j], u1);
                }
                const float u = u0 + u1;
                dc_split(u, UH + t * LD + j, UL + t * LD + j);
                dc_split(u * wv[t], WH + t * LD + j, WL + t * LD + j);
            }
            __syncthreads();
        }
        // O = exp(l_t) Q S_0 + P U, the tiles with the most steps first and dealt from the last warp down (the state's
        // tiles below are dealt from the first warp up)
        for (int job = DC_WARPS - 1 - warp; job < 4 * DT; job += DC_WARPS) {
            const int ti = 3 - job / DT, tj = job % DT;
            FragC acc;
            wmma::load_matrix_sync(acc, R2 + ti * 16 * FD + tj * 16, FD, wmma::mem_row_major);
            dc_mma3<FragA, FragB>(acc, PH + ti * 16 * LQ, PL + ti * 16 * LQ, LQ, 16, UH + tj * 16, UL + tj * 16, LD, 16 * LD,
                                  ti + 1);
            wmma::store_matrix_sync(R2 + ti * 16 * FD + tj * 16, acc, FD, wmma::mem_row_major);
        }
        // S = exp(l_Q) S + K^T (w * U); a tile of the state belongs to one warp, which also makes its two halves
        const float dec_end = ela[DC_Q - 1];
        for (int job = warp; job < (NP / 16) * DT; job += DC_WARPS) {
            const int ni = job / DT, tj = job % DT;
            FragC acc;
            wmma::load_matrix_sync(acc, Sf + ni * 16 * FD + tj * 16, FD, wmma::mem_row_major);
            for (int x = 0; x < acc.num_elements; ++x) acc.x[x] *= dec_end;
            dc_mma3<FragAT, FragB>(acc, KH + ni * 16, KL + ni * 16, LN, 16 * LN, WH + tj * 16, WL + tj * 16, LD, 16 * LD,
                                   DC_Q / 16);
            wmma::store_matrix_sync(Sf + ni * 16 * FD + tj * 16, acc, FD, wmma::mem_row_major);
            __syncwarp();
            for (int x = lane; x < 256; x += 32) {
                const int n = ni * 16 + (x >> 4), j = tj * 16 + (x & 15);
                dc_split(Sf[n * FD + j], SH + n * LD + j, SL + n * LD + j);
            }
        }
        __syncthreads();
        for (int i = tid; i < DC_Q * DV; i += DC_THREADS) {
            const int t = i / DV, j = i % DV;
            if (t < nt && col0 + j < e) out[((size_t)(a0 + t0 + t) * H + h) * e + col0 + j] = R2[t * FD + j];
        }
    }
    __syncthreads();
    if (live == nullptr || live[r] != 0) {
        for (int i = tid; i < NP * DV; i += DC_THREADS) {
            const int n = i / DV, j = i % DV;
            if (n < d && col0 + j < e) sp[(size_t)n * e + col0 + j] = Sf[n * FD + j];
        }
    }
}

template <int NP, int DV> static size_t dc_smem() {
    const int LN = NP + DC_PAD, LD = DV + DC_PAD, LQ = DC_Q + DC_PAD, FY = DC_Q + DC_PADF, FD = DV + DC_PADF;
    return (size_t)(4 * DC_Q * LN + 2 * NP * LD + 4 * DC_Q * LQ + 4 * DC_Q * LD) * sizeof(bf16) +
           (size_t)(2 * DC_Q * FY + 2 * DC_Q * FD + NP * FD + 8 * 256 + 4 * DC_Q) * sizeof(float);
}

// q, k [T, .] with head h's d channels at column (h / (H / G)) d of rows `ld` floats apart; v likewise with e columns a
// head at column h e; b_raw, a_raw [T, .] rows ldb, lda apart; state [max_slots, H, d, e]; out [T, H, e].  Requests that
// bring fewer than min_len tokens are left alone.  d <= 128.
extern "C" int aie_delta_rule_chunked(const float* q, const float* k, const float* v, int ld, const float* b_raw, int ldb,
                                      const float* a_raw, int lda, const float* a_log, const float* dt_bias, float q_scale,
                                      float unit_eps, float* state, float* out, const int* q_start, const int* q_len,
                                      const int* slots, const int* live, int R, int H, int G, int d, int e, int max_slots,
                                      int min_len, unsigned* err, cudaStream_t st) {
    if (R <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || d <= 0 || e <= 0) return AIE_BAD_ARG;
    if (d > 128) return AIE_UNSUPPORTED;
    // value columns a CTA: the widest of 64, 32 and 16 that the state's rows leave room for and that gives every SM a
    // CTA; narrower CTAs repeat the products of keys and queries, but a lone long prompt has few (request, head) pairs
    const int sms = aie_sm_count();
    int DVc = d > 64 ? 32 : 64;
    while (DVc > 16 && e > DVc / 2 && (long long)R * H * ((e + DVc - 1) / DVc) < sms) DVc /= 2;
    const int col_blocks = (e + DVc - 1) / DVc;
    const long long blocks = (long long)R * H * col_blocks;
    if (blocks > 0x7fffffffLL) return AIE_UNSUPPORTED;
    const int vec4 = d % 4 == 0 && ld % 4 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)k & 15) == 0;
#define GO(NP, DV)                                                                                                      \
    do {                                                                                                                \
        static bool set = false;                                                                                        \
        if (!set) {                                                                                                     \
            cudaError_t ce = cudaFuncSetAttribute(delta_rule_chunked_kernel<NP, DV>,                                    \
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dc_smem<NP, DV>()); \
            if (ce != cudaSuccess) return (int)ce;                                                                      \
            set = true;                                                                                                 \
        }                                                                                                               \
        delta_rule_chunked_kernel<NP, DV><<<(unsigned)blocks, DC_THREADS, dc_smem<NP, DV>(), st>>>(                     \
            q, k, v, ld, b_raw, ldb, a_raw, lda, a_log, dt_bias, q_scale, unit_eps, state, out, q_start, q_len, slots,  \
            live, H, G, d, e, col_blocks, max_slots, min_len, vec4, err);                                                \
    } while (0)
#define GO3(NP)                                  \
    do {                                         \
        if (DVc == 64) GO(NP < 128 ? NP : 64, 64); \
        else if (DVc == 32) GO(NP, 32);          \
        else GO(NP, 16);                         \
    } while (0)
    if (d <= 32) GO3(32);
    else if (d <= 64) GO3(64);
    else GO3(128);
#undef GO3
#undef GO
    AIE_LAUNCH_CHECK();
}
