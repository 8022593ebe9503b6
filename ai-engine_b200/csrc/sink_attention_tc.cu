// bfloat16 attention with a distance bias, a window that keeps the first tokens, a sink and a gate per head on
// tensor cores (mma.sync m16n8k16, bf16 in, float32 accumulate), over a paged cache of one plane whose rows hold
// a key (DK elements) and behind it a value (DV elements); DK and DV each 32, 64 or 128.
//
//   s(i, j) = (q_i . k_j) * scale * temp[h] - slope[h] * (i - j)
//   i reads j  iff  j <= i and (window <= 0 or i - j < window or j < keep_first)
//   out_i = gate[i, h] * sum_j exp(s(i, j)) v_j / (exp(sink[h]) + sum_j exp(s(i, j)))
//
// Scores, the running maximum and sum and the weights are float32.  A weight enters the product with the values
// as two bfloat16 numbers (its rounded value and the rounded rest: 16 bits of mantissa), so that the tensor
// cores add the same weights the float32 sum holds.
//
//   sink_prefill_kernel  one CTA of eight warps per (128 query tokens of a request, head); a warp owns 16 rows.
//                        Tiles of 64 keys come page by page through the block table into two shared-memory
//                        buffers with 16-byte cp.async copies (XOR-swizzled for ldmatrix).  With a window, the
//                        tiles that hold kept first keys are visited before the window's own; tiles between
//                        them are never read.
//   sink_decode_kernel   requests that bring one token: one CTA of four warps per (part of the keys, key/value
//                        head and up to 16 of its query heads, request).  The query heads are the rows of the
//                        16-row tile; every warp walks every fourth tile of 32 keys of the part through a ring
//                        of its own, and the warps are joined through shared memory.  With one part the CTA
//                        writes the result; with more, parts (maximum, sum, unnormalised output) go to scratch
//                        and sink_join_kernel joins them.  The sink enters once, where the parts are joined.
#include "common.cuh"
#include "attention_prefill.cuh"

#define SK_M 128
#define SK_WARPS 8

// row r, 16-byte chunk c of a [rows][D] bf16 tile; rows of 64 bytes (D = 32) share a 128-byte line in pairs
template <int D> __device__ __forceinline__ bf16* sk_at(bf16* base, int row, int chunk) {
    if (D >= 64) return base + row * D + ((chunk ^ (row & 7)) << 3);
    return base + row * D + ((chunk ^ ((row >> 1) & 3)) << 3);
}

// One warp, 16 query rows against a tile of N keys in shared memory.  The thread holds rows (lane / 4) and
// (lane / 4) + 8: their positions qp, factors qs (scale * temp) and slopes sl.  `masked`: apply the visibility
// rule (tiles wholly inside every row's sight skip it); keys above `key_end` are never visible.
template <int DK, int DV, int N>
__device__ __forceinline__ void sk_tile(const bf16* kb, const bf16* vb, const unsigned (&qf)[DK / 16][4],
                                        float (&o)[DV / 8][4], float (&m_run)[2], float (&l_run)[2], int kbase,
                                        const int (&qp)[2], const float (&qs)[2], const float (&sl)[2], int window,
                                        int keep_first, bool masked, int lane) {
    float s[N / 8][4];
#pragma unroll
    for (int j = 0; j < N / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < DK / 16; ++ks) {
#pragma unroll
        for (int j = 0; j < N / 8; j += 2) {
            const int mid = lane >> 3;
            unsigned b0, b1, b2, b3;
            ldsm_x4(b0, b1, b2, b3, sk_at<DK>(const_cast<bf16*>(kb), (j + (mid >> 1)) * 8 + (lane & 7), ks * 2 + (mid & 1)));
            mma16816(s[j], qf[ks], b0, b1);
            mma16816(s[j + 1], qf[ks], b2, b3);
        }
    }
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < N / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = e >> 1;
            const int key = kbase + j * 8 + 2 * (lane & 3) + (e & 1);
            float v = s[j][e] * qs[i] - sl[i] * (float)(qp[i] - key);
            if (masked) {
                const bool ok = key <= qp[i] && (window <= 0 || key > qp[i] - window || key < keep_first);
                if (!ok) v = -INFINITY;
            }
            s[j][e] = v;
            tmax[i] = fmaxf(tmax[i], v);
        }
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        float tm = tmax[i];
        tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 1));
        tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 2));
        const float m_new = fmaxf(m_run[i], tm);
        m_use[i] = (m_new == -INFINITY) ? 0.f : m_new;          // a row with nothing visible yet
        corr[i] = (m_run[i] == -INFINITY) ? 0.f : __expf(m_run[i] - m_use[i]);
        m_run[i] = m_new;
    }
    float psum[2] = {0.f, 0.f};
    unsigned ph[N / 16][4], pl[N / 16][4];
#pragma unroll
    for (int j = 0; j < N / 8; ++j) {
        float p[4], r[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            p[e] = __expf(s[j][e] - m_use[e >> 1]);             // exp(-inf) = 0 for keys out of sight
            psum[e >> 1] += p[e];
            r[e] = p[e] - __bfloat162float(__float2bfloat16_rn(p[e]));
        }
        ph[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p[0], p[1]);
        ph[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
        pl[j >> 1][(j & 1) * 2 + 0] = pack_bf16(r[0], r[1]);
        pl[j >> 1][(j & 1) * 2 + 1] = pack_bf16(r[2], r[3]);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        psum[i] += __shfl_xor_sync(0xffffffffu, psum[i], 1);
        psum[i] += __shfl_xor_sync(0xffffffffu, psum[i], 2);
        l_run[i] = l_run[i] * corr[i] + psum[i];
    }
#pragma unroll
    for (int j = 0; j < DV / 8; ++j) {
        o[j][0] *= corr[0];
        o[j][1] *= corr[0];
        o[j][2] *= corr[1];
        o[j][3] *= corr[1];
    }
#pragma unroll
    for (int kk = 0; kk < N / 16; ++kk) {
#pragma unroll
        for (int jd = 0; jd < DV / 8; jd += 2) {
            const int mid = lane >> 3;
            unsigned b0, b1, b2, b3;
            ldsm_x4_t(b0, b1, b2, b3, sk_at<DV>(const_cast<bf16*>(vb), kk * 16 + (mid & 1) * 8 + (lane & 7), jd + (mid >> 1)));
            mma16816(o[jd], ph[kk], b0, b1);
            mma16816(o[jd + 1], ph[kk], b2, b3);
            mma16816(o[jd], pl[kk], b0, b1);
            mma16816(o[jd + 1], pl[kk], b2, b3);
        }
    }
}

template <int DK, int DV>
__global__ void __launch_bounds__(SK_WARPS * 32)
sink_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pages, bf16* __restrict__ out,
                    const float* __restrict__ gate, const float* __restrict__ temp, const float* __restrict__ slope,
                    const float* __restrict__ sink, const int* __restrict__ tiles, const int* __restrict__ q_start,
                    const int* __restrict__ q_len, const int* __restrict__ ctx_len,
                    const int* __restrict__ block_table, int bt_width, int num_pages, int P, int H, int G,
                    int window, int keep_first, float scale, unsigned* err) {
    constexpr int N = 64, W = DK + DV;
    constexpr int CK = DK / 8, CV = DV / 8, CW = W / 8;      // 16-byte chunks of a key, a value, a cache row
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);            // [128][DK]
    bf16* k_s = q_s + SK_M * DK;                               // [2][64][DK]
    bf16* v_s = k_s + 2 * N * DK;                              // [2][64][DV]
    int* row_s = reinterpret_cast<int*>(v_s + 2 * N * DV);     // [2][64] cache rows of the tile's keys

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tile_i = (int)gridDim.y - 1 - (int)blockIdx.y;   // the list holds the tiles fewest keys first
    const int r = tiles[2 * tile_i], q_off = tiles[2 * tile_i + 1];
    const int h = blockIdx.x, g = h / (H / G);
    const int t0 = q_start[r] + q_off;
    const int rows_valid = min(SK_M, q_len[r] - q_off);
    const int p0 = ctx_len[r] + q_off;              // position of the tile's first query
    const int p_last = p0 + rows_valid - 1;         // and of its last valid one
    const int* bt = block_table + (size_t)r * bt_width;

    for (int i = tid; i < SK_M * CK; i += SK_WARPS * 32) {
        const int row = i / CK, c = i % CK;
        const bool ok = row < rows_valid;
        cp_async16(sk_at<DK>(q_s, row, c), q + ((size_t)(t0 + (ok ? row : 0)) * H + h) * DK + c * 8, ok);
    }
    cp_async_commit();

    int lo_min = 0;
    if (window > 0 && p0 - window + 1 > 0) lo_min = p0 - window + 1;
    const int kt_lo = lo_min / N, kt_hi = p_last / N;
    // tiles of kept first keys that lie before the window's first tile
    const int n_kept = (window > 0 && keep_first > 0) ? min(kt_lo, (keep_first + N - 1) / N) : 0;
    const int n_it = n_kept + kt_hi - kt_lo + 1;
    auto tile_of = [&](int it) { return it < n_kept ? it : kt_lo + (it - n_kept); };

    auto load_tile = [&](int kt, int buf) {
        if (tid < N) {
            const int key = kt * N + tid;
            int prow = -1;
            if (key <= p_last) {
                const int pidx = key / P;
                const int page = pidx < bt_width ? bt[pidx] : -1;
                if (page >= 0 && page < num_pages) prow = (page * G + g) * P + (key - pidx * P);
                else if (key >= lo_min || key < keep_first) atomicOr(err, AIE_DEV_PAGE_OOB);   // out of sight a page may be gone
            }
            row_s[buf * N + tid] = prow;
        }
        __syncthreads();
        bf16* kd = k_s + buf * N * DK;
        bf16* vd = v_s + buf * N * DV;
        for (int i = tid; i < N * CW; i += SK_WARPS * 32) {
            const int row = i / CW, c = i % CW;
            const int prow = row_s[buf * N + row];
            const bool ok = prow >= 0;
            const bf16* src = pages + (size_t)(ok ? prow : 0) * W + c * 8;
            if (c < CK) cp_async16(sk_at<DK>(kd, row, c), src, ok);
            else cp_async16(sk_at<DV>(vd, row, c - CK), src, ok);
        }
        cp_async_commit();
    };

    load_tile(tile_of(0), 0);

    float o[DV / 8][4];
#pragma unroll
    for (int j = 0; j < DV / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
    // the sink opens the running softmax: a weight exp(sink - m) = 1 at m = sink, with no value
    float m_run[2], l_run[2];
    m_run[0] = m_run[1] = sink ? sink[h] : -INFINITY;
    l_run[0] = l_run[1] = sink ? 1.f : 0.f;
    unsigned qf[DK / 16][4];
    int qp[2];
    qp[0] = p0 + warp * 16 + (lane >> 2);
    qp[1] = qp[0] + 8;
    float qs[2], sl[2];
    qs[0] = qs[1] = scale * (temp ? temp[h] : 1.f);
    sl[0] = sl[1] = slope ? slope[h] : 0.f;

    for (int it = 0; it < n_it; ++it) {
        const int kt = tile_of(it), buf = it & 1;
        if (it + 1 < n_it) {
            load_tile(tile_of(it + 1), buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (it == 0) {
#pragma unroll
            for (int ks = 0; ks < DK / 16; ++ks) {
                const int mid = lane >> 3;
                ldsm_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3],
                        sk_at<DK>(q_s, warp * 16 + (mid & 1) * 8 + (lane & 7), ks * 2 + (mid >> 1)));
            }
        }
        const int kbase = kt * N;
        // the rule is applied on tiles that touch the diagonal or the low edge of some row's window
        const bool masked = (kbase + N - 1 > p0) || (window > 0 && kbase < p_last - window + 1);
        sk_tile<DK, DV, N>(k_s + buf * N * DK, v_s + buf * N * DV, qf, o, m_run, l_run, kbase, qp, qs, sl, window,
                           keep_first, masked, lane);
        __syncthreads();     // everyone is done with this buffer before it is loaded again
    }

#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int row = warp * 16 + (lane >> 2) + i * 8;
        if (row >= rows_valid) continue;
        const float inv = (l_run[i] > 0.f ? 1.0f / l_run[i] : 0.f) * (gate ? gate[(size_t)(t0 + row) * H + h] : 1.f);
        bf16* dst = out + ((size_t)(t0 + row) * H + h) * DV + 2 * (lane & 3);
#pragma unroll
        for (int j = 0; j < DV / 8; ++j)
            *reinterpret_cast<unsigned*>(dst + j * 8) = pack_bf16(o[j][i * 2] * inv, o[j][i * 2 + 1] * inv);
    }
}

// ---------------------------------------------------------------------------
// requests that bring one token
#define SD_WARPS 4
#define SD_HEADS 8           // query heads of one key/value head that a CTA takes (rows 0 .. 7 of the 16-row tile)
#define SD_NST 3             // stages of a warp's ring
#define SD_MAX_SPLITS 64

// keys of one stage of a warp: about 8 KB of cache rows, a multiple of 16 keys
template <int W> struct SdStage { static constexpr int keys = W > 128 ? 16 : (W > 64 ? 32 : 64); };

template <int DK, int DV> struct SdSmem {
    static constexpr int W = DK + DV, STILE = SdStage<W>::keys;
    static constexpr size_t stage_bytes = (size_t)STILE * W * sizeof(bf16);
    static constexpr size_t rows_off = (size_t)SD_WARPS * SD_NST * stage_bytes;
    static constexpr size_t bytes = rows_off + (size_t)SD_WARPS * STILE * sizeof(int);
};

// The keys a lone token at `pos` reads are numbered u = 0 .. nk-1: first the `kept` first keys that the window
// has passed, then the window's own from `lo` on.  Every numbered key is visible, so no rule is applied to
// them; a key's true position enters the distance bias.
template <int DK, int DV>
__global__ void __launch_bounds__(SD_WARPS * 32)
sink_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pages, bf16* __restrict__ out,
                   float* __restrict__ part_o, float* __restrict__ part_lse, const float* __restrict__ gate,
                   const float* __restrict__ temp, const float* __restrict__ slope, const float* __restrict__ sink,
                   const int* __restrict__ dec_tokens, const int* __restrict__ positions,
                   const int* __restrict__ token_req, const int* __restrict__ block_table, int bt_width,
                   int num_pages, int P, int H, int G, int GC, int window, int keep_first, float scale, int S,
                   unsigned* err) {
    constexpr int W = DK + DV, CW = W / 8, CK = DK / 8;
    constexpr int STILE = SdStage<W>::keys, KS = DK / 16;
    extern __shared__ __align__(128) unsigned char sd_smem[];
    __shared__ float mrg_m[SD_WARPS][SD_HEADS], mrg_l[SD_WARPS][SD_HEADS];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int s = blockIdx.x, di = blockIdx.z;
    const int group = H / G, gchunks = (group + GC - 1) / GC;
    const int kvh = blockIdx.y / gchunks, g0 = (blockIdx.y % gchunks) * GC;
    const int ng = min(GC, group - g0);
    const int t = dec_tokens[di];
    const int pos = positions[t], row = token_req[t];
    const int hbase = kvh * group + g0;
    const int qrow = lane >> 2, qcol = (lane & 3) * 2;
    const int* bt = block_table + (size_t)row * bt_width;

    bf16* stage0 = reinterpret_cast<bf16*>(sd_smem + (size_t)warp * SD_NST * SdSmem<DK, DV>::stage_bytes);
    int* rows_w = reinterpret_cast<int*>(sd_smem + SdSmem<DK, DV>::rows_off) + warp * STILE;

    int lo = 0;
    if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
    const int kept = min(keep_first, lo);
    const int nk = kept + pos + 1 - lo;
    const int tiles_total = (nk + STILE - 1) / STILE;
    const int tps = (tiles_total + S - 1) / S;
    const int tile_begin = s * tps, tile_end = min((s + 1) * tps, tiles_total);
    const int first = tile_begin + warp;
    const int n_my = first < tile_end ? (tile_end - first + SD_WARPS - 1) / SD_WARPS : 0;

    auto issue = [&](int i) {
        if (i < n_my) {
            const int u0 = (first + i * SD_WARPS) * STILE;
            for (int j = lane; j < STILE; j += 32) {
                const int u = u0 + j;
                int prow = -1;
                if (u < nk) {
                    const int key = u < kept ? u : lo + (u - kept);
                    const int pidx = key / P;
                    const int page = pidx < bt_width ? bt[pidx] : -1;
                    if (page >= 0 && page < num_pages) prow = (page * G + kvh) * P + (key - pidx * P);
                    else atomicOr(err, AIE_DEV_PAGE_OOB);
                }
                rows_w[j] = prow;
            }
            __syncwarp();
            bf16* kd = stage0 + (size_t)(i % SD_NST) * STILE * W;
            bf16* vd = kd + STILE * DK;
#pragma unroll
            for (int r = 0; r < STILE * CW / 32; ++r) {
                const int idx = lane + r * 32;
                const int kr = idx / CW, c = idx % CW;
                const int prow = rows_w[kr];
                const bf16* src = pages + (size_t)(prow >= 0 ? prow : 0) * W + c * 8;
                if (c < CK) cp_async16(sk_at<DK>(kd, kr, c), src, prow >= 0);
                else cp_async16(sk_at<DV>(vd, kr, c - CK), src, prow >= 0);
            }
            __syncwarp();      // the rows are read before the next stage's are written
        }
        cp_async_commit();
    };

#pragma unroll
    for (int i = 0; i < SD_NST - 1; ++i) issue(i);

    // q as the A operand: row = head; rows ng .. 15 are zero
    unsigned qa[KS][2];
    {
        const bf16* qp = q + ((size_t)t * H + hbase + (qrow < ng ? qrow : 0)) * DK;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const unsigned a = *reinterpret_cast<const unsigned*>(qp + ks * 16 + qcol);
            const unsigned b = *reinterpret_cast<const unsigned*>(qp + ks * 16 + 8 + qcol);
            qa[ks][0] = qrow < ng ? a : 0u;
            qa[ks][1] = qrow < ng ? b : 0u;
        }
    }
    const int hq = hbase + (qrow < ng ? qrow : 0);
    const float qs = scale * (temp ? temp[hq] : 1.f), sl = slope ? slope[hq] : 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    float o[DV / 8][2];
#pragma unroll
    for (int j = 0; j < DV / 8; ++j) o[j][0] = o[j][1] = 0.f;

    for (int i = 0; i < n_my; ++i) {
        issue(i + SD_NST - 1);
        cp_async_wait<SD_NST - 1>();
        __syncwarp();
        bf16* kd = stage0 + (size_t)(i % SD_NST) * STILE * W;
        bf16* vd = kd + STILE * DK;
        const int u0 = (first + i * SD_WARPS) * STILE;
        const int mid = lane >> 3;
#pragma unroll
        for (int sub = 0; sub < STILE / 16; ++sub) {
            if (u0 + sub * 16 >= nk) break;
            float sc[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) sc[j][e] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                unsigned b0, b1, b2, b3;
                ldsm_x4(b0, b1, b2, b3, sk_at<DK>(kd, sub * 16 + (mid >> 1) * 8 + (lane & 7), ks * 2 + (mid & 1)));
                const unsigned a[4] = {qa[ks][0], 0u, qa[ks][1], 0u};
                mma16816(sc[0], a, b0, b1);
                mma16816(sc[1], a, b2, b3);
            }
            float tmax = -INFINITY;
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int u = u0 + sub * 16 + j * 8 + qcol + e;
                    const int key = u < kept ? u : lo + (u - kept);
                    sc[j][e] = u < nk ? sc[j][e] * qs - sl * (float)(pos - key) : -INFINITY;
                    tmax = fmaxf(tmax, sc[j][e]);
                }
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
            const float m_new = fmaxf(m_run, tmax);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            const float corr = (m_run == -INFINITY) ? 0.f : __expf(m_run - m_use);
            float p[2][2], rr[2][2], psum = 0.f;
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    p[j][e] = __expf(sc[j][e] - m_use);
                    psum += p[j][e];
                    rr[j][e] = p[j][e] - __bfloat162float(__float2bfloat16_rn(p[j][e]));
                }
            psum += __shfl_xor_sync(0xffffffffu, psum, 1);
            psum += __shfl_xor_sync(0xffffffffu, psum, 2);
            l_run = l_run * corr + psum;
            m_run = m_new;
            const unsigned ph[4] = {pack_bf16(p[0][0], p[0][1]), 0u, pack_bf16(p[1][0], p[1][1]), 0u};
            const unsigned pl[4] = {pack_bf16(rr[0][0], rr[0][1]), 0u, pack_bf16(rr[1][0], rr[1][1]), 0u};
#pragma unroll
            for (int jd = 0; jd < DV / 8; jd += 2) {
                float c0[4] = {o[jd][0] * corr, o[jd][1] * corr, 0.f, 0.f};
                float c1[4] = {o[jd + 1][0] * corr, o[jd + 1][1] * corr, 0.f, 0.f};
                unsigned b0, b1, b2, b3;
                ldsm_x4_t(b0, b1, b2, b3, sk_at<DV>(vd, sub * 16 + (mid & 1) * 8 + (lane & 7), jd + (mid >> 1)));
                mma16816(c0, ph, b0, b1);
                mma16816(c1, ph, b2, b3);
                mma16816(c0, pl, b0, b1);
                mma16816(c1, pl, b2, b3);
                o[jd][0] = c0[0];
                o[jd][1] = c0[1];
                o[jd + 1][0] = c1[0];
                o[jd + 1][1] = c1[1];
            }
        }
        __syncwarp();
    }
    cp_async_wait<0>();
    __syncthreads();

    // join the warps (the staging memory is free now)
    float* mrg_o = reinterpret_cast<float*>(sd_smem);      // [SD_WARPS][SD_HEADS][DV]
    if (qrow < SD_HEADS) {
        if ((lane & 3) == 0) { mrg_m[warp][qrow] = m_run; mrg_l[warp][qrow] = l_run; }
#pragma unroll
        for (int jd = 0; jd < DV / 8; ++jd) {
            mrg_o[((size_t)warp * SD_HEADS + qrow) * DV + jd * 8 + qcol] = o[jd][0];
            mrg_o[((size_t)warp * SD_HEADS + qrow) * DV + jd * 8 + qcol + 1] = o[jd][1];
        }
    }
    __syncthreads();
    for (int idx = tid; idx < ng * DV; idx += SD_WARPS * 32) {
        const int g = idx / DV, e = idx % DV;
        const int h = hbase + g;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < SD_WARPS; ++w) M = fmaxf(M, mrg_m[w][g]);
        const bool whole = S == 1;
        if (whole && sink) M = fmaxf(M, sink[h]);
        float L = 0.f, A = 0.f;
#pragma unroll
        for (int w = 0; w < SD_WARPS; ++w) {
            const float f = (mrg_m[w][g] == -INFINITY) ? 0.f : __expf(mrg_m[w][g] - M);
            L += mrg_l[w][g] * f;
            A += mrg_o[((size_t)w * SD_HEADS + g) * DV + e] * f;
        }
        if (whole) {
            if (sink) L += __expf(sink[h] - M);      // the sink counts once, with no value
            const float inv = (L > 0.f ? 1.0f / L : 0.f) * (gate ? gate[(size_t)t * H + h] : 1.f);
            out[((size_t)t * H + h) * DV + e] = __float2bfloat16_rn(A * inv);
        } else {
            const size_t pi = ((size_t)di * H + h) * S + s;
            part_o[pi * DV + e] = L > 0.f ? A / L : 0.f;
            if (e == 0) part_lse[pi] = L > 0.f ? M + __logf(L) : -INFINITY;
        }
    }
}

// out[t, h, :] = gate * sum_s w_s part_o[s] / (exp(sink - M) + sum_s w_s), w_s = exp(lse_s - M), M = max(lse, sink).
// One block per (lone token, head).
__global__ void sink_join_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                 bf16* __restrict__ out, const float* __restrict__ gate,
                                 const float* __restrict__ sink, const int* __restrict__ dec_tokens, int H, int DV,
                                 int S) {
    __shared__ float w_s[SD_MAX_SPLITS];
    __shared__ float wsum_s;
    const int di = blockIdx.x, h = blockIdx.y;
    const int t = dec_tokens[di];
    const size_t base = ((size_t)di * H + h) * S;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        const float l0 = lane < S ? part_lse[base + lane] : -INFINITY;
        const float l1 = lane + 32 < S ? part_lse[base + lane + 32] : -INFINITY;
        float M = warp_max(fmaxf(l0, l1));
        if (sink) M = fmaxf(M, sink[h]);
        const float w0 = (l0 == -INFINITY) ? 0.f : __expf(l0 - M);
        const float w1 = (l1 == -INFINITY) ? 0.f : __expf(l1 - M);
        if (lane < S) w_s[lane] = w0;
        if (lane + 32 < S) w_s[lane + 32] = w1;
        float Wt = warp_sum(w0 + w1);
        if (sink) Wt += __expf(sink[h] - M);
        if (lane == 0) wsum_s = Wt;
    }
    __syncthreads();
    const float inv = (wsum_s > 0.f ? 1.0f / wsum_s : 0.f) * (gate ? gate[(size_t)t * H + h] : 1.f);
    for (int e = threadIdx.x; e < DV; e += blockDim.x) {
        const float* src = part_o + base * DV + e;
        float A = 0.f;
        for (int s = 0; s < S; ++s) A += w_s[s] * src[(size_t)s * DV];
        out[((size_t)t * H + h) * DV + e] = __float2bfloat16_rn(A * inv);
    }
}

#define SK_DISPATCH(DK_, DV_, CALL)                                                        \
    if (d == DK_ && e == DV_) { CALL(DK_, DV_); }

#define SK_DISPATCH_ALL(CALL)                                                              \
    SK_DISPATCH(32, 32, CALL) else SK_DISPATCH(32, 64, CALL) else SK_DISPATCH(32, 128, CALL) \
    else SK_DISPATCH(64, 32, CALL) else SK_DISPATCH(64, 64, CALL) else SK_DISPATCH(64, 128, CALL) \
    else SK_DISPATCH(128, 32, CALL) else SK_DISPATCH(128, 64, CALL) else SK_DISPATCH(128, 128, CALL) \
    else return AIE_UNSUPPORTED;

// Portions of prompts.  tiles: int32 [n, 2] = (request row, offset of a tile of 128 tokens among the tokens it
// brings), fewest keys first.  q [T, H, d], out [T, H, e] bfloat16; pages [num_pages, G, P, d + e] bfloat16.
extern "C" int aie_sink_attention_prefill(const void* q, const void* pages, void* out, const float* gate,
                                          const float* temp, const float* slope, const float* sink, const int* tiles,
                                          int n_tiles, const int* q_start, const int* q_len, const int* ctx_len,
                                          const int* block_table, int bt_width, int num_pages, int P, int H, int G,
                                          int d, int e, int window, int keep_first, float scale, unsigned* err,
                                          cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (G <= 0 || H % G || n_tiles > 65535) return AIE_UNSUPPORTED;
    dim3 grid(H, n_tiles);
#define SK_PRE(DK_, DV_)                                                                                              \
    {                                                                                                                 \
        const size_t smem = (size_t)(SK_M * DK_ + 2 * 64 * DK_ + 2 * 64 * DV_) * sizeof(bf16) + 2 * 64 * sizeof(int);   \
        auto kern = sink_prefill_kernel<DK_, DV_>;                                                                    \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                           \
        kern<<<grid, SK_WARPS * 32, smem, stream>>>((const bf16*)q, (const bf16*)pages, (bf16*)out, gate, temp, slope, \
                                                    sink, tiles, q_start, q_len, ctx_len, block_table, bt_width,      \
                                                    num_pages, P, H, G, window, keep_first, scale, err);              \
    }
    SK_DISPATCH_ALL(SK_PRE)
#undef SK_PRE
    AIE_LAUNCH_CHECK();
}

// Lone tokens.  dec_tokens: rows of the n tokens; S parts of each one's keys; with S > 1 part_o [n, H, S, e] and
// part_lse [n, H, S] float32 are scratch and a second kernel joins them.
extern "C" int aie_sink_attention_decode(const void* q, const void* pages, void* out, float* part_o, float* part_lse,
                                         const float* gate, const float* temp, const float* slope, const float* sink,
                                         const int* dec_tokens, int n, const int* positions, const int* token_req,
                                         const int* block_table, int bt_width, int num_pages, int P, int H, int G,
                                         int d, int e, int window, int keep_first, float scale, int S, unsigned* err,
                                         cudaStream_t stream) {
    if (n <= 0) return 0;
    if (G <= 0 || H % G || S < 1 || S > SD_MAX_SPLITS || n > 65535 || (S > 1 && (!part_o || !part_lse)))
        return AIE_UNSUPPORTED;
    const int group = H / G, GC = group < SD_HEADS ? group : SD_HEADS;
    const int gchunks = (group + GC - 1) / GC;
    if ((long long)G * gchunks > 65535) return AIE_UNSUPPORTED;
    dim3 grid(S, G * gchunks, n);
#define SK_DEC(DK_, DV_)                                                                                              \
    {                                                                                                                 \
        const size_t smem = SdSmem<DK_, DV_>::bytes;                                                                  \
        auto kern = sink_decode_kernel<DK_, DV_>;                                                                     \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                           \
        kern<<<grid, SD_WARPS * 32, smem, stream>>>((const bf16*)q, (const bf16*)pages, (bf16*)out, part_o, part_lse, \
                                                    gate, temp, slope, sink, dec_tokens, positions, token_req,        \
                                                    block_table, bt_width, num_pages, P, H, G, GC, window,            \
                                                    keep_first, scale, S, err);                                       \
    }
    SK_DISPATCH_ALL(SK_DEC)
#undef SK_DEC
    if (S > 1) {
        const cudaError_t e1 = cudaGetLastError();
        if (e1 != cudaSuccess) return (int)e1;
        sink_join_kernel<<<dim3(n, H), 128, 0, stream>>>(part_o, part_lse, (bf16*)out, gate, sink, dec_tokens, H, e, S);
    }
    AIE_LAUNCH_CHECK();
}
