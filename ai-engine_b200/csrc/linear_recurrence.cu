// Linear attention with a decaying matrix state, per request and head:
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T        (S: [d, dv], a_t per key channel)
//     o_t = S_t^T q_t
// a_t is a constant per head (retention), a per-token, per-channel value (gated linear attention), or one number
// per token and head made here from a step size (a selective state space: dt = softplus(raw + bias),
// a = exp(-exp(a_log) dt), the value scaled by dt, queries and keys shared by `hpg` neighbouring heads, and
// skip[h] v added to the output).  The state is float32, lives in the request's slot and is carried from step
// to step.  A fourth form has no keys: what the forget gate lets go is what is written (fg_lower given):
// a_t = l + (1 - l) sigmoid(z_t + bias) with a lower bound l per channel, k_t = 1 - a_t, and the query is
// silu of its projection; z comes in place of the per-token decays, and the three are made in float32 while a
// token's rows are staged.
//
// The columns of S never mix: column j needs only v_t[j].  A warp owns 32 / lanes columns of one (request,
// head); `lanes` threads share a column, each with RPT consecutive rows of S in registers, and a token costs
// each thread 2 RPT multiply-adds and a shuffle reduction over its column's lanes.  Tokens of a portion run
// in order, so a portion of any length continues where the previous step left the state, and a request's
// result does not depend on what else is in the batch.  The eight warps of a block belong to one (request, head):
// they stage the queries, keys and decays of up to sixteen tokens at a time in shared memory with coalesced
// loads and then walk those tokens from there, so a token does not cost a round trip to memory.
#include "common.cuh"

#define LR_WARPS 8
#define LR_TOKENS 16        // most tokens staged at a time
#define LR_THREADS (LR_WARPS * 32)

// one update of a state element and one term of the output, in the state's type (float, or double for the exact path)
template <typename ST> __device__ __forceinline__ ST lr_update(ST a, ST s, float k, float v);
template <> __device__ __forceinline__ float lr_update<float>(float a, float s, float k, float v) { return fmaf(a, s, k * v); }
template <> __device__ __forceinline__ double lr_update<double>(double a, double s, float k, float v) {
    return fma(a, s, (double)k * (double)v);
}
template <typename ST> __device__ __forceinline__ ST lr_term(ST s, float q, ST o);
template <> __device__ __forceinline__ float lr_term<float>(float s, float q, float o) { return fmaf(s, q, o); }
template <> __device__ __forceinline__ double lr_term<double>(double s, float q, double o) { return fma(s, (double)q, o); }

// ST: the type the state is held in while a step's tokens are walked.  float: every update rounds to float32.  double
// (the float32 engine's state-space layers): step size and decay are worked out in double too.  A decay near one,
// rounded to float32, keeps few digits of its small rate, and where the step size hardly changes from token to token
// the same rounding repeats at every token: over a thousand tokens a far token's share drifts by a few 1e-5.  In
// double a portion's updates round once, when the state goes back to its float32 slot.
template <int RPT, typename ST>
__global__ void __launch_bounds__(LR_THREADS)
linear_recurrence_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, int ld,
                         const float* __restrict__ decay_tok, int ld_decay, const float* __restrict__ decay_head,
                         float q_scale, float k_scale, float* __restrict__ state, float* __restrict__ out,
                         const int* __restrict__ q_start, const int* __restrict__ q_len, const int* __restrict__ slots,
                         int H, int d, int dv, int lanes, int groups, int TT, int max_slots, int vec, int vec4, unsigned* err,
                         int hpg, const float* __restrict__ dt_raw, int ld_dt, const float* __restrict__ dt_bias,
                         const float* __restrict__ a_log, const float* __restrict__ skip, int max_len,
                         const float* __restrict__ fg_lower, const float* __restrict__ fg_bias) {
    extern __shared__ __align__(16) float lr_sm[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int bg = blockIdx.x % groups, h = (blockIdx.x / groups) % H, r = blockIdx.x / (groups * H);
    if (max_len > 0 && q_len[r] > max_len) return;               // a longer portion is another kernel's
    const int slot = slots[r];
    if (slot < 0 || slot >= max_slots) {
        if (tid == 0) atomicOr(err, AIE_DEV_SLOT_OOB);
        return;
    }
    const int cols = 32 / lanes, CB = LR_WARPS * cols;            // columns a warp / a block owns
    float* q_s = lr_sm;                                           // [TT][d]
    float* k_s = q_s + TT * d;
    float* a_s = k_s + TT * d;                                    // only with per-token decays
    float* v_s = decay_tok ? a_s + TT * d : a_s;                  // [TT][CB]
    float* sc_s = v_s + TT * (LR_WARPS * (32 / lanes));           // [TT][3]: decay, step size, the decay's rest (only with dt_raw)
    const int hq = h / hpg;                                       // the head whose queries and keys this one reads
    const float rate = dt_raw ? expf(a_log[h]) : 0.f, dtb = dt_raw ? dt_bias[h] : 0.f;
    const int g = lane % lanes, cb = warp * cols + lane / lanes, col = bg * CB + cb;
    const int row0 = g * RPT;
    const bool col_ok = col < dv;
    ST S[RPT];
    float* sp = state + (((size_t)slot * H + h) * d) * dv + col;
#pragma unroll
    for (int i = 0; i < RPT; ++i) S[i] = (col_ok && row0 + i < d) ? (ST)sp[(size_t)(row0 + i) * dv] : (ST)0;
    const float dh = decay_head ? decay_head[h] : 1.f;
    const int a = q_start[r], n = q_len[r];
    for (int t0 = 0; t0 < n; t0 += TT) {
        const int nt = min(TT, n - t0);
        __syncthreads();                                          // the previous tokens are done with
        for (int tok = warp; tok < nt; tok += LR_WARPS) {          // a warp stages a token's rows
            const size_t at = (size_t)(a + t0 + tok) * ld + hq * d;
            const size_t at_a = (size_t)(a + t0 + tok) * ld_decay + h * d;
            float vs = k_scale;
            if (dt_raw) {                                          // float32: softplus, then the decay of this token
                const float x = dt_raw[(size_t)(a + t0 + tok) * ld_dt + h] + dtb;
                float dtv = x > 20.f ? x : log1pf(expf(x));
                float ah = expf(-rate * dtv), al = 0.f;
                if (sizeof(ST) == 8) {                             // the exact path: step size and decay worked out in double
                    const double xd = (double)dt_raw[(size_t)(a + t0 + tok) * ld_dt + h] + (double)dtb;
                    const double dd = xd > 20.0 ? xd : log1p(exp(xd));
                    const double ad = exp(-exp((double)a_log[h]) * dd);
                    dtv = (float)dd;
                    ah = (float)ad;
                    al = (float)(ad - (double)ah);
                }
                if (lane == 0) {
                    sc_s[tok * 3] = ah;
                    sc_s[tok * 3 + 1] = dtv;
                    sc_s[tok * 3 + 2] = al;
                }
                vs *= dtv;
            }
            if (vec4) {
                for (int c = lane * 4; c < d; c += 128) {
                    *reinterpret_cast<float4*>(q_s + tok * d + c) = *reinterpret_cast<const float4*>(q + at + c);
                    if (k) *reinterpret_cast<float4*>(k_s + tok * d + c) = *reinterpret_cast<const float4*>(k + at + c);
                    if (decay_tok) *reinterpret_cast<float4*>(a_s + tok * d + c) = *reinterpret_cast<const float4*>(decay_tok + at_a + c);
                }
            } else {
                for (int c = lane; c < d; c += 32) {
                    q_s[tok * d + c] = q[at + c];
                    if (k) k_s[tok * d + c] = k[at + c];
                    if (decay_tok) a_s[tok * d + c] = decay_tok[at_a + c];
                }
            }
            if (fg_lower) {                                        // gate, key and query of the keyless form
                __syncwarp();
                for (int c = lane; c < d; c += 32) {
                    const float lo = fg_lower[h * d + c];
                    const float z = a_s[tok * d + c] + (fg_bias ? fg_bias[h * d + c] : 0.f);
                    const float f = lo + (1.0f - lo) * (1.0f / (1.0f + expf(-z)));
                    a_s[tok * d + c] = f;
                    k_s[tok * d + c] = 1.0f - f;
                    const float qq = q_s[tok * d + c];
                    q_s[tok * d + c] = qq / (1.0f + expf(-qq));
                }
            }
            for (int c = lane; c < CB; c += 32)
                v_s[tok * CB + c] = bg * CB + c < dv ? v[(size_t)(a + t0 + tok) * ld + h * dv + bg * CB + c] * vs : 0.f;
        }
        __syncthreads();
        // the staged tokens' updates first, then their reductions over the column's lanes side by side (sixteen
        // independent chains of shuffles instead of one after each token)
        ST oacc[LR_TOKENS];
#pragma unroll
        for (int tok = 0; tok < LR_TOKENS; ++tok) {
            oacc[tok] = (ST)0;
            if (tok >= nt) continue;
            const float* qr = q_s + tok * d + row0;
            const float* kr = k_s + tok * d + row0;
            const float* ar = decay_tok ? a_s + tok * d + row0 : nullptr;
            const float vv = v_s[tok * CB + cb];
            const ST dh_t = dt_raw ? (ST)sc_s[tok * 3] + (ST)sc_s[tok * 3 + 2] : (ST)dh;
            ST o = (ST)0, o2 = (ST)0;                              // two chains of additions
            if (vec) {
#pragma unroll
                for (int i = 0; i < RPT; i += 4) {
                    if (row0 + i < d) {
                        const float4 q4 = *reinterpret_cast<const float4*>(qr + i);
                        const float4 k4 = *reinterpret_cast<const float4*>(kr + i);
                        float4 a4 = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (ar) a4 = *reinterpret_cast<const float4*>(ar + i);
                        S[i] = lr_update<ST>(ar ? (ST)a4.x : dh_t, S[i], k4.x, vv);
                        S[i + 1] = lr_update<ST>(ar ? (ST)a4.y : dh_t, S[i + 1], k4.y, vv);
                        S[i + 2] = lr_update<ST>(ar ? (ST)a4.z : dh_t, S[i + 2], k4.z, vv);
                        S[i + 3] = lr_update<ST>(ar ? (ST)a4.w : dh_t, S[i + 3], k4.w, vv);
                        o = lr_term<ST>(S[i], q4.x, o);
                        o = lr_term<ST>(S[i + 1], q4.y, o);
                        o2 = lr_term<ST>(S[i + 2], q4.z, o2);
                        o2 = lr_term<ST>(S[i + 3], q4.w, o2);
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < RPT; ++i) {
                    if (row0 + i < d) {
                        const ST al = ar ? (ST)ar[i] : dh_t;
                        S[i] = lr_update<ST>(al, S[i], kr[i], vv);
                        o = lr_term<ST>(S[i], qr[i], o);
                    }
                }
            }
            oacc[tok] = o + o2;
        }
        for (int off = lanes >> 1; off > 0; off >>= 1) {
#pragma unroll
            for (int tok = 0; tok < LR_TOKENS; ++tok) oacc[tok] += __shfl_xor_sync(0xffffffffu, oacc[tok], off);
        }
        if (g == 0 && col_ok) {
#pragma unroll
            for (int tok = 0; tok < LR_TOKENS; ++tok)
                if (tok < nt) {
                    float o = (float)(oacc[tok] * (ST)q_scale);
                    if (skip) o = fmaf(skip[h], v[(size_t)(a + t0 + tok) * ld + h * dv + col], o);
                    out[((size_t)(a + t0 + tok) * H + h) * dv + col] = o;
                }
        }
    }
    if (col_ok) {
#pragma unroll
        for (int i = 0; i < RPT; ++i)
            if (row0 + i < d) sp[(size_t)(row0 + i) * dv] = (float)S[i];
    }
}

// ---------------------------------------------------------------------------
// One token per request of the state-space form (dt_raw given): the step reads and writes every state once, so it
// runs at the speed of memory when rows of the state are read whole.  One block per (request, head): a thread owns
// four neighbouring value columns (16 bytes) of every `rows_step`-th state row, updates them, and keeps its share
// of y = S^T q; the shares are added through shared memory in a fixed order.
// ---------------------------------------------------------------------------
#define SS_THREADS 256
__global__ void __launch_bounds__(SS_THREADS)
state_space_step_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, int ld,
                        const float* __restrict__ dt_raw, int ld_dt, const float* __restrict__ dt_bias,
                        const float* __restrict__ a_log, const float* __restrict__ skip, float* __restrict__ state,
                        float* __restrict__ out, const int* __restrict__ q_start, const int* __restrict__ slots, int H,
                        int d, int dv, int hpg, int max_slots, int wide, unsigned* err) {
    extern __shared__ __align__(16) float ss_sm[];
    const int tid = threadIdx.x, h = blockIdx.x % H, r = blockIdx.x / H;
    const int slot = slots[r];
    if (slot < 0 || slot >= max_slots) {
        if (tid == 0) atomicOr(err, AIE_DEV_SLOT_OOB);
        return;
    }
    const int t = q_start[r], hq = h / hpg;
    const int c4 = dv / 4;                            // float4 columns of a row
    const int rows_step = SS_THREADS / c4;            // rows the block covers at a time (c4 divides the block)
    float* k_s = ss_sm;                               // [d]  B dt
    float* q_s = k_s + d;                             // [d]  C
    float* y_s = q_s + d;                             // [rows_step][dv]
    const float x = dt_raw[(size_t)t * ld_dt + h] + dt_bias[h];
    float dtv = x > 20.f ? x : log1pf(expf(x));
    const float a = expf(-expf(a_log[h]) * dtv);
    double ad = (double)a;
    if (wide) {       // the exact path: a decay near one keeps the digits of its small rate only in double
        const double xd = (double)dt_raw[(size_t)t * ld_dt + h] + (double)dt_bias[h];
        const double dd = xd > 20.0 ? xd : log1p(exp(xd));
        ad = exp(-exp((double)a_log[h]) * dd);
        dtv = (float)dd;
    }
    for (int i = tid; i < d; i += SS_THREADS) {
        k_s[i] = k[(size_t)t * ld + (size_t)hq * d + i] * dtv;
        q_s[i] = q[(size_t)t * ld + (size_t)hq * d + i];
    }
    __syncthreads();
    const int col = (tid % c4) * 4, row0 = tid / c4;
    const float4 xv = *reinterpret_cast<const float4*>(v + (size_t)t * ld + (size_t)h * dv + col);
    float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
    float* sp = state + (((size_t)slot * H + h) * d) * dv + col;
    if (row0 < rows_step) {
        for (int n = row0; n < d; n += rows_step) {
            float4 s4 = *reinterpret_cast<float4*>(sp + (size_t)n * dv);
            const float kk = k_s[n], qq = q_s[n];
            if (wide) {
                s4.x = (float)fma(ad, (double)s4.x, (double)kk * (double)xv.x);
                s4.y = (float)fma(ad, (double)s4.y, (double)kk * (double)xv.y);
                s4.z = (float)fma(ad, (double)s4.z, (double)kk * (double)xv.z);
                s4.w = (float)fma(ad, (double)s4.w, (double)kk * (double)xv.w);
            } else {
                s4.x = fmaf(a, s4.x, kk * xv.x);
                s4.y = fmaf(a, s4.y, kk * xv.y);
                s4.z = fmaf(a, s4.z, kk * xv.z);
                s4.w = fmaf(a, s4.w, kk * xv.w);
            }
            *reinterpret_cast<float4*>(sp + (size_t)n * dv) = s4;
            y.x = fmaf(s4.x, qq, y.x);
            y.y = fmaf(s4.y, qq, y.y);
            y.z = fmaf(s4.z, qq, y.z);
            y.w = fmaf(s4.w, qq, y.w);
        }
        *reinterpret_cast<float4*>(y_s + (size_t)row0 * dv + col) = y;
    }
    __syncthreads();
    for (int c = tid; c < dv; c += SS_THREADS) {
        float acc = 0.f;
        for (int g = 0; g < rows_step; ++g) acc += y_s[(size_t)g * dv + c];
        if (skip) acc = fmaf(skip[h], v[(size_t)t * ld + (size_t)h * dv + c], acc);
        out[((size_t)t * H + h) * dv + c] = acc;
    }
}

// q, k [T, .] with head h's d channels at column h d of rows `ld` floats apart; v likewise with dv columns a
// head; decay_tok [T, .] rows `ld_decay` apart (or null: decay_head [H] constants).  The key is scaled by
// k_scale, the output by q_scale (both 1 or d^-1/2).  state [max_slots, H, d, dv]; out [T, H, dv].
// dt_raw [T, .] (rows ld_dt apart, head h at column h) with dt_bias, a_log [H]: the decay comes from the step size
// as the header says; hpg: heads that share one head of q and k (1: each its own); skip [H] or null.
// max_len > 0: requests that bring more tokens are left alone (the chunked kernel takes them).
// wide_state: the state is held in double while a step's tokens are walked (see the kernel's header).
extern "C" int aie_linear_recurrence(const float* q, const float* k, const float* v, int ld, const float* decay_tok,
                                     int ld_decay, const float* decay_head, float q_scale, float k_scale, float* state,
                                     float* out, const int* q_start, const int* q_len, const int* slots, int T, int R,
                                     int H, int d, int dv, int max_slots, unsigned* err, int hpg, const float* dt_raw,
                                     int ld_dt, const float* dt_bias, const float* a_log, const float* skip, int max_len,
                                     int wide_state, const float* fg_lower, const float* fg_bias, cudaStream_t st) {
    if (R <= 0) return 0;
    if (H <= 0 || d <= 0 || dv <= 0 || (!decay_tok && !decay_head && !dt_raw)) return AIE_BAD_ARG;
    if (fg_lower ? (!decay_tok || k || hpg != 1) : !k) return AIE_BAD_ARG;
    if (hpg < 1 || H % hpg || (dt_raw && (!dt_bias || !a_log || decay_tok))) return AIE_BAD_ARG;
    if (d > 1024) return AIE_UNSUPPORTED;
    // a step of single tokens in the state-space form: the kernel that reads rows of the state whole
    if (dt_raw && T == R && max_len <= 0 && dv % 4 == 0 && dv / 4 <= SS_THREADS && SS_THREADS % (dv / 4) == 0 && ld % 4 == 0 &&
        !((size_t)v & 15) && !((size_t)state & 15) && q_scale == 1.f && k_scale == 1.f) {
        const int rows_step = SS_THREADS / (dv / 4);
        const size_t smem = ((size_t)2 * d + (size_t)rows_step * dv) * sizeof(float);
        if (smem <= 48 * 1024 && (long long)R * H <= 0x7fffffffLL) {
            state_space_step_kernel<<<(unsigned)(R * H), SS_THREADS, smem, st>>>(q, k, v, ld, dt_raw, ld_dt, dt_bias, a_log, skip,
                                                                                 state, out, q_start, slots, H, d, dv, hpg,
                                                                                 max_slots, wide_state, err);
            AIE_LAUNCH_CHECK();
        }
    }
    // A step of single tokens is bound by reading and writing the states: many rows a thread, so that a warp's
    // accesses to a row of the state are wide.  A step of prompt portions is bound by the chain of dependent
    // updates token after token: few rows a thread, so that many warps hide one another's latency.
    int rpt = d <= 32 ? 8 : (d <= 128 ? 16 : 32);
    if (T >= 8 * R) rpt = d <= 128 ? 4 : (d <= 256 ? 8 : (d <= 512 ? 16 : 32));
    int lanes = 1;
    while (lanes * rpt < d) lanes <<= 1;
    const int cols = 32 / lanes, CB = LR_WARPS * cols, groups = (dv + CB - 1) / CB;
    const long long blocks = (long long)R * H * groups;
    if (blocks > 0x7fffffffLL) return AIE_UNSUPPORTED;
    int TT = 3072 / d;      // at most 36 KB of staged queries, keys and decays
    TT = TT < 1 ? 1 : (TT > LR_TOKENS ? LR_TOKENS : TT);
    const size_t smem = ((size_t)TT * d * (decay_tok ? 3 : 2) + (size_t)TT * CB + 3 * TT) * sizeof(float);
    // rows of the staged tokens are read as float4: the head's width and every thread's first row are multiples of 4
    const int vec = d % 4 == 0 ? 1 : 0;
    // ... and the rows in memory too when the row strides and base addresses allow 16-byte loads
    const int vec4 = (vec && ld % 4 == 0 && !((size_t)q & 15) && !((size_t)k & 15) &&
                      (!decay_tok || (ld_decay % 4 == 0 && !((size_t)decay_tok & 15)))) ? 1 : 0;
#define GO(N)                                                                                                       \
    do {                                                                                                            \
    if (wide_state)                                                                                                 \
        linear_recurrence_kernel<N, double><<<(unsigned)blocks, LR_THREADS, smem, st>>>(q, k, v, ld, decay_tok, ld_decay, decay_head,  \
                                                                     q_scale, k_scale, state, out, q_start, q_len,  \
                                                                     slots, H, d, dv, lanes, groups, TT, max_slots, \
                                                                     vec, vec4, err, hpg, dt_raw, ld_dt, dt_bias,   \
                                                                     a_log, skip, max_len, fg_lower, fg_bias);      \
    else                                                                                                            \
        linear_recurrence_kernel<N, float><<<(unsigned)blocks, LR_THREADS, smem, st>>>(q, k, v, ld, decay_tok, ld_decay, decay_head,  \
                                                                     q_scale, k_scale, state, out, q_start, q_len,  \
                                                                     slots, H, d, dv, lanes, groups, TT, max_slots, \
                                                                     vec, vec4, err, hpg, dt_raw, ld_dt, dt_bias,   \
                                                                     a_log, skip, max_len, fg_lower, fg_bias);      \
    } while (0)
    if (rpt == 4) GO(4);
    else if (rpt == 8) GO(8);
    else if (rpt == 16) GO(16);
    else GO(32);
#undef GO
    AIE_LAUNCH_CHECK();
}
