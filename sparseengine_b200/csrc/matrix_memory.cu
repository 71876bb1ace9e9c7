// Matrix memory with exponential gates (the mLSTM cell of xLSTM), 32-bit state.
//
// Per request and head a matrix S [d, dv], a vector n [d] and a running maximum m (all start at 0):
//
//     i_t = cap tanh(a_t / cap)                      log input gate   (a, b: the gates' projections plus bias)
//     f_t = logsigmoid(cap tanh(b_t / cap))          log forget gate
//     m_t = max(f_t + m_(t-1), i_t)
//     S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T ;  n_t likewise with k_t alone
//     o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//
// n is kept as one more column of S (a value column of ones), so the state row of a request is
// [head][d][dv + 1] followed by m [head].  Three kernels: the gates (the scalar recurrence of m, a warp
// per request and head, 32 tokens at a time by prefix sum and prefix maximum), the matrix recurrence
// (token by token for steps of single tokens, in chunks of 64 tokens for prompt portions),
// and the epilogue (denominator, each head's root mean square, weight, sigmoid gate).  q, k, v and the
// gate come from the projection in the activation type; everything else is 32-bit.
//
// A step brings any mix of prompt portions and single tokens: entry s owns the tokens
// cu_q[s] .. cu_q[s+1]-1 and the state row seq_rows[s].
#include "common.cuh"

namespace se {

__device__ __forceinline__ float log_sigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// gates[t][h] = (log keep, log take, exp(-m_t)) with keep = exp(f_t + m_(t-1) - m_t) and take = exp(i_t - m_t);
// the request's m is brought up to date.  One warp per (entry, head).
template <typename T>
__global__ void memory_gates_kernel(const T* proj, int pitch, int i_off, int f_off, const float* __restrict__ bias,
                                    float cap, float* state, long long state_pitch, int m_off,
                                    const int* __restrict__ cu_q, const int* __restrict__ seq_rows,
                                    float* __restrict__ gates, int H) {
    const int e = blockIdx.x, h = blockIdx.y, lane = threadIdx.x;
    const int t0 = cu_q[e], t1 = cu_q[e + 1];
    if (t1 <= t0) return;
    float* mp = state + (size_t)seq_rows[e] * state_pitch + m_off + h;
    float m_in = *mp;
    const float bi = bias != nullptr ? bias[h] : 0.f, bf = bias != nullptr ? bias[H + h] : 0.f;
    // the gates' projections of the next 32 tokens are asked for before the current 32 are used
    auto fetch = [&](int t, float& a, float& b) {
        if (t < t1) {
            const T* row = proj + (size_t)t * pitch;
            a = to_float(row[i_off + h]);
            b = to_float(row[f_off + h]);
        }
    };
    float a_next = 0.f, b_next = 0.f;
    fetch(t0 + lane, a_next, b_next);
    for (int base = t0; base < t1; base += 32) {
        const int t = base + lane;
        const bool valid = t < t1;
        const float a_now = a_next, b_now = b_next;
        fetch(base + 32 + lane, a_next, b_next);
        float gi = -INFINITY, gf = 0.f;
        if (valid) {
            gi = cap * tanhf((a_now + bi) / cap);
            gf = log_sigmoid_f(cap * tanhf((b_now + bf) / cap));
        }
        float F = gf;                       // sum of the log forget gates up to this token, within the 32
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float v = __shfl_up_sync(0xffffffffu, F, o);
            if (lane >= o) F += v;
        }
        float A = gi - F;                   // the largest i_s - F_s up to this token
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float v = __shfl_up_sync(0xffffffffu, A, o);
            if (lane >= o) A = fmaxf(A, v);
        }
        const float m = F + fmaxf(m_in, A);
        float m_prev = __shfl_up_sync(0xffffffffu, m, 1);
        if (lane == 0) m_prev = m_in;
        if (valid) {
            float* g = gates + ((size_t)t * H + h) * 3;
            g[0] = gf + m_prev - m;
            g[1] = gi - m;
            g[2] = expf(-m);
        }
        const int last = min(31, t1 - 1 - base);
        m_in = __shfl_sync(0xffffffffu, m, last);
    }
    if (lane == 0) *mp = m_in;
}

constexpr int kMemWarps = 8;        // the state's rows are dealt to the warps: warp r holds rows r, r + 8, ...
constexpr int kMemTokens = 8;       // tokens staged at a time

// One block per (entry, head, 32 columns of [values | 1]).  Thread (warp r, lane c) keeps rows r + 8 n of
// column c in registers; a token's partial sums over a warp's rows meet in shared memory, eight tokens at
// a time.  o [tokens, heads, dv + 1]: the last column is n . q.  Sums run in one fixed order whatever the
// batch or the portion.
template <typename T, int NPT>
__global__ void __launch_bounds__(32 * kMemWarps)
memory_scan_kernel(const T* proj, int pitch, int q_off, int k_off, int v_off, const float* __restrict__ gates,
                   float q_scale, float* state, long long state_pitch, const int* __restrict__ cu_q,
                   const int* __restrict__ seq_rows, float* __restrict__ o, int H, int d, int dv) {
    extern __shared__ float mem_smem[];
    float* qs = mem_smem;                                   // [kMemTokens][d]
    float* ks = qs + kMemTokens * d;                        // [kMemTokens][d], times the token's input gate
    float* vs = ks + kMemTokens * d;                        // [kMemTokens][32]
    float* red = vs + kMemTokens * 32;                      // [kMemTokens][kMemWarps][32]
    float* keep = red + kMemTokens * kMemWarps * 32;        // [kMemTokens]
    const int s = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int cols = dv + 1, col = c0 + lane;
    const bool col_ok = col < cols;
    const int t0 = cu_q[s], t1 = cu_q[s + 1];
    if (t1 <= t0) return;
    float* S = state + (size_t)seq_rows[s] * state_pitch + (size_t)h * d * cols;
    float st[NPT];
#pragma unroll
    for (int n = 0; n < NPT; ++n) {
        const int i = warp + kMemWarps * n;
        st[n] = (i < d && col_ok) ? S[(size_t)i * cols + col] : 0.f;
    }
    for (int tb = t0; tb < t1; tb += kMemTokens) {
        const int nt = min(kMemTokens, t1 - tb);
        __syncthreads();                                    // the last round's sums have been read
        for (int x = threadIdx.x; x < nt * d; x += blockDim.x) {
            const int tt = x / d, i = x - tt * d;
            const T* row = proj + (size_t)(tb + tt) * pitch;
            qs[x] = to_float(row[q_off + h * d + i]) * q_scale;
            ks[x] = to_float(row[k_off + h * d + i]) * expf(gates[((size_t)(tb + tt) * H + h) * 3 + 1]);
        }
        for (int x = threadIdx.x; x < nt * 32; x += blockDim.x) {
            const int tt = x >> 5, c = c0 + (x & 31);
            vs[x] = c < dv ? to_float(proj[(size_t)(tb + tt) * pitch + v_off + h * dv + c]) : (c == dv ? 1.f : 0.f);
        }
        if ((int)threadIdx.x < nt) keep[threadIdx.x] = expf(gates[((size_t)(tb + threadIdx.x) * H + h) * 3]);
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float v = vs[tt * 32 + lane], g = keep[tt];
            float acc = 0.f;
#pragma unroll
            for (int n = 0; n < NPT; ++n) {
                const int i = warp + kMemWarps * n;
                if (i < d) {
                    st[n] = g * st[n] + ks[tt * d + i] * v;
                    acc += st[n] * qs[tt * d + i];
                }
            }
            red[(tt * kMemWarps + warp) * 32 + lane] = acc;
        }
        __syncthreads();
        for (int x = threadIdx.x; x < nt * 32; x += blockDim.x) {
            const int tt = x >> 5, c = x & 31;
            if (c0 + c < cols) {
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < kMemWarps; ++w) sum += red[(tt * kMemWarps + w) * 32 + c];
                o[((size_t)(tb + tt) * H + h) * cols + c0 + c] = sum;
            }
        }
    }
#pragma unroll
    for (int n = 0; n < NPT; ++n) {
        const int i = warp + kMemWarps * n;
        if (i < d && col_ok) S[(size_t)i * cols + col] = st[n];
    }
}

// ---- prompt portions: the recurrence in chunks of 64 tokens -----------------------------------------
//
// With B_t the sum of the log keeps of a chunk's tokens 0..t and l_s the log take of token s, the recurrence
// over a chunk of n tokens has a closed form:
//
//     o_t   = exp(B_t) S_0^T q_t + sum_{s <= t} exp(B_t - B_s + l_s) (q_t . k_s) [v_s | 1]
//     S_new = exp(B_(n-1)) S_0 + sum_s exp(B_(n-1) - B_s + l_s) k_s [v_s | 1]^T
//
// which is three small matrix products per chunk instead of a chain of n dependent steps; every exponent
// is at most 0 (the running maximum sees to that).  The normaliser's column of ones needs no products: its share of
// o_t is the sum over s of the weighted scores, which the block of a head's first 32 value columns adds up.  All of it is 32-bit FMA arithmetic; the sums B are taken
// in 64-bit, so that their differences keep the digits of the single terms.  One block per (entry, head,
// 32 value columns): q and k of the chunk lie transposed in shared memory (`[dim][token]`, padded
// rows), the block's slice of the state stays in shared memory over all chunks.
constexpr int kChunk = 64;
constexpr int kChunkThreads = 256;
constexpr int kPitch = kChunk + 4;
__device__ __forceinline__ int swz(int i, int t) { return i * kPitch + t; }

template <typename T>
__global__ void __launch_bounds__(kChunkThreads, 2)
memory_chunk_kernel(const T* proj, int pitch, int q_off, int k_off, int v_off, const float* __restrict__ gates,
                    float q_scale, float* state, long long state_pitch, const int* __restrict__ cu_q,
                    const int* __restrict__ seq_rows, float* __restrict__ o, int H, int d, int dv, int max_seg, int seg_len,
                    float* __restrict__ seg_state, double* __restrict__ seg_logs) {
    extern __shared__ __align__(16) float chunk_smem[];
    float* qs = chunk_smem;                      // [d][kPitch]
    float* ks = qs + d * kPitch;                 // [d][kPitch]
    float* vs = ks + d * kPitch;                 // [64][32]
    float* As = vs + kChunk * 32;                // [64 s][64 t]: exp(B_t - B_s + l_s) q_t . k_s for s <= t, else 0
    float* Ss = As + kChunk * kChunk;            // [d][32]
    float* ls = Ss + d * 32;                     // [64] log takes
    double* Bs = reinterpret_cast<double*>(ls + kChunk);      // [64] sums of the log keeps (8-byte aligned: every part before is a multiple of 8 bytes)
    float* ws = reinterpret_cast<float*>(Bs + kChunk);        // [64] what token s adds to the state after the chunk: exp(B_(n-1) - B_s + l_s)
    float* Ns = ws + kChunk;                                  // [d] the normaliser n (the state's last column), kept by the block of the first columns
    // With segments (seg_state != nullptr) block x = entry * max_seg + segment walks `seg_len` tokens of its entry from
    // a zero state, leaves the state it ends with in seg_state and the sum of its log keeps in seg_logs; what the true
    // state at the segment's start adds to the outputs follows in memory_seg_fix_kernel.  Without, it walks the whole
    // entry from the carried state.
    const int e = blockIdx.x / max_seg, sg = blockIdx.x - e * max_seg;
    const int h = blockIdx.y, c0 = blockIdx.z * 32;
    const int lane = threadIdx.x & 31, wg = threadIdx.x >> 5;
    const int cols = dv + 1;
    const int t_first = seg_state != nullptr ? cu_q[e] + sg * seg_len : cu_q[e];
    const int t_last = seg_state != nullptr ? min(cu_q[e + 1], t_first + seg_len) : cu_q[e + 1];
    if (t_last <= t_first) return;
    float* S = seg_state != nullptr ? seg_state + (((size_t)e * max_seg + sg) * H + h) * d * cols
                                    : state + (size_t)seq_rows[e] * state_pitch + (size_t)h * d * cols;
    const bool col_ok = c0 + lane < dv;
    // the block of a head's first 32 value columns also keeps the normaliser: its "value column" is all ones, so its
    // share of an output is the sum of the chunk's weighted scores, and no block spends a column's work on it
    const bool has_n = blockIdx.z == 0;
    for (int x = threadIdx.x; x < d * 32; x += kChunkThreads)
        Ss[x] = (seg_state == nullptr && c0 + (x & 31) < dv) ? S[(size_t)(x >> 5) * cols + c0 + (x & 31)] : 0.f;
    if (has_n)
        for (int i = threadIdx.x; i < d; i += kChunkThreads) Ns[i] = seg_state == nullptr ? S[(size_t)i * cols + dv] : 0.f;
    double log_total = 0.0;                       // the sum of the log keeps of all chunks so far
    const bool vec = (d & 7) == 0 && (pitch & 7) == 0 && (q_off & 7) == 0 && (k_off & 7) == 0 && aligned8(proj);

    for (int tb = t_first; tb < t_last; tb += kChunk) {
        const int n = min(kChunk, t_last - tb);
        __syncthreads();                          // the chunk before is done with q, k, v and A; the state is up to date
        // Everything the chunk needs from memory is asked for before any of it is used (one trip to memory per
        // chunk, not one per kind of input): the gates by warp 0, the values, then q and k.
        float g_keep[2] = {0.f, 0.f}, g_take[2] = {-INFINITY, -INFINITY};
        if (wg == 0) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int t = half * 32 + lane;
                if (t < n) {
                    const float* g = gates + ((size_t)(tb + t) * H + h) * 3;
                    g_keep[half] = g[0];
                    g_take[half] = g[1];
                }
            }
        }
        float vv[kChunk * 32 / kChunkThreads];
#pragma unroll
        for (int r = 0; r < kChunk * 32 / kChunkThreads; ++r) {
            const int x = threadIdx.x + r * kChunkThreads, t = x >> 5, c = c0 + (x & 31);
            vv[r] = (t < n && c < dv) ? to_float(proj[(size_t)(tb + t) * pitch + v_off + h * dv + c]) : 0.f;
        }
        if (vec) {
            // eight elements a load; a warp's lanes take the same eight dims of 32 tokens in a row, so that the
            // transposing stores fall into 32 banks
            const int pieces = kChunk * (d >> 3);
            for (int base = threadIdx.x; base < pieces; base += 4 * kChunkThreads) {
                float qv[4][8], kv[4][8];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int x = base + r * kChunkThreads, t = x & (kChunk - 1), i = (x >> 6) * 8;
                    if (x < pieces && t < n) {
                        const T* row = proj + (size_t)(tb + t) * pitch + h * d + i;
                        load8(row + q_off, qv[r]);
                        load8(row + k_off, kv[r]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j) qv[r][j] = kv[r][j] = 0.f;
                    }
                }
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int x = base + r * kChunkThreads, t = x & (kChunk - 1), i = (x >> 6) * 8;
                    if (x < pieces) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            qs[swz(i + j, t)] = qv[r][j] * q_scale;
                            ks[swz(i + j, t)] = kv[r][j];
                        }
                    }
                }
            }
        } else {
            for (int x = threadIdx.x; x < kChunk * d; x += kChunkThreads) {
                const int t = x / d, i = x - t * d;
                float qv = 0.f, kv = 0.f;
                if (t < n) {
                    const T* row = proj + (size_t)(tb + t) * pitch;
                    qv = to_float(row[q_off + h * d + i]) * q_scale;
                    kv = to_float(row[k_off + h * d + i]);
                }
                qs[swz(i, t)] = qv;
                ks[swz(i, t)] = kv;
            }
        }
#pragma unroll
        for (int r = 0; r < kChunk * 32 / kChunkThreads; ++r) vs[threadIdx.x + r * kChunkThreads] = vv[r];
        if (wg == 0) {                            // the sums of the log keeps, 64-bit, by one warp
            double carry = 0.0;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int t = half * 32 + lane;
                double b = (double)g_keep[half];
                ls[t] = g_take[half];
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    const double v = __shfl_up_sync(0xffffffffu, b, off);
                    if (lane >= off) b += v;
                }
                b += carry;
                Bs[t] = b;
                carry = __shfl_sync(0xffffffffu, b, 31);
            }
        }
        __syncthreads();
        // scores of the chunk with their weights: a 4 x 4 tile per thread, tiles above the diagonal are zero
        {
            const int tt = (threadIdx.x >> 4) * 4, ss = (threadIdx.x & 15) * 4;
            float acc[4][4] = {};
            if (ss <= tt + 3) {
#pragma unroll 4
                for (int i = 0; i < d; ++i) {
                    const float4 qv = *reinterpret_cast<const float4*>(qs + swz(i, tt));
                    const float4 kv = *reinterpret_cast<const float4*>(ks + swz(i, ss));
                    const float qa[4] = {qv.x, qv.y, qv.z, qv.w}, ka[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
                    for (int a = 0; a < 4; ++a)
#pragma unroll
                        for (int b = 0; b < 4; ++b) acc[a][b] += qa[a] * ka[b];
                }
            }
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                float4 row;
                float* r = &row.x;
#pragma unroll
                for (int a = 0; a < 4; ++a)
                    r[a] = (ss + b <= tt + a && tt + a < n) ? acc[a][b] * expf((float)(Bs[tt + a] - Bs[ss + b]) + ls[ss + b]) : 0.f;
                *reinterpret_cast<float4*>(As + (ss + b) * kChunk + tt) = row;
            }
        }
        float vreg[kChunk];                        // this lane's value column of the chunk
#pragma unroll
        for (int s_ = 0; s_ < kChunk; ++s_) vreg[s_] = vs[s_ * 32 + lane];
        __syncthreads();
        // outputs: warp wg takes tokens 8 wg .. 8 wg + 7, lane c the column
        {
            const int tg = wg * 8;
            float acc[8] = {}, acc2[8] = {};
#pragma unroll
            for (int s_ = 0; s_ < kChunk; ++s_) {
                const float4 a0 = *reinterpret_cast<const float4*>(As + s_ * kChunk + tg);
                const float4 a1 = *reinterpret_cast<const float4*>(As + s_ * kChunk + tg + 4);
                const float v = vreg[s_];
                acc[0] += a0.x * v; acc[1] += a0.y * v; acc[2] += a0.z * v; acc[3] += a0.w * v;
                acc[4] += a1.x * v; acc[5] += a1.y * v; acc[6] += a1.z * v; acc[7] += a1.w * v;
            }
#pragma unroll 4
            for (int i = 0; i < d; ++i) {
                const float4 q0 = *reinterpret_cast<const float4*>(qs + swz(i, tg));
                const float4 q1 = *reinterpret_cast<const float4*>(qs + swz(i, tg + 4));
                const float sv = Ss[i * 32 + lane];
                acc2[0] += q0.x * sv; acc2[1] += q0.y * sv; acc2[2] += q0.z * sv; acc2[3] += q0.w * sv;
                acc2[4] += q1.x * sv; acc2[5] += q1.y * sv; acc2[6] += q1.z * sv; acc2[7] += q1.w * sv;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int t = tg + j;
                if (t < n && col_ok) o[((size_t)(tb + t) * H + h) * cols + c0 + lane] = acc[j] + expf((float)Bs[t]) * acc2[j];
            }
        }
        const double b_end = Bs[n - 1];
        log_total += b_end;
        if (threadIdx.x < kChunk) {
            const int t = threadIdx.x;
            if (has_n) {                          // n . q of token t: the column of ones
                float den = 0.f, dot = 0.f;
#pragma unroll 8
                for (int s_ = 0; s_ < kChunk; ++s_) den += As[s_ * kChunk + t];
#pragma unroll 4
                for (int i = 0; i < d; ++i) dot += qs[swz(i, t)] * Ns[i];
                if (t < n) o[((size_t)(tb + t) * H + h) * cols + dv] = den + expf((float)Bs[t]) * dot;
            }
            ws[t] = t < n ? expf((float)(b_end - Bs[t]) + ls[t]) : 0.f;
        }
        __syncthreads();                          // every read of the old state is done
        // the state after the chunk: warp wg takes rows wg, wg + 8, ...
#pragma unroll
        for (int s_ = 0; s_ < kChunk; ++s_) vreg[s_] *= ws[s_];
        const float gn = expf((float)b_end);
        if (has_n)
            for (int i = threadIdx.x; i < d; i += kChunkThreads) {
                float a = 0.f;
#pragma unroll
                for (int s4 = 0; s4 < kChunk; s4 += 4) {
                    const float4 kv = *reinterpret_cast<const float4*>(ks + swz(i, s4));
                    a += kv.x * ws[s4] + kv.y * ws[s4 + 1] + kv.z * ws[s4 + 2] + kv.w * ws[s4 + 3];
                }
                Ns[i] = gn * Ns[i] + a;
            }
        for (int i = wg; i < d; i += kChunkThreads / 32) {
            float a = 0.f;
#pragma unroll
            for (int s4 = 0; s4 < kChunk; s4 += 4) {
                const float4 kv = *reinterpret_cast<const float4*>(ks + swz(i, s4));
                a += kv.x * vreg[s4] + kv.y * vreg[s4 + 1] + kv.z * vreg[s4 + 2] + kv.w * vreg[s4 + 3];
            }
            Ss[i * 32 + lane] = gn * Ss[i * 32 + lane] + a;
        }
    }
    __syncthreads();
    for (int x = threadIdx.x; x < d * 32; x += kChunkThreads)
        if (c0 + (x & 31) < dv) S[(size_t)(x >> 5) * cols + c0 + (x & 31)] = Ss[x];
    if (has_n)
        for (int i = threadIdx.x; i < d; i += kChunkThreads) S[(size_t)i * cols + dv] = Ns[i];
    if (seg_logs != nullptr && threadIdx.x == 0 && blockIdx.z == 0) seg_logs[((size_t)e * max_seg + sg) * H + h] = log_total;
}

// The segments of an entry joined: seg_state[e, j] holds what segment j alone leaves; it becomes the state at
// segment j's start, S_0 = the carried state, S_(j+1) = exp(sum of segment j's log keeps) S_j + (what segment j
// leaves), and the last one goes back to the entry's state row.  One thread per state element.
__global__ void memory_seg_join_kernel(float* __restrict__ seg_state, const double* __restrict__ seg_logs, float* state,
                                       long long state_pitch, const int* __restrict__ cu_q, const int* __restrict__ seq_rows,
                                       int H, int d, int cols, int max_seg, int seg_len) {
    const int e = blockIdx.y, h = blockIdx.z;
    const int n = cu_q[e + 1] - cu_q[e];
    if (n <= 0) return;
    const int nseg = (n + seg_len - 1) / seg_len;
    float* S = state + (size_t)seq_rows[e] * state_pitch + (size_t)h * d * cols;
    for (int x = blockIdx.x * blockDim.x + threadIdx.x; x < d * cols; x += gridDim.x * blockDim.x) {
        float cur = S[x];
        for (int j = 0; j < nseg; ++j) {
            float* p = seg_state + (((size_t)e * max_seg + j) * H + h) * d * cols + x;
            const float left = *p;
            *p = cur;
            cur = expf((float)seg_logs[((size_t)e * max_seg + j) * H + h]) * cur + left;
        }
        S[x] = cur;
    }
}

// o_t += exp(B_t) S_start^T q_t for the tokens of a segment (B_t: the sum of the log keeps from the segment's start
// to t): what the state at the segment's start adds to outputs that were computed from a zero state.
template <typename T>
__global__ void __launch_bounds__(kChunkThreads, 2)
memory_seg_fix_kernel(const T* proj, int pitch, int q_off, const float* __restrict__ gates, float q_scale,
                      const float* __restrict__ seg_state, const int* __restrict__ cu_q, float* __restrict__ o, int H, int d,
                      int dv, int max_seg, int seg_len) {
    extern __shared__ __align__(16) float fix_smem[];
    float* qs = fix_smem;                        // [d][kPitch]
    float* Ss = qs + d * kPitch;                 // [d][32]
    double* Bs = reinterpret_cast<double*>(Ss + d * 32);      // [64]
    float* Ns = reinterpret_cast<float*>(Bs + kChunk);        // [d] the normaliser at the segment's start (block of the first columns)
    const int e = blockIdx.x / max_seg, sg = blockIdx.x - e * max_seg;
    const int h = blockIdx.y, c0 = blockIdx.z * 32;
    const int lane = threadIdx.x & 31, wg = threadIdx.x >> 5;
    const int cols = dv + 1;
    const int t_first = cu_q[e] + sg * seg_len, t_last = min(cu_q[e + 1], t_first + seg_len);
    if (t_last <= t_first) return;
    const float* S = seg_state + (((size_t)e * max_seg + sg) * H + h) * d * cols;
    for (int x = threadIdx.x; x < d * 32; x += kChunkThreads)
        Ss[x] = c0 + (x & 31) < dv ? S[(size_t)(x >> 5) * cols + c0 + (x & 31)] : 0.f;
    const bool has_n = blockIdx.z == 0;
    if (has_n)
        for (int i = threadIdx.x; i < d; i += kChunkThreads) Ns[i] = S[(size_t)i * cols + dv];
    const bool col_ok = c0 + lane < dv;
    const bool vec = (d & 7) == 0 && (pitch & 7) == 0 && (q_off & 7) == 0 && aligned8(proj);
    double base_log = 0.0;                        // the sum of the log keeps of the segment's earlier chunks (warp 0 keeps it)
    for (int tb = t_first; tb < t_last; tb += kChunk) {
        const int n = min(kChunk, t_last - tb);
        __syncthreads();
        if (vec) {
            const int pieces = kChunk * (d >> 3);
            for (int x = threadIdx.x; x < pieces; x += kChunkThreads) {
                const int t = x & (kChunk - 1), i = (x >> 6) * 8;
                float qv[8] = {};
                if (t < n) load8(proj + (size_t)(tb + t) * pitch + q_off + h * d + i, qv);
#pragma unroll
                for (int j = 0; j < 8; ++j) qs[swz(i + j, t)] = qv[j] * q_scale;
            }
        } else {
            for (int x = threadIdx.x; x < kChunk * d; x += kChunkThreads) {
                const int t = x / d, i = x - t * d;
                qs[swz(i, t)] = t < n ? to_float(proj[(size_t)(tb + t) * pitch + q_off + h * d + i]) * q_scale : 0.f;
            }
        }
        if (wg == 0) {
            double carry = base_log;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int t = half * 32 + lane;
                double b = t < n ? (double)gates[((size_t)(tb + t) * H + h) * 3] : 0.0;
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    const double v = __shfl_up_sync(0xffffffffu, b, off);
                    if (lane >= off) b += v;
                }
                b += carry;
                Bs[t] = b;
                carry = __shfl_sync(0xffffffffu, b, 31);
            }
            base_log = carry;
        }
        __syncthreads();
        const int tg = wg * 8;
        float acc2[8] = {};
#pragma unroll 4
        for (int i = 0; i < d; ++i) {
            const float4 q0 = *reinterpret_cast<const float4*>(qs + swz(i, tg));
            const float4 q1 = *reinterpret_cast<const float4*>(qs + swz(i, tg + 4));
            const float sv = Ss[i * 32 + lane];
            acc2[0] += q0.x * sv; acc2[1] += q0.y * sv; acc2[2] += q0.z * sv; acc2[3] += q0.w * sv;
            acc2[4] += q1.x * sv; acc2[5] += q1.y * sv; acc2[6] += q1.z * sv; acc2[7] += q1.w * sv;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int t = tg + j;
            if (t < n && col_ok) o[((size_t)(tb + t) * H + h) * cols + c0 + lane] += expf((float)Bs[t]) * acc2[j];
        }
        if (has_n && threadIdx.x < n) {
            const int t = threadIdx.x;
            float dot = 0.f;
#pragma unroll 4
            for (int i = 0; i < d; ++i) dot += qs[swz(i, t)] * Ns[i];
            o[((size_t)(tb + t) * H + h) * cols + dv] += expf((float)Bs[t]) * dot;
        }
    }
}

// out[t, h, :] = u / sqrt(mean(u^2) + eps) * w[h * dv + :] * sigmoid(gate[t, h, :]) * out_scale with
// u = o[t, h, :dv] / (max(|o[t, h, dv]|, exp(-m)) + den_eps); a warp per (token, head).
template <typename T>
__global__ void memory_out_kernel(const float* __restrict__ o, const float* __restrict__ gates, const T* proj, int pitch,
                                  int g_off, const float* __restrict__ w, T* __restrict__ out, int out_pitch, int rows,
                                  int H, int dv, float eps, float den_eps, float out_scale) {
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int t = r / H, h = r - t * H;
    const float* op = o + (size_t)r * (dv + 1);
    const float den = 1.f / (fmaxf(fabsf(op[dv]), gates[(size_t)r * 3 + 2]) + den_eps);
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) { const float u = op[i] * den; ss += u * u; }
    const float inv = den / sqrtf(warp_sum(ss) / (float)dv + eps) * out_scale;
    const T* gp = proj + (size_t)t * pitch + g_off + h * dv;
    for (int i = lane; i < dv; i += 32) {
        const float gv = to_float(gp[i]);
        out[(size_t)t * out_pitch + h * dv + i] = from_float<T>(op[i] * inv * w[h * dv + i] / (1.f + expf(-gv)));
    }
}

}  // namespace se

extern "C" int se_memory_max_head_dim() { return se::kMemWarps * 32; }

extern "C" int se_memory_gates(const void* proj, int pitch, int i_off, int f_off, const float* bias, float cap,
                               float* state, long long state_pitch, int m_off, const int* cu_q, const int* seq_rows,
                               float* gates, int entries, int H, int dtype, cudaStream_t stream) {
    if (entries <= 0) return 0;
    if (H <= 0 || H > 65535 || !(cap > 0.f)) return SE_ERR_ARGUMENT;
    SE_DISPATCH_DTYPE(dtype, T,
        se::memory_gates_kernel<T><<<dim3(entries, H), 32, 0, stream>>>((const T*)proj, pitch, i_off, f_off, bias, cap, state,
                                                                        state_pitch, m_off, cu_q, seq_rows, gates, H));
    SE_LAUNCH_CHECK();
}

extern "C" int se_memory_scan(const void* proj, int pitch, int q_off, int k_off, int v_off, const float* gates,
                              float q_scale, float* state, long long state_pitch, const int* cu_q, const int* seq_rows,
                              float* o, int entries, int H, int d, int dv, int dtype, cudaStream_t stream) {
    if (entries <= 0) return 0;
    if (d <= 0 || d > se_memory_max_head_dim() || dv <= 0 || H <= 0 || H > 65535 || (dv + 32) / 32 > 65535)
        return SE_ERR_UNSUPPORTED;
    dim3 grid(entries, H, (dv + 1 + 31) / 32);
    const size_t smem = (size_t)(2 * se::kMemTokens * d + se::kMemTokens * 32 + se::kMemTokens * se::kMemWarps * 32 +
                                 se::kMemTokens) * sizeof(float);
#define SE_MEM_LAUNCH(NPT)                                                                                       \
    se::memory_scan_kernel<T, NPT><<<grid, 32 * se::kMemWarps, smem, stream>>>(                                  \
        (const T*)proj, pitch, q_off, k_off, v_off, gates, q_scale, state, state_pitch, cu_q, seq_rows, o, H, d, dv)
    SE_DISPATCH_DTYPE(dtype, T, {
        if (d <= 8 * se::kMemWarps) SE_MEM_LAUNCH(8);
        else if (d <= 16 * se::kMemWarps) SE_MEM_LAUNCH(16);
        else SE_MEM_LAUNCH(32);
    });
#undef SE_MEM_LAUNCH
    SE_LAUNCH_CHECK();
}

// The same recurrence in chunks of 64 tokens (closed form per chunk): for steps with prompt portions.
extern "C" int se_memory_chunk(const void* proj, int pitch, int q_off, int k_off, int v_off, const float* gates,
                               float q_scale, float* state, long long state_pitch, const int* cu_q, const int* seq_rows,
                               float* o, int entries, int H, int d, int dv, int max_seg, int seg_len, float* seg_state,
                               double* seg_logs, int dtype, cudaStream_t stream) {
    // max_seg > 1: the entries' tokens in segments of seg_len (a multiple of 64) that run side by side, joined by
    // the sums of their log keeps (three launches); seg_state: float [entries, max_seg, H, d, dv + 1], seg_logs:
    // double [entries, max_seg, H].
    if (entries <= 0) return 0;
    if (d <= 0 || d > se_memory_max_head_dim() || dv <= 0 || H <= 0 || H > 65535 || (dv + 32) / 32 > 65535)
        return SE_ERR_UNSUPPORTED;
    if (max_seg < 1 || (max_seg > 1 && (seg_state == nullptr || seg_logs == nullptr || seg_len <= 0 || seg_len % se::kChunk)))
        return SE_ERR_ARGUMENT;
    if ((long long)entries * max_seg > 0x7fffffffLL || entries > 65535) return SE_ERR_UNSUPPORTED;
    const bool segments = max_seg > 1;
    dim3 grid(entries * max_seg, H, (dv + 31) / 32);
    const size_t smem = (size_t)(2 * d * se::kPitch + se::kChunk * 32 + se::kChunk * se::kChunk + d * 32 + 2 * se::kChunk + d) * sizeof(float) +
                        se::kChunk * sizeof(double);
    const size_t fix_smem = (size_t)(d * se::kPitch + d * 32 + d) * sizeof(float) + se::kChunk * sizeof(double);
    SE_DISPATCH_DTYPE(dtype, T, {
        cudaError_t e = cudaFuncSetAttribute(se::memory_chunk_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(se::memory_chunk_kernel<T>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        if (e != cudaSuccess) return (int)e;
        se::memory_chunk_kernel<T><<<grid, se::kChunkThreads, smem, stream>>>(
            (const T*)proj, pitch, q_off, k_off, v_off, gates, q_scale, state, state_pitch, cu_q, seq_rows, o, H, d, dv, max_seg,
            segments ? seg_len : 0, segments ? seg_state : nullptr, segments ? seg_logs : nullptr);
        if (segments) {
            const int per = d * (dv + 1);
            se::memory_seg_join_kernel<<<dim3((per + 255) / 256 < 64 ? (per + 255) / 256 : 64, entries, H), 256, 0, stream>>>(
                seg_state, seg_logs, state, state_pitch, cu_q, seq_rows, H, d, dv + 1, max_seg, seg_len);
            e = cudaFuncSetAttribute(se::memory_seg_fix_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fix_smem);
            if (e != cudaSuccess) return (int)e;
            se::memory_seg_fix_kernel<T><<<grid, se::kChunkThreads, fix_smem, stream>>>(
                (const T*)proj, pitch, q_off, gates, q_scale, seg_state, cu_q, o, H, d, dv, max_seg, seg_len);
        }
    });
    SE_LAUNCH_CHECK();
}

extern "C" int se_memory_out(const float* o, const float* gates, const void* proj, int pitch, int g_off, const float* w,
                             void* out, int out_pitch, int tokens, int H, int dv, float eps, float den_eps,
                             float out_scale, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const int rows = tokens * H;
    SE_DISPATCH_DTYPE(dtype, T,
        se::memory_out_kernel<T><<<(rows + 7) / 8, 256, 0, stream>>>(o, gates, (const T*)proj, pitch, g_off, w, (T*)out,
                                                                      out_pitch, rows, H, dv, eps, den_eps, out_scale));
    SE_LAUNCH_CHECK();
}
