// The gated delta rule with one decay per head, in chunks of 64 tokens (for prompt portions).
//
//     S_t = g_t S_(t-1) + k_t u_t^T,   u_t = beta_t (v_t - (g_t S_(t-1))^T k_t),   o_t = S_t^T q_t
//
// With B_t the sum of log g over a chunk's tokens 0..t and S_0 the state at the chunk's start, the writes u of a
// chunk solve a triangular system, and outputs and the new state follow as three small matrix products:
//
//     (I + A) U = W,   A[t][s] = beta_t exp(B_t - B_s) (k_t . k_s)  (s < t),   W_t = beta_t (v_t - exp(B_t) S_0^T k_t)
//     o_t   = exp(B_t) S_0^T q_t + sum_{s <= t} exp(B_t - B_s) (q_t . k_s) u_s
//     S_new = exp(B_(n-1)) S_0 + sum_s exp(B_(n-1) - B_s) k_s u_s^T
//
// All of it is 32-bit FMA arithmetic (state, decays and everything else that enters the recurrence are 32-bit);
// the sums B are taken in 64-bit so that their differences keep the digits of the single terms.  One block of 256
// threads per (entry, head, 32 value columns): q and k of the chunk lie transposed in shared memory ([dim][token],
// padded rows), the block's slice of the state stays in shared memory over all chunks.  The system is solved by
// forward substitution, one lane per value column with its u in registers (one warp; the rows of A are read as
// broadcasts); the seven other warps wait at the barrier meanwhile.
//
// qkv [tokens, 2 G d + H dv] (32-bit: q and k unit vectors, q scaled), log_dec [tokens, H] (log g), beta [tokens, H];
// the state row of a request starts with [H][dv][d].  Entry s owns the tokens cu_q[s] .. cu_q[s+1]-1 and the state row
// seq_rows[s].
#include "common.cuh"

namespace se {

constexpr int kDcChunk = 64;
constexpr int kDcThreads = 256;
constexpr int kDcPitch = kDcChunk + 4;
__device__ __forceinline__ int dc_at(int i, int t) { return i * kDcPitch + t; }

__global__ void __launch_bounds__(kDcThreads, 2)
delta_chunk_kernel(const float* __restrict__ qkv, const float* __restrict__ log_dec, const float* __restrict__ beta,
                   float* state, long long state_pitch, const int* __restrict__ cu_q, const int* __restrict__ seq_rows,
                   float* __restrict__ o, int H, int G, int d, int dv) {
    extern __shared__ __align__(16) float dc_smem[];
    float* qs = dc_smem;                         // [d][kDcPitch]
    float* ks = qs + d * kDcPitch;               // [d][kDcPitch]
    float* vs = ks + d * kDcPitch;               // [64][32]: v, then W, then U
    float* As = vs + kDcChunk * 32;              // [64][64]: A[t][s] for the solve, then P[s][t] for the outputs
    float* Ss = As + kDcChunk * kDcChunk;        // [d][32]
    float* bs = Ss + d * 32;                     // [64] beta
    float* ws = bs + kDcChunk;                   // [64] exp(B_(n-1) - B_s)
    double* Bs = reinterpret_cast<double*>(ws + kDcChunk);      // [64]
    const int e = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * 32, g = h / (H / G);
    const int lane = threadIdx.x & 31, wg = threadIdx.x >> 5;
    const int t_first = cu_q[e], t_last = cu_q[e + 1];
    if (t_last <= t_first) return;
    const int width = 2 * G * d + H * dv;
    float* S = state + (size_t)seq_rows[e] * state_pitch + (size_t)h * dv * d;
    const bool col_ok = c0 + lane < dv;
    for (int x = threadIdx.x; x < d * 32; x += kDcThreads) {      // Ss[i][c] = S[c0 + c][i]
        const int c = x / d, i = x - c * d;
        Ss[i * 32 + c] = c0 + c < dv ? S[(size_t)(c0 + c) * d + i] : 0.f;
    }
    const bool vec = (d & 3) == 0 && (width & 3) == 0 && ((G * d) & 3) == 0 && aligned8(qkv);

    for (int tb = t_first; tb < t_last; tb += kDcChunk) {
        const int n = min(kDcChunk, t_last - tb);
        __syncthreads();                          // the chunk before is done with its tiles; the state is up to date
        // everything the chunk needs from memory is asked for before any of it is used
        float g_log[2] = {0.f, 0.f}, g_beta[2] = {0.f, 0.f};
        if (wg == 0) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int t = half * 32 + lane;
                if (t < n) {
                    g_log[half] = log_dec[(size_t)(tb + t) * H + h];
                    g_beta[half] = beta[(size_t)(tb + t) * H + h];
                }
            }
        }
        float vv[kDcChunk * 32 / kDcThreads];
#pragma unroll
        for (int r = 0; r < kDcChunk * 32 / kDcThreads; ++r) {
            const int x = threadIdx.x + r * kDcThreads, t = x >> 5, c = c0 + (x & 31);
            vv[r] = (t < n && c < dv) ? qkv[(size_t)(tb + t) * width + 2 * G * d + h * dv + c] : 0.f;
        }
        if (vec) {
            // four elements a load; a warp's lanes take the same four dims of 32 tokens in a row, so that the
            // transposing stores fall into 32 banks
            const int pieces = kDcChunk * (d >> 2);
            for (int base = threadIdx.x; base < pieces; base += 4 * kDcThreads) {
                float4 qv[4], kv[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int x = base + r * kDcThreads, t = x & (kDcChunk - 1), i = (x >> 6) * 4;
                    qv[r] = kv[r] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (x < pieces && t < n) {
                        const float* row = qkv + (size_t)(tb + t) * width + g * d + i;
                        qv[r] = *reinterpret_cast<const float4*>(row);
                        kv[r] = *reinterpret_cast<const float4*>(row + G * d);
                    }
                }
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int x = base + r * kDcThreads, t = x & (kDcChunk - 1), i = (x >> 6) * 4;
                    if (x < pieces) {
                        qs[dc_at(i, t)] = qv[r].x; qs[dc_at(i + 1, t)] = qv[r].y; qs[dc_at(i + 2, t)] = qv[r].z; qs[dc_at(i + 3, t)] = qv[r].w;
                        ks[dc_at(i, t)] = kv[r].x; ks[dc_at(i + 1, t)] = kv[r].y; ks[dc_at(i + 2, t)] = kv[r].z; ks[dc_at(i + 3, t)] = kv[r].w;
                    }
                }
            }
        } else {
            for (int x = threadIdx.x; x < kDcChunk * d; x += kDcThreads) {
                const int t = x / d, i = x - t * d;
                const float* row = qkv + (size_t)(tb + t) * width + g * d + i;
                qs[dc_at(i, t)] = t < n ? row[0] : 0.f;
                ks[dc_at(i, t)] = t < n ? row[G * d] : 0.f;
            }
        }
#pragma unroll
        for (int r = 0; r < kDcChunk * 32 / kDcThreads; ++r) vs[threadIdx.x + r * kDcThreads] = vv[r];
        if (wg == 0) {                            // the sums of the log decays, 64-bit, by one warp
            double carry = 0.0;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int t = half * 32 + lane;
                double b = (double)g_log[half];
                bs[t] = g_beta[half];
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
        // A 4 x 4 tile (tokens tt.., keys ss..) per thread of q . k (kept in registers for later) and of k . k (the
        // system's matrix, to shared memory); tiles above the diagonal are zero.
        const int tt = (threadIdx.x >> 4) * 4, ss = (threadIdx.x & 15) * 4;
        float pq[4][4] = {};
        {
            float pk[4][4] = {};
            if (ss <= tt + 3) {
#pragma unroll 4
                for (int i = 0; i < d; ++i) {
                    const float4 qv = *reinterpret_cast<const float4*>(qs + dc_at(i, tt));
                    const float4 kt = *reinterpret_cast<const float4*>(ks + dc_at(i, tt));
                    const float4 kv = *reinterpret_cast<const float4*>(ks + dc_at(i, ss));
                    const float qa[4] = {qv.x, qv.y, qv.z, qv.w}, ta[4] = {kt.x, kt.y, kt.z, kt.w}, ka[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
                    for (int a = 0; a < 4; ++a)
#pragma unroll
                        for (int b = 0; b < 4; ++b) {
                            pq[a][b] += qa[a] * ka[b];
                            pk[a][b] += ta[a] * ka[b];
                        }
                }
            }
#pragma unroll
            for (int a = 0; a < 4; ++a) {         // A[t][s], row t contiguous over s
                float4 row;
                float* r = &row.x;
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const bool in = ss + b < tt + a && tt + a < n;
                    const float wgt = in ? expf((float)(Bs[tt + a] - Bs[ss + b])) : 0.f;
                    r[b] = in ? bs[tt + a] * wgt * pk[a][b] : 0.f;
                    pq[a][b] = (ss + b <= tt + a && tt + a < n) ? pq[a][b] * (ss + b == tt + a ? 1.f : wgt) : 0.f;
                }
                *reinterpret_cast<float4*>(As + (tt + a) * kDcChunk + ss) = row;
            }
        }
        // W_t = beta_t (v_t - exp(B_t) S_0^T k_t): warp wg takes tokens 8 wg .. 8 wg + 7, lane c the column
        float sq[8] = {};                         // S_0^T q_t, kept for the outputs
        {
            const int tg = wg * 8;
            float sk[8] = {};
#pragma unroll 4
            for (int i = 0; i < d; ++i) {
                const float4 k0 = *reinterpret_cast<const float4*>(ks + dc_at(i, tg));
                const float4 k1 = *reinterpret_cast<const float4*>(ks + dc_at(i, tg + 4));
                const float4 q0 = *reinterpret_cast<const float4*>(qs + dc_at(i, tg));
                const float4 q1 = *reinterpret_cast<const float4*>(qs + dc_at(i, tg + 4));
                const float sv = Ss[i * 32 + lane];
                sk[0] += k0.x * sv; sk[1] += k0.y * sv; sk[2] += k0.z * sv; sk[3] += k0.w * sv;
                sk[4] += k1.x * sv; sk[5] += k1.y * sv; sk[6] += k1.z * sv; sk[7] += k1.w * sv;
                sq[0] += q0.x * sv; sq[1] += q0.y * sv; sq[2] += q0.z * sv; sq[3] += q0.w * sv;
                sq[4] += q1.x * sv; sq[5] += q1.y * sv; sq[6] += q1.z * sv; sq[7] += q1.w * sv;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int t = tg + j;
                const float decay = expf((float)Bs[t]);
                vs[t * 32 + lane] = t < n ? bs[t] * (vs[t * 32 + lane] - decay * sk[j]) : 0.f;
                sq[j] *= decay;
            }
        }
        __syncthreads();
        // forward substitution: u_t = W_t - sum_{s < t} A[t][s] u_s, a lane per column
        if (wg == 0) {
            float u[kDcChunk];
#pragma unroll
            for (int t = 0; t < kDcChunk; ++t) {
                float acc = vs[t * 32 + lane];
#pragma unroll
                for (int s4 = 0; s4 + 4 <= t; s4 += 4) {
                    const float4 a = *reinterpret_cast<const float4*>(As + t * kDcChunk + s4);
                    acc -= a.x * u[s4] + a.y * u[s4 + 1] + a.z * u[s4 + 2] + a.w * u[s4 + 3];
                }
#pragma unroll
                for (int s_ = t & ~3; s_ < t; ++s_) acc -= As[t * kDcChunk + s_] * u[s_];
                u[t] = acc;
                vs[t * 32 + lane] = acc;
            }
        }
        __syncthreads();
        // the weighted q . k tiles go where A was: P[s][t], row s contiguous over t
#pragma unroll
        for (int b = 0; b < 4; ++b)
            *reinterpret_cast<float4*>(As + (ss + b) * kDcChunk + tt) = make_float4(pq[0][b], pq[1][b], pq[2][b], pq[3][b]);
        float vreg[kDcChunk];                      // this lane's column of U
#pragma unroll
        for (int s_ = 0; s_ < kDcChunk; ++s_) vreg[s_] = vs[s_ * 32 + lane];
        const double b_end = Bs[n - 1];
        if (threadIdx.x < kDcChunk) ws[threadIdx.x] = (int)threadIdx.x < n ? expf((float)(b_end - Bs[threadIdx.x])) : 0.f;
        __syncthreads();
        // outputs: warp wg takes tokens 8 wg .. 8 wg + 7, lane c the column
        {
            const int tg = wg * 8;
            float acc[8] = {};
#pragma unroll
            for (int s_ = 0; s_ < kDcChunk; ++s_) {
                const float4 a0 = *reinterpret_cast<const float4*>(As + s_ * kDcChunk + tg);
                const float4 a1 = *reinterpret_cast<const float4*>(As + s_ * kDcChunk + tg + 4);
                const float v = vreg[s_];
                acc[0] += a0.x * v; acc[1] += a0.y * v; acc[2] += a0.z * v; acc[3] += a0.w * v;
                acc[4] += a1.x * v; acc[5] += a1.y * v; acc[6] += a1.z * v; acc[7] += a1.w * v;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int t = tg + j;
                if (t < n && col_ok) o[((size_t)(tb + t) * H + h) * dv + c0 + lane] = acc[j] + sq[j];
            }
        }
        __syncthreads();                          // every read of the old state is done
        // the state after the chunk: warp wg takes rows wg, wg + 8, ...
#pragma unroll
        for (int s_ = 0; s_ < kDcChunk; ++s_) vreg[s_] *= ws[s_];
        const float gn = expf((float)b_end);
        for (int i = wg; i < d; i += kDcThreads / 32) {
            float a = 0.f;
#pragma unroll
            for (int s4 = 0; s4 < kDcChunk; s4 += 4) {
                const float4 kv = *reinterpret_cast<const float4*>(ks + dc_at(i, s4));
                a += kv.x * vreg[s4] + kv.y * vreg[s4 + 1] + kv.z * vreg[s4 + 2] + kv.w * vreg[s4 + 3];
            }
            Ss[i * 32 + lane] = gn * Ss[i * 32 + lane] + a;
        }
    }
    __syncthreads();
    for (int x = threadIdx.x; x < d * 32; x += kDcThreads) {
        const int c = x / d, i = x - c * d;
        if (c0 + c < dv) S[(size_t)(c0 + c) * d + i] = Ss[i * 32 + c];
    }
}

}  // namespace se

extern "C" int se_delta_chunk_max_head_dim() { return 256; }

extern "C" int se_delta_chunk(const float* qkv, const float* log_dec, const float* beta, float* state, long long state_pitch,
                              const int* cu_q, const int* seq_rows, float* o, int entries, int H, int G, int d, int dv,
                              cudaStream_t stream) {
    if (entries <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || d <= 0 || dv <= 0) return SE_ERR_ARGUMENT;
    if (d > se_delta_chunk_max_head_dim() || H > 65535 || entries > 65535 || (dv + 31) / 32 > 65535) return SE_ERR_UNSUPPORTED;
    const dim3 grid(entries, H, (dv + 31) / 32);
    const size_t smem = (size_t)(2 * d * se::kDcPitch + se::kDcChunk * 32 + se::kDcChunk * se::kDcChunk + d * 32 + 2 * se::kDcChunk) * sizeof(float) +
                        se::kDcChunk * sizeof(double);
    cudaError_t e = cudaFuncSetAttribute(se::delta_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(se::delta_chunk_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (e != cudaSuccess) return (int)e;
    se::delta_chunk_kernel<<<grid, se::kDcThreads, smem, stream>>>(qkv, log_dec, beta, state, state_pitch, cu_q, seq_rows, o, H, G, d, dv);
    SE_LAUNCH_CHECK();
}
