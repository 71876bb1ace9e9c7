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
// per request and head, 32 tokens at a time by prefix sum and prefix maximum), the matrix recurrence,
// and the epilogue (denominator, each head's root mean square, weight, sigmoid gate).  q, k, v and the
// gate come from the projection in the activation type; everything else is 32-bit.
//
// A step brings any mix of prompt portions and single tokens: entry s owns the tokens
// cu_q[s] .. cu_q[s+1]-1 and the state row seq_rows[s].
#include "common.cuh"

namespace se {

__device__ __forceinline__ float log_sigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// gates[t][h] = (keep, take, exp(-m_t)); the request's m is brought up to date.  One warp per (entry, head).
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
    for (int base = t0; base < t1; base += 32) {
        const int t = base + lane;
        const bool valid = t < t1;
        float gi = -INFINITY, gf = 0.f;
        if (valid) {
            const T* row = proj + (size_t)t * pitch;
            gi = cap * tanhf((to_float(row[i_off + h]) + bi) / cap);
            gf = log_sigmoid_f(cap * tanhf((to_float(row[f_off + h]) + bf) / cap));
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
            g[0] = expf(gf + m_prev - m);
            g[1] = expf(gi - m);
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
            ks[x] = to_float(row[k_off + h * d + i]) * gates[((size_t)(tb + tt) * H + h) * 3 + 1];
        }
        for (int x = threadIdx.x; x < nt * 32; x += blockDim.x) {
            const int tt = x >> 5, c = c0 + (x & 31);
            vs[x] = c < dv ? to_float(proj[(size_t)(tb + tt) * pitch + v_off + h * dv + c]) : (c == dv ? 1.f : 0.f);
        }
        if ((int)threadIdx.x < nt) keep[threadIdx.x] = gates[((size_t)(tb + threadIdx.x) * H + h) * 3];
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
