// Mixers with a recurrent state of fixed size per request: a short causal convolution over
// time with carried inputs, the selective state-space recurrence (scalar decay per head, state
// N x P) and the gated delta rule (one decay per head and key channel, state d x dv), with
// their prologues and epilogues.  Everything that enters a recurrence is 32-bit.
//
// A step's batch is ragged: entry e owns tokens cu_q[e] .. cu_q[e+1]-1 (consecutive positions of
// one request) and state row seq_rows[e]; token t belongs to entry token_seq[t].  Everything
// that changes from step to step is read from these device arrays, so the launches can be
// replayed from a CUDA graph.  A request's state row starts as zeros.
//
// State row of a mixer (32-bit floats): the recurrence's matrix per head, stored [head][column
// of the value side][row of the key/state side], followed by the convolution's last taps-1
// inputs [taps-1][channel].
#include "common.cuh"

namespace se {

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }
__device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); }
__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }
// silu of a value that is rounded to bfloat16 inputs' precision anyway: the fast exponential and
// division (a few units in the last place of 32-bit) where the activation type is bfloat16
template <typename T> __device__ __forceinline__ float silu_act(float v) { return silu_f(v); }
template <> __device__ __forceinline__ float silu_act<__nv_bfloat16>(float v) { return __fdividef(v, 1.f + __expf(-v)); }

// ---- causal convolution, silu ----------------------------------------------------------------
// out[t, c] = silu(bias[c] + sum_j w[c, j] * in[t - (taps-1-j), c]); inputs before the entry's first
// token of this step come from the carried inputs, which are zeros before the request's start.
// grid (ceil(tokens / tile), ceil(C / 128)).
// A block takes `tile` consecutive tokens of 128 channels (up to kConvTokens: the step's mean number of
// tokens per request, so that a step of single tokens spreads over many blocks): their inputs (and
// the taps-1 before them) go to shared memory once, so every input is read from memory once.
constexpr int kConvTokens = 16;
template <typename T>
__global__ void __launch_bounds__(128)
causal_conv_kernel(const T* x, int pitch, int c0, const float* __restrict__ w, const float* __restrict__ bias,
                   const float* state, long long state_pitch, int conv_off, const int* __restrict__ token_seq,
                   const int* __restrict__ cu_q, const int* __restrict__ seq_rows, float* __restrict__ out, int tokens,
                   int C, int taps, int tile_tokens) {
    extern __shared__ float tile[];           // [tile_tokens + taps - 1][128]
    const int t0 = blockIdx.x * tile_tokens, c = blockIdx.y * 128 + threadIdx.x;
    if (c >= C) return;                       // no barrier below: a thread only reads what it wrote itself
    const int nt = min(tile_tokens, tokens - t0);
    for (int k = 0; k < nt + taps - 1; ++k) {
        const int tt = t0 - (taps - 1) + k;
        tile[k * 128 + threadIdx.x] = tt >= 0 ? to_float(x[(size_t)tt * pitch + c0 + c]) : 0.f;
    }
    const float b = bias != nullptr ? bias[c] : 0.f;
    // Most tiles lie inside one request's tokens: its first token is then looked up once, not per token.
    const int e_first = token_seq[t0], e_last = token_seq[t0 + nt - 1];
    const bool one_entry = e_first == e_last;
    const int start_first = cu_q[e_first];
    constexpr int kRegTaps = 8;               // up to this many taps the weights stay in registers
    float wr[kRegTaps];
#pragma unroll
    for (int j = 0; j < kRegTaps; ++j) wr[j] = j < taps ? w[(size_t)c * taps + j] : 0.f;
    for (int i = 0; i < nt; ++i) {
        const int t = t0 + i;
        const int e = one_entry ? e_first : token_seq[t];
        const int start = one_entry ? start_first : cu_q[e];
        float acc = b;
        if (t - (taps - 1) >= start) {        // the whole window lies in this step's tokens
            if (taps <= kRegTaps) {
#pragma unroll
                for (int j = 0; j < kRegTaps; ++j)
                    if (j < taps) acc += wr[j] * tile[(i + j) * 128 + threadIdx.x];
            } else {
                for (int j = 0; j < taps; ++j) acc += w[(size_t)c * taps + j] * tile[(i + j) * 128 + threadIdx.x];
            }
        } else {
            const float* carried = state + (size_t)seq_rows[e] * state_pitch + conv_off;
            for (int j = 0; j < taps; ++j) {
                const int tt = t - (taps - 1 - j);
                const float v = tt >= start ? tile[(i + j) * 128 + threadIdx.x]
                                            : carried[(size_t)(taps - 1 - (start - tt)) * C + c];
                acc += w[(size_t)c * taps + j] * v;
            }
        }
        out[(size_t)t * C + c] = silu_act<T>(acc);
    }
}

// The carried inputs after the step: the last taps-1 inputs of each entry (older ones move up
// when the entry brought fewer tokens).  grid (entries, ceil(C / blockDim)); runs after the
// convolution has read the old ones.
template <typename T>
__global__ void conv_carry_kernel(const T* x, int pitch, int c0, float* state, long long state_pitch, int conv_off,
                                  const int* __restrict__ cu_q, const int* __restrict__ seq_rows, int C, int taps) {
    const int e = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int start = cu_q[e], end = cu_q[e + 1], n = end - start;
    float* carried = state + (size_t)seq_rows[e] * state_pitch + conv_off;
    for (int i = 0; i < taps - 1; ++i) {          // ascending: slot i + n is read before it is written
        const int tt = end - (taps - 1) + i;
        carried[(size_t)i * C + c] = tt >= start ? to_float(x[(size_t)tt * pitch + c0 + c]) : carried[(size_t)(i + n) * C + c];
    }
}

// ---- the two recurrences ---------------------------------------------------------------------
// A block owns (entry, head, tile of value columns).  Thread (column, s) keeps rows s, s + nsplit,
// ... (REGS of them) of its column in registers; the nsplit threads of a column (a power of two
// <= 32) are neighbouring lanes of one warp, so the state moves in coalesced accesses and the
// sums over rows end in shuffles.  In shared memory a token's row values are regrouped per
// thread: row n sits at (n % nsplit) * (REGS + 4) + n / nsplit, so a thread reads its values with
// 16-byte loads and the pad of 4 keeps the threads of a column on different banks.  Rows beyond
// the state's own are zeros in shared memory and stay zero in the registers, so the inner loops
// have no bounds.  The inputs of kChunk tokens at a time are staged in shared memory, in two
// buffers: the copies of the next chunk (cp.async) run while this one is computed.
//
// What bounds them is the 32-bit multiply-add rate: two (state space) or four (delta rule)
// operations per state element and token, in a chain along the tokens of a request.
constexpr int kChunk = 8;

__device__ __forceinline__ float split_sum(float v, int nsplit) {
    for (int o = nsplit >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ void copy_async4(float* dst_shared, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst_shared);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void copies_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Selective state space: S <- exp(-exp(A_log) dt) S + dt B x^T;  y = S^T C + D x.
// xbc [T, H*P + 2*G*N] holds x | B | C (after convolution and silu); dt_raw is column dt_off + h of
// the input projection.  y [T, H*P].
template <typename T, int REGS>
__global__ void __launch_bounds__(256)
ssm_scan_kernel(const float* __restrict__ xbc, const T* proj, int pitch, int dt_off, const float* __restrict__ dt_bias,
                const float* __restrict__ a_log, const float* __restrict__ d_skip, float* state, long long state_pitch,
                const int* __restrict__ cu_q, const int* __restrict__ seq_rows, float* __restrict__ y, int H, int P,
                int N, int G, int nsplit, int cols) {
    extern __shared__ __align__(16) float sm[];
    const int np = nsplit * (REGS + 4);
    const int buf = kChunk * (2 * np + cols + 2);     // per buffer: B [kChunk][np], C [kChunk][np], x [kChunk][cols], dt, decay
    const int e = blockIdx.x, h = blockIdx.y, g = h / (H / G);
    const int s = threadIdx.x % nsplit, pl = threadIdx.x / nsplit, p = blockIdx.z * cols + pl;
    const bool live = p < P;
    const int start = cu_q[e], end = cu_q[e + 1];
    const int width = H * P + 2 * G * N;
    float* Sp = state + (size_t)seq_rows[e] * state_pitch + ((size_t)h * P + (live ? p : 0)) * N;
    float S[REGS];
#pragma unroll
    for (int i = 0; i < REGS; ++i) {
        const int n = s + nsplit * i;
        S[i] = live && n < N ? Sp[n] : 0.f;
    }
    for (int i = threadIdx.x; i < 2 * buf; i += blockDim.x) sm[i] = 0.f;      // the rows beyond N stay zero
    __syncthreads();
    const float rate = expf(a_log[h]), skip = d_skip[h], bias = dt_bias[h];

    auto issue = [&](int t0, int nt, float* dst) {       // asynchronous copies of a chunk's B, C and x
        for (int i = threadIdx.x; i < nt * N; i += blockDim.x) {
            const int c = i / N, n = i - c * N;
            const float* r = xbc + (size_t)(t0 + c) * width + H * P + g * N + n;
            const int at = c * np + (n % nsplit) * (REGS + 4) + n / nsplit;
            copy_async4(dst + at, r);
            copy_async4(dst + kChunk * np + at, r + G * N);
        }
        for (int i = threadIdx.x; i < nt * cols; i += blockDim.x) {
            const int c = i / cols, j = i - c * cols, pp = blockIdx.z * cols + j;
            if (pp < P) copy_async4(dst + 2 * kChunk * np + c * cols + j, xbc + (size_t)(t0 + c) * width + h * P + pp);
        }
    };
    auto raw_dt = [&](int t0, int nt) {
        return (int)threadIdx.x < nt ? to_float(proj[(size_t)(t0 + threadIdx.x) * pitch + dt_off + h]) : 0.f;
    };
    auto put_dt = [&](float raw, int nt, float* dst) {
        if ((int)threadIdx.x < nt) {
            const float dt = softplus_f(raw + bias);
            dst[2 * kChunk * np + kChunk * cols + threadIdx.x] = dt;
            dst[2 * kChunk * np + kChunk * cols + kChunk + threadIdx.x] = expf(-rate * dt);
        }
    };

    if (start < end) {
        const int nt = min(kChunk, end - start);
        issue(start, nt, sm);
        put_dt(raw_dt(start, nt), nt, sm);
        copies_wait();
    }
    __syncthreads();
    int cur = 0;
    for (int t0 = start; t0 < end; t0 += kChunk, cur ^= 1) {
        const int nt = min(kChunk, end - t0);
        const int next_nt = min(kChunk, end - (t0 + kChunk));      // <= 0: this is the last chunk
        float* here = sm + cur * buf;
        float* there = sm + (cur ^ 1) * buf;
        float raw = 0.f;
        if (next_nt > 0) {
            issue(t0 + kChunk, next_nt, there);
            raw = raw_dt(t0 + kChunk, next_nt);
        }
        const float* sx = here + 2 * kChunk * np;
        const float* sdt = sx + kChunk * cols;
        for (int c = 0; c < nt; ++c) {
            const float a = sdt[kChunk + c], xv = sx[c * cols + pl];
            const float bx = sdt[c] * xv;
            const float4* B4 = reinterpret_cast<const float4*>(here + c * np + s * (REGS + 4));
            const float4* C4 = reinterpret_cast<const float4*>(here + kChunk * np + c * np + s * (REGS + 4));
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < REGS; i += 4) {
                const float4 bv = B4[i >> 2], cv = C4[i >> 2];
                S[i] = a * S[i] + bv.x * bx;         acc[0] += S[i] * cv.x;
                S[i + 1] = a * S[i + 1] + bv.y * bx; acc[1] += S[i + 1] * cv.y;
                S[i + 2] = a * S[i + 2] + bv.z * bx; acc[2] += S[i + 2] * cv.z;
                S[i + 3] = a * S[i + 3] + bv.w * bx; acc[3] += S[i + 3] * cv.w;
            }
            const float sum = split_sum((acc[0] + acc[1]) + (acc[2] + acc[3]), nsplit);
            if (s == 0 && live) y[(size_t)(t0 + c) * H * P + h * P + p] = sum + skip * xv;
        }
        if (next_nt > 0) {
            put_dt(raw, next_nt, there);
            copies_wait();
        }
        __syncthreads();
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < REGS; ++i) {
            const int n = s + nsplit * i;
            if (n < N) Sp[n] = S[i];
        }
    }
}

// Gated delta rule, per head: S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.
// qkv [T, 2*G*d + H*dv] holds q | k | v (q and k already unit vectors, q scaled); dec [T, H*d] the
// decays g; beta [T, H].  o [T, H*dv].
template <int REGS>
__global__ void __launch_bounds__(256)
delta_scan_kernel(const float* __restrict__ qkv, const float* __restrict__ dec, const float* __restrict__ beta,
                  float* state, long long state_pitch, const int* __restrict__ cu_q, const int* __restrict__ seq_rows,
                  float* __restrict__ o, int H, int G, int d, int dv, int nsplit, int cols) {
    extern __shared__ __align__(16) float sm[];
    const int np = nsplit * (REGS + 4);
    const int buf = kChunk * (3 * np + cols + 1);     // per buffer: q, k, g [kChunk][np] each, v [kChunk][cols], beta
    const int e = blockIdx.x, h = blockIdx.y, g = h / (H / G);
    const int s = threadIdx.x % nsplit, jl = threadIdx.x / nsplit, j = blockIdx.z * cols + jl;
    const bool live = j < dv;
    const int start = cu_q[e], end = cu_q[e + 1];
    const int width = 2 * G * d + H * dv;
    float* Sp = state + (size_t)seq_rows[e] * state_pitch + ((size_t)h * dv + (live ? j : 0)) * d;
    float S[REGS];
#pragma unroll
    for (int i = 0; i < REGS; ++i) {
        const int n = s + nsplit * i;
        S[i] = live && n < d ? Sp[n] : 0.f;
    }
    for (int i = threadIdx.x; i < 2 * buf; i += blockDim.x) sm[i] = 0.f;
    __syncthreads();

    auto issue = [&](int t0, int nt, float* dst) {
        for (int i = threadIdx.x; i < nt * d; i += blockDim.x) {
            const int c = i / d, n = i - c * d;
            const float* r = qkv + (size_t)(t0 + c) * width + g * d + n;
            const int at = c * np + (n % nsplit) * (REGS + 4) + n / nsplit;
            copy_async4(dst + at, r);
            copy_async4(dst + kChunk * np + at, r + G * d);
            copy_async4(dst + 2 * kChunk * np + at, dec + (size_t)(t0 + c) * H * d + h * d + n);
        }
        for (int i = threadIdx.x; i < nt * cols; i += blockDim.x) {
            const int c = i / cols, jj = i - c * cols, col = blockIdx.z * cols + jj;
            if (col < dv) copy_async4(dst + 3 * kChunk * np + c * cols + jj, qkv + (size_t)(t0 + c) * width + 2 * G * d + h * dv + col);
        }
        if ((int)threadIdx.x < nt) copy_async4(dst + 3 * kChunk * np + kChunk * cols + threadIdx.x, beta + (size_t)(t0 + threadIdx.x) * H + h);
    };

    if (start < end) {
        issue(start, min(kChunk, end - start), sm);
        copies_wait();
    }
    __syncthreads();
    int cur = 0;
    for (int t0 = start; t0 < end; t0 += kChunk, cur ^= 1) {
        const int nt = min(kChunk, end - t0);
        const int next_nt = min(kChunk, end - (t0 + kChunk));
        float* here = sm + cur * buf;
        if (next_nt > 0) issue(t0 + kChunk, next_nt, sm + (cur ^ 1) * buf);
        const float* sv = here + 3 * kChunk * np;
        const float* sb = sv + kChunk * cols;
        for (int c = 0; c < nt; ++c) {
            const float4* Q4 = reinterpret_cast<const float4*>(here + c * np + s * (REGS + 4));
            const float4* K4 = reinterpret_cast<const float4*>(here + kChunk * np + c * np + s * (REGS + 4));
            const float4* G4 = reinterpret_cast<const float4*>(here + 2 * kChunk * np + c * np + s * (REGS + 4));
            float r[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < REGS; i += 4) {
                const float4 gv = G4[i >> 2], kv = K4[i >> 2];
                S[i] *= gv.x;     r[0] += S[i] * kv.x;
                S[i + 1] *= gv.y; r[1] += S[i + 1] * kv.y;
                S[i + 2] *= gv.z; r[2] += S[i + 2] * kv.z;
                S[i + 3] *= gv.w; r[3] += S[i + 3] * kv.w;
            }
            const float rs = split_sum((r[0] + r[1]) + (r[2] + r[3]), nsplit);
            const float u = sb[c] * (sv[c * cols + jl] - rs);
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < REGS; i += 4) {
                const float4 kv = K4[i >> 2], qv = Q4[i >> 2];
                S[i] += kv.x * u;     acc[0] += S[i] * qv.x;
                S[i + 1] += kv.y * u; acc[1] += S[i + 1] * qv.y;
                S[i + 2] += kv.z * u; acc[2] += S[i + 2] * qv.z;
                S[i + 3] += kv.w * u; acc[3] += S[i + 3] * qv.w;
            }
            const float sum = split_sum((acc[0] + acc[1]) + (acc[2] + acc[3]), nsplit);
            if (s == 0 && live) o[(size_t)(t0 + c) * H * dv + h * dv + j] = sum;
        }
        if (next_nt > 0) copies_wait();
        __syncthreads();
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < REGS; ++i) {
            const int n = s + nsplit * i;
            if (n < d) Sp[n] = S[i];
        }
    }
}

// ---- the recurrences with a register tile of 8 rows x 4 columns per thread ----------------------
// One column per thread reads every row value from shared memory once per multiply-add pair, and
// the shared-memory pipe then sets the pace.  Here a thread keeps 8 rows (s, s + nsplit, ...) of 4
// neighbouring columns: a row value read once serves 4 columns.  The 4 sums a thread holds are
// reduced over the nsplit lanes crosswise (lanes trade the halves they do not keep: 2 + 1 shuffles
// leave one column's sum per lane, then one shuffle per further doubling), not one by one.
constexpr int kTileRows = 8, kTileCols = 4, kTilePad = kTileRows + 4;
#define SE_TILE_THREADS 128      // most threads of a block of the tiled kernels (their launch bound)

// acc[4] per lane -> the sum over the nsplit lanes of column (2 * (s & 1) + ((s >> 1) & 1)), in every lane;
// nsplit >= 4
__device__ __forceinline__ float cross_sum4(const float* acc, int s, int nsplit) {
    const bool b0 = s & 1, b1 = s & 2;
    float k0 = b0 ? acc[2] : acc[0], k1 = b0 ? acc[3] : acc[1];
    k0 += __shfl_xor_sync(0xffffffffu, b0 ? acc[0] : acc[2], 1);
    k1 += __shfl_xor_sync(0xffffffffu, b0 ? acc[1] : acc[3], 1);
    float kp = b1 ? k1 : k0;
    kp += __shfl_xor_sync(0xffffffffu, b1 ? k0 : k1, 2);
    for (int o = 4; o < nsplit; o <<= 1) kp += __shfl_xor_sync(0xffffffffu, kp, o);
    return kp;
}

// Step sizes and decays of the state-space recurrence, [T, H, 2] = (softplus(raw + bias),
// exp(-exp(A_log) * that)): taken out of the recurrence, where one warp computed them while the
// others waited.
template <typename T>
__global__ void ssm_steps_kernel(const T* proj, int pitch, int dt_off, const float* __restrict__ dt_bias,
                                 const float* __restrict__ a_log, float* __restrict__ steps, int tokens, int H) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= tokens * H) return;
    const int t = i / H, h = i - t * H;
    const float dt = softplus_f(to_float(proj[(size_t)t * pitch + dt_off + h]) + dt_bias[h]);
    steps[2 * (size_t)i] = dt;
    steps[2 * (size_t)i + 1] = expf(-expf(a_log[h]) * dt);
}

template <typename T>
__global__ void __launch_bounds__(SE_TILE_THREADS)
ssm_scan_tile_kernel(const float* __restrict__ xbc, const float* __restrict__ steps, const float* __restrict__ d_skip,
                     float* state, long long state_pitch, const int* __restrict__ cu_q, const int* __restrict__ seq_rows,
                     float* __restrict__ y, int H, int P, int N, int G, int nsplit, int cols) {
    constexpr int RN = kTileRows, RC = kTileCols;
    extern __shared__ __align__(16) float sm[];
    const int np = nsplit * kTilePad;
    const int buf = kChunk * (2 * np + cols + 2);     // per buffer: B, C [kChunk][np], x [kChunk][cols], (step, decay) [kChunk][2]
    const int e = blockIdx.x, h = blockIdx.y, g = h / (H / G);
    const int s = threadIdx.x % nsplit, cg = threadIdx.x / nsplit, p0 = blockIdx.z * cols + cg * RC;
    const int start = cu_q[e], end = cu_q[e + 1];
    const int width = H * P + 2 * G * N;
    float* Sp = state + (size_t)seq_rows[e] * state_pitch + (size_t)h * P * N;
    float S[RN][RC];
#pragma unroll
    for (int i = 0; i < RN; ++i)
#pragma unroll
        for (int c = 0; c < RC; ++c) {
            const int n = s + nsplit * i;
            S[i][c] = (p0 + c < P && n < N) ? Sp[(size_t)(p0 + c) * N + n] : 0.f;
        }
    if (N != nsplit * RN || blockIdx.z * cols + cols > P) {      // rows beyond N and columns beyond P read as zeros
        for (int i = threadIdx.x; i < 2 * buf; i += blockDim.x) sm[i] = 0.f;
        __syncthreads();
    }
    const float skip = d_skip[h];
    const int split_log2 = 31 - __clz(nsplit);

    auto issue = [&](int t0, int nt, float* dst) {
        // no division in here: nsplit is a power of two, and the loops run over rows, then tokens
        const float* r0 = xbc + (size_t)t0 * width + H * P + g * N;
        for (int n = threadIdx.x; n < N; n += blockDim.x) {
            const int at = (n & (nsplit - 1)) * kTilePad + (n >> split_log2);
            for (int c = 0; c < nt; ++c) {
                copy_async4(dst + c * np + at, r0 + (size_t)c * width + n);
                copy_async4(dst + kChunk * np + c * np + at, r0 + (size_t)c * width + G * N + n);
            }
        }
        const float* x0 = xbc + (size_t)t0 * width + h * P + blockIdx.z * cols;
        for (int j = threadIdx.x; j < cols; j += blockDim.x) {
            if (blockIdx.z * cols + j < P)
                for (int c = 0; c < nt; ++c) copy_async4(dst + 2 * kChunk * np + c * cols + j, x0 + (size_t)c * width + j);
        }
        if ((int)threadIdx.x < 2 * nt)
            copy_async4(dst + 2 * kChunk * np + kChunk * cols + threadIdx.x,
                        steps + 2 * ((size_t)(t0 + (threadIdx.x >> 1)) * H + h) + (threadIdx.x & 1));
    };
    if (start < end) {
        issue(start, min(kChunk, end - start), sm);
        copies_wait();
    }
    __syncthreads();
    const int col = 2 * (s & 1) + ((s >> 1) & 1);      // the column whose sum the crosswise reduction leaves in this lane
    int cur = 0;
    for (int t0 = start; t0 < end; t0 += kChunk, cur ^= 1) {
        const int nt = min(kChunk, end - t0);
        const int next_nt = min(kChunk, end - (t0 + kChunk));
        const float* here = sm + cur * buf;
        if (next_nt > 0) issue(t0 + kChunk, next_nt, sm + (cur ^ 1) * buf);
        const float* sx = here + 2 * kChunk * np;
        const float* sdt = sx + kChunk * cols;         // (step, decay) per token
        // One token: its inputs from shared memory, the state update, the four column sums.
        auto advance = [&](int c, float* sums) {
            const float a = sdt[2 * c + 1], dt = sdt[2 * c];
            const float4 xv = *reinterpret_cast<const float4*>(sx + c * cols + cg * RC);
            const float bx[RC] = {dt * xv.x, dt * xv.y, dt * xv.z, dt * xv.w};
            const float4* B4 = reinterpret_cast<const float4*>(here + c * np + s * kTilePad);
            const float4* C4 = reinterpret_cast<const float4*>(here + kChunk * np + c * np + s * kTilePad);
            const float4 b0 = B4[0], b1 = B4[1], c0 = C4[0], c1 = C4[1];
            const float Bv[RN] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
            const float Cv[RN] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
            for (int k = 0; k < RC; ++k) sums[k] = 0.f;
#pragma unroll
            for (int i = 0; i < RN; ++i)
#pragma unroll
                for (int k = 0; k < RC; ++k) {
                    S[i][k] = a * S[i][k] + Bv[i] * bx[k];
                    sums[k] += S[i][k] * Cv[i];
                }
        };
        auto finish = [&](int c, const float* sums) {       // the sums over the lanes, and the output
            float* yr = y + (size_t)(t0 + c) * H * P + h * P;
            if (nsplit >= 4) {
                const float total = cross_sum4(sums, s, nsplit);
                if (s < 4 && p0 + col < P) yr[p0 + col] = total + skip * sx[c * cols + cg * RC + col];
            } else {
#pragma unroll
                for (int k = 0; k < RC; ++k) {
                    const float total = split_sum(sums[k], nsplit);
                    if (s == 0 && p0 + k < P) yr[p0 + k] = total + skip * sx[c * cols + cg * RC + k];
                }
            }
        };
        if (nt == kChunk) {
            // A full chunk unrolled: the column sums of its tokens wait in registers and are reduced over
            // the lanes together after the loop, as independent shuffles instead of a chain per token.
            float sums[kChunk][RC];
#pragma unroll
            for (int c = 0; c < kChunk; ++c) advance(c, sums[c]);
#pragma unroll
            for (int c = 0; c < kChunk; ++c) finish(c, sums[c]);
        } else {
            for (int c = 0; c < nt; ++c) {
                float sums[RC];
                advance(c, sums);
                finish(c, sums);
            }
        }
        if (next_nt > 0) copies_wait();
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < RN; ++i)
#pragma unroll
        for (int c = 0; c < RC; ++c) {
            const int n = s + nsplit * i;
            if (p0 + c < P && n < N) Sp[(size_t)(p0 + c) * N + n] = S[i][c];
        }
}

__global__ void __launch_bounds__(SE_TILE_THREADS)
delta_scan_tile_kernel(const float* __restrict__ qkv, const float* __restrict__ dec, const float* __restrict__ beta,
                       float* state, long long state_pitch, const int* __restrict__ cu_q, const int* __restrict__ seq_rows,
                       float* __restrict__ o, int H, int G, int d, int dv, int nsplit, int cols) {
    constexpr int RN = kTileRows, RC = kTileCols;
    extern __shared__ __align__(16) float sm[];
    const int np = nsplit * kTilePad;
    const int buf = kChunk * (3 * np + cols + 1);
    const int e = blockIdx.x, h = blockIdx.y, g = h / (H / G);
    const int s = threadIdx.x % nsplit, cg = threadIdx.x / nsplit, j0 = blockIdx.z * cols + cg * RC;
    const int lane = threadIdx.x & 31;
    const int start = cu_q[e], end = cu_q[e + 1];
    const int width = 2 * G * d + H * dv;
    float* Sp = state + (size_t)seq_rows[e] * state_pitch + (size_t)h * dv * d;
    float S[RN][RC];
#pragma unroll
    for (int i = 0; i < RN; ++i)
#pragma unroll
        for (int c = 0; c < RC; ++c) {
            const int n = s + nsplit * i;
            S[i][c] = (j0 + c < dv && n < d) ? Sp[(size_t)(j0 + c) * d + n] : 0.f;
        }
    if (d != nsplit * RN || blockIdx.z * cols + cols > dv) {     // rows beyond d and columns beyond dv read as zeros
        for (int i = threadIdx.x; i < 2 * buf; i += blockDim.x) sm[i] = 0.f;
        __syncthreads();
    }
    const int split_log2 = 31 - __clz(nsplit);

    auto issue = [&](int t0, int nt, float* dst) {
        const float* r0 = qkv + (size_t)t0 * width + g * d;
        const float* g0 = dec + (size_t)t0 * H * d + h * d;
        for (int n = threadIdx.x; n < d; n += blockDim.x) {
            const int at = (n & (nsplit - 1)) * kTilePad + (n >> split_log2);
            for (int c = 0; c < nt; ++c) {
                copy_async4(dst + c * np + at, r0 + (size_t)c * width + n);
                copy_async4(dst + kChunk * np + c * np + at, r0 + (size_t)c * width + G * d + n);
                copy_async4(dst + 2 * kChunk * np + c * np + at, g0 + (size_t)c * H * d + n);
            }
        }
        const float* v0 = qkv + (size_t)t0 * width + 2 * G * d + h * dv + blockIdx.z * cols;
        for (int jj = threadIdx.x; jj < cols; jj += blockDim.x) {
            if (blockIdx.z * cols + jj < dv)
                for (int c = 0; c < nt; ++c) copy_async4(dst + 3 * kChunk * np + c * cols + jj, v0 + (size_t)c * width + jj);
        }
        if ((int)threadIdx.x < nt) copy_async4(dst + 3 * kChunk * np + kChunk * cols + threadIdx.x, beta + (size_t)(t0 + threadIdx.x) * H + h);
    };
    if (start < end) {
        issue(start, min(kChunk, end - start), sm);
        copies_wait();
    }
    __syncthreads();
    int cur = 0;
    for (int t0 = start; t0 < end; t0 += kChunk, cur ^= 1) {
        const int nt = min(kChunk, end - t0);
        const int next_nt = min(kChunk, end - (t0 + kChunk));
        float* here = sm + cur * buf;
        if (next_nt > 0) issue(t0 + kChunk, next_nt, sm + (cur ^ 1) * buf);
        const float* sv = here + 3 * kChunk * np;
        const float* sb = sv + kChunk * cols;
        auto token = [&](int c) {
            const float4* Q4 = reinterpret_cast<const float4*>(here + c * np + s * kTilePad);
            const float4* K4 = reinterpret_cast<const float4*>(here + kChunk * np + c * np + s * kTilePad);
            const float4* G4 = reinterpret_cast<const float4*>(here + 2 * kChunk * np + c * np + s * kTilePad);
            const float4 k0 = K4[0], k1 = K4[1], g0 = G4[0], g1 = G4[1];
            const float Kv[RN] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w};
            const float Gv[RN] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
            float r[RC] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < RN; ++i)
#pragma unroll
                for (int k = 0; k < RC; ++k) {
                    S[i][k] *= Gv[i];
                    r[k] += S[i][k] * Kv[i];
                }
            float rs[RC];
            if (nsplit >= 4) {          // one column's sum per lane, then every lane collects the four of its group
                const float mine = cross_sum4(r, s, nsplit);
                const int base = lane & ~3;
                rs[0] = __shfl_sync(0xffffffffu, mine, base);
                rs[1] = __shfl_sync(0xffffffffu, mine, base | 2);
                rs[2] = __shfl_sync(0xffffffffu, mine, base | 1);
                rs[3] = __shfl_sync(0xffffffffu, mine, base | 3);
            } else {
#pragma unroll
                for (int k = 0; k < RC; ++k) rs[k] = split_sum(r[k], nsplit);
            }
            const float bt = sb[c];
            const float4 vv = *reinterpret_cast<const float4*>(sv + c * cols + cg * RC);
            const float u[RC] = {bt * (vv.x - rs[0]), bt * (vv.y - rs[1]), bt * (vv.z - rs[2]), bt * (vv.w - rs[3])};
            const float4 q0 = Q4[0], q1 = Q4[1];
            const float Qv[RN] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
            float acc[RC] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < RN; ++i)
#pragma unroll
                for (int k = 0; k < RC; ++k) {
                    S[i][k] += Kv[i] * u[k];
                    acc[k] += S[i][k] * Qv[i];
                }
            float* orow = o + (size_t)(t0 + c) * H * dv + h * dv;
            if (nsplit >= 4) {
                const float total = cross_sum4(acc, s, nsplit);
                const int col = 2 * (s & 1) + ((s >> 1) & 1);
                if (s < 4 && j0 + col < dv) orow[j0 + col] = total;
            } else {
#pragma unroll
                for (int k = 0; k < RC; ++k) {
                    const float total = split_sum(acc[k], nsplit);
                    if (s == 0 && j0 + k < dv) orow[j0 + k] = total;
                }
            }
        };
        for (int c = 0; c < nt; ++c) token(c);
        if (next_nt > 0) copies_wait();
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < RN; ++i)
#pragma unroll
        for (int c = 0; c < RC; ++c) {
            const int n = s + nsplit * i;
            if (j0 + c < dv && n < d) Sp[(size_t)(j0 + c) * d + n] = S[i][c];
        }
}

// Plan of the tiled kernels, for up to 8 * 32 rows: threads per column group, columns per block.
static inline void tile_plan(int rows, int columns, int units, int* nsplit, int* cols) {
    int ns = 1;
    while (ns * kTileRows < rows) ns *= 2;
    *nsplit = ns;
    // Blocks of 128 threads (SE_SCAN_THREADS, a tuning aid, sets a smaller size): a head's columns spread
    // over several blocks, so that one long request reaches more SMs, and three such blocks share an
    // SM, so that one block's state and inputs are on their way while another computes.
    static const int block_threads = [] { const char* v = ::getenv("SE_SCAN_THREADS"); return v ? atoi(v) : 128; }();
    const int threads = block_threads < 32 ? 32 : block_threads > SE_TILE_THREADS ? SE_TILE_THREADS : block_threads;
    (void)units;
    int groups = threads / ns > 0 ? threads / ns : 1;        // column groups per block
    const int unit = 32 / ns;
    const int need = ((columns + kTileCols - 1) / kTileCols + unit - 1) / unit * unit;
    if (groups > need) groups = need;
    *cols = groups * kTileCols;
}

// ---- prologue of the delta rule ----------------------------------------------------------------
// One block per token: q and k heads (in qkv, in place) become unit vectors, x / sqrt(sum x^2 +
// unit_eps), q also times q_scale; dec = exp(-exp(A_log[h]) * softplus(a + dt_bias)); beta =
// sigmoid(b).  `a` (rows a_pitch apart) is the decay projection: [H*d], one decay per head and key
// channel, or, with `per_head`, [H], one decay per head (dt_bias likewise), which is written to all
// of the head's channels.  `proj` column b_off + h is the beta projection.
template <typename T>
__global__ void delta_prep_kernel(float* qkv, int width, const T* a, int a_pitch, const T* proj, int pitch, int b_off,
                                  const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                  float* __restrict__ dec, float* __restrict__ beta, int H, int G, int d,
                                  float unit_eps, float q_scale, int per_head, float* __restrict__ log_dec) {
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    float* row = qkv + (size_t)t * width;
    for (int hh = warp; hh < 2 * G; hh += warps) {          // q heads, then k heads
        float* v = row + (size_t)hh * d;
        float ss = 0.f;
        for (int i = lane; i < d; i += 32) ss += v[i] * v[i];
        ss = warp_sum(ss);
        const float f = (hh < G ? q_scale : 1.f) / sqrtf(ss + unit_eps);
        for (int i = lane; i < d; i += 32) v[i] *= f;
    }
    for (int i = threadIdx.x; i < H * d; i += blockDim.x) {
        const int h = i / d, j = per_head ? h : i;
        const float rate = expf(a_log[h]);
        dec[(size_t)t * H * d + i] = expf(-rate * softplus_f(to_float(a[(size_t)t * a_pitch + j]) + dt_bias[j]));
    }
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        beta[(size_t)t * H + h] = sigmoid_f(to_float(proj[(size_t)t * pitch + b_off + h]));
        // the decays' logarithms (one per head), for the chunked form of the recurrence
        if (log_dec != nullptr)
            log_dec[(size_t)t * H + h] = -expf(a_log[h]) * softplus_f(to_float(a[(size_t)t * a_pitch + h]) + dt_bias[h]);
    }
}

// ---- epilogues ---------------------------------------------------------------------------------
// Delta rule: each head's output divided by its root mean square over dv, times w[dv] (shared by
// the heads), times sigmoid(gate) or (`silu`) gate * sigmoid(gate); the gate's rows lie gate_pitch
// apart, a head's dv columns side by side.  One warp per (token, head).
template <typename T>
__global__ void delta_out_kernel(const float* __restrict__ o, const T* gate, int gate_pitch, const float* __restrict__ w,
                                 T* __restrict__ out, int rows, int H, int dv, float eps, int silu) {
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= rows) return;
    const float* v = o + (size_t)r * dv;
    const T* gp = gate + (size_t)(r / H) * gate_pitch + (size_t)(r % H) * dv;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) ss += v[i] * v[i];
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)dv + eps);
    for (int i = lane; i < dv; i += 32) {
        const float g = to_float(gp[i]);
        out[(size_t)r * dv + i] = from_float<T>(v[i] * inv * w[i] * (silu ? g * sigmoid_f(g) : sigmoid_f(g)));
    }
}

// State space: y * silu(z), then an RMS norm over each of `parts` equal parts of the row, times
// w.  z is column z_off + i of the input projection.  grid (tokens, parts).
template <typename T>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, const T* proj, int pitch, int z_off,
                                        const float* __restrict__ w, T* __restrict__ out, int inner, int parts, float eps,
                                        int keep) {
    extern __shared__ float gated[];          // the part's gated values, if they fit (`keep`)
    __shared__ float scratch[33];
    const int t = blockIdx.x, n = inner / parts, base = blockIdx.y * n;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = y[(size_t)t * inner + base + i] * silu_f(to_float(proj[(size_t)t * pitch + z_off + base + i]));
        if (keep) gated[i] = v;
        ss += v * v;
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = keep ? gated[i]
                             : y[(size_t)t * inner + base + i] * silu_f(to_float(proj[(size_t)t * pitch + z_off + base + i]));
        out[(size_t)t * inner + base + i] = from_float<T>(v * inv * w[base + i]);
    }
}

// rows of the key/state side a recurrence kernel takes (32 registers x 16 lanes)
constexpr int kMaxStateRows = 512;

// regs: rows a thread keeps (8, 16 or 32: the more, the fewer shuffles and shared-memory reads per
// multiply-add); nsplit: threads per column; cols: columns per block (a multiple of 32 / nsplit, at
// most what is there), blocks of 256 threads, so that the columns of a head spread over several
// blocks and one long request still fills the SMs.
static inline void scan_plan(int rows, int columns, int* regs, int* nsplit, int* cols) {
    *regs = rows > 64 ? 32 : rows > 16 ? 16 : 8;
    int ns = 1;
    while (ns * *regs < rows) ns *= 2;
    *nsplit = ns;
    int c = 256 / ns;
    const int unit = 32 / ns;
    const int need = (columns + unit - 1) / unit * unit;
    if (c > need) c = need;
    *cols = c;
}

#define SE_SCAN_DISPATCH(regs, ...)                               \
    if ((regs) == 8) { constexpr int R = 8; __VA_ARGS__; }        \
    else if ((regs) == 16) { constexpr int R = 16; __VA_ARGS__; } \
    else { constexpr int R = 32; __VA_ARGS__; }

}  // namespace se

extern "C" int se_recurrent_max_state_rows() { return se::kMaxStateRows; }

extern "C" int se_causal_conv(const void* x, int pitch, int c0, const float* w, const float* bias, float* state,
                              long long state_pitch, int conv_off, const int* token_seq, const int* cu_q,
                              const int* seq_rows, float* out, int tokens, int entries, int C, int taps, int dtype,
                              cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (C <= 0 || taps <= 0 || entries <= 0) return SE_ERR_ARGUMENT;
    const int threads = 128;
    int tile = tokens / entries;
    tile = tile < 1 ? 1 : tile > se::kConvTokens ? se::kConvTokens : tile;
    const dim3 grid(se::ceil_div(tokens, tile), se::ceil_div(C, threads)), grid2(entries, se::ceil_div(C, threads));
    if (grid.y > 65535 || taps > 64) return SE_ERR_UNSUPPORTED;
    const size_t smem = (size_t)(tile + taps - 1) * 128 * sizeof(float);
    SE_DISPATCH_DTYPE(dtype, T, {
        se::causal_conv_kernel<T><<<grid, threads, smem, stream>>>((const T*)x, pitch, c0, w, bias, state, state_pitch, conv_off,
                                                                   token_seq, cu_q, seq_rows, out, tokens, C, taps, tile);
        if (taps > 1)
            se::conv_carry_kernel<T><<<grid2, threads, 0, stream>>>((const T*)x, pitch, c0, state, state_pitch, conv_off, cu_q,
                                                                    seq_rows, C, taps);
    });
    SE_LAUNCH_CHECK();
}

// steps: workspace of 2 * tokens * H floats (step sizes and decays), or null (then the kernel with one
// column per thread computes them itself)
extern "C" int se_ssm_scan(const float* xbc, const void* proj, int pitch, int dt_off, const float* dt_bias,
                           const float* a_log, const float* d_skip, float* state, long long state_pitch, const int* cu_q,
                           const int* seq_rows, float* y, float* steps, int tokens, int entries, int H, int P, int N, int G,
                           int dtype, cudaStream_t stream) {
    if (entries <= 0) return 0;
    if (H <= 0 || P <= 0 || N <= 0 || G <= 0 || H % G) return SE_ERR_ARGUMENT;
    if (N > se::kMaxStateRows || H > 65535) return SE_ERR_UNSUPPORTED;
    int regs, nsplit, cols;
    if (N <= se::kTileRows * 32 && steps != nullptr) {
        se::tile_plan(N, P, entries * H, &nsplit, &cols);
        const dim3 grid(entries, H, se::ceil_div(P, cols));
        const size_t smem = (size_t)2 * se::kChunk * (2 * nsplit * se::kTilePad + cols + 2) * sizeof(float);
        SE_DISPATCH_DTYPE(dtype, T, {
            if (smem > 40 * 1024) {
                cudaError_t e = cudaFuncSetAttribute(se::ssm_scan_tile_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (e != cudaSuccess) return (int)e;
            }
            se::ssm_steps_kernel<T><<<se::ceil_div(tokens * H, 256), 256, 0, stream>>>((const T*)proj, pitch, dt_off, dt_bias, a_log,
                                                                                     steps, tokens, H);
            se::ssm_scan_tile_kernel<T><<<grid, nsplit * cols / se::kTileCols, smem, stream>>>(
                xbc, steps, d_skip, state, state_pitch, cu_q, seq_rows, y, H, P, N, G, nsplit, cols);
        });
        SE_LAUNCH_CHECK();
    }
    se::scan_plan(N, P, &regs, &nsplit, &cols);
    const dim3 grid(entries, H, se::ceil_div(P, cols));
    const size_t smem = (size_t)2 * se::kChunk * (2 * nsplit * (regs + 4) + cols + 2) * sizeof(float);
    SE_DISPATCH_DTYPE(dtype, T, {
        SE_SCAN_DISPATCH(regs, {
            if (smem > 40 * 1024) {
                cudaError_t e = cudaFuncSetAttribute(se::ssm_scan_kernel<T, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (e != cudaSuccess) return (int)e;
            }
            se::ssm_scan_kernel<T, R><<<grid, nsplit * cols, smem, stream>>>(xbc, (const T*)proj, pitch, dt_off, dt_bias, a_log,
                                                                             d_skip, state, state_pitch, cu_q, seq_rows, y, H, P,
                                                                             N, G, nsplit, cols);
        });
    });
    SE_LAUNCH_CHECK();
}

extern "C" int se_delta_prep(float* qkv, const void* a, int a_pitch, const void* proj, int pitch, int b_off,
                             const float* dt_bias, const float* a_log, float* dec, float* beta, int tokens, int H, int G,
                             int d, int dv, float unit_eps, float q_scale, int per_head, float* log_dec, int dtype,
                             cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || d <= 0 || dv <= 0 || a_pitch < (per_head ? H : H * d)) return SE_ERR_ARGUMENT;
    if (log_dec != nullptr && !per_head) return SE_ERR_ARGUMENT;
    SE_DISPATCH_DTYPE(dtype, T,
        se::delta_prep_kernel<T><<<tokens, 256, 0, stream>>>(qkv, 2 * G * d + H * dv, (const T*)a, a_pitch, (const T*)proj, pitch,
                                                            b_off, dt_bias, a_log, dec, beta, H, G, d, unit_eps, q_scale,
                                                            per_head, log_dec));
    SE_LAUNCH_CHECK();
}

extern "C" int se_delta_scan(const float* qkv, const float* dec, const float* beta, float* state, long long state_pitch,
                             const int* cu_q, const int* seq_rows, float* o, int entries, int H, int G, int d, int dv,
                             cudaStream_t stream) {
    if (entries <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || d <= 0 || dv <= 0) return SE_ERR_ARGUMENT;
    if (d > se::kMaxStateRows || H > 65535) return SE_ERR_UNSUPPORTED;
    int regs, nsplit, cols;
    if (d <= se::kTileRows * 32) {
        se::tile_plan(d, dv, entries * H, &nsplit, &cols);
        const dim3 grid(entries, H, se::ceil_div(dv, cols));
        const size_t smem = (size_t)2 * se::kChunk * (3 * nsplit * se::kTilePad + cols + 1) * sizeof(float);
        if (smem > 40 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(se::delta_scan_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        se::delta_scan_tile_kernel<<<grid, nsplit * cols / se::kTileCols, smem, stream>>>(qkv, dec, beta, state, state_pitch, cu_q,
                                                                                         seq_rows, o, H, G, d, dv, nsplit, cols);
        SE_LAUNCH_CHECK();
    }
    se::scan_plan(d, dv, &regs, &nsplit, &cols);
    const dim3 grid(entries, H, se::ceil_div(dv, cols));
    const size_t smem = (size_t)2 * se::kChunk * (3 * nsplit * (regs + 4) + cols + 1) * sizeof(float);
    SE_SCAN_DISPATCH(regs, {
        if (smem > 40 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(se::delta_scan_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        se::delta_scan_kernel<R><<<grid, nsplit * cols, smem, stream>>>(qkv, dec, beta, state, state_pitch, cu_q, seq_rows, o, H, G,
                                                                        d, dv, nsplit, cols);
    });
    SE_LAUNCH_CHECK();
}

extern "C" int se_delta_out(const float* o, const void* gate, int gate_pitch, const float* w, void* out, int rows, int H,
                            int dv, float eps, int silu, int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (H <= 0 || rows % H || gate_pitch < H * dv) return SE_ERR_ARGUMENT;
    SE_DISPATCH_DTYPE(dtype, T,
        se::delta_out_kernel<T><<<se::ceil_div(rows, 4), 128, 0, stream>>>(o, (const T*)gate, gate_pitch, w, (T*)out, rows, H, dv,
                                                                           eps, silu));
    SE_LAUNCH_CHECK();
}

extern "C" int se_gated_group_norm(const float* y, const void* proj, int pitch, int z_off, const float* w, void* out,
                                   int tokens, int inner, int parts, float eps, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (parts <= 0 || inner % parts || parts > 65535) return SE_ERR_ARGUMENT;
    const int n = inner / parts, keep = n * (int)sizeof(float) <= 40 * 1024;
    const int threads = n >= 1024 ? 256 : 128;
    SE_DISPATCH_DTYPE(dtype, T,
        se::gated_group_norm_kernel<T><<<dim3(tokens, parts), threads, keep ? n * sizeof(float) : 0, stream>>>(
            y, (const T*)proj, pitch, z_off, w, (T*)out, inner, parts, eps, keep));
    SE_LAUNCH_CHECK();
}
