// Several residual streams per token (hyper-connections), 32-bit.
//
// A token carries S copies x_1 .. x_S of the residual stream, laid out [token][stream][width].
// A sublayer reads one mixture of them and writes its result back into all of them:
//
//     read :  u   = sum_s a[s] x_s ;  h = u / sqrt(mean(u^2) + eps) * w        (w: the norm's 32-bit weight)
//     write:  x_t <- sum_s M[s][t] x_s + b[t] * y'                              (all t from the old x)
//     y' = y * sigmoid(g + c)  where a gate is given (g: the gate's projection, c its bias), else y
//
// One kernel does the write of the sublayer that has just run and the read for the next one, one
// block per token: the S stream values of a column are in registers between the two, the mixture u
// of the row waits in shared memory for the row's mean square.  Either half may be left out (the
// first read of a step has nothing to write, the last write of a step reads with a = 1 for the
// model's last norm).  S = 1 with M = a = b = 1 is the plain pre-norm residual.  Everything is
// 32-bit; y, g and h have the activation type.
#include "common.cuh"

namespace se {

constexpr int kMaxStreams = 16;      // up to 8 with four columns per thread, beyond that one column per thread

// V columns per thread at a time: 4 (16-byte accesses of the streams) where the width and the addresses allow, else 1.
template <typename T, int V>
__device__ __forceinline__ void load_act(const T* p, float* v) {
    if constexpr (V == 1) {
        v[0] = to_float(p[0]);
    } else if constexpr (sizeof(T) == 4) {
        const float4 a = *reinterpret_cast<const float4*>(p);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    } else {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float2 a = __bfloat1622float2(hh[0]), b = __bfloat1622float2(hh[1]);
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
}
template <typename T, int V>
__device__ __forceinline__ void store_act(T* p, const float* v) {
    if constexpr (V == 1) {
        p[0] = from_float<T>(v[0]);
    } else if constexpr (sizeof(T) == 4) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
        uint2 raw;
        __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&raw);
        hh[0] = __floats2bfloat162_rn(v[0], v[1]);
        hh[1] = __floats2bfloat162_rn(v[2], v[3]);
        *reinterpret_cast<uint2*>(p) = raw;
    }
}
template <int V>
__device__ __forceinline__ void load_f32(const float* p, float* v) {
    if constexpr (V == 1) {
        v[0] = p[0];
    } else {
        const float4 a = *reinterpret_cast<const float4*>(p);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    }
}
template <int V>
__device__ __forceinline__ void store_f32(float* p, const float* v) {
    if constexpr (V == 1) p[0] = v[0];
    else *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}

template <typename T, int V, int S>
__global__ void __launch_bounds__(256)
stream_mix_kernel(float* streams, int width, const T* __restrict__ y, const T* __restrict__ gate,
                  const float* __restrict__ gate_bias, const float* __restrict__ mix, const float* __restrict__ out_w,
                  const float* __restrict__ in_w, const float* __restrict__ norm_w, float eps, T* __restrict__ h,
                  int store) {
    extern __shared__ __align__(16) float urow[];
    __shared__ float scratch[33];
    __shared__ float sm_mix[S * S], sm_out[S], sm_in[S];
    const size_t t = blockIdx.x;
    if (y != nullptr)
        for (int i = threadIdx.x; i < S * S; i += blockDim.x) sm_mix[i] = mix[i];
    if (threadIdx.x < S) {
        if (y != nullptr) sm_out[threadIdx.x] = out_w[threadIdx.x];
        if (h != nullptr) sm_in[threadIdx.x] = in_w != nullptr ? in_w[threadIdx.x] : 1.f;
    }
    __syncthreads();
    float* base = streams + t * S * width;
    float ss = 0.f;
    for (int i = threadIdx.x * V; i < width; i += blockDim.x * V) {
        float x[S][V];
#pragma unroll
        for (int s = 0; s < S; ++s) load_f32<V>(base + (size_t)s * width + i, x[s]);
        if (y != nullptr) {
            float yv[V];
            load_act<T, V>(y + t * width + i, yv);
            if (gate != nullptr) {
                float z[V], b[V];
                load_act<T, V>(gate + t * width + i, z);
                if (gate_bias != nullptr) {
                    load_f32<V>(gate_bias + i, b);
#pragma unroll
                    for (int j = 0; j < V; ++j) z[j] += b[j];
                }
#pragma unroll
                for (int j = 0; j < V; ++j) yv[j] *= 1.f / (1.f + expf(-z[j]));
            }
            float nx[S][V];
#pragma unroll
            for (int d = 0; d < S; ++d)
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    float v = 0.f;
#pragma unroll
                    for (int s = 0; s < S; ++s) v += sm_mix[s * S + d] * x[s][j];
                    nx[d][j] = v + sm_out[d] * yv[j];
                }
#pragma unroll
            for (int d = 0; d < S; ++d) {
#pragma unroll
                for (int j = 0; j < V; ++j) x[d][j] = nx[d][j];
                if (store) store_f32<V>(base + (size_t)d * width + i, nx[d]);
            }
        }
        if (h != nullptr) {
#pragma unroll
            for (int j = 0; j < V; ++j) {
                float u = 0.f;
#pragma unroll
                for (int s = 0; s < S; ++s) u += sm_in[s] * x[s][j];
                urow[i + j] = u;
                ss += u * u;
            }
        }
    }
    if (h == nullptr) return;
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
    // every thread reads back the elements it wrote itself
    for (int i = threadIdx.x * V; i < width; i += blockDim.x * V) {
        float w[V], o[V];
        load_f32<V>(norm_w + i, w);
#pragma unroll
        for (int j = 0; j < V; ++j) o[j] = urow[i + j] * inv * w[j];
        store_act<T, V>(h + t * width + i, o);
    }
}

// streams[t][s] = table[ids[t]] * scale for every s (32-bit product)
template <typename T>
__global__ void stream_embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ streams,
                                    int S, int width, int vocab, float scale) {
    const size_t t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    const T* src = table + (size_t)(ok ? id : 0) * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = ok ? to_float(src[i]) * scale : 0.f;
        for (int s = 0; s < S; ++s) streams[(t * S + s) * width + i] = v;
    }
}

// out[t] = sum_s streams[t][s] (a debugging aid: the stream as one)
__global__ void stream_sum_kernel(const float* __restrict__ streams, float* __restrict__ out, int S, int width) {
    const size_t t = blockIdx.x;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < S; ++s) v += streams[(t * S + s) * width + i];
        out[t * width + i] = v;
    }
}

// out = a * x + b * y (+ bias), 32-bit, rounded once: the outputs of mixers that run side by side.  Eight elements
// per thread at a time where the width and the addresses allow it.
template <typename T>
__global__ void scaled_sum_kernel(const T* __restrict__ x, const T* __restrict__ y, float a, float b,
                                  const float* __restrict__ bias, T* __restrict__ out, size_t n, int width, int vec) {
    if (vec) {
        for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += (size_t)gridDim.x * blockDim.x * 8) {
            float xv[8], yv[8], o[8];
            load8(x + i, xv);
            load8(y + i, yv);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = a * xv[j] + b * yv[j];
            if (bias != nullptr) {
                float bv[8];
                load8(bias + i % width, bv);
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] += bv[j];
            }
            store8(out + i, o);
        }
        return;
    }
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float v = a * to_float(x[i]) + b * to_float(y[i]);
        if (bias != nullptr) v += bias[i % width];
        out[i] = from_float<T>(v);
    }
}

}  // namespace se

extern "C" int se_scaled_sum(const void* x, const void* y, float a, float b, const float* bias, void* out, int rows,
                             int width, int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const size_t n = (size_t)rows * width;
    auto aligned16 = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const int vec = width % 8 == 0 && aligned16(x) && aligned16(y) && aligned16(bias) && aligned16(out);
    const size_t work = vec ? n / 8 : n;
    const int blocks = (int)((work + 255) / 256 < 148 * 8 ? (work + 255) / 256 : 148 * 8);
    SE_DISPATCH_DTYPE(dtype, T,
        se::scaled_sum_kernel<T><<<blocks, 256, 0, stream>>>((const T*)x, (const T*)y, a, b, bias, (T*)out, n, width, vec));
    SE_LAUNCH_CHECK();
}

extern "C" int se_stream_mix_max_streams() { return se::kMaxStreams; }
extern "C" int se_stream_mix_max_width() { return 51200; }

// y == nullptr: no write; h == nullptr: no read.  store = 0: the new streams are not written back
// (rows gathered for the last norm).
extern "C" int se_stream_mix(float* streams, int tokens, int S, int width, const void* y, const void* gate,
                             const float* gate_bias, const float* mix, const float* out_w, const float* in_w,
                             const float* norm_w, float eps, void* h, int store, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (S <= 0 || S > se::kMaxStreams || width <= 0 || width > se_stream_mix_max_width()) return SE_ERR_UNSUPPORTED;
    if (y != nullptr && (mix == nullptr || out_w == nullptr)) return SE_ERR_ARGUMENT;
    if (h != nullptr && norm_w == nullptr) return SE_ERR_ARGUMENT;
    if (y == nullptr && h == nullptr) return 0;
    const size_t smem = h != nullptr ? (size_t)width * sizeof(float) : 0;
    auto aligned16 = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool vec = S <= 8 && width % 4 == 0 && aligned16(streams) && aligned16(y) && aligned16(gate) && aligned16(gate_bias) &&
                     aligned16(norm_w) && aligned16(h);
    const int per = vec ? 4 : 1;
    const int threads = width / per >= 256 ? 256 : width / per >= 128 ? 128 : 64;
#define SE_MIX_LAUNCH(V, SN)                                                                                             \
    {                                                                                                                    \
        if (smem > 40 * 1024) {                                                                                          \
            cudaError_t e = cudaFuncSetAttribute(se::stream_mix_kernel<T, V, SN>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                 (int)smem);                                                             \
            if (e != cudaSuccess) return (int)e;                                                                         \
        }                                                                                                                \
        se::stream_mix_kernel<T, V, SN><<<tokens, threads, smem, stream>>>(streams, width, (const T*)y, (const T*)gate,  \
                                                                           gate_bias, mix, out_w, in_w, norm_w, eps, (T*)h, store); \
    }
#define SE_MIX_STREAMS(V)                                                                                                \
    switch (S) {                                                                                                         \
        case 1: SE_MIX_LAUNCH(V, 1) break;                                                                               \
        case 2: SE_MIX_LAUNCH(V, 2) break;                                                                               \
        case 3: SE_MIX_LAUNCH(V, 3) break;                                                                               \
        case 4: SE_MIX_LAUNCH(V, 4) break;                                                                               \
        case 5: SE_MIX_LAUNCH(V, 5) break;                                                                               \
        case 6: SE_MIX_LAUNCH(V, 6) break;                                                                               \
        case 7: SE_MIX_LAUNCH(V, 7) break;                                                                               \
        default: SE_MIX_LAUNCH(V, 8) break;                                                                              \
    }
#define SE_MIX_MANY()                                                                                                    \
    switch (S) {                                                                                                         \
        case 9: SE_MIX_LAUNCH(1, 9) break;                                                                               \
        case 10: SE_MIX_LAUNCH(1, 10) break;                                                                             \
        case 11: SE_MIX_LAUNCH(1, 11) break;                                                                             \
        case 12: SE_MIX_LAUNCH(1, 12) break;                                                                             \
        case 13: SE_MIX_LAUNCH(1, 13) break;                                                                             \
        case 14: SE_MIX_LAUNCH(1, 14) break;                                                                             \
        case 15: SE_MIX_LAUNCH(1, 15) break;                                                                             \
        default: SE_MIX_LAUNCH(1, 16) break;                                                                             \
    }
    SE_DISPATCH_DTYPE(dtype, T, {
        if (S > 8) { SE_MIX_MANY() } else if (vec) { SE_MIX_STREAMS(4) } else { SE_MIX_STREAMS(1) }
    });
#undef SE_MIX_MANY
#undef SE_MIX_STREAMS
#undef SE_MIX_LAUNCH
    SE_LAUNCH_CHECK();
}

extern "C" int se_stream_embed(const void* table, const int* ids, float* streams, int tokens, int S, int width, int vocab,
                               float scale, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (S <= 0 || width <= 0) return SE_ERR_ARGUMENT;
    SE_DISPATCH_DTYPE(dtype, T,
        se::stream_embed_kernel<T><<<tokens, 256, 0, stream>>>((const T*)table, ids, streams, S, width, vocab, scale));
    SE_LAUNCH_CHECK();
}

extern "C" int se_stream_sum(const float* streams, float* out, int tokens, int S, int width, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    se::stream_sum_kernel<<<tokens, 256, 0, stream>>>(streams, out, S, width);
    SE_LAUNCH_CHECK();
}
