// Kernels for models that carry their residual stream in 32-bit whatever the activation type:
// scaled embedding gather into the stream, layer norm (weight and bias) of `alpha * stream + y`
// that writes the new stream in 32-bit and a copy in the activation type for the next matrix
// product, and the activations of an ungated feed-forward.
//
// Layer norm: (v - mean) / sqrt(var + eps) * w + b with var the mean of the squared deviations
// (two passes over the row, which is kept in shared memory in 32-bit).
#include "common.cuh"

namespace se {

// stream[t] = table[ids[t]] * scale (32-bit product), act[t] = the same rounded (optional).
template <typename T>
__global__ void embed_stream_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ stream,
                                    T* __restrict__ act, int hidden, int vocab, float scale) {
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    const T* src = table + (size_t)(ok ? id : 0) * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = ok ? to_float(src[i]) * scale : 0.f;
        stream[(size_t)t * hidden + i] = v;
        if (act != nullptr) act[(size_t)t * hidden + i] = from_float<T>(v);
    }
}

// One block per row.  v = alpha * x + y (y optional); out32 and out_act are optional.  Rows whose
// width is a multiple of 8 and whose pointers allow it move in groups of 8 elements.
template <typename T>
__global__ void add_layernorm_kernel(const float* x, const T* y, float alpha, const T* __restrict__ w,
                                     const T* __restrict__ b, float* out32, T* out_act, int hidden, float eps) {
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[33];
    grid_dependency_trigger();
    grid_dependency_wait();
    const size_t base = (size_t)blockIdx.x * hidden;
    const bool vec = (hidden & 7) == 0 && aligned8(x) && aligned8(w) && (y == nullptr || aligned8(y)) &&
                     (b == nullptr || aligned8(b)) && (out32 == nullptr || aligned8(out32)) &&
                     (out_act == nullptr || aligned8(out_act));
    float s = 0.f;
    if (vec) {
        for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
            float v[8];
            load8(x + base + i, v);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] *= alpha;
            if (y != nullptr) {
                float r[8];
                load8(y + base + i, r);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] += r[j];
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) { row[i + j] = v[j]; s += v[j]; }
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float v = alpha * x[base + i];
            if (y != nullptr) v += to_float(y[base + i]);
            row[i] = v;
            s += v;
        }
    }
    const float mean = block_sum(s, scratch) / (float)hidden;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {      // block_sum's barriers lie between the writes and here
        const float c = row[i] - mean;
        ss += c * c;
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)hidden + eps);
    if (vec) {
        for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
            float wv[8], bv[8], o[8];
            load8(w + i, wv);
            if (b != nullptr) load8(b + i, bv);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = (row[i + j] - mean) * inv * wv[j] + (b != nullptr ? bv[j] : 0.f);
            if (out32 != nullptr) store8(out32 + base + i, o);
            if (out_act != nullptr) store8(out_act + base + i, o);
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float o = (row[i] - mean) * inv * to_float(w[i]) + (b != nullptr ? to_float(b[i]) : 0.f);
            if (out32 != nullptr) out32[base + i] = o;
            if (out_act != nullptr) out_act[base + i] = from_float<T>(o);
        }
    }
}

// One block per row of a pre-norm model's 32-bit stream.  v = x + y (y optional) goes to out32
// (which may be x itself); with a weight, out_act = v / sqrt(mean(v^2) + eps) * w, without one
// out_act = v rounded (both optional).
template <typename T>
__global__ void add_rmsnorm_stream_kernel(const float* x, const T* y, const T* __restrict__ w, float* out32, T* out_act,
                                          int hidden, float eps) {
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * hidden;
    // rows whose width is a multiple of 8 and whose pointers allow it move in groups of 8 elements
    const bool vec = (hidden & 7) == 0 && aligned8(x) && (y == nullptr || aligned8(y)) && (w == nullptr || aligned8(w)) &&
                     (out32 == nullptr || aligned8(out32)) && (out_act == nullptr || aligned8(out_act));
    float ss = 0.f;
    if (vec) {
        for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
            float v[8];
            load8(x + base + i, v);
            if (y != nullptr) {
                float r[8];
                load8(y + base + i, r);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] += r[j];
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) { row[i + j] = v[j]; ss += v[j] * v[j]; }
            if (out32 != nullptr) store8(out32 + base + i, v);
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float v = x[base + i];
            if (y != nullptr) v += to_float(y[base + i]);
            row[i] = v;
            ss += v * v;
            if (out32 != nullptr) out32[base + i] = v;
        }
    }
    if (out_act == nullptr) return;
    // every thread reads back the elements of the row that it wrote itself
    const float inv = w != nullptr ? 1.0f / sqrtf(block_sum(ss, scratch) / (float)hidden + eps) : 1.f;
    if (vec) {
        for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
            float o[8];
            if (w != nullptr) {
                float wv[8];
                load8(w + i, wv);
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = row[i + j] * inv * wv[j];
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = row[i + j];
            }
            store8(out_act + base + i, o);
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x)
            out_act[base + i] = from_float<T>(w != nullptr ? row[i] * inv * to_float(w[i]) : row[i]);
    }
}

// One block per row of a 32-bit stream whose sublayers are normed on their way out:
// stream += y / sqrt(mean(y^2) + eps) * w (32-bit), and out_act (optional) receives the new stream
// rounded to the activation type, which is what the next sublayer reads.
template <typename T>
__global__ void rmsnorm_add_stream_kernel(float* stream, const T* y, const T* __restrict__ w, T* out_act, int hidden,
                                          float eps) {
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[33];
    grid_dependency_trigger();
    grid_dependency_wait();
    const size_t base = (size_t)blockIdx.x * hidden;
    const bool vec = (hidden & 7) == 0 && aligned8(stream) && aligned8(y) && aligned8(w) &&
                     (out_act == nullptr || aligned8(out_act));
    float ss = 0.f;
    if (vec) {
        for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
            float v[8];
            load8(y + base + i, v);
#pragma unroll
            for (int j = 0; j < 8; ++j) { row[i + j] = v[j]; ss += v[j] * v[j]; }
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float v = to_float(y[base + i]);
            row[i] = v;
            ss += v * v;
        }
    }
    // every thread reads back the elements of the row that it wrote itself
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)hidden + eps);
    if (vec) {
        for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
            float wv[8], x[8];
            load8(w + i, wv);
            load8(stream + base + i, x);
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] += row[i + j] * inv * wv[j];
            store8(stream + base + i, x);
            if (out_act != nullptr) store8(out_act + base + i, x);
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float x = stream[base + i] + row[i] * inv * to_float(w[i]);
            stream[base + i] = x;
            if (out_act != nullptr) out_act[base + i] = from_float<T>(x);
        }
    }
}

__device__ __forceinline__ float act_apply(float v, int kind) {
    if (kind == 0) { const float r = fmaxf(v, 0.f); return r * r; }                       // squared relu
    if (kind == 1) return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));   // gelu (tanh form)
    if (kind == 2) return v / (1.f + expf(-v));                                           // silu
    return fmaxf(v, 0.f);                                                                 // relu
}

template <typename T>
__global__ void activation_kernel(T* x, size_t n, int kind) {
    grid_dependency_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (aligned8(x)) {                        // groups of 8 elements, then the rest one by one
        const size_t groups = n / 8;
        for (size_t g = i0; g < groups; g += stride) {
            float v[8];
            load8(x + 8 * g, v);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = act_apply(v[j], kind);
            store8(x + 8 * g, v);
        }
        for (size_t i = groups * 8 + i0; i < n; i += stride) x[i] = from_float<T>(act_apply(to_float(x[i]), kind));
        return;
    }
    for (size_t i = i0; i < n; i += stride) x[i] = from_float<T>(act_apply(to_float(x[i]), kind));
}

// x <- cap * tanh(x / cap) in place (32-bit arithmetic, rounded once): the cap on a model's logits
template <typename T>
__global__ void softcap_kernel(T* x, size_t n, float cap) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        x[i] = from_float<T>(cap * tanhf(to_float(x[i]) / cap));
}

}  // namespace se

extern "C" int se_softcap(void* x, long long n, float cap, int dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!(cap > 0.f)) return SE_ERR_ARGUMENT;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    SE_DISPATCH_DTYPE(dtype, T, se::softcap_kernel<T><<<blocks, 256, 0, stream>>>((T*)x, (size_t)n, cap));
    SE_LAUNCH_CHECK();
}

extern "C" int se_embed_stream(const void* table, const int* ids, float* stream, void* act, int tokens, int hidden,
                               int vocab, float scale, int dtype, cudaStream_t stream_) {
    if (tokens <= 0) return 0;
    SE_DISPATCH_DTYPE(dtype, T,
        se::embed_stream_kernel<T><<<tokens, 256, 0, stream_>>>((const T*)table, ids, stream, (T*)act, hidden, vocab, scale));
    SE_LAUNCH_CHECK();
}

extern "C" int se_layernorm_max_width() { return 200 * 1024 / (int)sizeof(float); }

extern "C" int se_add_layernorm(const float* x, const void* y, float alpha, const void* w, const void* b, float* out32,
                                void* out_act, int rows, int hidden, float eps, int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0 || hidden > se_layernorm_max_width()) return SE_ERR_UNSUPPORTED;
    const size_t smem = (size_t)hidden * sizeof(float);
    const int threads = hidden >= 8192 ? 512 : hidden >= 1024 ? 256 : 128;
    SE_DISPATCH_DTYPE(dtype, T, {
        if (smem > 40 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(se::add_layernorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        cudaError_t e = SE_LAUNCH_DEPENDENT("norm", se::add_layernorm_kernel<T>, dim3(rows), dim3(threads), smem, stream, x,
                                             (const T*)y, alpha, (const T*)w, (const T*)b, out32, (T*)out_act, hidden, eps);
        if (e != cudaSuccess) return (int)e;
    });
    SE_LAUNCH_CHECK();
}

extern "C" int se_add_rmsnorm_stream(const float* x, const void* y, const void* w, float* out32, void* out_act, int rows,
                                     int hidden, float eps, int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0 || hidden > se_layernorm_max_width()) return SE_ERR_UNSUPPORTED;
    const size_t smem = (size_t)hidden * sizeof(float);
    const int threads = hidden >= 8192 ? 512 : hidden >= 1024 ? 256 : 128;
    SE_DISPATCH_DTYPE(dtype, T, {
        if (smem > 40 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(se::add_rmsnorm_stream_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        se::add_rmsnorm_stream_kernel<T><<<rows, threads, smem, stream>>>(x, (const T*)y, (const T*)w, out32, (T*)out_act,
                                                                          hidden, eps);
    });
    SE_LAUNCH_CHECK();
}

extern "C" int se_rmsnorm_add_stream(float* stream_, const void* y, const void* w, void* out_act, int rows, int hidden,
                                     float eps, int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0 || hidden > se_layernorm_max_width()) return SE_ERR_UNSUPPORTED;
    if (y == nullptr || w == nullptr) return SE_ERR_ARGUMENT;
    const size_t smem = (size_t)hidden * sizeof(float);
    const int threads = hidden >= 8192 ? 512 : hidden >= 1024 ? 256 : 128;
    SE_DISPATCH_DTYPE(dtype, T, {
        if (smem > 40 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(se::rmsnorm_add_stream_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        cudaError_t e = SE_LAUNCH_DEPENDENT("norm", se::rmsnorm_add_stream_kernel<T>, dim3(rows), dim3(threads), smem, stream,
                                             stream_, (const T*)y, (const T*)w, (T*)out_act, hidden, eps);
        if (e != cudaSuccess) return (int)e;
    });
    SE_LAUNCH_CHECK();
}

// kind: 0 squared relu, 1 gelu (tanh form), 2 silu, 3 relu; in place
extern "C" int se_activation(void* x, long long n, int kind, int dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (kind < 0 || kind > 3) return SE_ERR_ARGUMENT;
    const long long work = (n + 7) / 8;
    const int blocks = (int)((work + 255) / 256 < 148 * 16 ? (work + 255) / 256 : 148 * 16);
    SE_DISPATCH_DTYPE(dtype, T, {
        cudaError_t e = SE_LAUNCH_DEPENDENT("act", se::activation_kernel<T>, dim3(blocks), dim3(256), 0, stream, (T*)x, (size_t)n, kind);
        if (e != cudaSuccess) return (int)e;
    });
    SE_LAUNCH_CHECK();
}
