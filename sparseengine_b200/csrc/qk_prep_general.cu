// Query/key preparation in its general form, for attention variants the rotary kernel of
// qk_prep.cu does not cover: a value head size of its own, a query temperature that grows with
// the position, layers that bring queries only (they attend over another layer's keys), and
// values blended with those of an earlier layer.
//
//   q_out[t] = rot(q * inv_rms(q) * q_w, pos) * temp(pos)      (statistics over the whole projection)
//   K page   = rot(k * inv_rms(k) * k_w, pos)
//   V page   = v, or (1 - mix) * v + mix * v_first              (v_first: the same token's values elsewhere)
//   temp(p)  = 1 + coef * ln(floor((p + 1) / every) + 1)        (coef = 0: none)
//   rot      : on the first `rotary_dim` dims of every head, dim i paired with dim i + rotary_dim/2,
//              (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = pos * inv_freq[i]  (rotary_dim = 0: none)
//
// Everything is computed in 32-bit and rounded once.  The norm weights are
// optional.  The projection row is [q: hq*d | k: hkv*d | v: hkv*dv] (`has_kv`) or [q] alone.
//
// Cache layout of one cache layer: per page the keys [kv head][slot in page][d], then the values
// [kv head][slot in page][dv]; with dv = d this is the layout of the other attention kernels.
#include "common.cuh"

namespace se {

template <typename T>
__global__ void __launch_bounds__(256)
qk_prep_general_kernel(const T* proj, int pitch, const T* __restrict__ q_w, const T* __restrict__ k_w,
                       const float* __restrict__ inv_freq, int rotary_dim, const T* v_first, int v_first_pitch,
                       const float* __restrict__ v_mix,
                       const int* __restrict__ positions, const int* __restrict__ token_seq,
                       const int* __restrict__ seq_rows, const int* __restrict__ table, int table_stride,
                       T* __restrict__ cache, T* __restrict__ q_out, int hq, int hkv, int d, int dv, float eps,
                       float temp_coef, int temp_every, int page_size, int has_kv, int num_pages, int* __restrict__ error) {
    __shared__ float scratch[33];
    grid_dependency_trigger();
    grid_dependency_wait();      // proj is not __restrict__: its loads stay below this line
    const int t = blockIdx.x;
    const int qn = hq * d, kn = hkv * d, vn = hkv * dv;
    const int pos = positions[t];
    int page = 0;
    if (has_kv) {
        page = table[(size_t)seq_rows[token_seq[t]] * table_stride + pos / page_size];
        if (!page_in_pool(page, num_pages, error, SE_CODE_BAD_PAGE_QK_PREP)) has_kv = 0;
    }
    float temp = 1.f;
    if (temp_coef != 0.f && temp_every > 0) temp = 1.f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.f);
    const T* row = proj + (size_t)t * pitch;
    float inv_q = 1.f, inv_k = 1.f;
    if (q_w != nullptr) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < qn; i += blockDim.x) { const float v = to_float(row[i]); ss += v * v; }
        inv_q = 1.0f / sqrtf(block_sum(ss, scratch) / (float)qn + eps);
    }
    if (k_w != nullptr && has_kv) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < kn; i += blockDim.x) { const float v = to_float(row[qn + i]); ss += v * v; }
        inv_k = 1.0f / sqrtf(block_sum(ss, scratch) / (float)kn + eps);
    }
    const int half = rotary_dim / 2;
    // element i of a projection part (norm weights w, inverse root mean square inv), normed and rotated
    auto prepared = [&](const T* part, const T* w, float inv, int i) {
        float v = to_float(part[i]) * inv;
        if (w != nullptr) v *= to_float(w[i]);
        const int c = i % d;
        if (c >= rotary_dim) return v;
        const int j = c < half ? i + half : i - half;
        float u = to_float(part[j]) * inv;
        if (w != nullptr) u *= to_float(w[j]);
        float sn, cs;
        sincosf((float)pos * inv_freq[c < half ? c : c - half], &sn, &cs);
        return c < half ? v * cs - u * sn : v * cs + u * sn;
    };
    for (int i = threadIdx.x; i < qn; i += blockDim.x)
        q_out[(size_t)t * qn + i] = from_float<T>(prepared(row, q_w, inv_q, i) * temp);
    if (!has_kv) return;
    const size_t page_elems = (size_t)hkv * page_size * (d + dv);
    T* kbase = cache + (size_t)page * page_elems + (size_t)(pos % page_size) * d;
    T* vbase = cache + (size_t)page * page_elems + (size_t)hkv * page_size * d + (size_t)(pos % page_size) * dv;
    for (int i = threadIdx.x; i < kn; i += blockDim.x) {
        const int h = i / d, c = i - h * d;
        kbase[(size_t)h * page_size * d + c] = from_float<T>(prepared(row + qn, k_w, inv_k, i));
    }
    const float mix = v_first != nullptr ? v_mix[0] : 0.f;
    for (int i = threadIdx.x; i < vn; i += blockDim.x) {
        const int h = i / dv, c = i - h * dv;
        T v = row[qn + kn + i];
        if (v_first != nullptr)
            v = from_float<T>((1.f - mix) * to_float(v) + mix * to_float(v_first[(size_t)t * v_first_pitch + i]));
        vbase[(size_t)h * page_size * dv + c] = v;
    }
}

}  // namespace se

extern "C" int se_qk_prep_general(const void* proj, int pitch, const void* q_w, const void* k_w, const float* inv_freq,
                                  int rotary_dim, const void* v_first, int v_first_pitch, const float* v_mix,
                                  const int* positions,
                                  const int* token_seq, const int* seq_rows, const int* table, int table_stride,
                                  void* cache, void* q_out, int tokens, int hq, int hkv, int d, int dv, float eps,
                                  float temp_coef, int temp_every, int page_size, int has_kv, int num_pages, int* error,
                                  int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (hq <= 0 || d <= 0 || (has_kv && (hkv <= 0 || dv <= 0 || page_size <= 0))) return SE_ERR_ARGUMENT;
    if (pitch < hq * d + (has_kv ? hkv * (d + dv) : 0)) return SE_ERR_ARGUMENT;
    if (rotary_dim < 0 || rotary_dim > d || (rotary_dim & 1) || (rotary_dim > 0 && inv_freq == nullptr)) return SE_ERR_ARGUMENT;
    if (v_first != nullptr && (v_mix == nullptr || !has_kv || v_first_pitch < hkv * dv)) return SE_ERR_ARGUMENT;
    SE_DISPATCH_DTYPE(dtype, T, {
        cudaError_t e = SE_LAUNCH_DEPENDENT("qk", se::qk_prep_general_kernel<T>, dim3(tokens), dim3(256), 0, stream,
                                             (const T*)proj, pitch, (const T*)q_w, (const T*)k_w, inv_freq, rotary_dim, (const T*)v_first,
                                             v_first_pitch, v_mix, positions, token_seq, seq_rows,
                                             table, table_stride, (T*)cache, (T*)q_out, hq, hkv, d, dv, eps, temp_coef, temp_every,
                                             page_size, has_kv, num_pages, error);
        if (e != cudaSuccess) return (int)e;
    });
    SE_LAUNCH_CHECK();
}
