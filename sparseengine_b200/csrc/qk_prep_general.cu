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
// Options: `bias` (32-bit, [q | k | v] like the projection row) is added to the projection before
// anything else; `per_head` norms every head by its own root mean square, with weights of d elements
// shared by the heads, instead of the whole projection with a weight per column.
//
// Everything is computed in 32-bit and rounded once.  The norm weights are
// optional.  The projection row is [q: hq*d | k: hkv*d | v: hkv*dv] (`has_kv`) or [q] alone.
//
// Cache layout of one cache layer: per page the keys [kv head][slot in page][d], then the values
// [kv head][slot in page][dv]; with dv = d this is the layout of the other attention kernels.
#include "common.cuh"

namespace se {

constexpr int kMaxHalf = 128;       // half of the largest rotated width (head sizes up to 256)

template <typename T>
__global__ void __launch_bounds__(256)
qk_prep_general_kernel(const T* proj, int pitch, const T* __restrict__ q_w, const T* __restrict__ k_w,
                       const float* __restrict__ inv_freq, int rotary_dim, const T* v_first, int v_first_pitch,
                       const float* __restrict__ v_mix,
                       const int* __restrict__ positions, const int* __restrict__ token_seq,
                       const int* __restrict__ seq_rows, const int* __restrict__ table, int table_stride,
                       T* __restrict__ cache, T* __restrict__ q_out, int hq, int hkv, int d, int dv, float eps,
                       float temp_coef, int temp_every, int page_size, int has_kv, int num_pages, int* __restrict__ error,
                       const float* __restrict__ bias, int per_head) {
    extern __shared__ float inv_head[];      // per_head: the inverse root mean square of every q head, then every k head
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
    const int half = rotary_dim / 2;
    const T* vf = v_first != nullptr ? v_first + (size_t)t * v_first_pitch : nullptr;
    // Eight elements at a time where sizes and addresses allow it.
    const bool vec = (d & 7) == 0 && (half & 7) == 0 && (dv & 7) == 0 && (pitch & 7) == 0 && aligned8(proj) && aligned8(q_out) &&
                     (bias == nullptr || aligned8(bias)) &&
                     (q_w == nullptr || aligned8(q_w)) && (k_w == nullptr || aligned8(k_w)) && (cache == nullptr || aligned8(cache)) &&
                     (vf == nullptr || ((v_first_pitch & 7) == 0 && aligned8(v_first)));
    // element i of a part of the projection row (its bias starts at bias + b0)
    auto raw = [&](const T* part, int b0, int i) { return to_float(part[i]) + (bias != nullptr ? bias[b0 + i] : 0.f); };
    auto raw8 = [&](const T* part, int b0, int i, float* v) {
        load8(part + i, v);
        if (bias != nullptr) {
            float bb[8];
            load8(bias + b0 + i, bb);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] += bb[j];
        }
    };
    auto sum_squares = [&](const T* part, int b0, int n) {
        float ss = 0.f;
        if (vec) {
            for (int i = threadIdx.x * 8; i < n; i += blockDim.x * 8) {
                float v[8];
                raw8(part, b0, i, v);
#pragma unroll
                for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
            }
        } else {
            for (int i = threadIdx.x; i < n; i += blockDim.x) { const float v = raw(part, b0, i); ss += v * v; }
        }
        return block_sum(ss, scratch);
    };
    float inv_q = 1.f, inv_k = 1.f;
    if (per_head) {
        // a warp per head: q heads (if normed), then k heads
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
        const int heads = hq + (has_kv ? hkv : 0);
        for (int h = warp; h < heads; h += warps) {
            const bool is_q = h < hq;
            float ss = 0.f;
            if ((is_q ? q_w : k_w) != nullptr) {
                const T* part = is_q ? row + (size_t)h * d : row + qn + (size_t)(h - hq) * d;
                const int b0 = is_q ? h * d : qn + (h - hq) * d;
                for (int i = lane; i < d; i += 32) { const float v = raw(part, b0, i); ss += v * v; }
                ss = warp_sum(ss);
            }
            if (lane == 0) inv_head[h] = (is_q ? q_w : k_w) != nullptr ? 1.0f / sqrtf(ss / (float)d + eps) : 1.f;
        }
        __syncthreads();
    } else {
        if (q_w != nullptr) inv_q = 1.0f / sqrtf(sum_squares(row, 0, qn) / (float)qn + eps);
        if (k_w != nullptr && has_kv) inv_k = 1.0f / sqrtf(sum_squares(row + qn, qn, kn) / (float)kn + eps);
    }
    // cos and sin of the token's angles, once for all heads
    __shared__ float cs_t[kMaxHalf], sn_t[kMaxHalf];
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &sn_t[i], &cs_t[i]);
    __syncthreads();
    T* kbase = nullptr;
    T* vbase = nullptr;
    if (has_kv) {
        const size_t page_elems = (size_t)hkv * page_size * (d + dv);
        kbase = cache + (size_t)page * page_elems + (size_t)(pos % page_size) * d;
        vbase = cache + (size_t)page * page_elems + (size_t)hkv * page_size * d + (size_t)(pos % page_size) * dv;
    }
    const float mix = v_first != nullptr ? v_mix[0] : 0.f;
    T* qdst = q_out + (size_t)t * qn;

    // The 8-wide path: a work item is a pair of 8-element chunks that rotate into one another (columns c
    // and c + half of a head), or one chunk that passes.
    if (vec) {
        const int pair_items = half / 8, items = d / 8 - pair_items;          // per head
        auto normed8 = [&](const T* part, int b0, const T* w, float inv, int i, int wi, float* v) {
            raw8(part, b0, i, v);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] *= inv;
            if (w != nullptr) {
                float ww[8];
                load8(w + wi, ww);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] *= ww[j];
            }
        };
        // heads of the queries, then (with keys) heads of the keys
        const int heads = hq + (has_kv ? hkv : 0);
        for (int it = threadIdx.x; it < heads * items; it += blockDim.x) {
            const int h = it / items, k = it - h * items;
            const bool is_q = h < hq;
            const int hh = is_q ? h : h - hq;
            const T* part = is_q ? row : row + qn;
            const int b0 = is_q ? 0 : qn;
            const T* w = is_q ? q_w : k_w;
            const float inv = per_head ? inv_head[h] : (is_q ? inv_q : inv_k), mul = is_q ? temp : 1.f;
            const int w0 = per_head ? 0 : hh * d;        // where the head's weights start
            T* dst = is_q ? qdst + (size_t)hh * d : kbase + (size_t)hh * page_size * d;
            float a[8];
            if (k < pair_items) {
                const int c = k * 8;
                float b[8], ra[8], rb[8];
                normed8(part, b0, w, inv, hh * d + c, w0 + c, a);
                normed8(part, b0, w, inv, hh * d + c + half, w0 + c + half, b);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float cs = cs_t[c + j], sn = sn_t[c + j];
                    ra[j] = (a[j] * cs - b[j] * sn) * mul;
                    rb[j] = (b[j] * cs + a[j] * sn) * mul;
                }
                store8(dst + c, ra);
                store8(dst + c + half, rb);
            } else {
                const int c = rotary_dim + (k - pair_items) * 8;
                normed8(part, b0, w, inv, hh * d + c, w0 + c, a);
#pragma unroll
                for (int j = 0; j < 8; ++j) a[j] *= mul;
                store8(dst + c, a);
            }
        }
        if (!has_kv) return;
        for (int i = threadIdx.x * 8; i < vn; i += blockDim.x * 8) {
            const int h = i / dv, c = i - h * dv;
            if (vf == nullptr && bias == nullptr) {
                *reinterpret_cast<uint4*>(vbase + (size_t)h * page_size * dv + c) = *reinterpret_cast<const uint4*>(row + qn + kn + i);
                if (sizeof(T) == 4)
                    *reinterpret_cast<uint4*>(vbase + (size_t)h * page_size * dv + c + 4) = *reinterpret_cast<const uint4*>(row + qn + kn + i + 4);
            } else {
                float a[8], f[8];
                raw8(row + qn + kn, qn + kn, i, a);
                if (vf != nullptr) {
                    load8(vf + i, f);
#pragma unroll
                    for (int j = 0; j < 8; ++j) a[j] = (1.f - mix) * a[j] + mix * f[j];
                }
                store8(vbase + (size_t)h * page_size * dv + c, a);
            }
        }
        return;
    }

    // element i of a projection part (norm weights w, inverse root mean square inv), normed and rotated
    auto prepared = [&](const T* part, int b0, const T* w, float inv_whole, int h0, int i) {
        const int c = i % d;
        const float inv = per_head ? inv_head[h0 + i / d] : inv_whole;
        float v = raw(part, b0, i) * inv;
        if (w != nullptr) v *= to_float(w[per_head ? c : i]);
        if (c >= rotary_dim) return v;
        const int j = c < half ? i + half : i - half;
        float u = raw(part, b0, j) * inv;
        if (w != nullptr) u *= to_float(w[per_head ? j % d : j]);
        const float sn = sn_t[c < half ? c : c - half], cs = cs_t[c < half ? c : c - half];
        return c < half ? v * cs - u * sn : v * cs + u * sn;
    };
    for (int i = threadIdx.x; i < qn; i += blockDim.x)
        qdst[i] = from_float<T>(prepared(row, 0, q_w, inv_q, 0, i) * temp);
    if (!has_kv) return;
    for (int i = threadIdx.x; i < kn; i += blockDim.x) {
        const int h = i / d, c = i - h * d;
        kbase[(size_t)h * page_size * d + c] = from_float<T>(prepared(row + qn, qn, k_w, inv_k, hq, i));
    }
    for (int i = threadIdx.x; i < vn; i += blockDim.x) {
        const int h = i / dv, c = i - h * dv;
        float v = raw(row + qn + kn, qn + kn, i);
        if (vf != nullptr) v = (1.f - mix) * v + mix * to_float(vf[i]);
        vbase[(size_t)h * page_size * dv + c] = from_float<T>(v);
    }
}

}  // namespace se

extern "C" int se_qk_prep_general(const void* proj, int pitch, const void* q_w, const void* k_w, const float* inv_freq,
                                  int rotary_dim, const void* v_first, int v_first_pitch, const float* v_mix,
                                  const int* positions,
                                  const int* token_seq, const int* seq_rows, const int* table, int table_stride,
                                  void* cache, void* q_out, int tokens, int hq, int hkv, int d, int dv, float eps,
                                  float temp_coef, int temp_every, int page_size, int has_kv, int num_pages, int* error,
                                  const float* bias, int per_head, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (hq <= 0 || d <= 0 || (has_kv && (hkv <= 0 || dv <= 0 || page_size <= 0))) return SE_ERR_ARGUMENT;
    if (pitch < hq * d + (has_kv ? hkv * (d + dv) : 0)) return SE_ERR_ARGUMENT;
    if (rotary_dim < 0 || rotary_dim > d || (rotary_dim & 1) || (rotary_dim > 0 && inv_freq == nullptr)) return SE_ERR_ARGUMENT;
    if (rotary_dim > 2 * se::kMaxHalf) return SE_ERR_UNSUPPORTED;
    if (v_first != nullptr && (v_mix == nullptr || !has_kv || v_first_pitch < hkv * dv)) return SE_ERR_ARGUMENT;
    const size_t smem = per_head ? (size_t)(hq + (has_kv ? hkv : 0)) * sizeof(float) : 0;
    if (smem > 40 * 1024) return SE_ERR_UNSUPPORTED;
    SE_DISPATCH_DTYPE(dtype, T, {
        cudaError_t e = SE_LAUNCH_DEPENDENT("qk", se::qk_prep_general_kernel<T>, dim3(tokens), dim3(256), smem, stream,
                                             (const T*)proj, pitch, (const T*)q_w, (const T*)k_w, inv_freq, rotary_dim, (const T*)v_first,
                                             v_first_pitch, v_mix, positions, token_seq, seq_rows,
                                             table, table_stride, (T*)cache, (T*)q_out, hq, hkv, d, dv, eps, temp_coef, temp_every,
                                             page_size, has_kv, num_pages, error, bias, per_head);
        if (e != cudaSuccess) return (int)e;
    });
    SE_LAUNCH_CHECK();
}
