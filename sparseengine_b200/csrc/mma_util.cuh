// Warp-level tensor-core and asynchronous-copy helpers shared by the attention kernels.
#pragma once
#include "common.cuh"

namespace se {
namespace mma {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;     // 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of 16-byte chunk `c` of row `r` in a [rows][D] bf16 tile whose chunks are
// XOR-swizzled within each row (conflict-free ldmatrix; rows of fewer than eight chunks swizzle
// within what they have).
template <int D> __device__ __forceinline__ uint32_t tile_off(int r, int c) {
    constexpr int kChunks = D / 8;
    constexpr int kMask = kChunks < 8 ? kChunks - 1 : 7;
    static_assert((kChunks & (kChunks - 1)) == 0, "rows of a power-of-two number of chunks");
    return (uint32_t)((r * kChunks + (c ^ (r & kMask))) * 16);
}

// Options of the softmax that the tensor-core attention kernels share with the plain one.
//   cap_in, cap_out : scale / c and c / scale for scores capped by c tanh(s * scale / c); 0, 0: no cap.
//                     The kernels keep raw scores q.k and fold `scale` into their exponentials, so the
//                     capped score goes back to raw units: s <- cap_out * tanh(s * cap_in).
//   sink            : a key of score 0 without a value joins the softmax's denominator.
//   gate, gate_pitch: the output is multiplied element by element with sigmoid(gate[t][h * dv + i])
//                     (rows gate_pitch elements apart); nullptr: no gate.
//   sink_logits     : with `sink`, a learned logit per query head in the place of the sink's 0 (unscaled); nullptr: 0.
//   keep_first      : with a window, keys 0 .. keep_first-1 stay visible beside the window's.
struct SoftmaxOptions {
    float cap_in, cap_out;
    int sink;
    const __nv_bfloat16* gate;
    int gate_pitch;
    const float* sink_logits;
    int keep_first;
};
// the sink's logit of a head, times log2(e)
__device__ __forceinline__ float sink_log2(const SoftmaxOptions& opt, int head) {
    return opt.sink_logits != nullptr ? opt.sink_logits[head] * 1.4426950408889634f : 0.f;
}

// cap_out * tanh(s * cap_in) with tanh(x) = 1 - 2 / (exp(2x) + 1); beyond |x| = 15 tanh is 1 in 32-bit.
__device__ __forceinline__ float capped_score(float s, float cap_in, float cap_out) {
    const float x = fminf(fmaxf(s * cap_in, -15.f), 15.f);
    return cap_out * (1.f - __fdividef(2.f, __expf(2.f * x) + 1.f));
}
// Two 32-bit products or fused multiply-adds in one instruction (sm_100: `mul.rn.f32x2`, `fma.rn.f32x2`).
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    unsigned long long d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)));
    return reinterpret_cast<float2&>(d);
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(reinterpret_cast<unsigned long long&>(a)),
        "l"(reinterpret_cast<unsigned long long&>(b)), "l"(reinterpret_cast<unsigned long long&>(c)));
    return reinterpret_cast<float2&>(d);
}
// The cap without the special-function unit, two scores at a time: with x = s * cap_in,
// cap_out * tanh(x) = s * P(x^2) since cap_in * cap_out = 1 and tanh(x) = x P(x^2).  WIDE = false: P of degree 4,
// fitted on |x| <= 0.5; WIDE = true: degree 7, on |x| <= 1 (relative error 1.0e-7 and 1.2e-7 when evaluated in
// 32-bit).  Scores of a model are mostly far inside its cap, and the softmax warps of the tensor-core prompt kernel
// have no time to spare: their exponentials alone keep the special-function unit as busy as the matrix products keep
// the tensor cores.
template <bool WIDE>
__device__ __forceinline__ float2 capped_pair_small(float2 s, float cap_in) {
    const float2 x = mul2(s, make_float2(cap_in, cap_in));
    const float2 t = mul2(x, x);
    float2 p;
#define SE_C2(v) make_float2(v, v)
    if (WIDE) {
        p = fma2(SE_C2(-0.0003548834065441042f), t, SE_C2(0.0022876455914229155f));
        p = fma2(p, t, SE_C2(-0.007924946025013924f));
        p = fma2(p, t, SE_C2(0.021469980478286743f));
        p = fma2(p, t, SE_C2(-0.053872738033533096f));
        p = fma2(p, t, SE_C2(0.13332191109657288f));
        p = fma2(p, t, SE_C2(-0.3333328068256378f));
    } else {
        p = fma2(SE_C2(0.01723547652363777f), t, SE_C2(-0.0530422069132328f));
        p = fma2(p, t, SE_C2(0.13325822353363037f));
        p = fma2(p, t, SE_C2(-0.3333314061164856f));
    }
    p = fma2(p, t, SE_C2(1.f));
#undef SE_C2
    return mul2(s, p);
}
// N scores of a thread (N even), given the largest |s * cap_in| among them (or among a group of threads that
// decides as one): the short polynomial, the long one, or the exact form for all.
template <int N>
__device__ __forceinline__ void cap_scores_by(float* s, float xmax, float cap_in, float cap_out) {
    if (xmax <= 0.5f) {
#pragma unroll
        for (int i = 0; i < N; i += 2) {
            const float2 r = capped_pair_small<false>(make_float2(s[i], s[i + 1]), cap_in);
            s[i] = r.x; s[i + 1] = r.y;
        }
    } else if (xmax <= 1.f) {
#pragma unroll
        for (int i = 0; i < N; i += 2) {
            const float2 r = capped_pair_small<true>(make_float2(s[i], s[i + 1]), cap_in);
            s[i] = r.x; s[i + 1] = r.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) s[i] = capped_score(s[i], cap_in, cap_out);
    }
}
template <int N>
__device__ __forceinline__ void cap_scores(float* s, float cap_in, float cap_out) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < N; ++i) amax = fmaxf(amax, fabsf(s[i]));
    cap_scores_by<N>(s, amax * cap_in, cap_in, cap_out);
}
__device__ __forceinline__ float gated_by(float o, float g) {
    return __fdividef(o, 1.f + __expf(-g));
}
__device__ __forceinline__ float gated(float o, const __nv_bfloat16* gate) {
    return gated_by(o, __bfloat162float(*gate));
}
// Whether the gate's rows can be read 16 bytes (8 elements) or 4 bytes (2 elements) at a time, for head
// sizes that are multiples of 8.
__device__ __forceinline__ bool gate_rows_aligned(const SoftmaxOptions& opt, int bytes) {
    return (reinterpret_cast<uintptr_t>(opt.gate) & (bytes - 1)) == 0 && (opt.gate_pitch * 2) % bytes == 0;
}

}  // namespace mma
}  // namespace se
