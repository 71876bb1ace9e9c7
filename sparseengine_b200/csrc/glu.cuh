// The gated activations an expert's first product ends in.  `gate` and `up` arrive rounded to the
// activation type T; the result is 32-bit and the caller rounds it once more as it stores it.
//   kind 0  silu(gate) * up, silu rounded to T before the product (the rounding points of the
//           bfloat16 pipeline the other kernels keep)
//   kind 1  g = min(gate, limit), u = clamp(up, -limit, limit): g * sigmoid(alpha * g) * (u + 1)
#pragma once
#include "common.cuh"

#define SE_GLU_SILU 0
#define SE_GLU_CLAMPED 1

namespace se {

template <typename T>
__device__ __forceinline__ float glu_value(float gate, float up, int kind, float limit, float alpha) {
    if (kind == SE_GLU_CLAMPED) {
        const float g = fminf(gate, limit);
        const float u = fminf(fmaxf(up, -limit), limit);
        return g / (1.f + expf(-alpha * g)) * (u + 1.f);
    }
    return round_act<T>(gate / (1.f + expf(-gate))) * up;
}

}  // namespace se
