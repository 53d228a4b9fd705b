// Element arithmetic of the gated activations and of RMSNorm, shared by the stand-alone kernels and by the quantizer's
// fused prologue, so that "activation, then quantize" and the fused kernel produce the same bits.
//
// Formulas of the reference (all in fp32, result rounded to the tensor's type):
//   SwiGLU  out = (a / (1 + exp(-a))) * b * p        primus_turbo/triton/activation/swiglu_kernel.py:51-57
//   GeGLU   out = (0.5 * a * (1 + erf(a / sqrt 2))) * b * p   geglu_kernel.py:53, triton/utils/gelu.py:21-25
//   RMSNorm y = x * rstd * g, rstd = rsqrt(mean(x^2) + eps), g = gamma (or 1 + gamma)   normalization/rmsnorm_kernel.py:68-75
// with a = first half of the row ("up" in the reference's kernels), b = second half, p = the row's probability.
#pragma once
#include <cuda_runtime.h>

namespace ptb {

enum { PT_ACT_SILU = 0, PT_ACT_GELU = 1 };

template <int ACT> __device__ __forceinline__ float act_value(float a) {
    if constexpr (ACT == PT_ACT_SILU) return __fdividef(a, 1.0f + __expf(-a));
    else return 0.5f * a * (1.0f + erff(a * 0.7071067811f));
}
// d act(a) / d a
template <int ACT> __device__ __forceinline__ float act_grad(float a) {
    if constexpr (ACT == PT_ACT_SILU) {
        const float s = __fdividef(1.0f, 1.0f + __expf(-a));
        return s * (1.0f + a * (1.0f - s));
    } else {
        return 0.3989422803f * a * __expf(-(0.7071067811f * a) * (0.7071067811f * a)) + 0.5f * erff(0.7071067811f * a) + 0.5f;
    }
}
template <int ACT> __device__ __forceinline__ float glu_value(float a, float b, float p) { return act_value<ACT>(a) * b * p; }

__device__ __forceinline__ float rmsnorm_value(float x, float rstd, float g) { return x * rstd * g; }

}  // namespace ptb
