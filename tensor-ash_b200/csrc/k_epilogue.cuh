// Fused GEMM epilogue shared by every GEMM kernel in this library.
//
// Order and formulas follow the reference shader
// (shaders/matmul_epilogue_common.glsl:14-21, 30-39, 43-51):
//   v = alpha * acc (+ C_old)  ->  + bias[batch, col]  ->  act  ->  binary(D)
// with SiLU = x / (1 + exp(-x)), GELU = 0.5 x (1 + tanh(k0 * fma(0.044715 x^2, x, x))),
// AddScaled = fma(beta, D, v), Mul = v * D.  Full-precision expf/tanhf: the
// FP32 parity budget is 1e-5 relative, which the fast intrinsics do not meet.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace ta {

__device__ __forceinline__ float epi_activate(float x, uint32_t act) {
  switch (act) {
    case 1: return fmaxf(x, 0.0f);
    case 2: return x / (1.0f + expf(-x));
    case 3: {
      const float k0 = 0.7978845608028654f;
      return 0.5f * x * (1.0f + tanhf(k0 * fmaf(0.044715f * x * x, x, x)));
    }
    default: return x;
  }
}

// v already holds alpha*acc (+C_old).  bias_v / d_v are the loaded operands
// (ignored when the corresponding feature is off).
__device__ __forceinline__ float epi_apply(float v, bool has_bias, float bias_v, uint32_t act,
                                           uint32_t binary, float d_v, float beta) {
  if (has_bias) v += bias_v;
  v = epi_activate(v, act);
  if (binary == 1) v = fmaf(beta, d_v, v);
  else if (binary == 2) v *= d_v;
  return v;
}

}  // namespace ta
