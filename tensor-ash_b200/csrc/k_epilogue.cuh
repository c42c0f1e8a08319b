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

// Compile-time activation: the tile epilogues dispatch on the activation ONCE per tile and run a
// loop specialised for it.  With the runtime switch above inlined at every element of an unrolled
// epilogue, the expf / tanhf bodies of the untaken cases still sit in the instruction stream; on
// a 128 x 256 tile the loop then ran from instruction memory at ~3 us per 32-column chunk (25 us
// per tile) against 0.4 us specialised.
template <uint32_t ACT>
__device__ __forceinline__ float epi_activate_t(float x) {
  if constexpr (ACT == 1) {
    return fmaxf(x, 0.0f);
  } else if constexpr (ACT == 2) {
    return x / (1.0f + expf(-x));
  } else if constexpr (ACT == 3) {
    const float k0 = 0.7978845608028654f;
    return 0.5f * x * (1.0f + tanhf(k0 * fmaf(0.044715f * x * x, x, x)));
  } else {
    return x;
  }
}

template <uint32_t ACT>
__device__ __forceinline__ float epi_apply_t(float v, bool has_bias, float bias_v, uint32_t binary, float d_v,
                                             float beta) {
  if (has_bias) v += bias_v;
  v = epi_activate_t<ACT>(v);
  const float added = fmaf(beta, d_v, v), multiplied = v * d_v;   // selects, not branches
  return binary == 1 ? added : (binary == 2 ? multiplied : v);
}

template <uint32_t ACT>
struct ActTag {
  static constexpr uint32_t value = ACT;
};

// Calls f(ActTag<act>{}) for the runtime activation id (0..3).
template <typename F>
__device__ __forceinline__ void epi_dispatch_act(uint32_t act, F &&f) {
  switch (act) {
    case 1: f(ActTag<1>{}); break;
    case 2: f(ActTag<2>{}); break;
    case 3: f(ActTag<3>{}); break;
    default: f(ActTag<0>{}); break;
  }
}

}  // namespace ta
