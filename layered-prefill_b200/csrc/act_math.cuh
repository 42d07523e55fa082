// Gated activations with the reference's rounding points.
//
// silu_and_mul (csrc/activation_kernels.cu:9-25): silu is computed in fp32 from the bf16 gate,
// rounded to bf16, then multiplied with the bf16 up value and rounded to bf16 again.
// swigluoai_and_mul (csrc/activation_kernels.cu:27-45): clamp, sigmoid and product in fp32,
// one rounding to bf16 at the end.
// expf and the division are the full-precision ones (the library is built without fast-math,
// as the reference is: setup.py:46-47).
#pragma once

#include <cuda_bf16.h>

namespace moe_b200 {

__device__ __forceinline__ __nv_bfloat16 silu_mul_bf16(__nv_bfloat16 gate, __nv_bfloat16 up) {
  const float x = __bfloat162float(gate);
  const __nv_bfloat16 s = __float2bfloat16_rn(x / (1.0f + expf(-x)));
  return __float2bfloat16_rn(__bfloat162float(s) * __bfloat162float(up));
}

// Same roundings, with the SFU exponential and reciprocal (2 ulp in fp32 before the bf16 rounding).
__device__ __forceinline__ __nv_bfloat16 silu_mul_bf16_fast(__nv_bfloat16 gate, __nv_bfloat16 up) {
  const float x = __bfloat162float(gate);
  const __nv_bfloat16 s = __float2bfloat16_rn(__fdividef(x, 1.0f + __expf(-x)));
  return __float2bfloat16_rn(__bfloat162float(s) * __bfloat162float(up));
}

__device__ __forceinline__ __nv_bfloat16 swigluoai_bf16(__nv_bfloat16 gate, __nv_bfloat16 up, float alpha,
                                                        float limit) {
  const float g = __bfloat162float(gate);
  const float cg = g > limit ? limit : g;
  const float u = __bfloat162float(up);
  const float cu = u > limit ? limit : (u < -limit ? -limit : u);
  const float sig = 1.0f / (1.0f + expf(-cg * alpha));
  const float glu = cg * sig;
  return __float2bfloat16_rn((cu + 1.0f) * glu);
}

}  // namespace moe_b200
