// One row of RMSNorm (optionally with the residual add in front) with the reference kernels' arithmetic and
// summation order (csrc/layernorm_kernels.cu:10-36, 76-107; csrc/reduction_utils.cuh:61-86), as a device function:
// used by the norm kernels, by the fused call in front of the MoE block and by the all-reduce that ends in the
// next layer's add + norm.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "ptx.cuh"

namespace moe_b200 {

constexpr int kNormThreads = 128;  // x 8 elements = the reference's 1024 threads

union Bf16x8 {
  uint4 u;
  __nv_bfloat16 h[8];
};

// Sum over the reference's min(H, 1024) per-thread partials, p[i] being the partial of reference thread 8*t + i.
// Called by the kNormThreads first threads of the CTA (whole warps); `red` holds 32 floats. The result is valid
// in every calling thread after the CTA-wide barrier inside.
template <int kCtaThreads>
__device__ __forceinline__ float reference_block_sum(const float (&p_in)[8], int t, float* red, float* total_slot) {
  float c = 0.f;
  if (t < kNormThreads) {
    float p[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) p[i] = p_in[i];
#pragma unroll
    for (int i = 0; i < 8; ++i) p[i] += __shfl_xor_sync(0xffffffffu, p[i], 2);  // reference lane ^ 16
#pragma unroll
    for (int i = 0; i < 8; ++i) p[i] += __shfl_xor_sync(0xffffffffu, p[i], 1);  // reference lane ^ 8
    const float a0 = p[0] + p[4], a1 = p[1] + p[5], a2 = p[2] + p[6], a3 = p[3] + p[7];  // ^ 4
    const float b0 = a0 + a2, b1 = a1 + a3;                                              // ^ 2
    c = b0 + b1;                                                                         // ^ 1
    if ((t & 3) == 0) red[t >> 2] = c;  // reference warp t / 4
  }
  __syncthreads();
  if (t < 32) {
    float v = red[t];  // warps the reference block does not have hold 0 (their partials are 0)
#pragma unroll
    for (int mask = 16; mask > 0; mask >>= 1) v += __shfl_xor_sync(0xffffffffu, v, mask);
    if (t == 0) *total_slot = v;
  }
  __syncthreads();
  return *total_slot;
}

// residual <- bf16(input + residual) (or stays input when kAdd is false), out <- bf16(bf16(r * rsqrt(mean(r^2) + eps)) * w).
// `load_in(c)` returns 8 consecutive input values (a row in memory, or a row reduced over the ranks on the fly).
// The normalised row is also left in x_row (shared memory). Nothing is written to global memory before every
// thread has read its inputs; with kClusterSync that holds across the CTAs of a cluster working on the same row
// (each forms the row for itself, `write_global` picks the one that stores it).
template <bool kAdd, int kCtaThreads, bool kClusterSync, typename LoadIn>
__device__ __forceinline__ void rms_norm_row(LoadIn load_in, __nv_bfloat16* res_row,
                                             const __nv_bfloat16* __restrict__ weight, __nv_bfloat16* out_row,
                                             int H, float eps, __nv_bfloat16* x_row, float* red, float* total_slot,
                                             bool write_global) {
  const int t = threadIdx.x;
  float p[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) p[i] = 0.f;
  if (t < kNormThreads) {
    for (int c = 8 * t; c < H; c += 1024) {
      Bf16x8 a, r;
      a.u = load_in(c);  // 8 consecutive bf16 of the input row starting at column c
      if (kAdd) r.u = *reinterpret_cast<const uint4*>(res_row + c);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float x = kAdd ? __bfloat162float(a.h[i]) + __bfloat162float(r.h[i]) : __bfloat162float(a.h[i]);
        p[i] = fmaf(x, x, p[i]);
        a.h[i] = __float2bfloat16_rn(x);  // what the second pass of the reference reads back
      }
      *reinterpret_cast<uint4*>(x_row + c) = a.u;
    }
  }
  const float total = reference_block_sum<kCtaThreads>(p, t, red, total_slot);
  if (kClusterSync) cluster_sync_all();
  const float s = rsqrtf(total / H + eps);
  for (int c = 8 * t; c < H; c += 8 * kCtaThreads) {
    Bf16x8 xv, wv;
    xv.u = *reinterpret_cast<const uint4*>(x_row + c);
    wv.u = *reinterpret_cast<const uint4*>(weight + c);
    if (kAdd && write_global) *reinterpret_cast<uint4*>(res_row + c) = xv.u;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const __nv_bfloat16 scaled = __float2bfloat16_rn(__bfloat162float(xv.h[i]) * s);
      xv.h[i] = __float2bfloat16_rn(__bfloat162float(scaled) * __bfloat162float(wv.h[i]));
    }
    if (write_global) *reinterpret_cast<uint4*>(out_row + c) = xv.u;
    *reinterpret_cast<uint4*>(x_row + c) = xv.u;
  }
}

}  // namespace moe_b200
