// Stand-alone element-wise ops of the MoE block. Inside the fused path the activation lives
// in the gate_up GEMM epilogue; these kernels exist for the op-level boundary (the reference
// exports silu_and_mul / swigluoai_and_mul, csrc/ops.cpp:29-36) and for the k-slot sum
// (moe_sum, nanovllm/layers/for_moe/moe_easy_kernel.py:26-31). All are HBM-bound: 16-byte
// accesses, grid sized from the element count.
#include "act_math.cuh"
#include "launch.cuh"
#include "moe_b200_internal.cuh"

namespace moe_b200 {

namespace {

union Pack8 {
  uint4 u;
  __nv_bfloat16 h[8];
};

// out[r, c] = act(in[r, c], in[r, d + c]); rounding points as in csrc/activation_kernels.cu:9-25.
__global__ void silu_and_mul_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ in,
                                    long long rows, int d) {
  const int vec_per_row = d / 8;
  const long long total = rows * vec_per_row;
  for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < total;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = v / vec_per_row;
    const int c = static_cast<int>(v % vec_per_row) * 8;
    Pack8 g, u, o;
    g.u = *reinterpret_cast<const uint4*>(in + r * 2 * d + c);
    u.u = *reinterpret_cast<const uint4*>(in + r * 2 * d + d + c);
#pragma unroll
    for (int j = 0; j < 8; ++j) o.h[j] = silu_mul_bf16(g.h[j], u.h[j]);
    *reinterpret_cast<uint4*>(out + r * d + c) = o.u;
  }
}

__global__ void silu_and_mul_scalar_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ in,
                                           long long rows, int d) {
  const long long total = rows * d;
  for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < total;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = v / d;
    const int c = static_cast<int>(v % d);
    out[v] = silu_mul_bf16(in[r * 2 * d + c], in[r * 2 * d + d + c]);
  }
}

// gpt-oss gate: gate = in[r, 2c], up = in[r, 2c+1] (csrc/activation_kernels.cu:27-64).
__global__ void swigluoai_and_mul_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ in,
                                         long long rows, int d, float alpha, float limit) {
  const long long total = rows * d;
  for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < total;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    const __nv_bfloat162 p = *reinterpret_cast<const __nv_bfloat162*>(in + 2 * v);
    out[v] = swigluoai_bf16(p.x, p.y, alpha, limit);
  }
}

// out[t, :] = bf16(sum_j float(in[t, j, :])), j ascending.
__global__ void moe_sum_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, long long T,
                               int k, int H) {
  grid_dependency_launch();
  grid_dependency_wait();
  const int vec_per_row = H / 8;
  const long long total = T * vec_per_row;
  for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < total;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = v / vec_per_row;
    const int c = static_cast<int>(v % vec_per_row) * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; ++j) {
      Pack8 p;
      p.u = *reinterpret_cast<const uint4*>(in + (t * k + j) * H + c);
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] += __bfloat162float(p.h[q]);
    }
    Pack8 o;
#pragma unroll
    for (int q = 0; q < 8; ++q) o.h[q] = __float2bfloat16_rn(acc[q]);
    *reinterpret_cast<uint4*>(out + t * H + c) = o.u;
  }
}

int grid_for(long long work_items, int threads) {
  long long blocks = (work_items + threads - 1) / threads;
  const long long cap = static_cast<long long>(device_sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace

int launch_silu_and_mul(__nv_bfloat16* out, const __nv_bfloat16* in, int rows, int d, cudaStream_t stream) {
  if (rows < 0 || d <= 0) return set_error(kStatusInvalidArgument, "silu_and_mul: bad shape");
  if (rows == 0) return kStatusOk;
  const bool vec = d % 8 == 0 && (reinterpret_cast<uintptr_t>(out) % 16 == 0) && (reinterpret_cast<uintptr_t>(in) % 16 == 0);
  if (vec)
    silu_and_mul_kernel<<<grid_for(static_cast<long long>(rows) * (d / 8), 256), 256, 0, stream>>>(out, in, rows, d);
  else
    silu_and_mul_scalar_kernel<<<grid_for(static_cast<long long>(rows) * d, 256), 256, 0, stream>>>(out, in, rows, d);
  count_launches(1);
  return check_launch("silu_and_mul");
}

int launch_swigluoai_and_mul(__nv_bfloat16* out, const __nv_bfloat16* in, int rows, int d, float alpha, float limit,
                             cudaStream_t stream) {
  if (rows < 0 || d <= 0) return set_error(kStatusInvalidArgument, "swigluoai_and_mul: bad shape");
  if (rows == 0) return kStatusOk;
  swigluoai_and_mul_kernel<<<grid_for(static_cast<long long>(rows) * d, 256), 256, 0, stream>>>(out, in, rows, d, alpha,
                                                                                                limit);
  count_launches(1);
  return check_launch("swigluoai_and_mul");
}

int launch_moe_sum(const __nv_bfloat16* in, __nv_bfloat16* out, int T, int k, int H, cudaStream_t stream) {
  if (T < 0 || k <= 0 || H <= 0 || H % 8 != 0) return set_error(kStatusInvalidArgument, "moe_sum: H must be a multiple of 8");
  if (T == 0) return kStatusOk;
  launch_pdl(moe_sum_kernel, dim3(grid_for(static_cast<long long>(T) * (H / 8), 256)), dim3(256), 0, stream, in, out,
             static_cast<long long>(T), k, H);
  count_launches(1);
  return check_launch("moe_sum");
}

}  // namespace moe_b200
