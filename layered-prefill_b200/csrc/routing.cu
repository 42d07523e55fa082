// Router: softmax over all experts followed by k rounds of arg-max, one token row
// per group of lanes, everything in registers and warp shuffles.
//
// The arithmetic order is the one the reference's topkGatingSoftmax uses
// (csrc/moe_topk_softmax_kernels.cu:182-380), because topk_ids has to be bit-exact:
//   * a lane owns VPT experts, read as 16-byte groups that are THREADS_PER_ROW groups apart;
//   * max: sequential over the lane's values, then xor-butterfly from THREADS_PER_ROW/2 down to 1;
//   * e_i = expf(x_i - max) (libdevice expf, no fast-math), row sum = sequential add, same butterfly;
//   * p_i = e_i * (1.f / row_sum);
//   * arg-max: strict '>' inside a lane (lowest index wins), across lanes the larger value wins
//     and on equal values the smaller expert index; the winner is blanked with -10000.
// On top of that this kernel accepts bf16 logits directly (the reference upcasts with
// gating_output.float(), for_moe/fused_moe.py:414 -- the upcast is exact) and can fold in
// the renormalisation topk_weights / topk_weights.sum(-1) (for_moe/fused_moe.py:417-418).
#include "launch.cuh"
#include "moe_b200_internal.cuh"
#include "routing_core.cuh"

namespace moe_b200 {

namespace {

constexpr int kWarpsPerCta = 4;

template <int E, bool kBf16In>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
topk_softmax_pow2_kernel(const void* __restrict__ gating, float* __restrict__ topk_w, int* __restrict__ topk_ids,
                         int* __restrict__ token_expert_indices, int num_rows, int k, int renormalize) {
  grid_dependency_launch();
  grid_dependency_wait();
  using S = TopkShape<E>;
  constexpr int VPT = S::kVpt;
  constexpr int TPR = S::kThreadsPerRow;
  constexpr int ELTS = S::kEltsPerLdg;
  constexpr int LDGS = S::kVecsPerThread;

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  // Lanes past the last row keep running on a clamped row (their shuffles are still needed
  // by nobody, but a full-mask shuffle wants every lane present) and never store.
  const int raw_row = (blockIdx.x * kWarpsPerCta + warp) * S::kRowsPerWarp + lane / TPR;
  const bool row_ok = raw_row < num_rows;
  const int row = row_ok ? raw_row : num_rows - 1;
  const int g = lane % TPR;
  const int first_col = g * ELTS;

  float v[VPT];
#pragma unroll
  for (int ii = 0; ii < LDGS; ++ii) {
    const int col = first_col + ii * S::kColsPerGroupLdg;
    if constexpr (kBf16In) {
      const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(gating) + static_cast<size_t>(row) * E + col;
#pragma unroll
      for (int j = 0; j < ELTS; ++j) v[ii * ELTS + j] = __bfloat162float(src[j]);
    } else {
      const float* src = static_cast<const float*>(gating) + static_cast<size_t>(row) * E + col;
      if constexpr (ELTS == 4) {
        const float4 q = *reinterpret_cast<const float4*>(src);
        v[ii * 4 + 0] = q.x; v[ii * 4 + 1] = q.y; v[ii * 4 + 2] = q.z; v[ii * 4 + 3] = q.w;
      } else {
#pragma unroll
        for (int j = 0; j < ELTS; ++j) v[ii * ELTS + j] = src[j];
      }
    }
  }

  topk_softmax_row<E>(v, lane, row_ok, row, num_rows, k, renormalize, topk_w, topk_ids, token_expert_indices);
}

// Any expert count (not a power of two, or above 256): one warp per row, probabilities
// staged in shared memory. Same selection rule (larger probability, then smaller index).
// The reference takes its moeSoftmax + moeTopK pair here (csrc/moe_topk_softmax_kernels.cu:50-166),
// whose block-wide sum has a different association order, so weights agree to rounding only.
template <bool kBf16In>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
topk_softmax_generic_kernel(const void* __restrict__ gating, float* __restrict__ topk_w, int* __restrict__ topk_ids,
                            int* __restrict__ token_expert_indices, int num_rows, int num_experts, int k,
                            int renormalize) {
  extern __shared__ float probs_smem[];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int row = blockIdx.x * kWarpsPerCta + warp;
  if (row >= num_rows) return;
  float* probs = probs_smem + static_cast<size_t>(warp) * num_experts;

  float m = -3.402823466e+38f;
  for (int e = lane; e < num_experts; e += 32) {
    float x;
    if constexpr (kBf16In) x = __bfloat162float(static_cast<const __nv_bfloat16*>(gating)[static_cast<size_t>(row) * num_experts + e]);
    else x = static_cast<const float*>(gating)[static_cast<size_t>(row) * num_experts + e];
    probs[e] = x;
    m = fmaxf(m, x);
  }
  for (int mask = 16; mask > 0; mask /= 2) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, mask));
  float z = 0.f;
  for (int e = lane; e < num_experts; e += 32) z += expf(probs[e] - m);
  for (int mask = 16; mask > 0; mask /= 2) z += __shfl_xor_sync(0xffffffffu, z, mask);
  const float inv = 1.f / z;
  for (int e = lane; e < num_experts; e += 32) probs[e] = expf(probs[e] - m) * inv;
  __syncwarp();

  float picked_sum = 0.f;
  for (int k_idx = 0; k_idx < k; ++k_idx) {
    float best = -1.f;
    int expert = 0;
    for (int e = lane; e < num_experts; e += 32) {
      const float val = probs[e];
      if (val > best) {
        best = val;
        expert = e;
      }
    }
    for (int mask = 16; mask > 0; mask /= 2) {
      const float other = __shfl_xor_sync(0xffffffffu, best, mask);
      const int other_expert = __shfl_xor_sync(0xffffffffu, expert, mask);
      if (other > best || (other == best && other_expert < expert)) {
        best = other;
        expert = other_expert;
      }
    }
    if (lane == 0) {
      const size_t idx = static_cast<size_t>(k) * row + k_idx;
      topk_w[idx] = best;
      topk_ids[idx] = expert;
      if (token_expert_indices != nullptr) token_expert_indices[idx] = k_idx * num_rows + row;
      picked_sum += best;
      probs[expert] = -10000.f;
    }
    __syncwarp();
  }
  if (renormalize && lane == 0) {
    for (int k_idx = 0; k_idx < k; ++k_idx) {
      const size_t idx = static_cast<size_t>(k) * row + k_idx;
      topk_w[idx] = topk_w[idx] / picked_sum;
    }
  }
}

template <int E>
void launch_pow2(const void* gating, int bf16_in, float* w, int* ids, int* tei, int T, int k, int renorm,
                 cudaStream_t stream) {
  constexpr int rows_per_cta = kWarpsPerCta * TopkShape<E>::kRowsPerWarp;
  const int blocks = (T + rows_per_cta - 1) / rows_per_cta;
  if (bf16_in)
    launch_pdl(topk_softmax_pow2_kernel<E, true>, dim3(blocks), dim3(kWarpsPerCta * 32), 0, stream, gating, w, ids, tei, T, k, renorm);
  else
    launch_pdl(topk_softmax_pow2_kernel<E, false>, dim3(blocks), dim3(kWarpsPerCta * 32), 0, stream, gating, w, ids, tei, T, k, renorm);
}

}  // namespace

int launch_topk_softmax(const void* gating, int gating_is_bf16, float* topk_w, int* topk_ids,
                        int* token_expert_indices, int T, int E, int k, int renormalize, cudaStream_t stream) {
  if (T < 0 || E <= 0 || k <= 0 || k > E) return set_error(kStatusInvalidArgument, "topk_softmax: need 0 < k <= E");
  if (T == 0) return kStatusOk;
  switch (E) {
    case 1: launch_pow2<1>(gating, gating_is_bf16, topk_w, topk_ids, token_expert_indices, T, k, renormalize, stream); break;
    case 2: launch_pow2<2>(gating, gating_is_bf16, topk_w, topk_ids, token_expert_indices, T, k, renormalize, stream); break;
    case 4: launch_pow2<4>(gating, gating_is_bf16, topk_w, topk_ids, token_expert_indices, T, k, renormalize, stream); break;
    case 8: launch_pow2<8>(gating, gating_is_bf16, topk_w, topk_ids, token_expert_indices, T, k, renormalize, stream); break;
    case 16: launch_pow2<16>(gating, gating_is_bf16, topk_w, topk_ids, token_expert_indices, T, k, renormalize, stream); break;
    case 32: launch_pow2<32>(gating, gating_is_bf16, topk_w, topk_ids, token_expert_indices, T, k, renormalize, stream); break;
    case 64: launch_pow2<64>(gating, gating_is_bf16, topk_w, topk_ids, token_expert_indices, T, k, renormalize, stream); break;
    case 128: launch_pow2<128>(gating, gating_is_bf16, topk_w, topk_ids, token_expert_indices, T, k, renormalize, stream); break;
    case 256: launch_pow2<256>(gating, gating_is_bf16, topk_w, topk_ids, token_expert_indices, T, k, renormalize, stream); break;
    default: {
      if (E > 8192) return set_error(kStatusInvalidArgument, "topk_softmax: more than 8192 experts");
      const size_t smem = static_cast<size_t>(kWarpsPerCta) * E * sizeof(float);
      const int blocks = (T + kWarpsPerCta - 1) / kWarpsPerCta;
      if (gating_is_bf16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(topk_softmax_generic_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        topk_softmax_generic_kernel<true><<<blocks, kWarpsPerCta * 32, smem, stream>>>(gating, topk_w, topk_ids, token_expert_indices, T, E, k, renormalize);
      } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(topk_softmax_generic_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        topk_softmax_generic_kernel<false><<<blocks, kWarpsPerCta * 32, smem, stream>>>(gating, topk_w, topk_ids, token_expert_indices, T, E, k, renormalize);
      }
    }
  }
  count_launches(1);
  return check_launch("topk_softmax");
}

}  // namespace moe_b200
