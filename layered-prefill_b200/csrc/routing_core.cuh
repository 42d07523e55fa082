// Softmax + k rounds of arg-max for one token row whose logits already sit in registers, spread over the
// row's group of lanes the way topk_softmax_pow2_kernel (routing.cu) loads them. Shared by that kernel and by
// the fused pre-MoE kernel (pre_moe.cu), so both produce the same bits.
#pragma once

#include <cuda_runtime.h>

namespace moe_b200 {

template <int E>
struct TopkShape {
  static constexpr int kEltsPerLdg = E < 4 ? E : 4;
  static constexpr int kVecsPerThread = (E / (kEltsPerLdg * 32)) > 1 ? (E / (kEltsPerLdg * 32)) : 1;
  static constexpr int kVpt = kVecsPerThread * kEltsPerLdg;
  static constexpr int kThreadsPerRow = E / kVpt;
  static constexpr int kRowsPerWarp = 32 / kThreadsPerRow;
  static constexpr int kColsPerGroupLdg = kEltsPerLdg * kThreadsPerRow;
};

// v: the lane's VPT logits (16-byte groups, kThreadsPerRow groups apart); lane: lane in the warp; row_ok: whether
// this lane's row exists (lanes of missing rows run along and store nothing).
template <int E>
__device__ __forceinline__ void topk_softmax_row(float (&v)[TopkShape<E>::kVpt], int lane, bool row_ok, int row,
                                                 int num_rows, int k, int renormalize, float* __restrict__ topk_w,
                                                 int* __restrict__ topk_ids, int* __restrict__ token_expert_indices) {
  using S = TopkShape<E>;
  constexpr int VPT = S::kVpt;
  constexpr int TPR = S::kThreadsPerRow;
  constexpr int ELTS = S::kEltsPerLdg;
  constexpr int LDGS = S::kVecsPerThread;
  const int g = lane % TPR;
  const int first_col = g * ELTS;

  float row_max = v[0];
#pragma unroll
  for (int ii = 1; ii < VPT; ++ii) row_max = fmaxf(row_max, v[ii]);
#pragma unroll
  for (int mask = TPR / 2; mask > 0; mask /= 2) row_max = fmaxf(row_max, __shfl_xor_sync(0xffffffffu, row_max, mask, TPR));

  float row_sum = 0.f;
#pragma unroll
  for (int ii = 0; ii < VPT; ++ii) {
    v[ii] = expf(v[ii] - row_max);
    row_sum += v[ii];
  }
#pragma unroll
  for (int mask = TPR / 2; mask > 0; mask /= 2) row_sum += __shfl_xor_sync(0xffffffffu, row_sum, mask, TPR);

  const float inv_sum = 1.f / row_sum;
#pragma unroll
  for (int ii = 0; ii < VPT; ++ii) v[ii] = v[ii] * inv_sum;

  // Winner number k_idx is kept in registers by lane k_idx % TPR of the row's group (slot k_idx / TPR),
  // so the results leave the kernel as one store per lane and nothing is read back from memory.
  float keep_w[VPT];
  int keep_id[VPT];
#pragma unroll
  for (int s = 0; s < VPT; ++s) {
    keep_w[s] = 0.f;
    keep_id[s] = 0;
  }
  for (int k_idx = 0; k_idx < k; ++k_idx) {
    float best = v[0];
    int expert = first_col;
#pragma unroll
    for (int ldg = 0; ldg < LDGS; ++ldg) {
#pragma unroll
      for (int j = 0; j < ELTS; ++j) {
        const float val = v[ldg * ELTS + j];
        if (val > best) {
          best = val;
          expert = first_col + ldg * S::kColsPerGroupLdg + j;
        }
      }
    }
    // Consensus over the row's lanes: the largest value and, among the lanes that hold it, the smallest
    // expert index -- what the reference's compare-and-swap butterfly arrives at, in two warp reductions.
    // Values are softmax probabilities (>= 0) or the -10000 blanking mark, so their bit patterns order
    // like signed integers.
    if constexpr (TPR > 1) {
      const unsigned row_lanes = TPR == 32 ? 0xffffffffu : (((1u << TPR) - 1u) << ((lane / TPR) * TPR));
      const int top = __reduce_max_sync(row_lanes, __float_as_int(best));
      expert = __reduce_min_sync(row_lanes, __float_as_int(best) == top ? expert : 0x7fffffff);
      best = __int_as_float(top);
    }
    if (g == k_idx % TPR) {
      const int slot = k_idx / TPR;
#pragma unroll
      for (int s = 0; s < VPT; ++s) {
        if (s == slot) {
          keep_w[s] = best;
          keep_id[s] = expert;
        }
      }
    }
    if (k_idx + 1 < k) {
      const int ldg_group = expert / S::kColsPerGroupLdg;
      const int owner = (expert / ELTS) % TPR;
      const int at = ldg_group * ELTS + expert % ELTS;
      if (g == owner) {
#pragma unroll
        for (int s = 0; s < VPT; ++s)
          if (s == at) v[s] = -10000.f;
      }
    }
  }

  float inv_picked = 1.f;
  if (renormalize) {
    float picked_sum = 0.f;
#pragma unroll
    for (int s = 0; s < VPT; ++s) picked_sum += keep_w[s];
#pragma unroll
    for (int mask = TPR / 2; mask > 0; mask /= 2) picked_sum += __shfl_xor_sync(0xffffffffu, picked_sum, mask, TPR);
    inv_picked = picked_sum;
  }
  if (row_ok) {
#pragma unroll
    for (int s = 0; s < VPT; ++s) {
      const int k_idx = s * TPR + g;
      if (k_idx < k) {
        const size_t idx = static_cast<size_t>(k) * row + k_idx;
        topk_w[idx] = renormalize ? keep_w[s] / inv_picked : keep_w[s];
        topk_ids[idx] = keep_id[s];
        if (token_expert_indices != nullptr) token_expert_indices[idx] = k_idx * num_rows + row;
      }
    }
  }
}

}  // namespace moe_b200
