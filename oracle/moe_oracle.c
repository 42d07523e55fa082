/*
 * TEST INFRASTRUCTURE, NOT PRODUCT: CPU restatement of the routing and permutation steps of the
 * reference's MoE block, used only by tests/, the smoke check and the benchmark's cpu_baseline leg
 * to check the CUDA library. Nothing in layered-prefill_b200/ may call it.
 *
 * Parity status: the reference holds no golden vectors or tests for these functions (it has no
 * tests at all), so this file is pinned (a) against outputs of the reference's own torch helper
 * nanovllm/layers/for_moe/moe_easy_kernel.py:topk_softmax committed under tests/golden/, and
 * (b) on the GPU box against the reference's compiled CUDA ops when oracle/_ref holds them.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/*
 * Softmax + top-k of one row, following topkGatingSoftmax
 * (csrc/moe_topk_softmax_kernels.cu:182-380) for power-of-two expert counts up to 256:
 *   - a lane owns VPT experts: groups of ELTS consecutive experts, TPR*ELTS apart (:239-258);
 *   - row max (order-free); e_i = expf(x_i - max); lane sums are sequential over the lane's values
 *     (:277-282), lanes are then combined by an xor butterfly TPR/2..1 (:285-290) -- fp32 addition is
 *     commutative, so every lane ends with the same bits and lane 0 is enough;
 *   - p_i = e_i * (1.f / sum) (:297-303);
 *   - k rounds of arg-max, larger value first, equal values to the lower index (:325,343); the winner
 *     is blanked with -10000 (:376).
 * Other expert counts follow moeSoftmax/moeTopK (:50-166) with a plain sequential sum.
 */
static void softmax_row(const float* x, int E, float* p, float* lane_sum /* >= 32 floats */) {
  float m = x[0];
  for (int i = 1; i < E; ++i) m = fmaxf(m, x[i]);
  const int pow2 = (E & (E - 1)) == 0 && E <= 256;
  if (pow2) {
    const int elts = E < 4 ? E : 4;
    int vecs = E / (elts * 32);
    if (vecs < 1) vecs = 1;
    const int vpt = vecs * elts;
    const int tpr = E / vpt;
    for (int i = 0; i < E; ++i) p[i] = expf(x[i] - m);
    for (int g = 0; g < tpr; ++g) {
      float s = 0.f;
      for (int ii = 0; ii < vecs; ++ii)
        for (int j = 0; j < elts; ++j) s += p[ii * tpr * elts + g * elts + j];
      lane_sum[g] = s;
    }
    for (int mask = tpr / 2; mask > 0; mask /= 2) {
      float next[32];
      for (int g = 0; g < tpr; ++g) next[g] = lane_sum[g] + lane_sum[g ^ mask];
      memcpy(lane_sum, next, sizeof(float) * (size_t)tpr);
    }
    const float inv = 1.f / lane_sum[0];
    for (int i = 0; i < E; ++i) p[i] = p[i] * inv;
  } else {
    float z = 0.f;
    for (int i = 0; i < E; ++i) z += expf(x[i] - m);
    const float inv = 1.f / z;
    for (int i = 0; i < E; ++i) p[i] = expf(x[i] - m) * inv;
  }
}

/* logits fp32 [T,E] -> weights fp32 [T,k], ids int32 [T,k], token_expert_indices int32 [T,k] (may be NULL).
 * renormalize: weights /= sum of the k picked (nanovllm/layers/for_moe/fused_moe.py:417-418). */
void oracle_topk_softmax(const float* logits, int T, int E, int k, int renormalize, float* weights, int32_t* ids,
                         int32_t* token_expert_indices) {
  float* p = (float*)malloc(sizeof(float) * (size_t)E);
  float lane_sum[32];
  for (int t = 0; t < T; ++t) {
    softmax_row(logits + (size_t)t * E, E, p, lane_sum);
    float picked = 0.f;
    for (int j = 0; j < k; ++j) {
      int best = 0;
      for (int i = 1; i < E; ++i)
        if (p[i] > p[best]) best = i;
      weights[(size_t)t * k + j] = p[best];
      ids[(size_t)t * k + j] = best;
      if (token_expert_indices) token_expert_indices[(size_t)t * k + j] = j * T + t;
      picked += p[best];
      p[best] = -10000.f;
    }
    if (renormalize)
      for (int j = 0; j < k; ++j) weights[(size_t)t * k + j] = weights[(size_t)t * k + j] / picked;
  }
  free(p);
}

/*
 * moe_align_block_size (csrc/moe_align_block_size_kernels.cu:140-237): counts per expert (:165-173),
 * padded to block_size (:186), exclusive scan (:190-201), expert id per block and zero tail
 * (:205-217), every slot pre-filled with numel (:150-152), flat indices scattered to their expert's
 * segment (:229-236). The reference's scatter order inside a segment is atomic arrival order; this
 * restatement emits the ascending order, which is what the comparison canonicalises to.
 * Ids outside [0, E) are skipped (:170,231).
 */
void oracle_moe_align_block_size(const int32_t* topk_ids, int numel, int E, int block_size, int32_t* sorted_ids,
                                 int sorted_cap, int32_t* expert_ids, int expert_ids_cap, int32_t* num_post_pad) {
  int32_t* cum = (int32_t*)calloc((size_t)E + 1, sizeof(int32_t));
  int32_t* cnt = (int32_t*)calloc((size_t)E, sizeof(int32_t));
  for (int i = 0; i < sorted_cap; ++i) sorted_ids[i] = numel;
  for (int i = 0; i < numel; ++i) {
    const int e = topk_ids[i];
    if (e >= 0 && e < E) cnt[e]++;
  }
  for (int e = 0; e < E; ++e) cum[e + 1] = cum[e] + (cnt[e] + block_size - 1) / block_size * block_size;
  *num_post_pad = cum[E];
  for (int b = 0; b < expert_ids_cap; ++b) expert_ids[b] = 0;
  for (int e = 0; e < E; ++e)
    for (int i = cum[e]; i < cum[e + 1]; i += block_size) expert_ids[i / block_size] = e;
  for (int e = 0; e < E; ++e) cnt[e] = cum[e];
  for (int i = 0; i < numel; ++i) {
    const int e = topk_ids[i];
    if (e >= 0 && e < E) sorted_ids[cnt[e]++] = i;
  }
  free(cum);
  free(cnt);
}
