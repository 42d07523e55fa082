// Declarations shared by the translation units of libmoe_b200: status codes, the
// error-string slot behind moe_b200_last_error(), and the internal launchers that
// the extern "C" layer (c_api.cu) forwards to.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace moe_b200 {

enum : int {
  kStatusOk = 0,
  kStatusInvalidArgument = 1,
  kStatusCudaError = 2,
  kStatusWorkspaceTooSmall = 3,
  kStatusDeviceTimeout = 4,   // a bounded device-side wait ran out (see the kernel's status word)
  kStatusNotRegistered = 5,   // all-reduce: buffer address is not registered
  kStatusDriverEntryPoint = 6,
  kStatusTooLarge = 7,        // request exceeds a fixed capacity (static scratch)
};

int set_error(int status, const char* fmt, ...);
int check_launch(const char* what);
int check_cuda(cudaError_t e, const char* what);
const char* last_error_string();
// Host-side count of kernels this library has launched in this process (reported by the benchmark).
void count_launches(int n);
unsigned long long launch_count();

constexpr int kBlockM = 128;  // token rows per grouped-GEMM tile (and the internal permutation block)

// ---- routing.cu
int launch_topk_softmax(const void* gating, int gating_is_bf16, float* topk_w, int* topk_ids,
                        int* token_expert_indices, int T, int E, int k, int renormalize, cudaStream_t stream);

// ---- align.cu
size_t align_workspace_bytes(int numel, int E);
int launch_align_block_size(const int* topk_ids, int numel, int E, int block_size, int* sorted_ids, int sorted_cap,
                            int* expert_ids, int expert_ids_cap, int* num_post_pad, void* workspace,
                            size_t workspace_bytes, cudaStream_t stream);

int static_align_scratch_ints();
int launch_align_block_size_static(const int* topk_ids, int numel, int E, int block_size, int* sorted_ids,
                                   int sorted_cap, int* expert_ids, int expert_ids_cap, int* num_post_pad,
                                   cudaStream_t stream);

// ---- elementwise.cu
int launch_silu_and_mul(__nv_bfloat16* out, const __nv_bfloat16* in, int rows, int d, cudaStream_t stream);
int launch_swigluoai_and_mul(__nv_bfloat16* out, const __nv_bfloat16* in, int rows, int d, float alpha, float limit,
                             cudaStream_t stream);
int launch_moe_sum(const __nv_bfloat16* in, __nv_bfloat16* out, int T, int k, int H, cudaStream_t stream);

// ---- grouped_gemm.cu
struct GroupedGemmArgs {
  // permutation (block size kBlockM)
  const int* sorted_ids;
  const int* expert_ids;
  const int* num_post_pad;
  int numel;        // T * top_k
  int top_k;
  int max_m_blocks; // upper bound on number of kBlockM blocks (sizes the grid)
  int num_experts;
  // problem
  int hidden;       // H
  int inter;        // I per rank
  int activation;   // 0 silu, 1 swigluoai (interleaved gate/up)
  float act_alpha, act_limit;
  int* status;      // device status word (0 = ok)
};
// h_sorted[p, :] = act(x[sorted_ids[p] / top_k] @ w13[e]^T), p in permuted order, bf16 [rows_cap, inter]
int launch_grouped_gemm1(const GroupedGemmArgs& a, const __nv_bfloat16* x, const __nv_bfloat16* w13,
                         const __nv_bfloat16* w13_bias, __nv_bfloat16* h_sorted, int rows_cap, cudaStream_t stream);
// c3[f, :] = bf16((h_sorted[p] @ w2[e]^T) * topk_w[f]), f = sorted_ids[p], bf16 [numel, hidden]
int launch_grouped_gemm2(const GroupedGemmArgs& a, const __nv_bfloat16* h_sorted, int rows_cap,
                         const __nv_bfloat16* w2, const __nv_bfloat16* w2_bias, const float* topk_w,
                         __nv_bfloat16* c3, cudaStream_t stream);
int device_sm_count();

// ---- pre_moe.cu (the decoder layer's steps in front of the MoE block)
// residual != nullptr: residual <- bf16(input + residual) first (ops.add_rms_norm); else ops.rms_norm.
int launch_rms_norm(__nv_bfloat16* out, __nv_bfloat16* residual, const __nv_bfloat16* input, const __nv_bfloat16* weight,
                    float eps, int T, int H, cudaStream_t stream);
size_t pre_moe_workspace_bytes(int T, int H, int E);
int launch_add_rms_norm_router(const __nv_bfloat16* input, __nv_bfloat16* residual, const __nv_bfloat16* norm_weight, float eps,
                               const __nv_bfloat16* gate_weight, __nv_bfloat16* normed, __nv_bfloat16* logits_out,
                               float* topk_w, int* topk_ids, int T, int H, int E, int top_k, int renormalize,
                               void* workspace, size_t workspace_bytes, int* status_word, cudaStream_t stream);

// ---- grouped_gemm_fp8.cu (e4m3 weights with 128 x 128 block scales, activations quantised per row and 128 columns)
// q[r, c] = e4m3(x[r, c] / s[r, g]), s = max(|x| over the group, 1e-10) / 448; group g = columns
// [128 g - shift, 128 (g + 1) - shift) cut to the row. With sorted_ids given, rows that are padding of the
// permutation (or lie beyond *num_post_pad) are skipped; shift != 0 needs sorted_ids.
int launch_quant_rows_fp8(const __nv_bfloat16* x, int rows, int cols, int shift, uint8_t* q, float* s,
                          const int* sorted_ids, int numel, const int* num_post_pad, cudaStream_t stream);
// The weight scales are those of the UNSHARDED tensors ([E, 2 I/128, H/128] and [E, H/128, I/128]); the rank holds
// the slice [i_offset, i_offset + a.inter) of the intermediate dimension I = i_total.
int launch_grouped_gemm1_fp8(const GroupedGemmArgs& a, const uint8_t* x_q, const float* x_s, const uint8_t* w13_q,
                             const float* w13_s, int i_offset, int i_total, __nv_bfloat16* h_sorted, cudaStream_t stream);
int launch_grouped_gemm2_fp8(const GroupedGemmArgs& a, const uint8_t* h_q, const float* h_s, const uint8_t* w2_q,
                             const float* w2_s, int i_offset, int i_total, const float* topk_w, __nv_bfloat16* c3,
                             cudaStream_t stream);
// Tensor map of a dense bf16 (elem_bytes 2) or byte (elem_bytes 1) tensor, 128-byte swizzle; dims/box innermost first.
int make_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint32_t* box, int elem_bytes);
// Token blocks the permutation is expected to produce, and the share of SM-time a round-robin tile list keeps busy.
double expected_m_blocks(int numel, int top_k, int num_experts);
double wave_efficiency(double tiles, int sms);

}  // namespace moe_b200
