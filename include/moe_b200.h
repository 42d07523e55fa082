/*
 * libmoe_b200 -- C ABI of the B200 (sm_100a) MoE-block hot path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (as void*), launches on
 * that stream without synchronising the host, and returns 0 on success or one of the MOE_B200_*
 * status codes; moe_b200_last_error() gives the message of the calling thread's last failure.
 * Nothing here allocates device memory unless its description says so: callers pass outputs and
 * workspaces (sizes from the *_workspace_bytes functions).
 *
 * Each declaration names the reference interface it stands in for (paths inside the
 * scale-snu/layered-prefill tree).
 */
#ifndef MOE_B200_H_
#define MOE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MOE_B200_OK 0
#define MOE_B200_INVALID_ARGUMENT 1
#define MOE_B200_CUDA_ERROR 2
#define MOE_B200_WORKSPACE_TOO_SMALL 3
#define MOE_B200_DEVICE_TIMEOUT 4
#define MOE_B200_NOT_REGISTERED 5
#define MOE_B200_DRIVER_ENTRY_POINT 6
#define MOE_B200_TOO_LARGE 7

#define MOE_B200_ACT_SILU 0      /* silu(gate) * up, w13 rows = [gate | up] */
#define MOE_B200_ACT_SWIGLUOAI 1 /* gpt-oss gate, w13 rows interleaved gate/up, alpha 1.702, limit 7 */

/* Message of the last non-zero status returned to this thread ("" if none). */
const char* moe_b200_last_error(void);
/* Library ABI version (bumped when a signature changes). */
int moe_b200_abi_version(void);
/* Token rows per grouped-GEMM tile = block size of the internal permutation (128). */
int moe_b200_block_m(void);

/* Number of kernels this library has launched in the calling process so far. No reference counterpart
 * (the benchmark reports it). */
uint64_t moe_b200_launch_count(void);

/*
 * RMSNorm with the reference's rounding and summation order (bit-identical for H % 32 == 0). Replace
 * ops.rms_norm / ops.add_rms_norm (csrc/ops.cpp:16-27, csrc/layernorm_kernels.cu:10-36, 76-107).
 *   add_rms_norm: residual <- bf16(input + residual); out <- bf16(bf16(residual * rsqrt(mean(residual^2) + eps)) * weight)
 * bf16 [T, H] contiguous, weight bf16 [H]; H % 8 == 0, H <= 24000.
 */
int moe_b200_rms_norm(void* out, const void* input, const void* weight, float eps, int T, int H, void* stream);
int moe_b200_add_rms_norm(void* out, void* residual, const void* input, const void* weight, float eps, int T, int H,
                          void* stream);

/*
 * The decoder layer's three steps in front of the MoE block in one call: post-attention add + RMSNorm, the router's
 * gate projection and softmax/top-k. Replaces the sequence post_attention_layernorm -> gate -> select_experts
 * (nanovllm/models/qwen3_moe.py:276-282 and :100-110, nanovllm/layers/fused_moe.py:712-724).
 *   input bf16 [T, H] (attention output), residual bf16 [T, H] (updated in place), norm_weight bf16 [H],
 *   gate_weight bf16 [E, H] (ReplicatedLinear.weight), normed_out bf16 [T, H] (the MoE block's hidden states),
 *   logits_out bf16 [T, E] or NULL, topk_weights fp32 [T, k], topk_ids int32 [T, k].
 * One kernel for T <= 512 with E in {128, 256} and H % 256 == 0; otherwise norm, tensor-core GEMM and routing as
 * separate launches (needs the workspace; E % 16 == 0, H % 16 == 0). Logits are the bf16 rounding of an fp32
 * dot product whose summation order differs from the reference's cuBLAS call.
 */
size_t moe_b200_pre_moe_workspace_bytes(int T, int H, int E);
int moe_b200_add_rms_norm_router(const void* input, void* residual, const void* norm_weight, float eps,
                                 const void* gate_weight, void* normed_out, void* logits_out, float* topk_weights,
                                 int32_t* topk_ids, int T, int H, int E, int top_k, int renormalize, void* workspace,
                                 size_t workspace_bytes, int32_t* status_word, void* stream);

/*
 * Router. Replaces ops.topk_softmax (csrc/ops.cpp:46-51, csrc/moe_topk_softmax_kernels.cu:476-503)
 * and, with renormalize != 0, the division in fused_topk (nanovllm/layers/for_moe/fused_moe.py:417-418).
 * gating: [T, E] row-major, fp32 (gating_is_bf16 == 0) or bf16 (!= 0). Outputs [T, k]:
 * topk_weights fp32, topk_ids int32 (descending probability, ties to the lower expert id),
 * token_expert_indices int32 = j*T + t (may be NULL).
 */
int moe_b200_topk_softmax(const void* gating, int gating_is_bf16, float* topk_weights, int32_t* topk_ids,
                          int32_t* token_expert_indices, int T, int E, int k, int renormalize, void* stream);

/*
 * Permutation. Replaces ops.moe_align_block_size (csrc/ops.cpp:53-60,
 * csrc/moe_align_block_size_kernels.cu:239-291). sorted_token_ids has sorted_cap =
 * numel + E*(block_size-1) entries and is completely written (pads = numel); expert_ids has
 * expert_ids_cap = ceil(sorted_cap / block_size) entries. Within an expert, ids are ascending.
 * workspace: moe_b200_align_workspace_bytes(numel, E) bytes of device memory (the reference
 * allocates its cumsum buffer itself, csrc/moe_align_block_size_kernels.cu:258-259).
 */
size_t moe_b200_align_workspace_bytes(int numel, int E);
int moe_b200_moe_align_block_size(const int32_t* topk_ids, int numel, int E, int block_size,
                                  int32_t* sorted_token_ids, int sorted_cap, int32_t* expert_ids, int expert_ids_cap,
                                  int32_t* num_tokens_post_pad, void* workspace, size_t workspace_bytes, void* stream);

/*
 * The same permutation for callers that cannot hand over a workspace because they have no way to
 * allocate one. This entry point has no counterpart in the reference. It exists for hosts that bind the
 * reference's exact op signature (which carries no workspace argument) but, unlike the reference's op,
 * must not allocate inside the call: a serving engine that gave every free byte of device memory to
 * its KV-cache pool at start-up, or a hot path on which touching the CUDA allocator (and the implicit
 * synchronisation a cudaMalloc/cudaFree can bring) is not acceptable. The per-chunk histogram and the
 * cumsum table live in an array built into the library image instead; every GPU that loads the library
 * holds those moe_b200_moe_align_static_scratch_bytes() bytes (130 KiB) until the process exits.
 *
 * Limit: ceil(numel / 1024) * E + E + 1 <= 33280 words, e.g. 131072 flat indices (16384 tokens with
 * top-8) for up to 256 experts. Larger requests fail with MOE_B200_TOO_LARGE and a message; nothing is
 * launched then. Outputs and their sizes are exactly those of moe_b200_moe_align_block_size.
 *
 * The call performs no cudaMalloc, cudaFree or other allocating call. The first call on each device looks
 * up the device address of the built-in array (cudaGetSymbolAddress, with that device current); make that
 * first call outside of any stream capture. All calls on a device share the one array, which keeps
 * whatever the last call left in it; nothing in it needs clearing between calls, because each call writes
 * every word before reading it. Two calls that can overlap on the GPU (different streams, no ordering
 * between them) race on the array and give undefined results: order them.
 */
size_t moe_b200_moe_align_static_scratch_bytes(void);
int moe_b200_moe_align_block_size_static(const int32_t* topk_ids, int numel, int E, int block_size,
                                         int32_t* sorted_token_ids, int sorted_cap, int32_t* expert_ids,
                                         int expert_ids_cap, int32_t* num_tokens_post_pad, void* stream);

/*
 * Stand-alone gated activations on bf16. Replace ops.silu_and_mul / ops.swigluoai_and_mul
 * (csrc/ops.cpp:29-36, csrc/activation_kernels.cu:68-109). in: [rows, 2d], out: [rows, d].
 */
int moe_b200_silu_and_mul(void* out, const void* in, int rows, int d, void* stream);
int moe_b200_swigluoai_and_mul(void* out, const void* in, int rows, int d, float alpha, float limit, void* stream);

/*
 * Sum over the k slots. Replaces moe_sum (nanovllm/layers/for_moe/moe_easy_kernel.py:26-31).
 * in: bf16 [T, k, H]; out: bf16 [T, H]; fp32 accumulation in slot order.
 */
int moe_b200_moe_sum(const void* in, void* out, int T, int k, int H, void* stream);

/*
 * Both expert GEMMs, the activation, the routed-weight scaling and the k-slot sum.
 * Replaces fused_experts / fused_experts_impl (nanovllm/layers/for_moe/fused_moe.py:422-633).
 *   x    bf16 [T, H]           hidden states
 *   w13  bf16 [E, 2*I, H]      gate rows then up rows (interleaved for MOE_B200_ACT_SWIGLUOAI)
 *   w2   bf16 [E, H, I]        I = intermediate size held by this rank
 *   w13_bias bf16 [E, 2*I], w2_bias bf16 [E, H]  (NULL when absent)
 *   topk_weights fp32 [T, k], topk_ids int32 [T, k]
 *   out  bf16 [T, H]; may be x itself (the reference's inplace=True)
 *   status_word: one int32 of device memory that was zero when first handed to the library; a
 *   kernel whose bounded wait ran out stores a non-zero code there (see moe_b200_read_status).
 * Requires H % 16 == 0 and I % 16 == 0.
 */
size_t moe_b200_fused_experts_workspace_bytes(int T, int E, int top_k, int H, int I);
int moe_b200_fused_experts(const void* x, const void* w13, const void* w2, const void* w13_bias, const void* w2_bias,
                           const float* topk_weights, const int32_t* topk_ids, void* out, int T, int E, int top_k,
                           int H, int I, int activation, void* workspace, size_t workspace_bytes,
                           int32_t* status_word, void* stream);

/*
 * fp8 (e4m3, w8a8) variant of fused_experts with 128 x 128 block-scaled weights and activations quantised
 * per token and group of 128 columns, fp32 accumulation. No reference counterpart: the reference's fused_moe
 * asserts that no scales are passed (nanovllm/layers/for_moe/fused_moe.py:248-249); the signature follows the
 * block-quantised convention of its kernel arguments (A_scale / B_scale, block_shape [128, 128]).
 *   x          bf16 [T, H]                      quantised inside (the bf16 input is not modified)
 *   w13_q      e4m3 [E, 2*I, H] (one byte each), w13_scale fp32 [E, 2*I/128, H/128]
 *   w2_q       e4m3 [E, H, I],                   w2_scale  fp32 [E, H/128, I/128]
 *   out        bf16 [T, H]
 * Requires H % 128 == 0 and I % 128 == 0; SiLU only, no biases.
 */
size_t moe_b200_fused_experts_fp8_workspace_bytes(int T, int E, int top_k, int H, int I);
int moe_b200_fused_experts_fp8(const void* x, const void* w13_q, const float* w13_scale, const void* w2_q,
                               const float* w2_scale, const float* topk_weights, const int32_t* topk_ids, void* out,
                               int T, int E, int top_k, int H, int I, void* workspace, size_t workspace_bytes,
                               int32_t* status_word, void* stream);
/* The same on one tensor-parallel rank: this rank holds the slice [i_offset, i_offset + I) of an intermediate
 * dimension of i_total (w13_q [E, 2*I, H] = its gate rows then its up rows, w2_q [E, H, I]); the scales stay those
 * of the unsharded weights (w13_scale [E, 2*i_total/128, H/128], w2_scale [E, H/128, i_total/128]) and are indexed
 * by global position, so a slice may start or end inside a scale block (I = 192 at TP=8 of I = 1536). The
 * intermediate is quantised in groups that follow those blocks. out = this rank's partial sum (all-reduce it).
 * Requires i_total % 128 == 0, I % 64 == 0, i_offset % 64 == 0. */
int moe_b200_fused_experts_fp8_tp(const void* x, const void* w13_q, const float* w13_scale, const void* w2_q,
                                  const float* w2_scale, const float* topk_weights, const int32_t* topk_ids, void* out,
                                  int T, int E, int top_k, int H, int I, int i_offset, int i_total, void* workspace,
                                  size_t workspace_bytes, int32_t* status_word, void* stream);
/* The same with the k-slot sum fused into the peer-memory all-reduce (as moe_b200_fused_moe_forward_tp does for bf16):
 * out = the layer's output on every rank. */
int moe_b200_fused_experts_fp8_tp_reduce(const void* x, const void* w13_q, const float* w13_scale, const void* w2_q,
                                         const float* w2_scale, const float* topk_weights, const int32_t* topk_ids,
                                         void* out, int T, int E, int top_k, int H, int I, int i_offset, int i_total,
                                         void* workspace, size_t workspace_bytes, int64_t ar_handle, int64_t reg_buffer,
                                         int64_t reg_buffer_bytes, int ar_algo, int32_t* status_word, void* stream);
/* q[r, c] = e4m3(x[r, c] / s[r, c/128]), s[r, g] = max(|x[r, 128g .. 128g+127]|, 1e-10) / 448; x bf16 [rows, cols],
 * cols % 128 == 0. The activation quantisation the call above applies (exposed for tests and for callers
 * that keep quantised activations). */
int moe_b200_quant_fp8_per_token_group(const void* x, int rows, int cols, void* q, float* scales, void* stream);

/*
 * The two grouped GEMM passes on their own, for callers that keep the permutation (block size
 * moe_b200_block_m()) and the intermediates themselves. Each replaces one invoke_fused_moe_kernel call
 * of fused_experts_impl together with the element-wise kernel around it:
 *   gate_up: for_moe/fused_moe.py:579-599 (GEMM + ops.silu_and_mul / swigluoai_and_mul). h_sorted is bf16
 *            [rows_cap, I] in permuted order (row p belongs to flat index sorted_token_ids[p]); pad rows
 *            are not written.
 *   down:    for_moe/fused_moe.py:611-628 (GEMM with MUL_ROUTED_WEIGHT). c3 is bf16 [T*k, H] at flat index.
 * rows_cap: rows of h_sorted = entries of sorted_token_ids, a multiple of 128.
 */
int moe_b200_grouped_gemm_gate_up(const void* x, const void* w13, const void* w13_bias, const int32_t* sorted_token_ids,
                                  const int32_t* expert_ids, const int32_t* num_tokens_post_pad, void* h_sorted,
                                  int rows_cap, int T, int E, int top_k, int H, int I, int activation,
                                  int32_t* status_word, void* stream);
int moe_b200_grouped_gemm_down(const void* h_sorted, int rows_cap, const void* w2, const void* w2_bias,
                               const float* topk_weights, const int32_t* sorted_token_ids, const int32_t* expert_ids,
                               const int32_t* num_tokens_post_pad, void* c3, int T, int E, int top_k, int H, int I,
                               int32_t* status_word, void* stream);

/*
 * Router + fused_experts in one call: what FusedMoE.forward runs on one rank before the
 * tensor-parallel reduction (nanovllm/layers/fused_moe.py:163-216, 750-787).
 * router_logits: [T, E] bf16 (logits_is_bf16 != 0) or fp32. topk_weights_out / topk_ids_out may be
 * NULL (the routing result then lives in the workspace only).
 */
size_t moe_b200_fused_moe_workspace_bytes(int T, int E, int top_k, int H, int I);
int moe_b200_fused_moe_forward(const void* x, const void* router_logits, int logits_is_bf16, const void* w13,
                               const void* w2, const void* w13_bias, const void* w2_bias, void* out,
                               float* topk_weights_out, int32_t* topk_ids_out, int T, int E, int top_k, int H, int I,
                               int renormalize, int activation, void* workspace, size_t workspace_bytes,
                               int32_t* status_word, void* stream);

/*
 * Copies the device status word to the host after synchronising `stream`. Returns MOE_B200_OK and
 * stores the word in *value; a non-zero word means a device-side wait timed out
 * (1 operand stage never filled, 2 never drained, 3 accumulator never completed, 4 never released,
 * 6 peer flag never arrived).
 */
int moe_b200_read_status(const int32_t* status_word, int32_t* value, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Tensor-parallel all-reduce over NVLink peer memory.
 * Replaces the custom all-reduce ops (csrc/ops.cpp:77-95, csrc/custom_all_reduce_kernels.cu:15-191,
 * csrc/custom_all_reduce.cuh:372-624). Handles are opaque int64 values, as in the reference (fptr_t).
 * ---------------------------------------------------------------------------------------------- */

/* Bytes of the synchronisation header at the start of every rank's metadata buffer
 * (ops.meta_size, custom_all_reduce_kernels.cu:109). */
int64_t moe_b200_ar_meta_size(void);
/* cudaMalloc + cudaIpcGetMemHandle; writes 64 handle bytes (ops.allocate_shared_buffer_and_handle,
 * custom_all_reduce_kernels.cu:148-179). This one allocates device memory by design. */
int moe_b200_ar_allocate_shared_buffer(int64_t size_bytes, int64_t* ptr_out, uint8_t* handle_out /*[64]*/);
/* cudaIpcOpenMemHandle (ops.open_mem_handle, custom_all_reduce_kernels.cu:181-187). */
int moe_b200_ar_open_mem_handle(const uint8_t* handle /*[64]*/, int64_t* ptr_out);
int moe_b200_ar_close_mem_handle(int64_t ptr);
/* cudaFree (ops.free_shared_buffer, custom_all_reduce_kernels.cu:189-191). */
int moe_b200_ar_free_shared_buffer(int64_t ptr);
/* meta_ptrs[world_size]: every rank's metadata buffer as seen from this process (own pointer at
 * [rank]); each must hold meta_size() + max_size bytes and start zeroed. rank_data: device scratch
 * for registered pointer tuples (ops.init_custom_ar, custom_all_reduce_kernels.cu:15-33). */
int moe_b200_ar_init(const int64_t* meta_ptrs, int world_size, void* rank_data, int64_t rank_data_bytes, int rank,
                     int fully_connected, int64_t* handle_out);
int moe_b200_ar_dispose(int64_t handle);
/* ptrs[world_size]: one IPC-shared buffer per rank (ops.register_buffer, :115-123). */
int moe_b200_ar_register_buffer(int64_t handle, const int64_t* ptrs);
/* Hands the communicator a second registered buffer (same layout of arguments as register_buffer) that only the
 * fused k-slot-sum + one-shot all-reduce uses, as two halves in alternation: that kernel then needs no closing
 * barrier (the next call's opening barrier proves that every peer has finished the previous one). Optional; without
 * it the fused call keeps both barriers. No reference counterpart. bytes: size of the buffer, a multiple of 32. */
int moe_b200_ar_register_fused_buffer(int64_t handle, const int64_t* ptrs, int64_t bytes);
/* Receive areas (one per rank, zero-initialised, used by nothing else) of the flag-in-data one-shot reduction that
 * moe_b200_ar_moe_sum_all_reduce takes for tensors of up to bytes / (4 * world) bytes: every 16-byte vector travels
 * as two packets {data, flag, data, flag} stored straight into the peers' areas, and a receiver polls its own
 * memory, so the call needs no barrier at all. No counterpart in the reference (its kernels all use the two
 * flag barriers of csrc/custom_all_reduce.cuh:199-241). Pass algo = 3 to a reduction to keep it off this path. */
int moe_b200_ar_register_ll_buffer(int64_t handle, const int64_t* ptrs, int64_t bytes);
/* out = sum over ranks of inp (bf16/fp16/fp32 by element_size+is_bf16), fp32 accumulation in rank
 * order, identical bits on every rank. If reg_buffer != 0 the input is first copied there
 * (ops.all_reduce, custom_all_reduce_kernels.cu:64-107). algo: 0 auto (size and world size decide, as in
 * custom_all_reduce.cuh:589-597, unless VLLM_CUSTOM_ALLREDUCE_ALGO forced a choice when the communicator was
 * created), 1 one-shot, 2 two-shot, 3 one-shot with flag barriers (keeps moe_b200_ar_moe_sum_all_reduce off its
 * flag-in-data path). */
int moe_b200_ar_all_reduce(int64_t handle, const void* inp, void* out, int64_t numel, int dtype /*0 bf16,1 f16,2 f32*/,
                           int64_t reg_buffer, int64_t reg_buffer_bytes, int algo, int32_t* status_word, void* stream);
/* k-slot sum of this rank's down-projection output fused with the all-reduce: one launch computes
 * partial[t,:] = bf16(sum_j c3[t,j,:]) into this rank's registered buffer, meets the peers at a flag
 * barrier and reduces across ranks into out. No reference counterpart as a single op: it stands for
 * moe_sum (moe_easy_kernel.py:26-31) followed by tensor_model_parallel_all_reduce
 * (nanovllm/layers/custom_all_reduce.py:343-366). */
int moe_b200_ar_moe_sum_all_reduce(int64_t handle, const void* c3, void* out, int T, int k, int H, int64_t reg_buffer,
                                   int64_t reg_buffer_bytes, int algo, int32_t* status_word, void* stream);
/* Wall-clock limit of every device-side wait on a peer flag (default 2 s). After a wait ran out the
 * status word is non-zero and the communicator's counters are out of step: dispose of it.
 * (The reference spins without limit, csrc/custom_all_reduce.cuh:209,231-234.) */
int moe_b200_ar_set_wait_limit_ns(int64_t handle, uint64_t limit_ns);
/* Launches one thread that waits, with the given limit, on a flag of this rank's metadata buffer that
 * nobody advances: a one-GPU check that a lost peer ends in a status word, not in a hang. No reference
 * counterpart. */
int moe_b200_ar_wait_probe(int64_t meta_ptr, uint64_t limit_ns, int32_t* status_word, void* stream);
/* CUDA-graph support (ops.get_graph_buffer_ipc_meta / register_graph_buffers, :125-146):
 * number of buffers captured since the last registration, their IPC handles (64 bytes each) and offsets. */
int moe_b200_ar_graph_buffer_count(int64_t handle, int* count_out);
int moe_b200_ar_get_graph_buffer_ipc_meta(int64_t handle, uint8_t* handles_out, int64_t* offsets_out, int capacity);
int moe_b200_ar_register_graph_buffers(int64_t handle, const uint8_t* handles /*[world][count][64]*/,
                                       const int64_t* offsets /*[world][count]*/, int count);

/*
 * Whole block on one tensor-parallel rank: router + experts + (moe_sum fused with all-reduce).
 * ar_handle == 0 or world size 1: same as moe_b200_fused_moe_forward.
 */
int moe_b200_fused_moe_forward_tp(const void* x, const void* router_logits, int logits_is_bf16, const void* w13,
                                  const void* w2, const void* w13_bias, const void* w2_bias, void* out, int T, int E,
                                  int top_k, int H, int I, int renormalize, int activation, void* workspace,
                                  size_t workspace_bytes, int64_t ar_handle, int64_t reg_buffer,
                                  int64_t reg_buffer_bytes, int ar_algo, int32_t* status_word, void* stream);

/*
 * All-reduce that ends in the NEXT decoder layer's residual add + RMSNorm, i.e. the reference's sequence
 *   hidden = tensor_model_parallel_all_reduce(hidden)          (nanovllm/layers/fused_moe.py:614-624)
 *   hidden, residual = input_layernorm(hidden, residual)       (nanovllm/models/qwen3_moe.py:262-270, ops.add_rms_norm)
 * in one launch for messages the one-shot algorithm takes (a block reduces whole token rows over the ranks and
 * normalises them; the reduced tensor never goes to memory), and as all-reduce into scratch_out + norm kernel for
 * larger ones. Results are bit-identical to running the two steps. bf16 only.
 *   inp bf16 [T, H] (staged into reg_buffer unless it is reg_buffer itself), residual bf16 [T, H] in/out,
 *   norm_weight bf16 [H], normed_out bf16 [T, H], scratch_out bf16 [T, H] (may be NULL when T*H*2 bytes is within the
 *   one-shot limit: 256 KiB at 8 ranks, 512 KiB at 4, any size at 2).
 * The second form starts from the block's [T, k, H] slot tensor (k-slot sum fused in front); the third is
 * moe_b200_fused_moe_forward_tp with that tail instead of the plain all-reduce.
 */
int moe_b200_ar_all_reduce_add_rms_norm(int64_t handle, const void* inp, void* scratch_out, void* residual,
                                        const void* norm_weight, float eps, void* normed_out, int T, int H,
                                        int64_t reg_buffer, int64_t reg_buffer_bytes, int algo, int32_t* status_word,
                                        void* stream);
int moe_b200_ar_moe_sum_all_reduce_add_rms_norm(int64_t handle, const void* c3, void* scratch_out, void* residual,
                                                const void* norm_weight, float eps, void* normed_out, int T, int k,
                                                int H, int64_t reg_buffer, int64_t reg_buffer_bytes, int algo,
                                                int32_t* status_word, void* stream);
int moe_b200_fused_moe_forward_tp_add_rms_norm(const void* x, const void* router_logits, int logits_is_bf16,
                                               const void* w13, const void* w2, const void* w13_bias,
                                               const void* w2_bias, void* residual, const void* norm_weight, float eps,
                                               void* normed_out, void* scratch_out, int T, int E, int top_k, int H, int I,
                                               int renormalize, int activation, void* workspace, size_t workspace_bytes,
                                               int64_t ar_handle, int64_t reg_buffer, int64_t reg_buffer_bytes,
                                               int ar_algo, int32_t* status_word, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* MOE_B200_H_ */
