// extern "C" layer of libmoe_b200 (declared in include/moe_b200.h): argument checks, workspace
// carving and the launch sequence of the fused MoE block. No torch types, no allocation.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "../../include/moe_b200.h"
#include "moe_b200_internal.cuh"

namespace moe_b200 {

namespace {
thread_local char g_error[512] = "";
}

int set_error(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return status;
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return kStatusOk;
  return set_error(kStatusCudaError, "%s: %s", what, cudaGetErrorString(e));
}

int check_launch(const char* what) { return check_cuda(cudaGetLastError(), what); }

const char* last_error_string() { return g_error; }

namespace {
std::atomic<unsigned long long> g_launches{0};
}
void count_launches(int n) { g_launches.fetch_add(static_cast<unsigned long long>(n), std::memory_order_relaxed); }
unsigned long long launch_count() { return g_launches.load(std::memory_order_relaxed); }

namespace {

constexpr size_t kAlign = 256;
size_t align_up(size_t v) { return (v + kAlign - 1) / kAlign * kAlign; }

// Sizes of the permutation buffers for block size kBlockM.
struct PermSizes {
  int numel;
  int sorted_cap;   // multiple of kBlockM
  int blocks_cap;
};

PermSizes perm_sizes(int T, int E, int top_k) {
  PermSizes s;
  s.numel = T * top_k;
  const int nonempty = s.numel < E ? s.numel : E;
  const long long cap = static_cast<long long>(s.numel) + static_cast<long long>(nonempty) * (kBlockM - 1);
  s.sorted_cap = static_cast<int>((cap + kBlockM - 1) / kBlockM * kBlockM);
  s.blocks_cap = s.sorted_cap / kBlockM;
  return s;
}

struct ExpertsWorkspace {
  int* sorted_ids;
  int* expert_ids;
  int* num_post_pad;
  void* align_ws;
  size_t align_ws_bytes;
  __nv_bfloat16* h_sorted;
  __nv_bfloat16* c3;
  size_t total;
};

ExpertsWorkspace carve_experts(void* base, int T, int E, int top_k, int H, int I) {
  const PermSizes ps = perm_sizes(T, E, top_k);
  uint8_t* p = static_cast<uint8_t*>(base);
  size_t off = 0;
  ExpertsWorkspace w;
  w.sorted_ids = reinterpret_cast<int*>(p + off); off += align_up(sizeof(int) * static_cast<size_t>(ps.sorted_cap > 0 ? ps.sorted_cap : 1));
  w.expert_ids = reinterpret_cast<int*>(p + off); off += align_up(sizeof(int) * static_cast<size_t>(ps.blocks_cap > 0 ? ps.blocks_cap : 1));
  w.num_post_pad = reinterpret_cast<int*>(p + off); off += kAlign;
  w.align_ws_bytes = align_up(align_workspace_bytes(ps.numel, E));
  w.align_ws = p + off; off += w.align_ws_bytes;
  w.h_sorted = reinterpret_cast<__nv_bfloat16*>(p + off); off += align_up(sizeof(__nv_bfloat16) * static_cast<size_t>(ps.sorted_cap) * I);
  w.c3 = reinterpret_cast<__nv_bfloat16*>(p + off); off += align_up(sizeof(__nv_bfloat16) * static_cast<size_t>(ps.numel) * H);
  w.total = off;
  return w;
}

// fp8 path: the bf16 workspace plus the quantised copies of the hidden states and of the permuted intermediate.
struct Fp8Workspace {
  ExpertsWorkspace base;
  uint8_t* x_q;
  float* x_s;
  uint8_t* h_q;
  float* h_s;
  size_t total;
};

Fp8Workspace carve_fp8(void* ws, int T, int E, int top_k, int H, int I) {
  Fp8Workspace w;
  w.base = carve_experts(ws, T, E, top_k, H, I);
  const PermSizes ps = perm_sizes(T, E, top_k);
  uint8_t* p = static_cast<uint8_t*>(ws);
  size_t off = w.base.total;
  const size_t rows_t = static_cast<size_t>(T > 0 ? T : 1);
  const size_t rows_p = static_cast<size_t>(ps.sorted_cap > 0 ? ps.sorted_cap : 1);
  w.x_q = p + off; off += align_up(rows_t * H);
  w.x_s = reinterpret_cast<float*>(p + off); off += align_up(sizeof(float) * rows_t * ((H + 127) / 128));
  w.h_q = p + off; off += align_up(rows_p * I);
  w.h_s = reinterpret_cast<float*>(p + off); off += align_up(sizeof(float) * rows_p * ((I + 127) / 128 + 1));
  w.total = off;
  return w;
}

int check_block_shapes(int T, int E, int top_k, int H, int I) {
  if (T < 0 || E <= 0 || top_k <= 0 || top_k > E || H <= 0 || I <= 0)
    return set_error(kStatusInvalidArgument, "fused MoE: bad sizes T=%d E=%d k=%d H=%d I=%d", T, E, top_k, H, I);
  if (H % 16 != 0 || I % 16 != 0)
    return set_error(kStatusInvalidArgument, "fused MoE: H and the per-rank I must be multiples of 16 (H=%d I=%d)", H, I);
  if (static_cast<long long>(T) * top_k > (1ll << 30))
    return set_error(kStatusInvalidArgument, "fused MoE: T*k too large");
  return kStatusOk;
}

}  // namespace

// Everything of fused_experts up to (not including) the k-slot sum; leaves C3 in the workspace.
int run_experts_until_c3(const void* x, const void* w13, const void* w2, const void* w13_bias, const void* w2_bias,
                         const float* topk_weights, const int* topk_ids, int T, int E, int top_k, int H, int I,
                         int activation, const ExpertsWorkspace& w, int* status_word, cudaStream_t stream) {
  const PermSizes ps = perm_sizes(T, E, top_k);
  if (int st = launch_align_block_size(topk_ids, ps.numel, E, kBlockM, w.sorted_ids, ps.sorted_cap, w.expert_ids,
                                       ps.blocks_cap, w.num_post_pad, w.align_ws, w.align_ws_bytes, stream))
    return st;
  GroupedGemmArgs a{};
  a.sorted_ids = w.sorted_ids; a.expert_ids = w.expert_ids; a.num_post_pad = w.num_post_pad;
  a.numel = ps.numel; a.top_k = top_k; a.max_m_blocks = ps.blocks_cap; a.num_experts = E;
  a.hidden = H; a.inter = I; a.activation = activation; a.act_alpha = 1.702f; a.act_limit = 7.0f;
  a.status = status_word;
  if (int st = launch_grouped_gemm1(a, static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w13),
                                    static_cast<const __nv_bfloat16*>(w13_bias), w.h_sorted, ps.sorted_cap, stream))
    return st;
  return launch_grouped_gemm2(a, w.h_sorted, ps.sorted_cap, static_cast<const __nv_bfloat16*>(w2),
                              static_cast<const __nv_bfloat16*>(w2_bias), topk_weights, w.c3, stream);
}

size_t experts_workspace_bytes(int T, int E, int top_k, int H, int I) {
  return carve_experts(nullptr, T, E, top_k, H, I).total;
}

const __nv_bfloat16* experts_workspace_c3(void* base, int T, int E, int top_k, int H, int I) {
  return carve_experts(base, T, E, top_k, H, I).c3;
}

int run_experts_until_c3_ws(const void* x, const void* w13, const void* w2, const void* w13_bias, const void* w2_bias,
                            const float* topk_weights, const int* topk_ids, int T, int E, int top_k, int H, int I,
                            int activation, void* workspace, int* status_word, cudaStream_t stream) {
  return run_experts_until_c3(x, w13, w2, w13_bias, w2_bias, topk_weights, topk_ids, T, E, top_k, H, I, activation,
                              carve_experts(workspace, T, E, top_k, H, I), status_word, stream);
}

// all_reduce.cu
int ar_moe_sum_all_reduce_impl(int64_t handle, const void* c3, void* out, int T, int k, int H, int64_t reg_buffer,
                               int64_t reg_buffer_bytes, int algo, int* status_word, cudaStream_t stream);
int ar_all_reduce_add_rms_norm_impl(int64_t handle, const void* c3, int k, void* scratch_out, __nv_bfloat16* residual,
                                    const __nv_bfloat16* weight, float eps, __nv_bfloat16* normed, int T, int H,
                                    int64_t reg_buffer, int64_t reg_buffer_bytes, int algo, int* status_word,
                                    cudaStream_t stream);

}  // namespace moe_b200

using namespace moe_b200;

extern "C" {

const char* moe_b200_last_error(void) { return last_error_string(); }
int moe_b200_abi_version(void) { return 1; }
int moe_b200_block_m(void) { return kBlockM; }
uint64_t moe_b200_launch_count(void) { return launch_count(); }

int moe_b200_grouped_gemm_gate_up(const void* x, const void* w13, const void* w13_bias, const int32_t* sorted_token_ids,
                                  const int32_t* expert_ids, const int32_t* num_tokens_post_pad, void* h_sorted,
                                  int rows_cap, int T, int E, int top_k, int H, int I, int activation,
                                  int32_t* status_word, void* stream) {
  if (int st = check_block_shapes(T, E, top_k, H, I)) return st;
  if (x == nullptr || w13 == nullptr || sorted_token_ids == nullptr || expert_ids == nullptr ||
      num_tokens_post_pad == nullptr || h_sorted == nullptr || status_word == nullptr)
    return set_error(kStatusInvalidArgument, "grouped_gemm_gate_up: null pointer");
  if (rows_cap % kBlockM != 0) return set_error(kStatusInvalidArgument, "grouped_gemm_gate_up: rows_cap must be a multiple of %d", kBlockM);
  GroupedGemmArgs a{};
  a.sorted_ids = sorted_token_ids; a.expert_ids = expert_ids; a.num_post_pad = num_tokens_post_pad;
  a.numel = T * top_k; a.top_k = top_k; a.max_m_blocks = rows_cap / kBlockM; a.num_experts = E;
  a.hidden = H; a.inter = I; a.activation = activation; a.act_alpha = 1.702f; a.act_limit = 7.0f; a.status = status_word;
  return launch_grouped_gemm1(a, static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w13),
                              static_cast<const __nv_bfloat16*>(w13_bias), static_cast<__nv_bfloat16*>(h_sorted),
                              rows_cap, static_cast<cudaStream_t>(stream));
}

int moe_b200_grouped_gemm_down(const void* h_sorted, int rows_cap, const void* w2, const void* w2_bias,
                               const float* topk_weights, const int32_t* sorted_token_ids, const int32_t* expert_ids,
                               const int32_t* num_tokens_post_pad, void* c3, int T, int E, int top_k, int H, int I,
                               int32_t* status_word, void* stream) {
  if (int st = check_block_shapes(T, E, top_k, H, I)) return st;
  if (h_sorted == nullptr || w2 == nullptr || topk_weights == nullptr || sorted_token_ids == nullptr ||
      expert_ids == nullptr || num_tokens_post_pad == nullptr || c3 == nullptr || status_word == nullptr)
    return set_error(kStatusInvalidArgument, "grouped_gemm_down: null pointer");
  if (rows_cap % kBlockM != 0) return set_error(kStatusInvalidArgument, "grouped_gemm_down: rows_cap must be a multiple of %d", kBlockM);
  GroupedGemmArgs a{};
  a.sorted_ids = sorted_token_ids; a.expert_ids = expert_ids; a.num_post_pad = num_tokens_post_pad;
  a.numel = T * top_k; a.top_k = top_k; a.max_m_blocks = rows_cap / kBlockM; a.num_experts = E;
  a.hidden = H; a.inter = I; a.activation = 0; a.status = status_word;
  return launch_grouped_gemm2(a, static_cast<const __nv_bfloat16*>(h_sorted), rows_cap,
                              static_cast<const __nv_bfloat16*>(w2), static_cast<const __nv_bfloat16*>(w2_bias),
                              topk_weights, static_cast<__nv_bfloat16*>(c3), static_cast<cudaStream_t>(stream));
}

int moe_b200_topk_softmax(const void* gating, int gating_is_bf16, float* topk_weights, int32_t* topk_ids,
                          int32_t* token_expert_indices, int T, int E, int k, int renormalize, void* stream) {
  if (T > 0 && (gating == nullptr || topk_weights == nullptr || topk_ids == nullptr))
    return set_error(kStatusInvalidArgument, "topk_softmax: null pointer");
  return launch_topk_softmax(gating, gating_is_bf16, topk_weights, topk_ids, token_expert_indices, T, E, k,
                             renormalize, static_cast<cudaStream_t>(stream));
}

size_t moe_b200_align_workspace_bytes(int numel, int E) { return align_workspace_bytes(numel, E); }

int moe_b200_moe_align_block_size(const int32_t* topk_ids, int numel, int E, int block_size,
                                  int32_t* sorted_token_ids, int sorted_cap, int32_t* expert_ids, int expert_ids_cap,
                                  int32_t* num_tokens_post_pad, void* workspace, size_t workspace_bytes,
                                  void* stream) {
  if (sorted_token_ids == nullptr || expert_ids == nullptr || num_tokens_post_pad == nullptr ||
      (numel > 0 && topk_ids == nullptr))
    return set_error(kStatusInvalidArgument, "moe_align_block_size: null pointer");
  if (block_size > 0 && E > 0) {
    const long long need = static_cast<long long>(numel) + static_cast<long long>(numel < E ? numel : E) * (block_size - 1);
    if (sorted_cap < need)
      return set_error(kStatusInvalidArgument, "moe_align_block_size: sorted_token_ids holds %d entries, %lld needed", sorted_cap, need);
    if (static_cast<long long>(expert_ids_cap) * block_size < need)
      return set_error(kStatusInvalidArgument, "moe_align_block_size: expert_ids holds %d entries, too few", expert_ids_cap);
  }
  return launch_align_block_size(topk_ids, numel, E, block_size, sorted_token_ids, sorted_cap, expert_ids,
                                 expert_ids_cap, num_tokens_post_pad, workspace, workspace_bytes,
                                 static_cast<cudaStream_t>(stream));
}

size_t moe_b200_moe_align_static_scratch_bytes(void) { return sizeof(int) * static_cast<size_t>(static_align_scratch_ints()); }

int moe_b200_moe_align_block_size_static(const int32_t* topk_ids, int numel, int E, int block_size,
                                         int32_t* sorted_token_ids, int sorted_cap, int32_t* expert_ids,
                                         int expert_ids_cap, int32_t* num_tokens_post_pad, void* stream) {
  if (sorted_token_ids == nullptr || expert_ids == nullptr || num_tokens_post_pad == nullptr ||
      (numel > 0 && topk_ids == nullptr))
    return set_error(kStatusInvalidArgument, "moe_align_block_size_static: null pointer");
  if (block_size > 0 && E > 0) {
    const long long need = static_cast<long long>(numel) + static_cast<long long>(numel < E ? numel : E) * (block_size - 1);
    if (sorted_cap < need)
      return set_error(kStatusInvalidArgument, "moe_align_block_size_static: sorted_token_ids holds %d entries, %lld needed", sorted_cap, need);
    if (static_cast<long long>(expert_ids_cap) * block_size < need)
      return set_error(kStatusInvalidArgument, "moe_align_block_size_static: expert_ids holds %d entries, too few", expert_ids_cap);
  }
  return launch_align_block_size_static(topk_ids, numel, E, block_size, sorted_token_ids, sorted_cap, expert_ids,
                                        expert_ids_cap, num_tokens_post_pad, static_cast<cudaStream_t>(stream));
}

int moe_b200_silu_and_mul(void* out, const void* in, int rows, int d, void* stream) {
  if (rows > 0 && (out == nullptr || in == nullptr)) return set_error(kStatusInvalidArgument, "silu_and_mul: null pointer");
  return launch_silu_and_mul(static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(in), rows, d,
                             static_cast<cudaStream_t>(stream));
}

int moe_b200_swigluoai_and_mul(void* out, const void* in, int rows, int d, float alpha, float limit, void* stream) {
  if (rows > 0 && (out == nullptr || in == nullptr)) return set_error(kStatusInvalidArgument, "swigluoai_and_mul: null pointer");
  return launch_swigluoai_and_mul(static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(in), rows, d,
                                  alpha, limit, static_cast<cudaStream_t>(stream));
}

int moe_b200_moe_sum(const void* in, void* out, int T, int k, int H, void* stream) {
  if (T > 0 && (out == nullptr || in == nullptr)) return set_error(kStatusInvalidArgument, "moe_sum: null pointer");
  return launch_moe_sum(static_cast<const __nv_bfloat16*>(in), static_cast<__nv_bfloat16*>(out), T, k, H,
                        static_cast<cudaStream_t>(stream));
}

size_t moe_b200_fused_experts_workspace_bytes(int T, int E, int top_k, int H, int I) {
  if (T < 0 || E <= 0 || top_k <= 0 || H <= 0 || I <= 0) return 0;
  return experts_workspace_bytes(T, E, top_k, H, I);
}

int moe_b200_fused_experts(const void* x, const void* w13, const void* w2, const void* w13_bias, const void* w2_bias,
                           const float* topk_weights, const int32_t* topk_ids, void* out, int T, int E, int top_k,
                           int H, int I, int activation, void* workspace, size_t workspace_bytes,
                           int32_t* status_word, void* stream) {
  if (int st = check_block_shapes(T, E, top_k, H, I)) return st;
  if (T == 0) return kStatusOk;
  if (x == nullptr || w13 == nullptr || w2 == nullptr || topk_weights == nullptr || topk_ids == nullptr ||
      out == nullptr || status_word == nullptr)
    return set_error(kStatusInvalidArgument, "fused_experts: null pointer");
  if (activation != MOE_B200_ACT_SILU && activation != MOE_B200_ACT_SWIGLUOAI)
    return set_error(kStatusInvalidArgument, "fused_experts: unsupported activation code %d", activation);
  const size_t need = experts_workspace_bytes(T, E, top_k, H, I);
  if (workspace == nullptr || workspace_bytes < need)
    return set_error(kStatusWorkspaceTooSmall, "fused_experts: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int st = run_experts_until_c3_ws(x, w13, w2, w13_bias, w2_bias, topk_weights, topk_ids, T, E, top_k, H, I,
                                       activation, workspace, status_word, s))
    return st;
  return launch_moe_sum(experts_workspace_c3(workspace, T, E, top_k, H, I), static_cast<__nv_bfloat16*>(out), T, top_k,
                        H, s);
}

int moe_b200_rms_norm(void* out, const void* input, const void* weight, float eps, int T, int H, void* stream) {
  if (out == nullptr || input == nullptr || weight == nullptr) return set_error(kStatusInvalidArgument, "rms_norm: null pointer");
  return launch_rms_norm(static_cast<__nv_bfloat16*>(out), nullptr, static_cast<const __nv_bfloat16*>(input),
                         static_cast<const __nv_bfloat16*>(weight), eps, T, H, static_cast<cudaStream_t>(stream));
}

int moe_b200_add_rms_norm(void* out, void* residual, const void* input, const void* weight, float eps, int T, int H,
                          void* stream) {
  if (out == nullptr || residual == nullptr || input == nullptr || weight == nullptr)
    return set_error(kStatusInvalidArgument, "add_rms_norm: null pointer");
  return launch_rms_norm(static_cast<__nv_bfloat16*>(out), static_cast<__nv_bfloat16*>(residual),
                         static_cast<const __nv_bfloat16*>(input), static_cast<const __nv_bfloat16*>(weight), eps, T, H,
                         static_cast<cudaStream_t>(stream));
}

size_t moe_b200_pre_moe_workspace_bytes(int T, int H, int E) {
  if (T < 0 || H <= 0 || E <= 0) return 0;
  return pre_moe_workspace_bytes(T, H, E);
}

int moe_b200_add_rms_norm_router(const void* input, void* residual, const void* norm_weight, float eps,
                                 const void* gate_weight, void* normed_out, void* logits_out, float* topk_weights,
                                 int32_t* topk_ids, int T, int H, int E, int top_k, int renormalize, void* workspace,
                                 size_t workspace_bytes, int32_t* status_word, void* stream) {
  if (input == nullptr || residual == nullptr || norm_weight == nullptr || gate_weight == nullptr || normed_out == nullptr ||
      topk_weights == nullptr || topk_ids == nullptr || status_word == nullptr)
    return set_error(kStatusInvalidArgument, "add_rms_norm_router: null pointer");
  return launch_add_rms_norm_router(static_cast<const __nv_bfloat16*>(input), static_cast<__nv_bfloat16*>(residual),
                                    static_cast<const __nv_bfloat16*>(norm_weight), eps,
                                    static_cast<const __nv_bfloat16*>(gate_weight), static_cast<__nv_bfloat16*>(normed_out),
                                    static_cast<__nv_bfloat16*>(logits_out), topk_weights, topk_ids, T, H, E, top_k,
                                    renormalize, workspace, workspace_bytes, status_word, static_cast<cudaStream_t>(stream));
}

int moe_b200_quant_fp8_per_token_group(const void* x, int rows, int cols, void* q, float* scales, void* stream) {
  if (x == nullptr || q == nullptr || scales == nullptr) return set_error(kStatusInvalidArgument, "quant_fp8_per_token_group: null pointer");
  return launch_quant_rows_fp8(static_cast<const __nv_bfloat16*>(x), rows, cols, 0, static_cast<uint8_t*>(q), scales, nullptr,
                               0, nullptr, static_cast<cudaStream_t>(stream));
}

size_t moe_b200_fused_experts_fp8_workspace_bytes(int T, int E, int top_k, int H, int I) {
  if (T < 0 || E <= 0 || top_k <= 0 || H <= 0 || I <= 0) return 0;
  return carve_fp8(nullptr, T, E, top_k, H, I).total;
}

// Everything of the fp8 experts up to (not including) the k-slot sum; returns the C3 slot tensor in the workspace.
static int run_experts_fp8_until_c3(const void* x, const void* w13_q, const float* w13_scale, const void* w2_q,
                                    const float* w2_scale, const float* topk_weights, const int32_t* topk_ids, int T, int E,
                                    int top_k, int H, int I, int i_offset, int i_total, void* workspace,
                                    size_t workspace_bytes, int32_t* status_word, cudaStream_t s,
                                    const __nv_bfloat16** c3_out) {
  if (int st = check_block_shapes(T, E, top_k, H, I)) return st;
  if (H % 128 != 0 || I % 64 != 0 || i_total % 128 != 0 || i_offset % 64 != 0 || i_offset < 0 || i_offset + I > i_total)
    return set_error(kStatusInvalidArgument, "fused_experts_fp8: H must be a multiple of 128, the intermediate size %d of 128, this rank's slice [%d, %d) of 64 (H=%d)", i_total, i_offset, i_offset + I, H);
  if (x == nullptr || w13_q == nullptr || w13_scale == nullptr || w2_q == nullptr || w2_scale == nullptr ||
      topk_weights == nullptr || topk_ids == nullptr || status_word == nullptr)
    return set_error(kStatusInvalidArgument, "fused_experts_fp8: null pointer");
  const size_t need = moe_b200_fused_experts_fp8_workspace_bytes(T, E, top_k, H, I);
  if (workspace == nullptr || workspace_bytes < need)
    return set_error(kStatusWorkspaceTooSmall, "fused_experts_fp8: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  const Fp8Workspace w = carve_fp8(workspace, T, E, top_k, H, I);
  const PermSizes ps = perm_sizes(T, E, top_k);
  if (int st = launch_quant_rows_fp8(static_cast<const __nv_bfloat16*>(x), T, H, 0, w.x_q, w.x_s, nullptr, 0, nullptr, s)) return st;
  if (int st = launch_align_block_size(topk_ids, ps.numel, E, kBlockM, w.base.sorted_ids, ps.sorted_cap, w.base.expert_ids,
                                       ps.blocks_cap, w.base.num_post_pad, w.base.align_ws, w.base.align_ws_bytes, s))
    return st;
  GroupedGemmArgs a{};
  a.sorted_ids = w.base.sorted_ids; a.expert_ids = w.base.expert_ids; a.num_post_pad = w.base.num_post_pad;
  a.numel = ps.numel; a.top_k = top_k; a.max_m_blocks = ps.blocks_cap; a.num_experts = E;
  a.hidden = H; a.inter = I; a.activation = 0; a.status = status_word;
  if (int st = launch_grouped_gemm1_fp8(a, w.x_q, w.x_s, static_cast<const uint8_t*>(w13_q), w13_scale, i_offset, i_total,
                                        w.base.h_sorted, s))
    return st;
  if (int st = launch_quant_rows_fp8(w.base.h_sorted, ps.sorted_cap, I, i_offset % 128, w.h_q, w.h_s, w.base.sorted_ids,
                                     ps.numel, w.base.num_post_pad, s))
    return st;
  if (int st = launch_grouped_gemm2_fp8(a, w.h_q, w.h_s, static_cast<const uint8_t*>(w2_q), w2_scale, i_offset, i_total,
                                        topk_weights, w.base.c3, s))
    return st;
  *c3_out = w.base.c3;
  return kStatusOk;
}

int moe_b200_fused_experts_fp8_tp(const void* x, const void* w13_q, const float* w13_scale, const void* w2_q,
                                  const float* w2_scale, const float* topk_weights, const int32_t* topk_ids, void* out,
                                  int T, int E, int top_k, int H, int I, int i_offset, int i_total, void* workspace,
                                  size_t workspace_bytes, int32_t* status_word, void* stream) {
  if (T == 0) return check_block_shapes(T, E, top_k, H, I);
  if (out == nullptr) return set_error(kStatusInvalidArgument, "fused_experts_fp8: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* c3 = nullptr;
  if (int st = run_experts_fp8_until_c3(x, w13_q, w13_scale, w2_q, w2_scale, topk_weights, topk_ids, T, E, top_k, H, I,
                                        i_offset, i_total, workspace, workspace_bytes, status_word, s, &c3))
    return st;
  return launch_moe_sum(c3, static_cast<__nv_bfloat16*>(out), T, top_k, H, s);
}

int moe_b200_fused_experts_fp8_tp_reduce(const void* x, const void* w13_q, const float* w13_scale, const void* w2_q,
                                         const float* w2_scale, const float* topk_weights, const int32_t* topk_ids,
                                         void* out, int T, int E, int top_k, int H, int I, int i_offset, int i_total,
                                         void* workspace, size_t workspace_bytes, int64_t ar_handle, int64_t reg_buffer,
                                         int64_t reg_buffer_bytes, int ar_algo, int32_t* status_word, void* stream) {
  if (T == 0) return check_block_shapes(T, E, top_k, H, I);
  if (out == nullptr || ar_handle == 0) return set_error(kStatusInvalidArgument, "fused_experts_fp8_tp_reduce: null pointer or no communicator");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* c3 = nullptr;
  if (int st = run_experts_fp8_until_c3(x, w13_q, w13_scale, w2_q, w2_scale, topk_weights, topk_ids, T, E, top_k, H, I,
                                        i_offset, i_total, workspace, workspace_bytes, status_word, s, &c3))
    return st;
  return ar_moe_sum_all_reduce_impl(ar_handle, c3, out, T, top_k, H, reg_buffer, reg_buffer_bytes, ar_algo, status_word, s);
}

int moe_b200_fused_experts_fp8(const void* x, const void* w13_q, const float* w13_scale, const void* w2_q,
                               const float* w2_scale, const float* topk_weights, const int32_t* topk_ids, void* out,
                               int T, int E, int top_k, int H, int I, void* workspace, size_t workspace_bytes,
                               int32_t* status_word, void* stream) {
  return moe_b200_fused_experts_fp8_tp(x, w13_q, w13_scale, w2_q, w2_scale, topk_weights, topk_ids, out, T, E, top_k, H,
                                       I, 0, I, workspace, workspace_bytes, status_word, stream);
}

size_t moe_b200_fused_moe_workspace_bytes(int T, int E, int top_k, int H, int I) {
  if (T < 0 || E <= 0 || top_k <= 0 || H <= 0 || I <= 0) return 0;
  const size_t routing = 2 * align_up(sizeof(float) * static_cast<size_t>(T > 0 ? T : 1) * top_k);
  return routing + experts_workspace_bytes(T, E, top_k, H, I);
}

int moe_b200_fused_moe_forward(const void* x, const void* router_logits, int logits_is_bf16, const void* w13,
                               const void* w2, const void* w13_bias, const void* w2_bias, void* out,
                               float* topk_weights_out, int32_t* topk_ids_out, int T, int E, int top_k, int H, int I,
                               int renormalize, int activation, void* workspace, size_t workspace_bytes,
                               int32_t* status_word, void* stream) {
  if (int st = check_block_shapes(T, E, top_k, H, I)) return st;
  if (T == 0) return kStatusOk;
  if (router_logits == nullptr) return set_error(kStatusInvalidArgument, "fused_moe_forward: null router_logits");
  const size_t need = moe_b200_fused_moe_workspace_bytes(T, E, top_k, H, I);
  if (workspace == nullptr || workspace_bytes < need)
    return set_error(kStatusWorkspaceTooSmall, "fused_moe_forward: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  uint8_t* base = static_cast<uint8_t*>(workspace);
  const size_t slot = align_up(sizeof(float) * static_cast<size_t>(T) * top_k);
  float* tw = topk_weights_out ? topk_weights_out : reinterpret_cast<float*>(base);
  int32_t* ti = topk_ids_out ? topk_ids_out : reinterpret_cast<int32_t*>(base + slot);
  if (int st = launch_topk_softmax(router_logits, logits_is_bf16, tw, ti, nullptr, T, E, top_k, renormalize,
                                   static_cast<cudaStream_t>(stream)))
    return st;
  return moe_b200_fused_experts(x, w13, w2, w13_bias, w2_bias, tw, ti, out, T, E, top_k, H, I, activation,
                                base + 2 * slot, workspace_bytes - 2 * slot, status_word, stream);
}

int moe_b200_fused_moe_forward_tp(const void* x, const void* router_logits, int logits_is_bf16, const void* w13,
                                  const void* w2, const void* w13_bias, const void* w2_bias, void* out, int T, int E,
                                  int top_k, int H, int I, int renormalize, int activation, void* workspace,
                                  size_t workspace_bytes, int64_t ar_handle, int64_t reg_buffer,
                                  int64_t reg_buffer_bytes, int ar_algo, int32_t* status_word, void* stream) {
  if (ar_handle == 0)
    return moe_b200_fused_moe_forward(x, router_logits, logits_is_bf16, w13, w2, w13_bias, w2_bias, out, nullptr,
                                      nullptr, T, E, top_k, H, I, renormalize, activation, workspace, workspace_bytes,
                                      status_word, stream);
  if (int st = check_block_shapes(T, E, top_k, H, I)) return st;
  if (T == 0) return kStatusOk;
  if (x == nullptr || router_logits == nullptr || w13 == nullptr || w2 == nullptr || out == nullptr ||
      status_word == nullptr)
    return set_error(kStatusInvalidArgument, "fused_moe_forward_tp: null pointer");
  if (activation != MOE_B200_ACT_SILU && activation != MOE_B200_ACT_SWIGLUOAI)
    return set_error(kStatusInvalidArgument, "fused_moe_forward_tp: unsupported activation code %d", activation);
  const size_t need = moe_b200_fused_moe_workspace_bytes(T, E, top_k, H, I);
  if (workspace == nullptr || workspace_bytes < need)
    return set_error(kStatusWorkspaceTooSmall, "fused_moe_forward_tp: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* base = static_cast<uint8_t*>(workspace);
  const size_t slot = align_up(sizeof(float) * static_cast<size_t>(T) * top_k);
  float* tw = reinterpret_cast<float*>(base);
  int32_t* ti = reinterpret_cast<int32_t*>(base + slot);
  if (int st = launch_topk_softmax(router_logits, logits_is_bf16, tw, ti, nullptr, T, E, top_k, renormalize, s)) return st;
  void* ews = base + 2 * slot;
  if (int st = run_experts_until_c3_ws(x, w13, w2, w13_bias, w2_bias, tw, ti, T, E, top_k, H, I, activation, ews,
                                       status_word, s))
    return st;
  return ar_moe_sum_all_reduce_impl(ar_handle, experts_workspace_c3(ews, T, E, top_k, H, I), out, T, top_k, H,
                                    reg_buffer, reg_buffer_bytes, ar_algo, status_word, s);
}

int moe_b200_fused_moe_forward_tp_add_rms_norm(const void* x, const void* router_logits, int logits_is_bf16,
                                               const void* w13, const void* w2, const void* w13_bias,
                                               const void* w2_bias, void* residual, const void* norm_weight, float eps,
                                               void* normed_out, void* scratch_out, int T, int E, int top_k, int H, int I,
                                               int renormalize, int activation, void* workspace, size_t workspace_bytes,
                                               int64_t ar_handle, int64_t reg_buffer, int64_t reg_buffer_bytes,
                                               int ar_algo, int32_t* status_word, void* stream) {
  if (int st = check_block_shapes(T, E, top_k, H, I)) return st;
  if (T == 0) return kStatusOk;
  if (x == nullptr || router_logits == nullptr || w13 == nullptr || w2 == nullptr || residual == nullptr ||
      norm_weight == nullptr || normed_out == nullptr || status_word == nullptr || ar_handle == 0)
    return set_error(kStatusInvalidArgument, "fused_moe_forward_tp_add_rms_norm: null pointer or no communicator");
  if (activation != MOE_B200_ACT_SILU && activation != MOE_B200_ACT_SWIGLUOAI)
    return set_error(kStatusInvalidArgument, "fused_moe_forward_tp_add_rms_norm: unsupported activation code %d", activation);
  const size_t need = moe_b200_fused_moe_workspace_bytes(T, E, top_k, H, I);
  if (workspace == nullptr || workspace_bytes < need)
    return set_error(kStatusWorkspaceTooSmall, "fused_moe_forward_tp_add_rms_norm: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* base = static_cast<uint8_t*>(workspace);
  const size_t slot = align_up(sizeof(float) * static_cast<size_t>(T) * top_k);
  float* tw = reinterpret_cast<float*>(base);
  int32_t* ti = reinterpret_cast<int32_t*>(base + slot);
  if (int st = launch_topk_softmax(router_logits, logits_is_bf16, tw, ti, nullptr, T, E, top_k, renormalize, s)) return st;
  void* ews = base + 2 * slot;
  if (int st = run_experts_until_c3_ws(x, w13, w2, w13_bias, w2_bias, tw, ti, T, E, top_k, H, I, activation, ews,
                                       status_word, s))
    return st;
  return ar_all_reduce_add_rms_norm_impl(ar_handle, experts_workspace_c3(ews, T, E, top_k, H, I), top_k, scratch_out,
                                         static_cast<__nv_bfloat16*>(residual), static_cast<const __nv_bfloat16*>(norm_weight),
                                         eps, static_cast<__nv_bfloat16*>(normed_out), T, H, reg_buffer, reg_buffer_bytes,
                                         ar_algo, status_word, s);
}

int moe_b200_read_status(const int32_t* status_word, int32_t* value, void* stream) {
  if (status_word == nullptr || value == nullptr) return set_error(kStatusInvalidArgument, "read_status: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int st = check_cuda(cudaMemcpyAsync(value, status_word, sizeof(int32_t), cudaMemcpyDeviceToHost, s), "read_status copy")) return st;
  return check_cuda(cudaStreamSynchronize(s), "read_status synchronize");
}

}  // extern "C"
