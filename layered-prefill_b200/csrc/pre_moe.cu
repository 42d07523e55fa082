// The decoder layer's steps right in front of the MoE block, as the reference's Qwen3MoeDecoderLayer runs them
// (nanovllm/models/qwen3_moe.py:276-282 and :100-110):
//   hidden, residual = post_attention_layernorm(hidden, residual)     ops.add_rms_norm, csrc/layernorm_kernels.cu:76-107
//   router_logits    = gate(hidden)                                   bf16 linear [T,H] x [E,H]^T, layers/linear.py:53-60
//   topk_weights/ids = softmax + top-k (+ renormalise)                the routing kernel of this library
// For decode-sized batches one kernel does all three per token row (a cluster of eight CTAs per row): the
// normalised row stays in shared memory, each CTA forms an eighth of the E dot products with the lanes striding
// along H and hands them to the first CTA through distributed shared memory, whose first warp picks the experts. For large batches the same results come from three launches: the norm kernel, the tensor-core
// grouped GEMM of this library run as a plain GEMM (one "expert" = the gate weight, identity permutation), and
// the routing kernel.
//
// The norm is bit-identical to the reference kernel, which needs its summation order: reference thread `tid` of
// min(H, 1024) accumulates x[tid], x[tid + 1024], ... with fused multiply-adds, a warp adds its 32 partials in
// an xor butterfly (16, 8, 4, 2, 1), warp 0 adds the warp sums the same way (csrc/reduction_utils.cuh:61-86).
// Here a thread owns 8 consecutive reference threads (16-byte accesses), so butterfly steps 16 and 8 are
// shuffles across 4 neighbouring threads and steps 4, 2, 1 are adds inside the thread, in that order.
#include <cmath>

#include "launch.cuh"
#include "moe_b200_internal.cuh"
#include "ptx.cuh"
#include "rms_norm_row.cuh"
#include "routing_core.cuh"

namespace moe_b200 {

namespace {

template <bool kAdd>
__global__ void __launch_bounds__(kNormThreads)
rms_norm_kernel(__nv_bfloat16* out, __nv_bfloat16* residual, const __nv_bfloat16* input,  // out may be input
                const __nv_bfloat16* __restrict__ weight, float eps, int H) {
  extern __shared__ uint4 norm_smem[];
  grid_dependency_launch();
  grid_dependency_wait();
  __nv_bfloat16* x_row = reinterpret_cast<__nv_bfloat16*>(norm_smem);
  float* red = reinterpret_cast<float*>(x_row + H);
  if (threadIdx.x < 33) red[threadIdx.x] = 0.f;
  __syncthreads();
  const size_t off = static_cast<size_t>(blockIdx.x) * H;
  const __nv_bfloat16* in_row = input + off;
  rms_norm_row<kAdd, kNormThreads, false>([in_row](int c) { return *reinterpret_cast<const uint4*>(in_row + c); },
                                          kAdd ? residual + off : nullptr, weight, out + off, H, eps, x_row, red, red + 32,
                                          true);
}

// Decode-sized batches: a cluster of 8 CTAs per token row. Every CTA forms the normalised row in its own shared
// memory (the row is 4 KB; re-reading the gate weight per row is what costs, so that is what is split), computes
// E/8 of the gate logits with its four warps, and stores them into CTA 0's shared memory; after the cluster
// barrier CTA 0's first warp runs the routing. (One CTA per row took 17 us at T=64: 512 KB of gate weight through
// one SM; the reference's three launches take 12 us.)
constexpr int kClusterCtas = 8;
constexpr int kClusterThreads = 128;

template <int E>
__global__ void __launch_bounds__(kClusterThreads)
pre_moe_cluster_kernel(const __nv_bfloat16* input, __nv_bfloat16* residual, const __nv_bfloat16* __restrict__ norm_weight,
                       float eps, const __nv_bfloat16* __restrict__ gate_weight, __nv_bfloat16* normed,
                       __nv_bfloat16* __restrict__ logits_out, float* __restrict__ topk_w, int* __restrict__ topk_ids, int T,
                       int H, int k, int renormalize) {
  extern __shared__ uint4 fused_smem[];
  grid_dependency_launch();
  grid_dependency_wait();
  __nv_bfloat16* x_row = reinterpret_cast<__nv_bfloat16*>(fused_smem);
  float* red = reinterpret_cast<float*>(x_row + H);
  float* logit_s = red + 40;
  const uint32_t rank = cluster_ctarank();
  const int row = blockIdx.x / kClusterCtas;
  const size_t off = static_cast<size_t>(row) * H;
  const __nv_bfloat16* in_row = input + off;
  rms_norm_row<true, kClusterThreads, true>([in_row](int c) { return *reinterpret_cast<const uint4*>(in_row + c); },
                                            residual + off, norm_weight, normed + off, H, eps, x_row, red, red + 32,
                                            rank == 0);
  __syncthreads();

  // gate projection: this CTA's E/8 experts, E/32 per warp in groups of four; a lane covers 8 columns of every
  // 256-column slice of the row
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  constexpr int kPerCta = E / kClusterCtas;
  constexpr int kPerWarp = kPerCta / 4;
  const int slices = H / 256;
  for (int e0 = static_cast<int>(rank) * kPerCta + warp * kPerWarp; e0 < static_cast<int>(rank) * kPerCta + (warp + 1) * kPerWarp;
       e0 += 4) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int c = 0; c < slices; ++c) {
      Bf16x8 xv;
      xv.u = *reinterpret_cast<const uint4*>(x_row + 256 * c + 8 * lane);
      Bf16x8 wv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        wv[u].u = __ldg(reinterpret_cast<const uint4*>(gate_weight + static_cast<size_t>(e0 + u) * H + 256 * c + 8 * lane));
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[u] = fmaf(__bfloat162float(xv.h[i]), __bfloat162float(wv[u].h[i]), acc[u]);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
#pragma unroll
      for (int mask = 16; mask > 0; mask >>= 1) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], mask);
    }
    if (lane < 4) {
      const float mine = lane == 0 ? acc[0] : lane == 1 ? acc[1] : lane == 2 ? acc[2] : acc[3];
      const __nv_bfloat16 l = __float2bfloat16_rn(mine);  // the linear layer's bf16 output
      st_cluster_f32(&logit_s[e0 + lane], 0, __bfloat162float(l));
      if (logits_out != nullptr) logits_out[static_cast<size_t>(row) * E + e0 + lane] = l;
    }
  }
  cluster_sync_all();  // every CTA's logits have landed in CTA 0; nobody leaves before CTA 0 could be written

  if (rank == 0 && warp == 0) {
    using S = TopkShape<E>;
    static_assert(S::kThreadsPerRow == 32, "one warp routes the row");
    float v[S::kVpt];
#pragma unroll
    for (int ii = 0; ii < S::kVecsPerThread; ++ii)
#pragma unroll
      for (int j = 0; j < S::kEltsPerLdg; ++j)
        v[ii * S::kEltsPerLdg + j] = logit_s[lane * S::kEltsPerLdg + ii * S::kColsPerGroupLdg + j];
    topk_softmax_row<E>(v, lane, true, row, T, k, renormalize, topk_w, topk_ids, nullptr);
  }
}

// identity permutation + unit routed weights, so that the grouped down-pass kernel computes a plain [T, K] x [N, K]^T
__global__ void identity_routing_kernel(int* sorted_ids, int* expert_ids, int* num_post_pad, float* ones, int T, int T_pad) {
  grid_dependency_launch();
  grid_dependency_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < T_pad) sorted_ids[i] = i < T ? i : T;
  if (i < T) ones[i] = 1.0f;
  if (i < T_pad / kBlockM) expert_ids[i] = 0;
  if (i == 0) *num_post_pad = T_pad;
}

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

struct PreMoeWorkspace {
  int* sorted_ids;
  int* expert_ids;
  int* num_post_pad;
  float* ones;
  __nv_bfloat16* logits;
  size_t total;
};

PreMoeWorkspace carve_pre_moe(void* base, int T, int E) {
  const int t_pad = (T + kBlockM - 1) / kBlockM * kBlockM;
  uint8_t* p = static_cast<uint8_t*>(base);
  size_t off = 0;
  PreMoeWorkspace w;
  w.sorted_ids = reinterpret_cast<int*>(p + off); off += align256(sizeof(int) * static_cast<size_t>(t_pad > 0 ? t_pad : 1));
  w.expert_ids = reinterpret_cast<int*>(p + off); off += align256(sizeof(int) * static_cast<size_t>(t_pad / kBlockM + 1));
  w.num_post_pad = reinterpret_cast<int*>(p + off); off += 256;
  w.ones = reinterpret_cast<float*>(p + off); off += align256(sizeof(float) * static_cast<size_t>(T > 0 ? T : 1));
  w.logits = reinterpret_cast<__nv_bfloat16*>(p + off); off += align256(sizeof(__nv_bfloat16) * static_cast<size_t>(T > 0 ? T : 1) * E);
  w.total = off;
  return w;
}

bool fused_shape_ok(int T, int H, int E) {
  return (E == 128 || E == 256) && H % 256 == 0 && H <= 16384 && T <= 512;
}

}  // namespace

size_t pre_moe_workspace_bytes(int T, int H, int E) {
  (void)H;
  return carve_pre_moe(nullptr, T, E).total;
}

int launch_rms_norm(__nv_bfloat16* out, __nv_bfloat16* residual, const __nv_bfloat16* input, const __nv_bfloat16* weight,
                    float eps, int T, int H, cudaStream_t stream) {
  if (T < 0 || H <= 0 || H % 8 != 0) return set_error(kStatusInvalidArgument, "rms_norm: hidden size must be a multiple of 8 (got %d)", H);
  if (T == 0) return kStatusOk;
  const size_t smem = static_cast<size_t>(H) * 2 + 40 * sizeof(float);
  if (smem > 48 * 1024) return set_error(kStatusInvalidArgument, "rms_norm: hidden size %d is above this kernel's 24000", H);
  const cudaError_t e = residual != nullptr
                            ? launch_pdl(rms_norm_kernel<true>, dim3(T), dim3(kNormThreads), smem, stream, out, residual, input, weight, eps, H)
                            : launch_pdl(rms_norm_kernel<false>, dim3(T), dim3(kNormThreads), smem, stream, out, residual, input, weight, eps, H);
  if (int st = check_cuda(e, "rms_norm launch")) return st;
  count_launches(1);
  return check_launch("rms_norm");
}

int launch_add_rms_norm_router(const __nv_bfloat16* input, __nv_bfloat16* residual, const __nv_bfloat16* norm_weight, float eps,
                               const __nv_bfloat16* gate_weight, __nv_bfloat16* normed, __nv_bfloat16* logits_out,
                               float* topk_w, int* topk_ids, int T, int H, int E, int top_k, int renormalize,
                               void* workspace, size_t workspace_bytes, int* status_word, cudaStream_t stream) {
  if (T < 0 || H <= 0 || E <= 0 || top_k <= 0 || top_k > E || H % 16 != 0)
    return set_error(kStatusInvalidArgument, "add_rms_norm_router: bad sizes T=%d H=%d E=%d k=%d (H must be a multiple of 16)", T, H, E, top_k);
  if (T == 0) return kStatusOk;
  if (fused_shape_ok(T, H, E)) {
    const size_t smem = static_cast<size_t>(H) * 2 + (40 + E) * sizeof(float);
    const dim3 grid(static_cast<unsigned>(T) * kClusterCtas);
    const cudaError_t e =
        E == 128 ? launch_pdl_cluster(pre_moe_cluster_kernel<128>, grid, dim3(kClusterThreads), smem, stream, kClusterCtas, input,
                                      residual, norm_weight, eps, gate_weight, normed, logits_out, topk_w, topk_ids, T, H,
                                      top_k, renormalize)
                 : launch_pdl_cluster(pre_moe_cluster_kernel<256>, grid, dim3(kClusterThreads), smem, stream, kClusterCtas, input,
                                      residual, norm_weight, eps, gate_weight, normed, logits_out, topk_w, topk_ids, T, H,
                                      top_k, renormalize);
    if (int st = check_cuda(e, "pre_moe_cluster launch")) return st;
    count_launches(1);
    return check_launch("pre_moe_cluster");
  }
  // large batches (or other expert counts): norm, tensor-core GEMM, routing as three launches
  if (E % 16 != 0) return set_error(kStatusInvalidArgument, "add_rms_norm_router: the expert count must be a multiple of 16 (got %d)", E);
  const size_t need = pre_moe_workspace_bytes(T, H, E);
  if (workspace == nullptr || workspace_bytes < need)
    return set_error(kStatusWorkspaceTooSmall, "add_rms_norm_router: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  const PreMoeWorkspace w = carve_pre_moe(workspace, T, E);
  const int t_pad = (T + kBlockM - 1) / kBlockM * kBlockM;
  if (int st = launch_rms_norm(normed, residual, input, norm_weight, eps, T, H, stream)) return st;
  if (int st = check_cuda(launch_pdl(identity_routing_kernel, dim3((t_pad + 255) / 256), dim3(256), 0, stream, w.sorted_ids,
                                     w.expert_ids, w.num_post_pad, w.ones, T, t_pad),
                          "identity_routing launch"))
    return st;
  count_launches(1);
  __nv_bfloat16* logits = logits_out != nullptr ? logits_out : w.logits;
  GroupedGemmArgs a{};
  a.sorted_ids = w.sorted_ids; a.expert_ids = w.expert_ids; a.num_post_pad = w.num_post_pad;
  a.numel = T; a.top_k = 1; a.max_m_blocks = t_pad / kBlockM; a.num_experts = 1;
  a.hidden = E; a.inter = H; a.activation = 0; a.status = status_word;
  // "down" pass with K = H and N = E: logits[t, :] = bf16((normed[t] . gate_weight^T) * 1.0)
  if (int st = launch_grouped_gemm2(a, normed, t_pad, gate_weight, nullptr, w.ones, logits, stream)) return st;
  return launch_topk_softmax(logits, 1, topk_w, topk_ids, nullptr, T, E, top_k, renormalize, stream);
}

}  // namespace moe_b200
