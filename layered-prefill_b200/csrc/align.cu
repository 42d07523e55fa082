// moe_align_block_size: token-to-expert permutation padded to a block size.
//
// Same outputs as the reference op (csrc/moe_align_block_size_kernels.cu:140-291):
//   sorted_token_ids[cumsum[e] + r] = r-th flat index i = t*k + j routed to expert e,
//   every other slot = numel, expert_ids[b] = owner of block b (0 past the end),
//   num_tokens_post_pad = sum of per-expert counts rounded up to block_size.
// Differences in how it gets there: the scatter is a stable counting sort (the r-th index
// is the r-th in ascending order, where the reference's atomicAdd scatter leaves the order
// to arrival time), and for large inputs the histogram and the scatter run on many CTAs
// (one per 1024 flat indices) around a one-CTA scan, instead of one CTA for everything.
// Three size classes: up to 1024 flat indices and 256 experts (decode) one CTA that ranks by warp match,
// up to 4096 one CTA with warp-ordered placement, above that the three multi-CTA kernels.
#include "launch.cuh"
#include "moe_b200_internal.cuh"

namespace moe_b200 {

namespace {

constexpr int kThreads = 1024;
constexpr int kMaxExperts = 1024;
constexpr int kSmallNumel = 4096;  // up to here one CTA does the whole job in one launch

__device__ __forceinline__ int ceil_to(int v, int b) { return (v + b - 1) / b * b; }

// Exclusive scan of one value per thread over the whole 1024-thread block.
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_totals, int* total_out) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += n;
  }
  if (lane == 31) warp_totals[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int t = warp_totals[lane];
    int ti = t;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, ti, d);
      if (lane >= d) ti += n;
    }
    warp_totals[lane] = ti - t;  // exclusive prefix of warp totals
    if (lane == 31) *total_out = ti;
  }
  __syncthreads();
  return warp_totals[warp] + incl - v;
}

// Stable placement of up to 1024 consecutive flat indices [base, base+1024). running[e] holds the
// next free slot of expert e and is advanced. Warps take turns in index order, so within an
// expert the slots are handed out in ascending flat index.
__device__ __forceinline__ void stable_place_chunk(const int* __restrict__ topk_ids, int base, int numel, int E,
                                                   int* running, int* __restrict__ sorted_ids) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int i = base + threadIdx.x;
  int e = -1;
  if (i < numel) {
    const int id = topk_ids[i];
    if (id >= 0 && id < E) e = id;
  }
  const int key = e >= 0 ? e : -1 - lane;  // lanes without a valid expert match nobody
  const unsigned peers = __match_any_sync(0xffffffffu, key);
  const int rank = __popc(peers & ((1u << lane) - 1u));
  const int leader = __ffs(peers) - 1;
  int slot = 0;
  // warps past the end of the input hold no index: the turn-taking stops at the last warp that does
  const int live_warps = min(kThreads / 32, (numel - base + 31) / 32);
  for (int w = 0; w < live_warps; ++w) {
    if (warp == w) {
      if (e >= 0 && lane == leader) {
        slot = running[e];
        running[e] = slot + __popc(peers);
      }
      slot = __shfl_sync(0xffffffffu, slot, leader);
    }
    __syncthreads();
  }
  if (e >= 0) sorted_ids[slot + rank] = i;
}

// cumsum[e] given padded counts; also writes expert_ids, its zero tail and num_post_pad.
__device__ __forceinline__ int scan_and_publish(int count, int E, int block_size, int sorted_cap, int expert_ids_cap,
                                                int* __restrict__ expert_ids, int* __restrict__ num_post_pad,
                                                int* warp_totals, int* total_smem) {
  const int e = threadIdx.x;
  const int padded = e < E ? ceil_to(count, block_size) : 0;
  const int start = block_exclusive_scan(padded, warp_totals, total_smem);
  const int total = *total_smem;
  if (e < E) {
    for (int i = start; i < start + padded; i += block_size) expert_ids[i / block_size] = e;
  }
  for (int b = total / block_size + threadIdx.x; b < expert_ids_cap; b += kThreads) expert_ids[b] = 0;
  if (threadIdx.x == 0) *num_post_pad = total;
  (void)sorted_cap;
  return start;
}

__global__ void __launch_bounds__(kThreads)
align_single_cta_kernel(const int* __restrict__ topk_ids, int numel, int E, int block_size,
                        int* __restrict__ sorted_ids, int sorted_cap, int* __restrict__ expert_ids, int expert_ids_cap,
                        int* __restrict__ num_post_pad) {
  __shared__ int counts[kMaxExperts];
  __shared__ int warp_totals[32];
  __shared__ int total_smem;
  grid_dependency_launch();
  grid_dependency_wait();

  for (int i = threadIdx.x; i < sorted_cap; i += kThreads) sorted_ids[i] = numel;
  for (int e = threadIdx.x; e < E; e += kThreads) counts[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < numel; i += kThreads) {
    const int id = topk_ids[i];
    if (id >= 0 && id < E) atomicAdd(&counts[id], 1);
  }
  __syncthreads();
  const int my_count = threadIdx.x < E ? counts[threadIdx.x] : 0;
  const int start = scan_and_publish(my_count, E, block_size, sorted_cap, expert_ids_cap, expert_ids, num_post_pad,
                                     warp_totals, &total_smem);
  __syncthreads();  // the fill of sorted_ids above is complete for every thread before any placement
  if (threadIdx.x < E) counts[threadIdx.x] = start;  // counts[] now = next free slot per expert
  __syncthreads();
  for (int base = 0; base < numel; base += kThreads) stable_place_chunk(topk_ids, base, numel, E, counts, sorted_ids);
}

// Decode-sized inputs (up to 1024 flat indices, one per thread; up to 256 experts): no turn-taking at all. A warp
// ranks its 32 indices among themselves with one match instruction, per-warp counts go to a [warp][expert] table,
// one thread per expert turns its column into a prefix over the warps, and an index lands at
// cumsum[expert] + (indices of that expert in earlier warps) + (rank inside its warp): ascending order again.
constexpr int kTinyExperts = 256;

__global__ void __launch_bounds__(kThreads)
align_tiny_kernel(const int* __restrict__ topk_ids, int numel, int E, int block_size, int* __restrict__ sorted_ids,
                  int sorted_cap, int* __restrict__ expert_ids, int expert_ids_cap, int* __restrict__ num_post_pad) {
  __shared__ int warp_cnt[32 * kTinyExperts];  // [warp][expert]
  __shared__ int counts[kTinyExperts];
  __shared__ int warp_totals[32];
  __shared__ int total_smem;
  grid_dependency_launch();
  grid_dependency_wait();

  const int i = threadIdx.x;
  const int lane = i & 31;
  const int warp = i >> 5;
  const int live_warps = (numel + 31) / 32;
  for (int s = threadIdx.x; s < sorted_cap; s += kThreads) sorted_ids[s] = numel;
  for (int c = threadIdx.x; c < live_warps * E; c += kThreads) warp_cnt[(c / E) * kTinyExperts + c % E] = 0;
  int e = -1;
  if (i < numel) {
    const int id = topk_ids[i];
    if (id >= 0 && id < E) e = id;
  }
  __syncthreads();
  int rank = 0;
  if (warp < live_warps) {
    const int key = e >= 0 ? e : -1 - lane;  // lanes without a valid expert match nobody
    const unsigned peers = __match_any_sync(0xffffffffu, key);
    rank = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0 && rank == 0) warp_cnt[warp * kTinyExperts + e] = __popc(peers);
  }
  __syncthreads();
  int my_count = 0;
  if (threadIdx.x < E) {
    for (int w = 0; w < live_warps; ++w) {
      const int c = warp_cnt[w * kTinyExperts + threadIdx.x];
      warp_cnt[w * kTinyExperts + threadIdx.x] = my_count;
      my_count += c;
    }
  }
  const int start = scan_and_publish(my_count, E, block_size, sorted_cap, expert_ids_cap, expert_ids, num_post_pad,
                                     warp_totals, &total_smem);
  if (threadIdx.x < E) counts[threadIdx.x] = start;
  __syncthreads();  // also orders the fill of sorted_ids above before the placements below
  if (e >= 0) sorted_ids[counts[e] + warp_cnt[warp * kTinyExperts + e] + rank] = i;
}

// ---- large inputs: histogram per 1024-index chunk / one-CTA scan / stable scatter per chunk
__global__ void __launch_bounds__(kThreads)
align_chunk_hist_kernel(const int* __restrict__ topk_ids, int numel, int E, int* __restrict__ sorted_ids,
                        int sorted_cap, int* __restrict__ chunk_hist) {
  __shared__ int counts[kMaxExperts];
  grid_dependency_launch();
  grid_dependency_wait();
  for (int i = blockIdx.x * kThreads + threadIdx.x; i < sorted_cap; i += gridDim.x * kThreads) sorted_ids[i] = numel;
  for (int e = threadIdx.x; e < E; e += kThreads) counts[e] = 0;
  __syncthreads();
  const int i = blockIdx.x * kThreads + threadIdx.x;
  if (i < numel) {
    const int id = topk_ids[i];
    if (id >= 0 && id < E) atomicAdd(&counts[id], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += kThreads) chunk_hist[static_cast<size_t>(blockIdx.x) * E + e] = counts[e];
}

__global__ void __launch_bounds__(kThreads)
align_scan_kernel(int num_chunks, int E, int block_size, int sorted_cap, int* __restrict__ expert_ids,
                  int expert_ids_cap, int* __restrict__ num_post_pad, int* __restrict__ chunk_hist,
                  int* __restrict__ cumsum) {
  __shared__ int warp_totals[32];
  __shared__ int total_smem;
  grid_dependency_launch();
  grid_dependency_wait();
  int run = 0;
  if (threadIdx.x < E) {
    // exclusive prefix over chunks: chunk_hist[c][e] becomes the first slot (within the expert) of
    // chunk c. Loads go out in batches of 16 before the stores, so their latencies overlap.
    constexpr int kBatch = 16;
    for (int c0 = 0; c0 < num_chunks; c0 += kBatch) {
      int n[kBatch];
#pragma unroll
      for (int u = 0; u < kBatch; ++u)
        n[u] = c0 + u < num_chunks ? chunk_hist[static_cast<size_t>(c0 + u) * E + threadIdx.x] : 0;
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        if (c0 + u < num_chunks) chunk_hist[static_cast<size_t>(c0 + u) * E + threadIdx.x] = run;
        run += n[u];
      }
    }
  }
  const int start = scan_and_publish(run, E, block_size, sorted_cap, expert_ids_cap, expert_ids, num_post_pad,
                                     warp_totals, &total_smem);
  if (threadIdx.x < E) cumsum[threadIdx.x] = start;
}

__global__ void __launch_bounds__(kThreads)
align_chunk_scatter_kernel(const int* __restrict__ topk_ids, int numel, int E, const int* __restrict__ chunk_hist,
                           const int* __restrict__ cumsum, int* __restrict__ sorted_ids) {
  __shared__ int running[kMaxExperts];
  grid_dependency_launch();
  grid_dependency_wait();
  for (int e = threadIdx.x; e < E; e += kThreads)
    running[e] = cumsum[e] + chunk_hist[static_cast<size_t>(blockIdx.x) * E + e];
  __syncthreads();
  stable_place_chunk(topk_ids, blockIdx.x * kThreads, numel, E, running, sorted_ids);
}

}  // namespace

size_t align_workspace_bytes(int numel, int E) {
  if (numel <= kSmallNumel) return 16;
  const size_t chunks = (static_cast<size_t>(numel) + kThreads - 1) / kThreads;
  return (chunks * E + E + 1) * sizeof(int);
}

int launch_align_block_size(const int* topk_ids, int numel, int E, int block_size, int* sorted_ids, int sorted_cap,
                            int* expert_ids, int expert_ids_cap, int* num_post_pad, void* workspace,
                            size_t workspace_bytes, cudaStream_t stream) {
  if (E <= 0 || E > kMaxExperts) return set_error(kStatusInvalidArgument, "moe_align_block_size: 1..1024 experts");
  if (block_size <= 0 || numel < 0) return set_error(kStatusInvalidArgument, "moe_align_block_size: bad sizes");
  if (numel <= kThreads && E <= kTinyExperts) {
    launch_pdl(align_tiny_kernel, dim3(1), dim3(kThreads), 0, stream, topk_ids, numel, E, block_size, sorted_ids,
               sorted_cap, expert_ids, expert_ids_cap, num_post_pad);
    count_launches(1);
    return check_launch("moe_align_block_size");
  }
  if (numel <= kSmallNumel) {
    launch_pdl(align_single_cta_kernel, dim3(1), dim3(kThreads), 0, stream, topk_ids, numel, E, block_size, sorted_ids,
               sorted_cap, expert_ids, expert_ids_cap, num_post_pad);
    count_launches(1);
    return check_launch("moe_align_block_size");
  }
  if (workspace == nullptr || workspace_bytes < align_workspace_bytes(numel, E))
    return set_error(kStatusWorkspaceTooSmall, "moe_align_block_size: workspace of %zu bytes needed",
                     align_workspace_bytes(numel, E));
  const int chunks = (numel + kThreads - 1) / kThreads;
  int* chunk_hist = static_cast<int*>(workspace);
  int* cumsum = chunk_hist + static_cast<size_t>(chunks) * E;
  launch_pdl(align_chunk_hist_kernel, dim3(chunks), dim3(kThreads), 0, stream, topk_ids, numel, E, sorted_ids, sorted_cap,
             chunk_hist);
  launch_pdl(align_scan_kernel, dim3(1), dim3(kThreads), 0, stream, chunks, E, block_size, sorted_cap, expert_ids,
             expert_ids_cap, num_post_pad, chunk_hist, cumsum);
  launch_pdl(align_chunk_scatter_kernel, dim3(chunks), dim3(kThreads), 0, stream, topk_ids, numel, E,
             static_cast<const int*>(chunk_hist), static_cast<const int*>(cumsum), sorted_ids);
  count_launches(3);
  return check_launch("moe_align_block_size");
}

// ---------------------------------------------------------------- allocation-free variant
// Same three kernels, with the per-chunk histogram and the cumsum table in a fixed array that lives in
// the library image instead of in memory the caller had to allocate. Every GPU that loads the library
// carries these kStaticScratchInts * 4 bytes (130 KiB) until the process exits.
constexpr int kStaticScratchInts = 33280;  // e.g. 128 chunks (131072 flat indices) x 256 experts + 257
static __device__ __align__(256) int g_align_scratch[kStaticScratchInts];

int static_align_scratch_ints() { return kStaticScratchInts; }

int launch_align_block_size_static(const int* topk_ids, int numel, int E, int block_size, int* sorted_ids,
                                   int sorted_cap, int* expert_ids, int expert_ids_cap, int* num_post_pad,
                                   cudaStream_t stream) {
  if (E <= 0 || E > kMaxExperts) return set_error(kStatusInvalidArgument, "moe_align_block_size_static: 1..1024 experts");
  if (block_size <= 0 || numel < 0) return set_error(kStatusInvalidArgument, "moe_align_block_size_static: bad sizes");
  const int chunks = numel > 0 ? (numel + kThreads - 1) / kThreads : 1;
  const long long need = static_cast<long long>(chunks) * E + E + 1;
  if (need > kStaticScratchInts)
    return set_error(kStatusTooLarge,
                     "moe_align_block_size_static: %d flat indices x %d experts need %lld scratch words, the built-in "
                     "scratch holds %d (use moe_b200_moe_align_block_size with a caller workspace)",
                     numel, E, need, kStaticScratchInts);
  // In host code g_align_scratch is only a handle for the symbol; the address kernels can use has to be
  // asked for, once per device, while that device is current.
  static int* scratch_of_device[64] = {nullptr};
  int dev = 0;
  if (int st = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return st;
  if (dev < 0 || dev >= 64) return set_error(kStatusInvalidArgument, "moe_align_block_size_static: device index %d", dev);
  if (scratch_of_device[dev] == nullptr) {
    int* ptr = nullptr;
    if (int st = check_cuda(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_align_scratch),
                            "cudaGetSymbolAddress(g_align_scratch)"))
      return st;
    scratch_of_device[dev] = ptr;
  }
  int* chunk_hist = scratch_of_device[dev];
  int* cumsum = chunk_hist + static_cast<size_t>(chunks) * E;
  // Nothing in the scratch has to start at zero: the histogram kernel writes every chunk_hist word of
  // this call and the scan kernel every cumsum word before anything reads them.
  align_chunk_hist_kernel<<<chunks, kThreads, 0, stream>>>(topk_ids, numel, E, sorted_ids, sorted_cap, chunk_hist);
  align_scan_kernel<<<1, kThreads, 0, stream>>>(chunks, E, block_size, sorted_cap, expert_ids, expert_ids_cap,
                                                num_post_pad, chunk_hist, cumsum);
  align_chunk_scatter_kernel<<<chunks, kThreads, 0, stream>>>(topk_ids, numel, E, chunk_hist, cumsum, sorted_ids);
  count_launches(3);
  return check_launch("moe_align_block_size_static");
}

}  // namespace moe_b200
