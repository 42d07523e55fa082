// Tensor-parallel all-reduce over NVLink peer memory, and the k-slot sum fused with it.
//
// Role in the block: the reference sums the down-projection slots with torch.sum
// (nanovllm/layers/for_moe/moe_easy_kernel.py:26-31) and then calls its CUDA-IPC all-reduce
// (csrc/custom_all_reduce.cuh:298-366, dispatch :579-601). Here both are one launch:
//   phase 0  partial[t,:] = bf16(sum_j c3[t,j,:]) straight into this rank's IPC-registered buffer
//   barrier  every block meets the same-numbered block of every peer (release/acquire flags)
//   one-shot every rank reads all peers' partials, fp32 sum in rank order 0..N-1, writes out
//   two-shot rank r reduces slice r into its scratch, second barrier, everybody gathers all slices
// The plain all-reduce (input already in a registered buffer) is the same without phase 0.
//
// Synchronisation: one monotonically increasing counter per (block, peer) slot; a waiter accepts any
// value at or past the one it expects (signed difference), so a peer that is one barrier ahead cannot
// be missed and a single slot array serves every barrier of a launch. Data written before a barrier
// by block b is read after it only by block b of the peers (every kernel below maps elements, or whole token
// rows, to blocks the same way on both sides of a barrier), which is what the block-level
// release/acquire (__syncthreads + st.release / ld.acquire + __syncthreads) guarantees. Every spin is bounded by a wall-clock limit; when it runs
// out the kernel stores a status word and finishes without waiting further.
//
// Peer data is read with ordinary 16-byte loads (ld.global.cg) from IPC-mapped buffers: no TMA, no
// cluster features, nothing that depends on which GPU owns the memory.
#include <array>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/moe_b200.h"
#include "launch.cuh"
#include "moe_b200_internal.cuh"
#include "ptx.cuh"
#include "rms_norm_row.cuh"

namespace moe_b200 {

namespace {

constexpr int kMaxRanks = 8;
constexpr int kMaxArBlocks = 160;  // up to one block per SM (148 on B200) for large messages
constexpr int kArThreads = 512;
constexpr int kFusedBlocks = 32;  // fixed grid of the barrier-saving one-shot kernel (its per-block call counters rely on it)
constexpr int kLLBlocks = 64;     // fixed grid of the flag-in-data kernel (same reason), 256 threads each
constexpr int kLLThreads = 256;

struct alignas(128) Signal {
  uint32_t arrive[kMaxArBlocks][kMaxRanks];  // arrive[b][r]: written by block b of rank r
  uint32_t epoch[kMaxArBlocks];              // this rank's barrier count per block
  uint32_t fused_calls[kFusedBlocks];        // this rank's count of barrier-saving one-shot calls, per block
  uint32_t ll_calls[kLLBlocks];              // this rank's count of flag-in-data one-shot calls, per block
};
constexpr size_t kMetaBytes = (sizeof(Signal) + 255) / 256 * 256;

struct alignas(16) RankData {
  const void* ptrs[kMaxRanks];
};
struct RankSignals {
  Signal* signals[kMaxRanks];
};

union Vec16 {
  uint4 u;
  __nv_bfloat16 b[8];
  __half h[8];
  float f[4];
};

template <typename T> struct VecTraits;
template <> struct VecTraits<__nv_bfloat16> {
  static constexpr int kElems = 8;
  __device__ static void add(float* acc, const Vec16& v) {
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += __bfloat162float(v.b[i]);
  }
  __device__ static void set(float* acc, const Vec16& v) {
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = __bfloat162float(v.b[i]);
  }
  __device__ static void pack(Vec16& v, const float* acc) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v.b[i] = __float2bfloat16_rn(acc[i]);
  }
};
template <> struct VecTraits<__half> {
  static constexpr int kElems = 8;
  __device__ static void add(float* acc, const Vec16& v) {
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += __half2float(v.h[i]);
  }
  __device__ static void set(float* acc, const Vec16& v) {
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = __half2float(v.h[i]);
  }
  __device__ static void pack(Vec16& v, const float* acc) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v.h[i] = __float2half_rn(acc[i]);
  }
};
template <> struct VecTraits<float> {
  static constexpr int kElems = 4;
  __device__ static void add(float* acc, const Vec16& v) {
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] += v.f[i];
  }
  __device__ static void set(float* acc, const Vec16& v) {
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = v.f[i];
  }
  __device__ static void pack(Vec16& v, const float* acc) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v.f[i] = acc[i];
  }
};

struct ArParams {
  RankData* rank_data;   // device tuple of the N input buffers
  RankSignals sg;
  Signal* self_sg;
  void* out;
  int rank;
  long long nvec;        // 16-byte vectors
  unsigned long long wait_limit_ns;
  int* status;
  // fused k-slot sum (phase 0); c3 == nullptr for the plain all-reduce
  const __nv_bfloat16* c3;
  int top_k;
  int hidden_vecs;       // H / 8
};

// All threads of the block call this. Returns false if a wait ran out.
template <int N>
__device__ __forceinline__ bool peer_barrier(const ArParams& p, bool ordered, bool* timed_out_smem) {
  __syncthreads();
  const uint32_t next = p.self_sg->epoch[blockIdx.x] + 1u;
  if (threadIdx.x < N) {
    uint32_t* peer_slot = &p.sg.signals[threadIdx.x]->arrive[blockIdx.x][p.rank];
    if (ordered) st_release_sys(peer_slot, next); else st_relaxed_sys(peer_slot, next);
    const uint32_t* my_slot = &p.self_sg->arrive[blockIdx.x][threadIdx.x];
    const unsigned long long t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
      const uint32_t v = ordered ? ld_acquire_sys(my_slot) : ld_relaxed_sys(my_slot);
      if (static_cast<int32_t>(v - next) >= 0) break;
      if ((++spins & 255u) == 0u && globaltimer_ns() - t0 > p.wait_limit_ns) {
        *timed_out_smem = true;
        atomicCAS(p.status, 0, kErrPeerWait);
        break;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) p.self_sg->epoch[blockIdx.x] = next;
  return !*timed_out_smem;
}

__device__ __forceinline__ uint4 ld_cg(const uint4* p) { return __ldcg(p); }

template <typename T, int N>
__device__ __forceinline__ uint4 reduce_ranks(const uint4* const* ptrs, long long idx) {
  float acc[VecTraits<T>::kElems];
  Vec16 v[N];
#pragma unroll
  for (int r = 0; r < N; ++r) v[r].u = ld_cg(ptrs[r] + idx);
  VecTraits<T>::set(acc, v[0]);
#pragma unroll
  for (int r = 1; r < N; ++r) VecTraits<T>::add(acc, v[r]);
  Vec16 o;
  VecTraits<T>::pack(o, acc);
  return o.u;
}

// How many vectors a thread keeps in flight per rank: about sixteen 16-byte peer loads per thread before the
// first add, which is what it takes to cover the NVLink round trip at two and four ranks.
template <int N> struct Unroll { static constexpr int kU = N <= 2 ? 8 : N <= 4 ? 4 : 2; };

// dst[j] = sum over ranks of ptrs[r][base + j] for j in [0, count), fp32 in rank order, this thread's share.
template <typename T, int N>
__device__ __forceinline__ void reduce_span(const uint4* const* ptrs, long long base, long long count, uint4* dst,
                                            long long tid, long long stride) {
  constexpr int U = Unroll<N>::kU;
  for (long long j = tid; j < count; j += stride * U) {
    Vec16 v[U][N];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long jj = j + u * stride;
      if (jj < count) {
#pragma unroll
        for (int r = 0; r < N; ++r) v[u][r].u = ld_cg(ptrs[r] + base + jj);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long jj = j + u * stride;
      if (jj < count) {
        float acc[VecTraits<T>::kElems];
        VecTraits<T>::set(acc, v[u][0]);
#pragma unroll
        for (int r = 1; r < N; ++r) VecTraits<T>::add(acc, v[u][r]);
        Vec16 o;
        VecTraits<T>::pack(o, acc);
        dst[jj] = o.u;
      }
    }
  }
}

// partial[t, 8 cols] = bf16(sum over k slots), written to this rank's registered buffer
__device__ __forceinline__ void slot_sum_vec(const ArParams& p, uint4* own, long long v) {
  const long long t = v / p.hidden_vecs;
  const int c = static_cast<int>(v % p.hidden_vecs);
  const uint4* src = reinterpret_cast<const uint4*>(p.c3) + (t * p.top_k) * p.hidden_vecs + c;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int j = 0; j < p.top_k; ++j) {
    Vec16 x;
    x.u = src[static_cast<long long>(j) * p.hidden_vecs];
    VecTraits<__nv_bfloat16>::add(acc, x);
  }
  Vec16 o;
  VecTraits<__nv_bfloat16>::pack(o, acc);
  own[v] = o.u;
}

template <typename T, int N>
__global__ void __launch_bounds__(kArThreads, 1) ar_oneshot_kernel(const ArParams p) {
  __shared__ bool timed_out;
  if (threadIdx.x == 0) timed_out = false;
  grid_dependency_launch();
  grid_dependency_wait();
  const RankData rd = *p.rank_data;
  const uint4* ptrs[N];
#pragma unroll
  for (int r = 0; r < N; ++r) ptrs[r] = static_cast<const uint4*>(rd.ptrs[r]);
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  if (p.c3 != nullptr) {
    uint4* own = const_cast<uint4*>(ptrs[p.rank]);
    for (long long v = tid; v < p.nvec; v += stride) slot_sum_vec(p, own, v);
  }
  peer_barrier<N>(p, true, &timed_out);
  reduce_span<T, N>(ptrs, 0, p.nvec, static_cast<uint4*>(p.out), tid, stride);
  // nobody may overwrite its input while a peer still reads it
  peer_barrier<N>(p, false, &timed_out);
}

// k-slot sum + one-shot all-reduce with ONE barrier per call. The closing barrier of the kernel above only keeps a
// rank from overwriting its buffer while a peer still reads it; here every rank owns two buffers (the halves of a
// registered buffer that nothing else uses) and call n works in half n % 2. When a rank writes half n % 2 again, in
// call n + 2, it has passed the opening barrier of call n + 1, which a peer's block reaches only after that peer's
// call n has finished completely (kernels of a stream do not overlap past the dependency wait), so every peer is
// done reading. The call counter lives in device memory, one copy per block, advanced by the kernel itself, so a
// captured graph can be replayed any number of times; it stays equal across blocks and ranks because every such
// launch has exactly kFusedBlocks blocks on every rank.
template <int N>
__global__ void __launch_bounds__(kArThreads, 1) ar_oneshot_sum_kernel(const ArParams p, long long half_vecs) {
  __shared__ bool timed_out;
  if (threadIdx.x == 0) timed_out = false;
  grid_dependency_launch();
  grid_dependency_wait();
  const uint32_t call = p.self_sg->fused_calls[blockIdx.x];
  const long long off = (call & 1u) ? half_vecs : 0;
  const RankData rd = *p.rank_data;
  const uint4* ptrs[N];
#pragma unroll
  for (int r = 0; r < N; ++r) ptrs[r] = static_cast<const uint4*>(rd.ptrs[r]) + off;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  uint4* own = const_cast<uint4*>(ptrs[p.rank]);
  for (long long v = tid; v < p.nvec; v += stride) slot_sum_vec(p, own, v);
  peer_barrier<N>(p, true, &timed_out);
  uint4* out = static_cast<uint4*>(p.out);
  for (long long v = tid; v < p.nvec; v += stride) out[v] = reduce_ranks<__nv_bfloat16, N>(ptrs, v);
  if (threadIdx.x == 0) p.self_sg->fused_calls[blockIdx.x] = call + 1u;
}

// k-slot sum + one-shot all-reduce with NO barrier: every 16-byte vector of this rank's partial sum travels as two
// 16-byte packets {data, flag, data, flag} whose flag words carry the call number, pushed with plain stores into a
// receive area of every rank (its own included); a receiver polls ITS OWN memory until both packets of a vector
// show the current call number, so the data needs no fence, no flag round trip and no remote load: one NVLink
// crossing per rank pair instead of three. (Eight-byte stores arrive whole over NVLink, which is what NCCL's
// low-latency protocol relies on as well; twice the bytes on the wire, which is why this path is for
// decode-sized tensors only.) Receive areas alternate with the parity of the call number, and a rank cannot be
// two calls ahead of a peer (to finish call n + 1 it needs that peer's packets of call n + 1, sent by a kernel that
// started after the peer's call n had finished), so nobody overwrites packets that are still being read. The sum
// is fp32 in rank order, one rounding: the bits of the barrier kernels.
struct LLParams {
  RankData* areas;        // device tuple: the receive area of every rank
  long long slot_vecs;    // vectors per (parity, source rank) slot of a receive area
};

__device__ __forceinline__ void st_ll(uint4* dst, uint32_t a, uint32_t b, uint32_t flag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(a), "r"(flag), "r"(b), "r"(flag) : "memory");
}
__device__ __forceinline__ uint4 ld_ll(const uint4* src) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src) : "memory");
  return v;
}

// Index of vector v's first packet inside a slot (the second one is 32 packets further): vectors are taken in groups
// of 32 (one per lane), a group owns 64 consecutive packets.
__device__ __forceinline__ long long ll_packet(long long v) { return (v & ~31ll) * 2 + (v & 31ll); }

template <int N>
__global__ void __launch_bounds__(kLLThreads, 1) ar_ll_sum_kernel(const ArParams p, const LLParams ll) {
  grid_dependency_launch();
  grid_dependency_wait();
  const uint32_t epoch = p.self_sg->ll_calls[blockIdx.x] + 1u;
  const long long parity_off = (epoch & 1u) ? static_cast<long long>(N) * ll.slot_vecs : 0;
  const RankData areas = *ll.areas;
  uint4* area[N];
#pragma unroll
  for (int r = 0; r < N; ++r) area[r] = static_cast<uint4*>(const_cast<void*>(areas.ptrs[r]));
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  // push: this rank's slot in everybody's receive area, two packets per vector
  for (long long v = tid; v < p.nvec; v += stride) {
    const long long t = v / p.hidden_vecs;
    const int c = static_cast<int>(v % p.hidden_vecs);
    const uint4* src = reinterpret_cast<const uint4*>(p.c3) + (t * p.top_k) * p.hidden_vecs + c;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < p.top_k; ++j) {
      Vec16 x;
      x.u = src[static_cast<long long>(j) * p.hidden_vecs];
      VecTraits<__nv_bfloat16>::add(acc, x);
    }
    Vec16 o;
    VecTraits<__nv_bfloat16>::pack(o, acc);
    // packets of the warp's 32 vectors: first halves in 32 consecutive packets, second halves in the next 32, so
    // that each store instruction of the warp covers 512 contiguous bytes of the peer's memory
    const long long slot = (parity_off + static_cast<long long>(p.rank) * ll.slot_vecs) * 2 + ll_packet(v);
#pragma unroll
    for (int r = 0; r < N; ++r) {
      st_ll(area[r] + slot, o.u.x, o.u.y, epoch);
      st_ll(area[r] + slot + 32, o.u.z, o.u.w, epoch);
    }
  }
  // receive: poll this rank's own area until every rank's packets of this call are there
  const uint4* mine = area[0];
#pragma unroll
  for (int r = 1; r < N; ++r)
    if (r == p.rank) mine = area[r];
  uint4* out = static_cast<uint4*>(p.out);
  bool ok = true;
  for (long long v = tid; v < p.nvec && ok; v += stride) {
    uint4 lo[N], hi[N];
    const unsigned long long t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
      bool all = true;
#pragma unroll
      for (int r = 0; r < N; ++r) {
        const long long slot = (parity_off + static_cast<long long>(r) * ll.slot_vecs) * 2 + ll_packet(v);
        lo[r] = ld_ll(mine + slot);
        hi[r] = ld_ll(mine + slot + 32);
        all = all && lo[r].y == epoch && lo[r].w == epoch && hi[r].y == epoch && hi[r].w == epoch;
      }
      if (all) break;
      if ((++spins & 63u) == 0u && globaltimer_ns() - t0 > p.wait_limit_ns) {
        atomicCAS(p.status, 0, kErrPeerWait);
        ok = false;
        break;
      }
    }
    if (!ok) break;
    float acc[8];
    Vec16 x;
    x.u = make_uint4(lo[0].x, lo[0].z, hi[0].x, hi[0].z);
    VecTraits<__nv_bfloat16>::set(acc, x);
#pragma unroll
    for (int r = 1; r < N; ++r) {
      x.u = make_uint4(lo[r].x, lo[r].z, hi[r].x, hi[r].z);
      VecTraits<__nv_bfloat16>::add(acc, x);
    }
    Vec16 o;
    VecTraits<__nv_bfloat16>::pack(o, acc);
    out[v] = o.u;
  }
  __syncthreads();
  if (threadIdx.x == 0) p.self_sg->ll_calls[blockIdx.x] = epoch;
}

// One-shot all-reduce that ends in the next layer's residual add + RMSNorm (what the decoder layer after the MoE
// block does first with the reduced tensor: nanovllm/models/qwen3_moe.py:262-270, ops.add_rms_norm): a block owns
// whole token rows, reduces a row over the ranks (fp32, rank order, bf16 rounding = the all-reduce's output), and
// runs the norm's row code on it; the reduced tensor itself never goes to memory. Optional phase 0 as in the plain
// kernel (k-slot sum into this rank's registered buffer).
struct NormTail {
  __nv_bfloat16* residual;      // [T, H], updated in place
  const __nv_bfloat16* weight;  // [H]
  __nv_bfloat16* normed;        // [T, H]
  float eps;
  int T;
  int H;
};

template <int N>
__global__ void __launch_bounds__(kArThreads, 1) ar_oneshot_add_rms_norm_kernel(const ArParams p, const NormTail nt) {
  extern __shared__ uint4 ar_norm_smem[];
  __shared__ bool timed_out;
  if (threadIdx.x == 0) timed_out = false;
  grid_dependency_launch();
  grid_dependency_wait();
  __nv_bfloat16* x_row = reinterpret_cast<__nv_bfloat16*>(ar_norm_smem);
  float* red = reinterpret_cast<float*>(x_row + nt.H);
  const RankData rd = *p.rank_data;
  const uint4* ptrs[N];
#pragma unroll
  for (int r = 0; r < N; ++r) ptrs[r] = static_cast<const uint4*>(rd.ptrs[r]);
  if (p.c3 != nullptr) {
    // Phase 0 is row-owned like the reduction below: block b of a peer reads, after the barrier, exactly the
    // rows that block b of this rank wrote before it (the barrier pairs same-numbered blocks only).
    uint4* own = const_cast<uint4*>(ptrs[p.rank]);
    for (int row = blockIdx.x; row < nt.T; row += gridDim.x) {
      const long long row_vec = static_cast<long long>(row) * p.hidden_vecs;
      for (int c = threadIdx.x; c < p.hidden_vecs; c += blockDim.x) slot_sum_vec(p, own, row_vec + c);
    }
  }
  peer_barrier<N>(p, true, &timed_out);
  for (int row = blockIdx.x; row < nt.T; row += gridDim.x) {
    const long long row_vec = static_cast<long long>(row) * (nt.H / 8);
    const size_t off = static_cast<size_t>(row) * nt.H;
    rms_norm_row<true, kArThreads, false>(
        [&ptrs, row_vec](int c) { return reduce_ranks<__nv_bfloat16, N>(ptrs, row_vec + c / 8); }, nt.residual + off,
        nt.weight, nt.normed + off, nt.H, nt.eps, x_row, red, red + 32, true);
    __syncthreads();  // x_row and the reduction slots are reused by the next row
  }
  // nobody may overwrite its input while a peer still reads it
  peer_barrier<N>(p, false, &timed_out);
}

template <typename T, int N>
__global__ void __launch_bounds__(kArThreads, 1) ar_twoshot_kernel(const ArParams p) {
  __shared__ bool timed_out;
  if (threadIdx.x == 0) timed_out = false;
  grid_dependency_launch();
  grid_dependency_wait();
  const RankData rd = *p.rank_data;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long part = p.nvec / N;
  const long long my_start = p.rank * part;
  const long long my_len = p.rank == N - 1 ? p.nvec - my_start : part;
  const long long largest = p.nvec - (N - 1) * part;

  const uint4* ptrs[N];
  uint4* tmps[N];
#pragma unroll
  for (int r = 0; r < N; ++r) {
    ptrs[r] = static_cast<const uint4*>(rd.ptrs[r]);
    tmps[r] = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.sg.signals[r]) + kMetaBytes);
  }
  if (p.c3 != nullptr) {
    // slice-relative mapping: element start_s + j is produced by the thread that will reduce offset j
    uint4* own = const_cast<uint4*>(ptrs[p.rank]);
    for (int s = 0; s < N; ++s) {
      const long long s_start = s * part;
      const long long s_len = s == N - 1 ? p.nvec - s_start : part;
      for (long long j = tid; j < s_len; j += stride) slot_sum_vec(p, own, s_start + j);
    }
  }
  peer_barrier<N>(p, true, &timed_out);
  // reduce-scatter: this rank's slice from every peer into its own scratch
  reduce_span<T, N>(ptrs, my_start, my_len, tmps[p.rank], tid, stride);
  peer_barrier<N>(p, true, &timed_out);
  // all-gather: the loads of several slices' vectors go out before the first store
  uint4* out = static_cast<uint4*>(p.out);
  constexpr int U = Unroll<N>::kU;
  for (long long j = tid; j < largest; j += stride * U) {
    uint4 g[U][N];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long jj = j + u * stride;
#pragma unroll
      for (int r = 0; r < N; ++r)
        if (jj < largest && (r == N - 1 || jj < part)) g[u][r] = ld_cg(tmps[r] + jj);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long jj = j + u * stride;
#pragma unroll
      for (int r = 0; r < N; ++r)
        if (jj < largest && (r == N - 1 || jj < part)) out[r * part + jj] = g[u][r];
    }
  }
}

// Waits on a flag slot nobody writes: exercises the bounded-wait path on a single GPU.
__global__ void ar_wait_probe_kernel(const uint32_t* slot, uint32_t expected, unsigned long long limit_ns,
                                     int* status) {
  const unsigned long long t0 = globaltimer_ns();
  while (static_cast<int32_t>(ld_acquire_sys(slot) - expected) < 0) {
    if (globaltimer_ns() - t0 > limit_ns) {
      atomicCAS(status, 0, kErrPeerWait);
      break;
    }
  }
}

using IpcKey = std::array<uint8_t, sizeof(cudaIpcMemHandle_t)>;

struct Comm {
  int rank = 0;
  int world = 0;
  bool fully_connected = true;
  RankSignals sg{};
  Signal* self_sg = nullptr;
  RankData* rank_data_next = nullptr;
  RankData* rank_data_end = nullptr;
  std::unordered_map<const void*, RankData*> buffers;
  std::vector<void*> graph_unreg;
  std::map<IpcKey, char*> ipc_opened;
  unsigned long long wait_limit_ns = kWaitLimitNs;
  int env_algo = 0;               // 1 = one-shot, 2 = two-shot forced by VLLM_CUSTOM_ALLREDUCE_ALGO at init time
  RankData* fused_rd = nullptr;   // the double buffer of the barrier-saving one-shot kernel (registered, used by nothing else)
  long long fused_bytes = 0;
  RankData* ll_rd = nullptr;      // receive areas of the flag-in-data one-shot kernel
  long long ll_bytes = 0;
};

typedef CUresult (*PointerGetAttributeFn)(void*, CUpointer_attribute, CUdeviceptr);
PointerGetAttributeFn pointer_get_attribute_fn() {
  static PointerGetAttributeFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuPointerGetAttribute", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PointerGetAttributeFn>(sym);
  }
  return fn;
}

int pick_blocks(long long nvec) {
  long long b = (nvec + kArThreads - 1) / kArThreads;
  if (b > kMaxArBlocks) b = kMaxArBlocks;
  const int sms = device_sm_count();
  if (b > sms) b = sms;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

bool use_oneshot(const Comm& c, long long bytes, int algo) {
  if (algo == 0) algo = c.env_algo;  // a call's own choice wins over the environment's
  if (algo == 1 || algo == 3) return true;  // 3: one-shot with barriers (never the flag-in-data kernel)
  if (algo == 2) return false;
  if (c.world == 2) return true;
  if (c.world <= 4) return bytes <= 512 * 1024;
  return bytes <= 256 * 1024;
}

template <typename T>
int launch_ar(const Comm& c, const ArParams& p, bool oneshot, cudaStream_t stream) {
  const int blocks = pick_blocks(p.nvec);
#define MOE_B200_AR_CASE(n)                                                              \
  case n:                                                                                \
    if (oneshot) launch_pdl(ar_oneshot_kernel<T, n>, dim3(blocks), dim3(kArThreads), 0, stream, p); \
    else launch_pdl(ar_twoshot_kernel<T, n>, dim3(blocks), dim3(kArThreads), 0, stream, p);        \
    break;
  switch (c.world) {
    MOE_B200_AR_CASE(2)
    MOE_B200_AR_CASE(4)
    MOE_B200_AR_CASE(6)
    MOE_B200_AR_CASE(8)
    default:
      return set_error(kStatusInvalidArgument, "custom allreduce only supports num gpus in (2,4,6,8). Actual num gpus = %d", c.world);
  }
#undef MOE_B200_AR_CASE
  count_launches(1);
  return check_launch("all_reduce");
}

// Resolves the device tuple of peer pointers for `input` (registered, or being captured into a graph).
int resolve_rank_data(Comm& c, const void* input, cudaStream_t stream, RankData** out) {
  // a buffer registered up front (the staging buffer) is usable as is, inside a capture too
  auto it = c.buffers.find(input);
  if (it != c.buffers.end()) {
    *out = it->second;
    return kStatusOk;
  }
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (int st = check_cuda(cudaStreamIsCapturing(stream, &cap), "cudaStreamIsCapturing")) return st;
  if (cap == cudaStreamCaptureStatusActive) {
    // an address met during graph capture: its peers' addresses are filled in by register_graph_buffers
    if (c.rank_data_next + c.graph_unreg.size() + 1 > c.rank_data_end)
      return set_error(kStatusTooLarge, "all_reduce: rank data buffer is full");
    *out = c.rank_data_next + c.graph_unreg.size();
    c.graph_unreg.push_back(const_cast<void*>(input));
    return kStatusOk;
  }
  return set_error(kStatusNotRegistered, "buffer address %llu is not registered!", static_cast<unsigned long long>(reinterpret_cast<uintptr_t>(input)));
}

Comm* as_comm(int64_t h) { return reinterpret_cast<Comm*>(static_cast<intptr_t>(h)); }

}  // namespace

int ar_moe_sum_all_reduce_impl(int64_t handle, const void* c3, void* out, int T, int k, int H, int64_t reg_buffer,
                               int64_t reg_buffer_bytes, int algo, int* status_word, cudaStream_t stream) {
  Comm* c = as_comm(handle);
  if (c == nullptr) return set_error(kStatusInvalidArgument, "moe_sum_all_reduce: null communicator");
  if (H % 8 != 0 || T < 0 || k <= 0) return set_error(kStatusInvalidArgument, "moe_sum_all_reduce: H must be a multiple of 8");
  if (T == 0) return kStatusOk;
  const long long bytes = static_cast<long long>(T) * H * 2;
  if (reg_buffer == 0 || reg_buffer_bytes < bytes)
    return set_error(kStatusTooLarge, "moe_sum_all_reduce: registered buffer holds %lld bytes, %lld needed", static_cast<long long>(reg_buffer_bytes), bytes);
  RankData* rd = nullptr;
  if (int st = resolve_rank_data(*c, reinterpret_cast<const void*>(static_cast<intptr_t>(reg_buffer)), stream, &rd)) return st;
  ArParams p{};
  p.rank_data = rd; p.sg = c->sg; p.self_sg = c->self_sg; p.out = out; p.rank = c->rank;
  p.nvec = bytes / 16; p.wait_limit_ns = c->wait_limit_ns; p.status = status_word;
  p.c3 = static_cast<const __nv_bfloat16*>(c3); p.top_k = k; p.hidden_vecs = H / 8;
  const bool oneshot = use_oneshot(*c, bytes, algo);
  // flag-in-data path: a receive area holds 2 parities x world slots of 32-byte packet pairs
  const long long ll_slot_vecs = c->ll_rd != nullptr ? c->ll_bytes / (2ll * c->world * 32) : 0;
  if (oneshot && algo != 3 && ll_slot_vecs >= bytes / 16) {
    LLParams ll{c->ll_rd, ll_slot_vecs};
#define MOE_B200_ARL_CASE(n) \
  case n: launch_pdl(ar_ll_sum_kernel<n>, dim3(kLLBlocks), dim3(kLLThreads), 0, stream, p, ll); break;
    switch (c->world) {
      MOE_B200_ARL_CASE(2)
      MOE_B200_ARL_CASE(4)
      MOE_B200_ARL_CASE(6)
      MOE_B200_ARL_CASE(8)
      default:
        return set_error(kStatusInvalidArgument, "custom allreduce only supports num gpus in (2,4,6,8). Actual num gpus = %d", c->world);
    }
#undef MOE_B200_ARL_CASE
    count_launches(1);
    return check_launch("moe_sum_all_reduce (flag-in-data)");
  }
  if (oneshot && c->fused_rd != nullptr && bytes <= c->fused_bytes / 2) {
    p.rank_data = c->fused_rd;
    const long long half_vecs = c->fused_bytes / 2 / 16;
#define MOE_B200_ARS_CASE(n) \
  case n: launch_pdl(ar_oneshot_sum_kernel<n>, dim3(kFusedBlocks), dim3(kArThreads), 0, stream, p, half_vecs); break;
    switch (c->world) {
      MOE_B200_ARS_CASE(2)
      MOE_B200_ARS_CASE(4)
      MOE_B200_ARS_CASE(6)
      MOE_B200_ARS_CASE(8)
      default:
        return set_error(kStatusInvalidArgument, "custom allreduce only supports num gpus in (2,4,6,8). Actual num gpus = %d", c->world);
    }
#undef MOE_B200_ARS_CASE
    count_launches(1);
    return check_launch("moe_sum_all_reduce (one barrier)");
  }
  return launch_ar<__nv_bfloat16>(*c, p, oneshot, stream);
}

// All-reduce (optionally with the k-slot sum in front) followed by residual add + RMSNorm. Small messages take the
// fused one-shot kernel; anything else runs the all-reduce into `scratch_out` and the norm kernel after it.
int ar_all_reduce_add_rms_norm_impl(int64_t handle, const void* c3, int k, void* scratch_out, __nv_bfloat16* residual,
                                    const __nv_bfloat16* weight, float eps, __nv_bfloat16* normed, int T, int H,
                                    int64_t reg_buffer, int64_t reg_buffer_bytes, int algo, int* status_word,
                                    cudaStream_t stream) {
  Comm* c = as_comm(handle);
  if (c == nullptr) return set_error(kStatusInvalidArgument, "all_reduce_add_rms_norm: null communicator");
  if (H % 8 != 0 || T < 0) return set_error(kStatusInvalidArgument, "all_reduce_add_rms_norm: H must be a multiple of 8");
  if (T == 0) return kStatusOk;
  const long long bytes = static_cast<long long>(T) * H * 2;
  if (reg_buffer == 0 || reg_buffer_bytes < bytes)
    return set_error(kStatusTooLarge, "all_reduce_add_rms_norm: registered buffer holds %lld bytes, %lld needed", static_cast<long long>(reg_buffer_bytes), bytes);
  RankData* rd = nullptr;
  if (int st = resolve_rank_data(*c, reinterpret_cast<const void*>(static_cast<intptr_t>(reg_buffer)), stream, &rd)) return st;
  ArParams p{};
  p.rank_data = rd; p.sg = c->sg; p.self_sg = c->self_sg; p.out = scratch_out; p.rank = c->rank;
  p.nvec = bytes / 16; p.wait_limit_ns = c->wait_limit_ns; p.status = status_word;
  p.c3 = static_cast<const __nv_bfloat16*>(c3); p.top_k = k; p.hidden_vecs = H / 8;
  const size_t smem = static_cast<size_t>(H) * 2 + 40 * sizeof(float);
  if (use_oneshot(*c, bytes, algo) && smem <= 48 * 1024) {
    NormTail nt{residual, weight, normed, eps, T, H};
    int blocks = T < kMaxArBlocks ? T : kMaxArBlocks;
    if (blocks > device_sm_count()) blocks = device_sm_count();
#define MOE_B200_ARN_CASE(n) \
  case n: launch_pdl(ar_oneshot_add_rms_norm_kernel<n>, dim3(blocks), dim3(kArThreads), smem, stream, p, nt); break;
    switch (c->world) {
      MOE_B200_ARN_CASE(2)
      MOE_B200_ARN_CASE(4)
      MOE_B200_ARN_CASE(6)
      MOE_B200_ARN_CASE(8)
      default:
        return set_error(kStatusInvalidArgument, "custom allreduce only supports num gpus in (2,4,6,8). Actual num gpus = %d", c->world);
    }
#undef MOE_B200_ARN_CASE
    count_launches(1);
    return check_launch("all_reduce_add_rms_norm");
  }
  if (scratch_out == nullptr) return set_error(kStatusInvalidArgument, "all_reduce_add_rms_norm: this size needs the scratch output");
  if (int st = launch_ar<__nv_bfloat16>(*c, p, use_oneshot(*c, bytes, algo), stream)) return st;
  return launch_rms_norm(normed, residual, static_cast<const __nv_bfloat16*>(scratch_out), weight, eps, T, H, stream);
}

}  // namespace moe_b200

using namespace moe_b200;

extern "C" {

int64_t moe_b200_ar_meta_size(void) { return static_cast<int64_t>(kMetaBytes); }

int moe_b200_ar_allocate_shared_buffer(int64_t size_bytes, int64_t* ptr_out, uint8_t* handle_out) {
  if (size_bytes <= 0 || ptr_out == nullptr || handle_out == nullptr)
    return set_error(kStatusInvalidArgument, "allocate_shared_buffer: bad arguments");
  void* buffer = nullptr;
  if (int st = check_cuda(cudaMalloc(&buffer, static_cast<size_t>(size_bytes)), "cudaMalloc(shared buffer)")) return st;
  if (int st = check_cuda(cudaMemset(buffer, 0, static_cast<size_t>(size_bytes)), "cudaMemset(shared buffer)")) {
    cudaFree(buffer);
    return st;
  }
  cudaIpcMemHandle_t h;
  if (int st = check_cuda(cudaIpcGetMemHandle(&h, buffer), "cudaIpcGetMemHandle")) {
    cudaFree(buffer);
    return st;
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  memcpy(handle_out, &h, sizeof(h));
  *ptr_out = static_cast<int64_t>(reinterpret_cast<intptr_t>(buffer));
  return kStatusOk;
}

int moe_b200_ar_open_mem_handle(const uint8_t* handle, int64_t* ptr_out) {
  if (handle == nullptr || ptr_out == nullptr) return set_error(kStatusInvalidArgument, "open_mem_handle: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  if (int st = check_cuda(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle")) return st;
  *ptr_out = static_cast<int64_t>(reinterpret_cast<intptr_t>(p));
  return kStatusOk;
}

int moe_b200_ar_close_mem_handle(int64_t ptr) {
  return check_cuda(cudaIpcCloseMemHandle(reinterpret_cast<void*>(static_cast<intptr_t>(ptr))), "cudaIpcCloseMemHandle");
}

int moe_b200_ar_free_shared_buffer(int64_t ptr) {
  return check_cuda(cudaFree(reinterpret_cast<void*>(static_cast<intptr_t>(ptr))), "cudaFree(shared buffer)");
}

int moe_b200_ar_init(const int64_t* meta_ptrs, int world_size, void* rank_data, int64_t rank_data_bytes, int rank,
                     int fully_connected, int64_t* handle_out) {
  if (meta_ptrs == nullptr || handle_out == nullptr || rank_data == nullptr)
    return set_error(kStatusInvalidArgument, "init_custom_ar: null pointer");
  if (world_size > kMaxRanks) return set_error(kStatusInvalidArgument, "world size > 8 is not supported");
  if (world_size % 2 == 1) return set_error(kStatusInvalidArgument, "Odd num gpus is not supported for now");
  if (rank < 0 || rank >= world_size) return set_error(kStatusInvalidArgument, "invalid rank passed in");
  // The reference's environment override of the algorithm choice (csrc/custom_all_reduce.cuh:561-577), read once.
  int env_algo = 0;
  if (const char* env = getenv("VLLM_CUSTOM_ALLREDUCE_ALGO")) {
    if (strcmp(env, "1stage") == 0 || strcmp(env, "oneshot") == 0) env_algo = 1;
    else if (strcmp(env, "2stage") == 0 || strcmp(env, "twoshot") == 0) env_algo = 2;
    else return set_error(kStatusInvalidArgument, "Invalid VLLM_CUSTOM_ALLREDUCE_ALGO: %s. Valid values: 1stage, oneshot, 2stage, twoshot", env);
  }
  Comm* c = new Comm();
  c->env_algo = env_algo;
  c->rank = rank;
  c->world = world_size;
  c->fully_connected = fully_connected != 0;
  for (int i = 0; i < world_size; ++i) c->sg.signals[i] = reinterpret_cast<Signal*>(static_cast<intptr_t>(meta_ptrs[i]));
  c->self_sg = c->sg.signals[rank];
  c->rank_data_next = static_cast<RankData*>(rank_data);
  c->rank_data_end = c->rank_data_next + rank_data_bytes / static_cast<int64_t>(sizeof(RankData));
  *handle_out = static_cast<int64_t>(reinterpret_cast<intptr_t>(c));
  return kStatusOk;
}

int moe_b200_ar_dispose(int64_t handle) {
  Comm* c = as_comm(handle);
  if (c == nullptr) return kStatusOk;
  for (auto& kv : c->ipc_opened) cudaIpcCloseMemHandle(kv.second);
  delete c;
  return kStatusOk;
}

int moe_b200_ar_register_buffer(int64_t handle, const int64_t* ptrs) {
  Comm* c = as_comm(handle);
  if (c == nullptr || ptrs == nullptr) return set_error(kStatusInvalidArgument, "register_buffer: null argument");
  if (c->rank_data_next + 1 > c->rank_data_end) return set_error(kStatusTooLarge, "register_buffer: rank data buffer is full");
  RankData data{};
  for (int i = 0; i < c->world; ++i) data.ptrs[i] = reinterpret_cast<const void*>(static_cast<intptr_t>(ptrs[i]));
  RankData* d = c->rank_data_next++;
  if (int st = check_cuda(cudaMemcpy(d, &data, sizeof(RankData), cudaMemcpyHostToDevice), "register_buffer copy")) return st;
  c->buffers[data.ptrs[c->rank]] = d;
  return kStatusOk;
}

int moe_b200_ar_register_fused_buffer(int64_t handle, const int64_t* ptrs, int64_t bytes) {
  Comm* c = as_comm(handle);
  if (c == nullptr || ptrs == nullptr || bytes < 32 || bytes % 32 != 0)
    return set_error(kStatusInvalidArgument, "register_fused_buffer: null argument or a size that is not a multiple of 32");
  if (int st = moe_b200_ar_register_buffer(handle, ptrs)) return st;
  c->fused_rd = c->buffers[reinterpret_cast<const void*>(static_cast<intptr_t>(ptrs[c->rank]))];
  c->fused_bytes = bytes;
  return kStatusOk;
}

int moe_b200_ar_register_ll_buffer(int64_t handle, const int64_t* ptrs, int64_t bytes) {
  Comm* c = as_comm(handle);
  if (c == nullptr || ptrs == nullptr || bytes < 64 * c->world || bytes % 64 != 0)
    return set_error(kStatusInvalidArgument, "register_ll_buffer: null argument or a size that is not a multiple of 64");
  if (int st = moe_b200_ar_register_buffer(handle, ptrs)) return st;
  c->ll_rd = c->buffers[reinterpret_cast<const void*>(static_cast<intptr_t>(ptrs[c->rank]))];
  c->ll_bytes = bytes;
  return kStatusOk;
}

int moe_b200_ar_set_wait_limit_ns(int64_t handle, uint64_t limit_ns) {
  Comm* c = as_comm(handle);
  if (c == nullptr) return set_error(kStatusInvalidArgument, "set_wait_limit: null communicator");
  c->wait_limit_ns = limit_ns;
  return kStatusOk;
}

int moe_b200_ar_all_reduce(int64_t handle, const void* inp, void* out, int64_t numel, int dtype, int64_t reg_buffer,
                           int64_t reg_buffer_bytes, int algo, int32_t* status_word, void* stream_v) {
  Comm* c = as_comm(handle);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (c == nullptr || inp == nullptr || out == nullptr || status_word == nullptr)
    return set_error(kStatusInvalidArgument, "all_reduce: null argument");
  const int esize = dtype == 2 ? 4 : 2;
  const long long bytes = numel * esize;
  if (bytes % 16 != 0)
    return set_error(kStatusInvalidArgument, "custom allreduce currently requires input length to be multiple of %d", 16 / esize);
  if (numel == 0) return kStatusOk;
  const void* src = inp;
  if (reg_buffer != 0) {
    if (bytes > reg_buffer_bytes)
      return set_error(kStatusTooLarge, "all_reduce: registered buffer is too small to contain the input");
    void* reg = reinterpret_cast<void*>(static_cast<intptr_t>(reg_buffer));
    if (int st = check_cuda(cudaMemcpyAsync(reg, inp, static_cast<size_t>(bytes), cudaMemcpyDeviceToDevice, stream), "all_reduce staging copy")) return st;
    src = reg;
  }
  RankData* rd = nullptr;
  if (int st = resolve_rank_data(*c, src, stream, &rd)) return st;
  ArParams p{};
  p.rank_data = rd; p.sg = c->sg; p.self_sg = c->self_sg; p.out = out; p.rank = c->rank;
  p.nvec = bytes / 16; p.wait_limit_ns = c->wait_limit_ns; p.status = status_word; p.c3 = nullptr;
  const bool oneshot = use_oneshot(*c, bytes, algo);
  switch (dtype) {
    case 0: return launch_ar<__nv_bfloat16>(*c, p, oneshot, stream);
    case 1: return launch_ar<__half>(*c, p, oneshot, stream);
    case 2: return launch_ar<float>(*c, p, oneshot, stream);
    default: return set_error(kStatusInvalidArgument, "custom allreduce only supports float32, float16 and bfloat16");
  }
}

int moe_b200_ar_moe_sum_all_reduce(int64_t handle, const void* c3, void* out, int T, int k, int H, int64_t reg_buffer,
                                   int64_t reg_buffer_bytes, int algo, int32_t* status_word, void* stream) {
  if (c3 == nullptr || out == nullptr || status_word == nullptr) return set_error(kStatusInvalidArgument, "moe_sum_all_reduce: null pointer");
  return ar_moe_sum_all_reduce_impl(handle, c3, out, T, k, H, reg_buffer, reg_buffer_bytes, algo, status_word,
                                    static_cast<cudaStream_t>(stream));
}

int moe_b200_ar_all_reduce_add_rms_norm(int64_t handle, const void* inp, void* scratch_out, void* residual,
                                        const void* norm_weight, float eps, void* normed_out, int T, int H,
                                        int64_t reg_buffer, int64_t reg_buffer_bytes, int algo, int32_t* status_word,
                                        void* stream_v) {
  if (inp == nullptr || residual == nullptr || norm_weight == nullptr || normed_out == nullptr || status_word == nullptr)
    return set_error(kStatusInvalidArgument, "all_reduce_add_rms_norm: null pointer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const long long bytes = static_cast<long long>(T) * H * 2;
  if (reg_buffer == 0 || bytes > reg_buffer_bytes)
    return set_error(kStatusTooLarge, "all_reduce_add_rms_norm: registered buffer is too small to contain the input");
  void* reg = reinterpret_cast<void*>(static_cast<intptr_t>(reg_buffer));
  if (inp != reg && bytes > 0) {
    if (int st = check_cuda(cudaMemcpyAsync(reg, inp, static_cast<size_t>(bytes), cudaMemcpyDeviceToDevice, stream), "all_reduce staging copy")) return st;
  }
  return ar_all_reduce_add_rms_norm_impl(handle, nullptr, 0, scratch_out, static_cast<__nv_bfloat16*>(residual),
                                         static_cast<const __nv_bfloat16*>(norm_weight), eps,
                                         static_cast<__nv_bfloat16*>(normed_out), T, H, reg_buffer, reg_buffer_bytes, algo,
                                         status_word, stream);
}

int moe_b200_ar_moe_sum_all_reduce_add_rms_norm(int64_t handle, const void* c3, void* scratch_out, void* residual,
                                                const void* norm_weight, float eps, void* normed_out, int T, int k,
                                                int H, int64_t reg_buffer, int64_t reg_buffer_bytes, int algo,
                                                int32_t* status_word, void* stream) {
  if (c3 == nullptr || residual == nullptr || norm_weight == nullptr || normed_out == nullptr || status_word == nullptr || k <= 0)
    return set_error(kStatusInvalidArgument, "moe_sum_all_reduce_add_rms_norm: null pointer");
  return ar_all_reduce_add_rms_norm_impl(handle, c3, k, scratch_out, static_cast<__nv_bfloat16*>(residual),
                                         static_cast<const __nv_bfloat16*>(norm_weight), eps,
                                         static_cast<__nv_bfloat16*>(normed_out), T, H, reg_buffer, reg_buffer_bytes, algo,
                                         status_word, static_cast<cudaStream_t>(stream));
}

int moe_b200_ar_graph_buffer_count(int64_t handle, int* count_out) {
  Comm* c = as_comm(handle);
  if (c == nullptr || count_out == nullptr) return set_error(kStatusInvalidArgument, "graph_buffer_count: null argument");
  *count_out = static_cast<int>(c->graph_unreg.size());
  return kStatusOk;
}

int moe_b200_ar_get_graph_buffer_ipc_meta(int64_t handle, uint8_t* handles_out, int64_t* offsets_out, int capacity) {
  Comm* c = as_comm(handle);
  if (c == nullptr) return set_error(kStatusInvalidArgument, "get_graph_buffer_ipc_meta: null communicator");
  const int n = static_cast<int>(c->graph_unreg.size());
  if (capacity < n) return set_error(kStatusTooLarge, "get_graph_buffer_ipc_meta: %d buffers, capacity %d", n, capacity);
  PointerGetAttributeFn get_attr = pointer_get_attribute_fn();
  if (n > 0 && get_attr == nullptr) return set_error(kStatusDriverEntryPoint, "cuPointerGetAttribute is not available");
  for (int i = 0; i < n; ++i) {
    void* ptr = c->graph_unreg[i];
    void* base = nullptr;
    // the IPC handle names the whole allocation, so share its base and the offset into it
    if (get_attr(&base, CU_POINTER_ATTRIBUTE_RANGE_START_ADDR, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS)
      return set_error(kStatusCudaError, "failed to get pointer attr");
    cudaIpcMemHandle_t h;
    if (int st = check_cuda(cudaIpcGetMemHandle(&h, base), "cudaIpcGetMemHandle(graph buffer)")) return st;
    memcpy(handles_out + static_cast<size_t>(i) * 64, &h, 64);
    offsets_out[i] = static_cast<char*>(ptr) - static_cast<char*>(base);
  }
  return kStatusOk;
}

int moe_b200_ar_register_graph_buffers(int64_t handle, const uint8_t* handles, const int64_t* offsets, int count) {
  Comm* c = as_comm(handle);
  if (c == nullptr) return set_error(kStatusInvalidArgument, "register_graph_buffers: null communicator");
  const int n = static_cast<int>(c->graph_unreg.size());
  if (count != n) return set_error(kStatusInvalidArgument, "register_graph_buffers: %d buffers captured, %d described", n, count);
  if (n == 0) return kStatusOk;
  if (c->rank_data_next + n > c->rank_data_end) return set_error(kStatusTooLarge, "register_graph_buffers: rank data buffer is full");
  std::vector<RankData> rd(n);
  for (int i = 0; i < n; ++i) {
    for (int j = 0; j < c->world; ++j) {
      if (j == c->rank) {
        rd[i].ptrs[j] = c->graph_unreg[i];
        continue;
      }
      IpcKey key;
      memcpy(key.data(), handles + (static_cast<size_t>(j) * n + i) * 64, 64);
      auto it = c->ipc_opened.find(key);
      if (it == c->ipc_opened.end()) {
        cudaIpcMemHandle_t h;
        memcpy(&h, key.data(), 64);
        void* p = nullptr;
        if (int st = check_cuda(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle(graph buffer)")) return st;
        it = c->ipc_opened.emplace(key, static_cast<char*>(p)).first;
      }
      rd[i].ptrs[j] = it->second + offsets[static_cast<size_t>(j) * n + i];
    }
  }
  if (int st = check_cuda(cudaMemcpy(c->rank_data_next, rd.data(), sizeof(RankData) * n, cudaMemcpyHostToDevice), "register_graph_buffers copy")) return st;
  c->rank_data_next += n;
  c->graph_unreg.clear();
  return kStatusOk;
}

// Single-GPU check of the bounded wait: spins on a slot of this rank's own signal area that nobody
// advances, with the given limit, and reports through the status word.
int moe_b200_ar_wait_probe(int64_t meta_ptr, uint64_t limit_ns, int32_t* status_word, void* stream) {
  if (meta_ptr == 0 || status_word == nullptr) return set_error(kStatusInvalidArgument, "wait_probe: null argument");
  Signal* s = reinterpret_cast<Signal*>(static_cast<intptr_t>(meta_ptr));
  ar_wait_probe_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(&s->arrive[kMaxArBlocks - 1][kMaxRanks - 1], 1u, limit_ns, status_word);
  return check_launch("wait_probe");
}

}  // extern "C"
