// fp8 (e4m3, w8a8) variant of the grouped expert GEMMs, block-scaled the way DeepSeek-style checkpoints are:
//   weights      w_q [E, N, K] e4m3 with one fp32 scale per 128 x 128 block, w_s [E, ceil(N/128), K/128]
//   activations  a_q [rows, K] e4m3 with one fp32 scale per row and group of 128 along K, a_s [rows, K/128],
//                quantised on the fly (quant_rows_fp8_kernel: s = max(|x|, 1e-10) / 448, q = e4m3(x / s))
//   C[r, n] = sum over K blocks kb of  a_s[r, kb] * w_s[n / 128, kb] * (a_q[r, kb-block] . w_q[n, kb-block])
// The reference has no fp8 path (its fused_moe asserts the scales are None: for_moe/fused_moe.py:248-249), so
// this follows the published block-quantisation scheme and is checked against a CPU emulation of it.
//
// Kernel: same skeleton as the bf16 kernels (grouped_gemm.cu): 128 permuted token rows per tile, weights by
// TMA (byte tensor map, 128-byte swizzle), token rows by cp.async, static tile list. What
// differs: a shared-memory stage holds 128 K elements = exactly one scale block, so the tensor core cannot
// accumulate across stages. Each stage's product (4 tcgen05.mma kind::f8f6f4, K = 32 each) goes into one of
// four 128-column TMEM buffers, and eight warps (two per TMEM lane quarter, 64 accumulator columns each) read it
// back, multiply by the two scales and accumulate in registers; the same warps then run the epilogue (SiLU * up
// with the bf16 kernels' rounding points, or x routed weight). The first purpose is the weight-streaming
// regime, where halving the bytes halves the time; at prefill sizes the register accumulation costs about as
// much as the tensor cores save. On a tensor-parallel rank the K blocks and the scale indices follow the scale
// blocks of the UNSHARDED weights (a slice of the intermediate dimension may begin or end inside a block), and two
// threads issue the MMAs of alternate K blocks.
#include <cuda_fp8.h>

#include <cmath>
#include <cstdio>

#include "act_math.cuh"
#include "launch.cuh"
#include "moe_b200_internal.cuh"
#include "ptx.cuh"

namespace moe_b200 {

namespace {

constexpr int BM = kBlockM;
constexpr int kGroup = 128;            // K elements per scale block = bytes per swizzle row = K per stage
constexpr int kStageA = BM * kGroup;   // 16 KB of token rows
constexpr int kStageB = 128 * kGroup;  // 16 KB of weight rows (64 gate + 64 up, or 128 down)
constexpr int kStageBytes = kStageA + kStageB;
constexpr int kStages = 6;
constexpr int kPartCols = 128;         // accumulator columns per stage product
constexpr int kPartBufs = 4;           // stage products in flight between the MMA thread and the accumulating warps
constexpr int kTmemCols = kPartBufs * kPartCols;
constexpr int kBarrierBytes = 1024;
constexpr int kSmemBytes = kBarrierBytes + 1024 /*alignment slack*/ + kStages * kStageBytes;

constexpr int kWarpTma = 0;
constexpr int kWarpMma = 1;       // 2 warps: issuer i takes the K blocks j with j % 2 == i
constexpr int kMmaIssuers = 2;
constexpr int kWarpPromote0 = 4;  // 8 warps (starting at a multiple of 4: a warp reads TMEM lane quarter warp % 4)
constexpr int kWarpGather0 = 12;  // 4 warps
constexpr int kThreads = 512;

struct ParamsF8 {
  const int* sorted_ids;
  const int* expert_ids;
  const int* num_post_pad;
  const uint8_t* a_q;  // [T, K] (gate_up: indexed by token) or [rows, K] (down: indexed by permuted row)
  const float* a_s;    // [.., K / 128]
  const float* w_s;    // [E, w_s_rows, w_s_ld]: the UNSHARDED scale tensor, indexed by global block
  int w_s_rows;
  int w_s_ld;
  int a_s_ld;          // scale groups per activation row = K blocks of this launch
  int num_kb;
  int k_shift;         // columns by which this rank's K range starts inside a scale block (0 unless K is sharded)
  int w_kb_off;        // global index of this rank's first K block
  int row_blk0;        // scale-row block of this tile family's first weight row (gate half, or the down rows)
  int row_blk1;        // same for the up half
  int numel;
  int top_k;
  int K;
  int n_tiles;
  int tile_cols;  // output columns per tile: 64 (gate_up) or 128 (down)
  int out_cols;
  int inter;      // row offset of the up half inside w13[e]
  __nv_bfloat16* out;
  long long out_ld;
  const float* topk_w;
  int* status;
};

union Pack8 {
  uint4 u;
  __nv_bfloat16 h[8];
};

__device__ __forceinline__ void report(int* status, int code) { atomicCAS(status, 0, code); }

template <int kMode>  // 1 = gate_up, 2 = down
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_b, const ParamsF8 p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* bar_empty = bar_full + kStages;
  uint64_t* bar_part_full = bar_empty + kStages;
  uint64_t* bar_part_free = bar_part_full + kPartBufs;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_part_free + kPartBufs);
  uint8_t* ring = smem + kBarrierBytes;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bar_full[s], 1 + 128);
      mbar_init(&bar_empty[s], 1);
    }
    for (int b = 0; b < kPartBufs; ++b) {
      mbar_init(&bar_part_full[b], 1);
      mbar_init(&bar_part_free[b], 8);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == kWarpMma) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  grid_dependency_launch();
  grid_dependency_wait();

  const int num_m_blocks = *p.num_post_pad / BM;
  const int total_tiles = num_m_blocks * p.n_tiles;
  const int num_kb = p.num_kb;

  if (warp == kWarpTma) {
    // ------------------------------------------------------------------ TMA producer (weights)
    if (lane == 0) {
      uint32_t s = 0, ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int m_blk = tile / p.n_tiles;
        const int n0 = (tile % p.n_tiles) * p.tile_cols;
        const int e = p.expert_ids[m_blk];
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&bar_empty[s], ph ^ 1u)) {
            report(p.status, kErrWaitEmpty);
            ok = false;
            break;
          }
          uint8_t* b_dst = ring + s * kStageBytes + kStageA;
          mbar_arrive_expect_tx(&bar_full[s], kStageB);
          if (kMode == 1) {
            tma_load_3d(b_dst, &tmap_b, kb * kGroup - p.k_shift, n0, e, &bar_full[s]);
            tma_load_3d(b_dst + 64 * kGroup, &tmap_b, kb * kGroup - p.k_shift, p.inter + n0, e, &bar_full[s]);
          } else {
            // a sharded K range may start inside a scale block: the box then begins at a negative (16-byte aligned)
            // coordinate and the part outside the tensor is zero-filled
            tma_load_3d(b_dst, &tmap_b, kb * kGroup - p.k_shift, n0, e, &bar_full[s]);
          }
          if (++s == kStages) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp >= kWarpMma && warp < kWarpMma + kMmaIssuers) {
    // ------------------------------------------------------------------ MMA issuers: one stage = one product buffer
    // Issuing a tcgen05.mma costs its thread about 110 cycles, more than the 64 cycles an N = 128 instruction
    // runs; the stage products are independent (nothing accumulates across K blocks in TMEM), so two threads
    // take alternate K blocks.
    if (lane == 0) {
      const uint32_t me = static_cast<uint32_t>(warp - kWarpMma);
      const uint32_t idesc = umma_idesc_e4m3(BM, kPartCols);
      bool ok = true;
      uint32_t j = 0;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < num_kb; ++kb, ++j) {
          if (j % kMmaIssuers != me) continue;
          const uint32_t s = j % kStages;
          const uint32_t ph = (j / kStages) & 1u;
          const uint32_t b = j % kPartBufs;
          const uint32_t bph = (j / kPartBufs) & 1u;
          if (!mbar_wait(&bar_part_free[b], bph ^ 1u)) {
            report(p.status, kErrWaitTmemEmpty);
            ok = false;
            break;
          }
          if (!mbar_wait(&bar_full[s], ph)) {
            report(p.status, kErrWaitFull);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(ring + s * kStageBytes);
          const uint64_t adesc = umma_desc_k_sw128(a_addr);
          const uint64_t bdesc = umma_desc_k_sw128(a_addr + kStageA);
          const uint32_t d_tmem = tmem_base + b * kPartCols;
          // 32 e4m3 = 32 bytes along K per instruction: +2 in the descriptor's 16-byte units
          umma_e4m3(d_tmem, adesc, bdesc, idesc, 0u);
          umma_e4m3(d_tmem, adesc + 2, bdesc + 2, idesc, 1u);
          umma_e4m3(d_tmem, adesc + 4, bdesc + 4, idesc, 1u);
          umma_e4m3(d_tmem, adesc + 6, bdesc + 6, idesc, 1u);
          umma_commit(&bar_empty[s]);
          umma_commit(&bar_part_full[b]);
        }
      }
    }
    __syncwarp();
  } else if (warp >= kWarpPromote0 && warp < kWarpPromote0 + 8) {
    // ------------------------------------------------------------------ scale-and-accumulate, then epilogue
    const int q = warp & 3;                        // TMEM lane quarter this warp may read
    const int hf = (warp - kWarpPromote0) >> 2;    // which half of the tile's output columns
    const int row_in_tile = q * 32 + lane;
    uint32_t j = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const int m_blk = tile / p.n_tiles;
      const int n0 = (tile % p.n_tiles) * p.tile_cols;
      const int e = p.expert_ids[m_blk];
      const long long pos = static_cast<long long>(m_blk) * BM + row_in_tile;
      const int flat = p.sorted_ids[pos];
      const bool valid = flat < p.numel;
      const bool any_valid = __any_sync(0xffffffffu, valid);
      const float* a_s_row =
          p.a_s + (kMode == 1 ? static_cast<long long>(valid ? flat / p.top_k : 0) : (valid ? pos : 0)) * p.a_s_ld;
      // weight scales by global position: row block of (rank offset + n0), K block of (rank's first block + kb)
      const float* w_s0 = p.w_s + (static_cast<long long>(e) * p.w_s_rows + (p.row_blk0 + n0) / kGroup) * p.w_s_ld + p.w_kb_off;
      const float* w_s1 = p.w_s + (static_cast<long long>(e) * p.w_s_rows + (p.row_blk1 + n0) / kGroup) * p.w_s_ld + p.w_kb_off;

      float acc[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) acc[i] = 0.f;

      // scales of the next K block are fetched while this one is processed (an L2 round trip is about as long
      // as a whole K block at streaming rate)
      float sa_n = valid ? a_s_row[0] : 0.f;
      float w0_n = __ldg(w_s0);
      float w1_n = kMode == 1 ? __ldg(w_s1) : 0.f;
      for (int kb = 0; kb < num_kb; ++kb, ++j) {
        const uint32_t b = j % kPartBufs;
        const uint32_t bph = (j / kPartBufs) & 1u;
        const float s0 = sa_n * w0_n;
        const float s1 = kMode == 1 ? sa_n * w1_n : s0;
        if (kb + 1 < num_kb) {
          sa_n = valid ? a_s_row[kb + 1] : 0.f;
          w0_n = __ldg(w_s0 + kb + 1);
          if (kMode == 1) w1_n = __ldg(w_s1 + kb + 1);
        }
        ok = mbar_wait(&bar_part_full[b], bph);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) report(p.status, kErrWaitTmemFull);
          break;
        }
        tc_fence_after_sync();
        if (any_valid) {
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + b * kPartCols;
          // gate_up: columns [32 hf, +32) of the gate half and of the up half (at +64); down: columns [64 hf, +64)
          const uint32_t c0 = kMode == 1 ? 32u * hf : 64u * hf;
          const uint32_t c1 = kMode == 1 ? 64u + 32u * hf : 64u * hf + 32u;
          uint32_t v0[16], v1[16];
          tmem_ld_x16(taddr + c0, v0);
          tmem_ld_x16(taddr + c0 + 16, v1);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            acc[i] = fmaf(__uint_as_float(v0[i]), s0, acc[i]);
            acc[16 + i] = fmaf(__uint_as_float(v1[i]), s0, acc[16 + i]);
          }
          tmem_ld_x16(taddr + c1, v0);
          tmem_ld_x16(taddr + c1 + 16, v1);
          tmem_ld_wait();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bar_part_free[b]);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            acc[32 + i] = fmaf(__uint_as_float(v0[i]), s1, acc[32 + i]);
            acc[48 + i] = fmaf(__uint_as_float(v1[i]), s1, acc[48 + i]);
          }
        } else {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bar_part_free[b]);
        }
      }
      if (!ok) break;

      if (valid) {
        if (kMode == 1) {
          // acc[0..31] = gate columns n0 + 32 hf + i, acc[32..63] = the matching up columns
          __nv_bfloat16* dst = p.out + pos * p.out_ld + n0 + 32 * hf;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            Pack8 o;
#pragma unroll
            for (int i = 0; i < 8; ++i)
              o.h[i] = silu_mul_bf16_fast(__float2bfloat16_rn(acc[8 * v + i]), __float2bfloat16_rn(acc[32 + 8 * v + i]));
            if (n0 + 32 * hf + 8 * v < p.out_cols) *reinterpret_cast<uint4*>(dst + 8 * v) = o.u;
          }
        } else {
          const float w = p.topk_w[flat];
          __nv_bfloat16* dst = p.out + static_cast<long long>(flat) * p.out_ld + n0 + 64 * hf;
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            Pack8 o;
#pragma unroll
            for (int i = 0; i < 8; ++i) o.h[i] = __float2bfloat16_rn(acc[8 * v + i] * w);
            if (n0 + 64 * hf + 8 * v < p.out_cols) *reinterpret_cast<uint4*>(dst + 8 * v) = o.u;
          }
        }
      }
    }
  } else if (warp >= kWarpGather0) {
    // ------------------------------------------------------------------ token-row gather (128 bytes per row and stage)
    const int gw = warp - kWarpGather0;
    const int sub = lane >> 3;
    const int ch = lane & 7;
    const int row0 = gw * 4 + sub;
    const uint32_t swz = static_cast<uint32_t>((ch ^ (row0 & 7)) << 4);
    uint32_t s = 0, ph = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const int m_blk = tile / p.n_tiles;
      const uint8_t* src[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const long long pos = static_cast<long long>(m_blk) * BM + row0 + 16 * i;
        const int flat = p.sorted_ids[pos];
        if (kMode == 1)
          src[i] = flat < p.numel ? p.a_q + static_cast<long long>(flat / p.top_k) * p.K : nullptr;
        else
          src[i] = flat < p.numel ? p.a_q + pos * p.K : nullptr;
      }
      for (int kb = 0; kb < num_kb; ++kb) {
        ok = mbar_wait(&bar_empty[s], ph ^ 1u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) report(p.status, kErrWaitEmpty);
          break;
        }
        const uint32_t a_base = smem_u32(ring + s * kStageBytes);
        const int col = kb * kGroup - p.k_shift + ch * 16;  // this lane's 16 columns of the stage, in the rank's K range
        const bool in_k = col >= 0 && col + 16 <= p.K;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t dst = a_base + static_cast<uint32_t>(row0 + 16 * i) * 128u + swz;
          const bool live = in_k && src[i] != nullptr;
          cp_async_16(dst, live ? static_cast<const void*>(src[i] + col) : static_cast<const void*>(p.a_q), live ? 16u : 0u);
        }
        // the stage's barrier counts this thread as arrived once the copies above have landed
        cp_async_mbar_arrive_noinc(&bar_full[s]);
        if (++s == kStages) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
    cp_async_wait_all();
  }

  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == kWarpMma) tmem_dealloc(tmem_base, kTmemCols);
}

// One warp per (row, group of 128 columns): 4 values per lane.
__global__ void __launch_bounds__(256)
quant_rows_fp8_kernel(const __nv_bfloat16* __restrict__ x, int rows, int cols, uint8_t* __restrict__ q,
                      float* __restrict__ s) {
  grid_dependency_launch();
  grid_dependency_wait();
  const int groups = cols / kGroup;
  const long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= static_cast<long long>(rows) * groups) return;
  const int row = static_cast<int>(w / groups);
  const int g = static_cast<int>(w % groups);
  const __nv_bfloat16* src = x + static_cast<long long>(row) * cols + g * kGroup + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  const float v[4] = {__low2float(p0), __high2float(p0), __low2float(p1), __high2float(p1)};
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
  const float scale = fmaxf(amax, 1e-10f) / 448.0f;
  uint32_t packed = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    packed |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(v[i] / scale, __NV_SATFINITE, __NV_E4M3)) << (8 * i);
  *reinterpret_cast<uint32_t*>(q + static_cast<long long>(row) * cols + g * kGroup + lane * 4) = packed;
  if (lane == 0) s[static_cast<long long>(row) * groups + g] = scale;
}

// Same quantisation for the permuted intermediate: one CTA per 128-row block of the permutation. A block's
// valid rows come first (the permutation pads each expert at the end), so the CTA counts them once and its warps
// walk (valid row, group) pairs only; decode batches have ~4 valid rows in a block of 128.
__global__ void __launch_bounds__(256)
quant_permuted_rows_fp8_kernel(const __nv_bfloat16* __restrict__ x, int cols, int shift, uint8_t* __restrict__ q,
                               float* __restrict__ s, const int* __restrict__ sorted_ids, int numel,
                               const int* __restrict__ num_post_pad) {
  grid_dependency_launch();
  grid_dependency_wait();
  const int blk = blockIdx.x;
  if (blk * BM >= *num_post_pad) return;
  const int n_valid = __syncthreads_count(threadIdx.x < BM && sorted_ids[blk * BM + threadIdx.x] < numel);
  // group g covers columns [128 g - shift, 128 (g + 1) - shift) of the row, cut to [0, cols): with a sharded
  // intermediate dimension the groups follow the scale blocks of the unsharded tensor
  const int groups = (shift + cols + kGroup - 1) / kGroup;
  const int lane = threadIdx.x & 31;
  // gridDim.y CTAs share a block's tasks (prefill-sized batches: up to 128 valid rows per block)
  for (int task = (threadIdx.x >> 5) + 8 * blockIdx.y; task < n_valid * groups; task += 8 * gridDim.y) {
    const long long row = static_cast<long long>(blk) * BM + task / groups;
    const int g = task % groups;
    const int c = g * kGroup - shift + lane * 4;
    const bool in = c >= 0 && c + 4 <= cols;
    uint2 raw = make_uint2(0u, 0u);
    if (in) raw = *reinterpret_cast<const uint2*>(x + row * cols + c);
    const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    const float v[4] = {__low2float(p0), __high2float(p0), __low2float(p1), __high2float(p1)};
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    const float scale = fmaxf(amax, 1e-10f) / 448.0f;
    uint32_t packed = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i)
      packed |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(v[i] / scale, __NV_SATFINITE, __NV_E4M3)) << (8 * i);
    if (in) *reinterpret_cast<uint32_t*>(q + row * cols + c) = packed;
    if (lane == 0) s[row * groups + g] = scale;
  }
}

template <int kMode>
int ensure_smem_attr_f8() {
  // per device, not per process: the attribute belongs to the function on one device
  static bool done[64] = {false};
  int dev = 0;
  if (int st = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return st;
  if (dev < 0 || dev >= 64 || !done[dev]) {
    const cudaError_t e = cudaFuncSetAttribute(grouped_gemm_fp8_kernel<kMode>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(grouped_gemm_fp8_kernel)");
    if (dev >= 0 && dev < 64) done[dev] = true;
  }
  return kStatusOk;
}

int check_fp8_shapes(const GroupedGemmArgs& a, int i_offset, int i_total) {
  if (a.hidden <= 0 || a.inter <= 0 || a.hidden % kGroup != 0 || a.inter % 64 != 0)
    return set_error(kStatusInvalidArgument, "fp8 grouped GEMM: hidden must be a multiple of %d and the per-rank intermediate size of 64 (got %d, %d)", kGroup, a.hidden, a.inter);
  if (i_total % kGroup != 0 || i_offset < 0 || i_offset % 64 != 0 || i_offset + a.inter > i_total)
    return set_error(kStatusInvalidArgument, "fp8 grouped GEMM: shard [%d, %d) of an intermediate size %d (which must be a multiple of %d, the offset of 64)", i_offset, i_offset + a.inter, i_total, kGroup);
  if (a.top_k <= 0 || a.numel < 0 || a.max_m_blocks < 0 || a.status == nullptr)
    return set_error(kStatusInvalidArgument, "fp8 grouped GEMM: bad routing sizes or null status word");
  if (a.activation != 0) return set_error(kStatusInvalidArgument, "fp8 grouped GEMM: only the silu activation is built");
  return kStatusOk;
}

}  // namespace

int launch_quant_rows_fp8(const __nv_bfloat16* x, int rows, int cols, int shift, uint8_t* q, float* s,
                          const int* sorted_ids, int numel, const int* num_post_pad, cudaStream_t stream) {
  if (rows < 0 || cols <= 0 || cols % 4 != 0 || shift < 0 || shift >= kGroup || shift % 4 != 0 ||
      (sorted_ids == nullptr && (cols % kGroup != 0 || shift != 0)))
    return set_error(kStatusInvalidArgument, "fp8 quantisation: unsupported row length %d / shift %d", cols, shift);
  if (rows == 0) return kStatusOk;
  if (sorted_ids != nullptr) {
    if (rows % BM != 0) return set_error(kStatusInvalidArgument, "fp8 quantisation of permuted rows: %d rows is not a multiple of %d", rows, BM);
    if (int st = check_cuda(launch_pdl(quant_permuted_rows_fp8_kernel, dim3(static_cast<unsigned>(rows / BM), numel > 4096 ? 8u : 1u), dim3(256), 0,
                                       stream, x, cols, shift, q, s, sorted_ids, numel, num_post_pad),
                            "quant_permuted_rows_fp8 launch"))
      return st;
    count_launches(1);
    return check_launch("quant_permuted_rows_fp8");
  }
  const long long warps = static_cast<long long>(rows) * (cols / kGroup);
  const unsigned blocks = static_cast<unsigned>((warps + 7) / 8);
  if (int st = check_cuda(launch_pdl(quant_rows_fp8_kernel, dim3(blocks), dim3(256), 0, stream, x, rows, cols, q, s),
                          "quant_rows_fp8 launch"))
    return st;
  count_launches(1);
  return check_launch("quant_rows_fp8");
}

int launch_grouped_gemm1_fp8(const GroupedGemmArgs& a, const uint8_t* x_q, const float* x_s, const uint8_t* w13_q,
                             const float* w13_s, int i_offset, int i_total, __nv_bfloat16* h_sorted, cudaStream_t stream) {
  if (int st = check_fp8_shapes(a, i_offset, i_total)) return st;
  if (a.numel == 0 || a.max_m_blocks == 0) return kStatusOk;
  if (int st = ensure_smem_attr_f8<1>()) return st;
  CUtensorMap map_b;
  const uint64_t dims[3] = {static_cast<uint64_t>(a.hidden), static_cast<uint64_t>(2 * a.inter), static_cast<uint64_t>(a.num_experts)};
  const uint32_t box[3] = {kGroup, 64, 1};
  if (int st = make_map(&map_b, w13_q, 3, dims, box, 1)) return st;
  ParamsF8 p{};
  p.sorted_ids = a.sorted_ids; p.expert_ids = a.expert_ids; p.num_post_pad = a.num_post_pad;
  p.a_q = x_q; p.a_s = x_s; p.w_s = w13_s;
  // scales of the unsharded [E, 2 I, H] weight: gate rows of this shard start at i_offset, up rows at I + i_offset
  p.w_s_rows = 2 * i_total / kGroup; p.w_s_ld = a.hidden / kGroup; p.a_s_ld = a.hidden / kGroup;
  p.num_kb = a.hidden / kGroup; p.k_shift = 0; p.w_kb_off = 0; p.row_blk0 = i_offset; p.row_blk1 = i_total + i_offset;
  p.numel = a.numel; p.top_k = a.top_k; p.K = a.hidden;
  p.tile_cols = 64; p.n_tiles = a.inter / 64; p.out_cols = a.inter; p.inter = a.inter;
  p.out = h_sorted; p.out_ld = a.inter; p.topk_w = nullptr; p.status = a.status;
  const long long tiles = static_cast<long long>(a.max_m_blocks) * p.n_tiles;
  const int grid = static_cast<int>(tiles < device_sm_count() ? tiles : device_sm_count());
  if (int st = check_cuda(launch_pdl(grouped_gemm_fp8_kernel<1>, dim3(grid), dim3(kThreads), kSmemBytes, stream, map_b, p),
                          "grouped_gemm_fp8 gate_up launch"))
    return st;
  count_launches(1);
  return check_launch("grouped_gemm_fp8 gate_up");
}

int launch_grouped_gemm2_fp8(const GroupedGemmArgs& a, const uint8_t* h_q, const float* h_s, const uint8_t* w2_q,
                             const float* w2_s, int i_offset, int i_total, const float* topk_w, __nv_bfloat16* c3,
                             cudaStream_t stream) {
  if (int st = check_fp8_shapes(a, i_offset, i_total)) return st;
  if (a.numel == 0 || a.max_m_blocks == 0) return kStatusOk;
  if (int st = ensure_smem_attr_f8<2>()) return st;
  CUtensorMap map_b;
  const uint64_t dims[3] = {static_cast<uint64_t>(a.inter), static_cast<uint64_t>(a.hidden), static_cast<uint64_t>(a.num_experts)};
  const uint32_t box[3] = {kGroup, 128, 1};
  if (int st = make_map(&map_b, w2_q, 3, dims, box, 1)) return st;
  ParamsF8 p{};
  p.sorted_ids = a.sorted_ids; p.expert_ids = a.expert_ids; p.num_post_pad = a.num_post_pad;
  p.a_q = h_q; p.a_s = h_s; p.w_s = w2_s;
  // K = this rank's slice [i_offset, i_offset + inter) of I: K blocks follow the scale blocks of the unsharded weight
  p.k_shift = i_offset % kGroup;
  p.num_kb = (p.k_shift + a.inter + kGroup - 1) / kGroup;
  p.w_kb_off = i_offset / kGroup;
  p.w_s_rows = a.hidden / kGroup; p.w_s_ld = i_total / kGroup; p.a_s_ld = p.num_kb; p.row_blk0 = 0; p.row_blk1 = 0;
  p.numel = a.numel; p.top_k = a.top_k; p.K = a.inter;
  p.tile_cols = 128; p.n_tiles = a.hidden / 128; p.out_cols = a.hidden; p.inter = 0;
  p.out = c3; p.out_ld = a.hidden; p.topk_w = topk_w; p.status = a.status;
  const long long tiles = static_cast<long long>(a.max_m_blocks) * p.n_tiles;
  const int grid = static_cast<int>(tiles < device_sm_count() ? tiles : device_sm_count());
  if (int st = check_cuda(launch_pdl(grouped_gemm_fp8_kernel<2>, dim3(grid), dim3(kThreads), kSmemBytes, stream, map_b, p),
                          "grouped_gemm_fp8 down launch"))
    return st;
  count_launches(1);
  return check_launch("grouped_gemm_fp8 down");
}

}  // namespace moe_b200
