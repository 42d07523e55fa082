// Grouped expert GEMMs of the MoE block on the 5th-generation tensor cores.
//
// What the reference does with one Triton kernel called twice plus two element-wise kernels
// (nanovllm/layers/for_moe/fused_moe.py:84-223, 575-631; csrc/activation_kernels.cu:9-25):
//   pass 1 (gate_up): C1[r, :] = bf16(x[r / k] . w13[e]^T), h = bf16(bf16(silu(gate)) * up)
//   pass 2 (down):    C3[r, :] = bf16((h[r] . w2[e]^T) * topk_w[r])
// Here each pass is one persistent, warp-specialised kernel:
//   * tiles are 128 permuted token rows (one block of the moe_align_block_size permutation with
//     block size 128, so a tile never mixes experts) by up to 256 weight rows;
//   * weights stream through TMA (3-D map [K, rows, expert], 128-byte swizzle, no cluster fan-out)
//     into a shared-memory ring that takes all 227 KB (4 stages at N=256, 5 at N=192, 7 at N=128); the
//     token rows (hidden states gathered through the permutation in pass 1, rows of the permuted
//     intermediate in pass 2) come in with 16-byte cp.async from four warps, written straight into the
//     same swizzled K-major layout, and signal the stage's barrier asynchronously
//     (cp.async.mbarrier.arrive.noinc: the arrival fires when the thread's copies have landed), which is how
//     CUTLASS's sm_100 collectives hand cp.async-filled stages to tcgen05.mma
//     (cutlass/gemm/collective/sm100_mma_cpasync_warpspecialized.hpp, ..._mixed_tma_cpasync_...: producer_commit
//     with cpasync_barrier_arrive, consumer_wait, UMMA, no proxy fence in between). A variant that waited for
//     the copies (cp.async.wait_group), issued fence.proxy.async and arrived one stage late measured 5 % slower
//     at decode and 10 % at prefill (the gather thread then keeps two stages in flight instead of the whole
//     ring) with bit-identical results, and was not kept. Splitting the operands over the TMA unit and the LSU
//     path measured faster than TMA for both, and padding rows cost no traffic (zero-fill);
//   * one thread issues tcgen05.mma (M=128, N<=256, K=16 per instruction) into one of two 256-column
//     TMEM accumulators, so the epilogue of tile i overlaps the main loop of tile i+1;
//   * pass 1 keeps the gate rows and the matching up rows of w13 in the same tile (columns [0,BNH)
//     and [BNH,2BNH) of the accumulator), so the activation is applied in registers with the
//     reference's three bf16 roundings and only h is written, in permuted order;
//   * pass 2 scales by the routed weight and writes bf16 rows at their flat index t*k+j; an epilogue warp owns
//     one row per lane (the TMEM layout), so it turns 64 columns of its 32 rows around in a 4 KB shared-memory
//     patch and stores whole 128-byte lines (four rows per instruction) instead of 32 scattered 16-byte pieces.
//   * roles by warp: 0 = TMA producer, 1 = MMA issuer, then the epilogue warps, then the gather warps. The kernel is
//     instantiated with four epilogue + four gather warps, and for the down pass over a rank's thin slice of I
//     (two to four K blocks per tile, where the epilogue sets the pace) with eight epilogue warps - two per TMEM lane
//     quarter, half of the tile's columns each - and two gather warps;
//   * whatever a role reads from global memory per tile (expert id, permutation entries, routed weight) is fetched
//     one or two tiles ahead.
// The tile list is static: tile = blockIdx.x + i*gridDim.x over (m_block, n_tile), n fastest.
#include <cmath>
#include <cstdio>
#include <cstring>

#include "act_math.cuh"
#include "launch.cuh"
#include "moe_b200_internal.cuh"
#include "ptx.cuh"

namespace moe_b200 {

namespace {

constexpr int BM = kBlockM;
constexpr int BK = 64;  // bf16 elements per K block = one 128-byte swizzle row
constexpr int kMaxStages = 8;
constexpr int kABytes = BM * BK * 2;
constexpr int kAccCols = 256;
constexpr int kTmemCols = 512;
constexpr int kBarrierBytes = 1024;                      // barriers + TMEM slot, in front of the ring
constexpr int kSmemLimit = 227 * 1024;                   // opt-in shared memory per CTA on sm_100
constexpr int kPatchBytes = 32 * 128;                    // one transposition patch (down pass): 32 rows x 64 bf16 columns
constexpr int kPatchesPerWarp = 2;                       // used in turn by each epilogue warp
constexpr int kRingBudget = kSmemLimit - kBarrierBytes - 1024 /*alignment slack*/;

constexpr int kWarpTma = 0;
constexpr int kWarpMma = 1;
constexpr int kWarpEpilogue0 = 2;  // kEpiWarps warps (4, or 8 for thin K: two per TMEM lane quarter, half the columns each)
// after them kGatherWarps warps (4, or 2) bring the token rows in by cp.async
constexpr int role_threads(int epi_warps, int gather_warps) { return 32 * (2 + epi_warps + gather_warps); }

struct KernelParams {
  const int* sorted_ids;
  const int* expert_ids;
  const int* num_post_pad;
  const __nv_bfloat16* x;  // token-side operand: hidden states [T, K] (gate_up) or permuted intermediate [rows, K] (down)
  int numel;
  int top_k;
  int K;
  int n_tiles;      // tiles along the output columns per m block
  int tile_cols;    // output columns per tile
  int mma_n;        // accumulator columns per tile (2*tile_cols for gate_up)
  int out_cols;     // valid output columns (inter for gate_up, hidden for down)
  int inter;        // row offset of the up half inside w13[e]
  int interleaved;  // gate/up rows interleaved (swigluoai layout)
  __nv_bfloat16* out;
  long long out_ld;
  const float* topk_w;
  const __nv_bfloat16* bias;  // [E, 2*inter] (gate_up) or [E, hidden] (down), may be null
  float alpha, limit;
  int* status;
  int stages;       // ring depth (2..kMaxStages)
  int stage_bytes;  // kABytes + mma_n * 128
};

union Pack8 {
  uint4 u;
  __nv_bfloat16 h[8];
};

__device__ __forceinline__ void report(int* status, int code) { atomicCAS(status, 0, code); }

// Epilogue of one 128-row tile for the 32 rows one warp may read from TMEM (taddr = its lane quarter and
// the accumulator's first column). pos = permuted row, flat = t*k+j of that row (>= numel on padding rows);
// patch = shared-memory address of this warp's transposition patches, [c_begin, c_end) = the tile columns this
// warp handles (down pass only; the gate_up pass always takes the whole tile).
template <int kMode>
__device__ __forceinline__ void epilogue_rows(const KernelParams& p, uint32_t taddr, long long pos, int flat,
                                              bool valid, float w, int e, int n0, uint32_t patch, int c_begin,
                                              int c_end) {
  if (kMode == 1) {
    __nv_bfloat16* out_row = p.out + pos * p.out_ld;
    if (!p.interleaved) {
      const __nv_bfloat16* bias_g = p.bias ? p.bias + static_cast<long long>(e) * 2 * p.inter : nullptr;
      // Two 16-column chunks in flight: the TMEM loads of the next chunk overlap the math of this one.
      uint32_t g0[16], u0[16], g1[16], u1[16];
      auto finish = [&](const uint32_t (&g)[16], const uint32_t (&u)[16], int c) {
        const int col = n0 + c;
        if (valid && col < p.out_cols) {
          Pack8 o[2];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float gf = __uint_as_float(g[j]);
            float uf = __uint_as_float(u[j]);
            if (bias_g) {
              gf += __bfloat162float(bias_g[col + j]);
              uf += __bfloat162float(bias_g[p.inter + col + j]);
            }
            o[j >> 3].h[j & 7] = silu_mul_bf16_fast(__float2bfloat16_rn(gf), __float2bfloat16_rn(uf));
          }
          *reinterpret_cast<uint4*>(out_row + col) = o[0].u;
          *reinterpret_cast<uint4*>(out_row + col + 8) = o[1].u;
        }
      };
      tmem_ld_x16(taddr, g0);
      tmem_ld_x16(taddr + p.tile_cols, u0);
      for (int c = 0; c < p.tile_cols; c += 32) {
        tmem_ld_wait();
        if (c + 16 < p.tile_cols) {
          tmem_ld_x16(taddr + c + 16, g1);
          tmem_ld_x16(taddr + p.tile_cols + c + 16, u1);
        }
        finish(g0, u0, c);
        tmem_ld_wait();
        if (c + 32 < p.tile_cols) {
          tmem_ld_x16(taddr + c + 32, g0);
          tmem_ld_x16(taddr + p.tile_cols + c + 32, u0);
        }
        if (c + 16 < p.tile_cols) finish(g1, u1, c + 16);
      }
    } else {
      const __nv_bfloat16* bias_g = p.bias ? p.bias + static_cast<long long>(e) * 2 * p.inter : nullptr;
      for (int c = 0; c < p.tile_cols; c += 8) {
        uint32_t gu[16];
        tmem_ld_x16(taddr + 2 * c, gu);
        tmem_ld_wait();
        const int col = n0 + c;
        if (valid && col < p.out_cols) {
          Pack8 o;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float gf = __uint_as_float(gu[2 * j]);
            float uf = __uint_as_float(gu[2 * j + 1]);
            if (bias_g) {
              gf += __bfloat162float(bias_g[2 * (col + j)]);
              uf += __bfloat162float(bias_g[2 * (col + j) + 1]);
            }
            o.h[j] = swigluoai_bf16(__float2bfloat16_rn(gf), __float2bfloat16_rn(uf), p.alpha, p.limit);
          }
          *reinterpret_cast<uint4*>(out_row + col) = o.u;
        }
      }
    }
  } else {
    const __nv_bfloat16* bias_d = p.bias ? p.bias + static_cast<long long>(e) * p.out_cols : nullptr;
    const int lane = threadIdx.x & 31;
    if (__popc(__ballot_sync(0xffffffffu, valid)) <= 8) {
      // decode-sized batches: a handful of live rows among the 32 of this warp. Each live lane converts and
      // stores its own row; turning all 32 rows around in shared memory would cost more than it saves.
      // Four TMEM loads (64 columns) per wait: with a short K the tile's main loop is a thousand cycles and a
      // wait per 16 columns made this epilogue the longest stage of the pipeline.
      __nv_bfloat16* out_row = p.out + static_cast<long long>(valid ? flat : 0) * p.out_ld;
      for (int c0 = c_begin; c0 < c_end; c0 += 64) {
        uint32_t d[4][16];
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) tmem_ld_x16(taddr + c0 + 16 * q4, d[q4]);
        tmem_ld_wait();
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int col = n0 + c0 + 16 * q4;
          if (valid && c0 + 16 * q4 < c_end && col < p.out_cols) {
            Pack8 o[2];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              float v = __uint_as_float(d[q4][j]);
              if (bias_d) v += __bfloat162float(bias_d[col + j]);
              o[j >> 3].h[j & 7] = __float2bfloat16_rn(v * w);
            }
            *reinterpret_cast<uint4*>(out_row + col) = o[0].u;
            *reinterpret_cast<uint4*>(out_row + col + 8) = o[1].u;
          }
        }
      }
      return;
    }
    // Two patches per warp, used in turn, and the TMEM loads of the next 64 columns issued as soon as the current
    // ones are converted: TMEM latency, shared-memory round trip and global stores of neighbouring chunks overlap.
    const int chunk = lane & 7;   // read side: 16-byte piece of a row
    const int rsub = lane >> 3;   // read side: row inside a group of four
    int flat_r[8];                // flat index of the eight rows this lane stores pieces of
#pragma unroll
    for (int i = 0; i < 8; ++i) flat_r[i] = __shfl_sync(0xffffffffu, flat, rsub + 4 * i);
    uint32_t d[4][16];
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) tmem_ld_x16(taddr + c_begin + 16 * q4, d[q4]);
    int buf = 0;
    for (int c0 = c_begin; c0 < c_end; c0 += 64, buf ^= 1) {
      const uint32_t patch_b = patch + static_cast<uint32_t>(buf) * kPatchBytes;
      const uint32_t patch_w = patch_b + static_cast<uint32_t>(lane) * 128u;  // this lane's row of the patch
      tmem_ld_wait();
      const int col0 = n0 + c0;
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        Pack8 o[2];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float v = __uint_as_float(d[q4][j]);
          if (bias_d && col0 + 16 * q4 + j < p.out_cols) v += __bfloat162float(bias_d[col0 + 16 * q4 + j]);
          o[j >> 3].h[j & 7] = __float2bfloat16_rn(v * w);
        }
        // row `lane`, pieces 2*q4 and 2*q4+1, xor-swizzled so that a quarter warp covers all 32 banks
        st_shared_v4(patch_w + (static_cast<uint32_t>((2 * q4) ^ (lane & 7)) << 4), o[0].u);
        st_shared_v4(patch_w + (static_cast<uint32_t>((2 * q4 + 1) ^ (lane & 7)) << 4), o[1].u);
      }
      if (c0 + 64 < c_end) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) tmem_ld_x16(taddr + c0 + 64 + 16 * q4, d[q4]);
      }
      __syncwarp();  // this patch is complete. (Its previous contents were read two chunks ago: every lane finished
                     // those reads before it arrived at the barrier of the chunk in between.)
      const int col = col0 + chunk * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = rsub + 4 * i;
        const uint4 v = ld_shared_v4(patch_b + static_cast<uint32_t>(r) * 128u + (static_cast<uint32_t>(chunk ^ (r & 7)) << 4));
        if (flat_r[i] < p.numel && col < p.out_cols && c0 + chunk * 8 < c_end)
          *reinterpret_cast<uint4*>(p.out + static_cast<long long>(flat_r[i]) * p.out_ld + col) = v;
      }
    }
  }
}

template <int kMode, int kEpiWarps, int kGatherWarps>  // kMode: 1 = gate_up, 2 = down
__global__ void __launch_bounds__(role_threads(kEpiWarps, kGatherWarps), 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_b, const KernelParams p) {
  constexpr int kWarpGather0 = kWarpEpilogue0 + kEpiWarps;
  constexpr int kRowsPerStep = 4 * kGatherWarps;       // token rows one gather instruction of all warps covers
  constexpr int kGatherSteps = BM / kRowsPerStep;       // copies per thread and stage
  extern __shared__ uint8_t smem_raw[];
  // operand stages want 1024-byte alignment in the shared window (swizzle atoms, descriptor base offset 0)
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* bar_empty = bar_full + kMaxStages;
  uint64_t* bar_tmem_full = bar_empty + kMaxStages;
  uint64_t* bar_tmem_empty = bar_tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_tmem_empty + 2);
  uint8_t* ring = smem + kBarrierBytes;
  const uint32_t num_stages = static_cast<uint32_t>(p.stages);
  const uint32_t stage_bytes = static_cast<uint32_t>(p.stage_bytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(&bar_full[s], 1 + 32 * kGatherWarps);
      mbar_init(&bar_empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bar_tmem_full[a], 1);
      mbar_init(&bar_tmem_empty[a], kEpiWarps);
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
  // set-up done: let the next kernel start its own, then wait for the previous kernel's results
  grid_dependency_launch();
  grid_dependency_wait();

  const int num_m_blocks = *p.num_post_pad / BM;
  const int total_tiles = num_m_blocks * p.n_tiles;
  const int num_kb = (p.K + BK - 1) / BK;

  if (warp == kWarpTma) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t s = 0, ph = 0;
      bool ok = true;
      // the expert of the next tile is fetched while this tile's loads are issued: with a short K (a rank's slice
      // of I in the down pass) a tile is a few stages, and a dependent global load per tile would show
      int e_next = static_cast<int>(blockIdx.x) < total_tiles ? p.expert_ids[blockIdx.x / p.n_tiles] : 0;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int m_blk = tile / p.n_tiles;
        const int n0 = (tile % p.n_tiles) * p.tile_cols;
        const int e = e_next;
        if (tile + static_cast<int>(gridDim.x) < total_tiles) e_next = p.expert_ids[(tile + gridDim.x) / p.n_tiles];
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&bar_empty[s], ph ^ 1u)) {
            report(p.status, kErrWaitEmpty);
            ok = false;
            break;
          }
          uint8_t* b_dst = ring + s * stage_bytes + kABytes;
          mbar_arrive_expect_tx(&bar_full[s], static_cast<uint32_t>(p.mma_n) * 128u);
          if (kMode == 1 && !p.interleaved) {
            tma_load_3d(b_dst, &tmap_b, kb * BK, n0, e, &bar_full[s]);
            tma_load_3d(b_dst + p.tile_cols * 128, &tmap_b, kb * BK, p.inter + n0, e, &bar_full[s]);
          } else {
            tma_load_3d(b_dst, &tmap_b, kb * BK, kMode == 1 ? 2 * n0 : n0, e, &bar_full[s]);
          }
          if (++s == num_stages) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == kWarpMma) {
    // ------------------------------------------------------------------ MMA issuer
    // One thread runs the whole loop. The tensor pipe queues next to nothing: a gap of ~100 cycles between
    // two tcgen05.mma of this thread is a bubble (measured: four dependent shared-memory accesses per K
    // block cost 22 % of the MMA rate). So the barrier needed next is probed while MMAs just issued still
    // execute, and the loop only blocks when the probe failed.
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(BM, static_cast<uint32_t>(p.mma_n));
      const uint64_t adesc0 = umma_desc_k_sw128(smem_u32(ring));
      const uint64_t bdesc0 = umma_desc_k_sw128(smem_u32(ring) + kABytes);
      const uint64_t stage_step = stage_bytes >> 4;  // descriptors address shared memory in 16-byte units
      const int my_tiles = static_cast<int>(blockIdx.x) < total_tiles
                               ? (total_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x)
                               : 0;
      uint32_t s = 0, ph = 0;
      uint64_t stage_off = 0;
      bool ok = true;
      bool acc_ready = false, stage_ready = false;
      for (int t = 0; t < my_tiles && ok; ++t) {
        const uint32_t acc = static_cast<uint32_t>(t) & 1u;
        const uint32_t acc_ph = (static_cast<uint32_t>(t) >> 1) & 1u;
        if (!acc_ready && !mbar_wait(&bar_tmem_empty[acc], acc_ph ^ 1u)) {
          report(p.status, kErrWaitTmemEmpty);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kAccCols;
        uint32_t accumulate = 0;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!stage_ready && !mbar_wait(&bar_full[s], ph)) {
            report(p.status, kErrWaitFull);
            ok = false;
            break;
          }
          const uint64_t adesc = adesc0 + stage_off;
          const uint64_t bdesc = bdesc0 + stage_off;
          // advancing 16 bf16 = 32 bytes along K inside the swizzled row: +2 in 16-byte units
          umma_bf16(d_tmem, adesc, bdesc, idesc, accumulate);
          umma_bf16(d_tmem, adesc + 2, bdesc + 2, idesc, 1u);
          uint32_t s_next = s + 1, ph_next = ph;
          if (s_next == num_stages) {
            s_next = 0;
            ph_next ^= 1u;
          }
          const bool last_kb = kb + 1 == num_kb;
          if (!last_kb || t + 1 < my_tiles) stage_ready = mbar_try_wait(&bar_full[s_next], ph_next);
          if (last_kb && t + 1 < my_tiles)
            acc_ready = mbar_try_wait(&bar_tmem_empty[acc ^ 1u], ((static_cast<uint32_t>(t + 1) >> 1) & 1u) ^ 1u);
          umma_bf16(d_tmem, adesc + 4, bdesc + 4, idesc, 1u);
          umma_bf16(d_tmem, adesc + 6, bdesc + 6, idesc, 1u);
          accumulate = 1u;
          umma_commit(&bar_empty[s]);
          stage_off = s_next == 0 ? 0 : stage_off + stage_step;
          s = s_next;
          ph = ph_next;
        }
        if (ok) umma_commit(&bar_tmem_full[acc]);
      }
    }
    __syncwarp();
  } else if (warp >= kWarpEpilogue0 && warp < kWarpEpilogue0 + kEpiWarps) {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int row_in_tile = q * 32 + lane;
    // with eight warps two share a lane quarter and take half of the tile's columns each
    const int col_part = (warp - kWarpEpilogue0) / 4;
    const int cols_per_part = kEpiWarps == 8 ? (p.tile_cols / 2 + 63) / 64 * 64 : p.tile_cols;
    const int c_begin = col_part * cols_per_part;
    const int c_end = min(p.tile_cols, c_begin + cols_per_part);
    const uint32_t patch = smem_u32(ring) + num_stages * stage_bytes +
                           static_cast<uint32_t>(warp - kWarpEpilogue0) * (kPatchesPerWarp * kPatchBytes);
    // A tile's permutation entry, routed weight and expert come from global memory, the weight through the entry.
    // These warps handle the tiles one after the other, so with a short main loop (a rank's slice of I in the down
    // pass: two K blocks) two dependent loads at the head of every tile would set the pace of the whole kernel:
    // the entry is fetched two tiles ahead, the weight and the expert one tile ahead.
    const int step = static_cast<int>(gridDim.x);
    auto load_flat = [&](int tile) {
      return tile < total_tiles ? p.sorted_ids[static_cast<long long>(tile / p.n_tiles) * BM + row_in_tile] : p.numel;
    };
    auto load_expert = [&](int tile) { return tile < total_tiles ? p.expert_ids[tile / p.n_tiles] : 0; };
    int flat_cur = load_flat(blockIdx.x);
    int flat_nx = load_flat(static_cast<int>(blockIdx.x) + step);
    int e_cur = load_expert(blockIdx.x);
    float w_cur = (kMode == 2 && flat_cur < p.numel) ? p.topk_w[flat_cur] : 0.f;
    uint32_t tile_iter = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += step, ++tile_iter) {
      const uint32_t acc = tile_iter & 1u;
      const uint32_t acc_ph = (tile_iter >> 1) & 1u;
      const int m_blk = tile / p.n_tiles;
      const int n0 = (tile % p.n_tiles) * p.tile_cols;
      const int e = e_cur;
      const long long pos = static_cast<long long>(m_blk) * BM + row_in_tile;
      const int flat = flat_cur;
      const bool valid = flat < p.numel;
      const float w = w_cur;
      // prefetch for the next tiles (consumed after this tile's epilogue)
      flat_cur = flat_nx;
      w_cur = (kMode == 2 && flat_nx < p.numel) ? p.topk_w[flat_nx] : 0.f;
      e_cur = load_expert(tile + step);
      flat_nx = load_flat(tile + 2 * step);

      bool ok = mbar_wait(&bar_tmem_full[acc], acc_ph);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) report(p.status, kErrWaitTmemFull);
        break;
      }
      tc_fence_after_sync();

      if (__any_sync(0xffffffffu, valid) && c_begin < c_end) {
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * kAccCols;
        epilogue_rows<kMode>(p, taddr, pos, flat, valid, w, e, n0, patch, c_begin, c_end);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_tmem_empty[acc]);
    }
  } else if (warp >= kWarpGather0) {
    // ------------------------------------------------------------------ token-row gather (gate_up pass)
    const int gw = warp - kWarpGather0;  // 0..kGatherWarps-1
    const int sub = lane >> 3;           // row inside a group of 4
    const int ch = lane & 7;             // 16-byte chunk inside the 128-byte row
    const int row0 = gw * 4 + sub;       // rows handled: row0 + kRowsPerStep*i
    const uint32_t swz = static_cast<uint32_t>((ch ^ (row0 & 7)) << 4);
    uint32_t s = 0, ph = 0;
    bool ok = true;
    // the permutation entries of the next tile are fetched one tile ahead (same reason as in the producer)
    int flat_next[kGatherSteps];
#pragma unroll
    for (int i = 0; i < kGatherSteps; ++i)
      flat_next[i] = static_cast<int>(blockIdx.x) < total_tiles
                         ? p.sorted_ids[static_cast<long long>(blockIdx.x / p.n_tiles) * BM + row0 + kRowsPerStep * i]
                         : p.numel;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const int m_blk = tile / p.n_tiles;
      const __nv_bfloat16* src[kGatherSteps];
      const bool more = tile + static_cast<int>(gridDim.x) < total_tiles;
      const long long next_base = more ? static_cast<long long>((tile + gridDim.x) / p.n_tiles) * BM + row0 : 0;
#pragma unroll
      for (int i = 0; i < kGatherSteps; ++i) {
        const int flat = flat_next[i];
        if (more) flat_next[i] = p.sorted_ids[next_base + kRowsPerStep * i];
        if (kMode == 1)
          src[i] = flat < p.numel ? p.x + static_cast<long long>(flat / p.top_k) * p.K + ch * 8 : nullptr;
        else  // down pass: row p of the permuted intermediate
          src[i] = flat < p.numel ? p.x + (static_cast<long long>(m_blk) * BM + row0 + kRowsPerStep * i) * p.K + ch * 8 : nullptr;
      }
      for (int kb = 0; kb < num_kb; ++kb) {
        ok = mbar_wait(&bar_empty[s], ph ^ 1u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) report(p.status, kErrWaitEmpty);
          break;
        }
        const uint32_t a_base = smem_u32(ring + s * stage_bytes);
        const bool in_k = kb * BK + ch * 8 < p.K;
#pragma unroll
        for (int i = 0; i < kGatherSteps; ++i) {
          const uint32_t dst = a_base + static_cast<uint32_t>(row0 + kRowsPerStep * i) * 128u + swz;
          const bool live = in_k && src[i] != nullptr;
          cp_async_16(dst, live ? static_cast<const void*>(src[i] + kb * BK) : static_cast<const void*>(p.x),
                      live ? 16u : 0u);
        }
        // the stage's barrier counts this thread as arrived once the copies above have landed
        cp_async_mbar_arrive_noinc(&bar_full[s]);
        if (++s == num_stages) {
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

// ---------------------------------------------------------------- host side
template <int kMode, int kEpiWarps, int kGatherWarps>
int ensure_smem_attr() {
  // the attribute belongs to the function on one device: a process that drives several GPUs sets it on each
  static bool done[64] = {false};
  int dev = 0;
  if (int st = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return st;
  if (dev < 0 || dev >= 64 || !done[dev]) {
    const cudaError_t e = cudaFuncSetAttribute(grouped_gemm_kernel<kMode, kEpiWarps, kGatherWarps>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(grouped_gemm_kernel)");
    if (dev >= 0 && dev < 64) done[dev] = true;
  }
  return kStatusOk;
}

// Widest gate_up tile (output columns, a multiple of 16 dividing `inter`) among those within 2 % of the
// best wave efficiency: for decode-sized batches the tile count is a handful of waves, and a width that
// leaves the last wave nearly empty costs more than the narrower MMA.
int pick_gate_up_tile(int inter, double m_blocks) {
  const int sms = device_sm_count();
  double best = 0.0;
  for (int c = 128; c >= 16; c -= 16)
    if (inter % c == 0 && (c >= 64 || inter < 64)) best = fmax(best, wave_efficiency(m_blocks * (inter / c), sms));
  for (int c = 128; c >= 16; c -= 16)
    if (inter % c == 0 && (c >= 64 || inter < 64) && wave_efficiency(m_blocks * (inter / c), sms) >= best - 0.02) return c;
  for (int c = 128; c >= 16; c -= 16)
    if (inter % c == 0) return c;
  return 0;
}

int pick_down_tile(int hidden, int inter, double m_blocks) {
  if (hidden <= 128) return (hidden + 15) / 16 * 16;
  // a rank's thin slice of I: a tile's main loop is a few K blocks and per-tile costs set the pace, so fewer,
  // wider tiles win whatever the wave count says
  if (inter <= 256) return 256;
  const int sms = device_sm_count();
  const double e256 = wave_efficiency(m_blocks * ((hidden + 255) / 256), sms);
  const double e128 = wave_efficiency(m_blocks * ((hidden + 127) / 128), sms);
  return e256 >= e128 - 0.02 ? 256 : 128;
}

// Ring depth that fits the shared-memory budget for a given accumulator width.
void pick_ring(int mma_n, int reserve_bytes, int* stages, int* stage_bytes) {
  *stage_bytes = kABytes + mma_n * 128;
  int s = (kRingBudget - reserve_bytes) / *stage_bytes;
  if (s > kMaxStages) s = kMaxStages;
  *stages = s;
}

int check_common(const GroupedGemmArgs& a) {
  if (a.hidden <= 0 || a.inter <= 0 || a.hidden % 8 != 0 || a.inter % 16 != 0)
    return set_error(kStatusInvalidArgument, "grouped GEMM: hidden must be a multiple of 8 and the per-rank intermediate size a multiple of 16 (got %d, %d)", a.hidden, a.inter);
  if (a.top_k <= 0 || a.numel < 0 || a.max_m_blocks < 0 || a.status == nullptr)
    return set_error(kStatusInvalidArgument, "grouped GEMM: bad routing sizes or null status word");
  return kStatusOk;
}

}  // namespace

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// Tensor map of a dense tensor (bf16, or bytes when elem_bytes == 1), innermost dimension contiguous, 128-byte
// swizzle; dims/box given innermost first.
int make_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint32_t* box, int elem_bytes) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return set_error(kStatusDriverEntryPoint, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[3];
  cuuint64_t gstride[2];
  cuuint32_t bdim[3];
  cuuint32_t estr[3] = {1, 1, 1};
  uint64_t stride = static_cast<uint64_t>(elem_bytes);
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    stride *= dims[i];
    if (i + 1 < rank) gstride[i] = stride;
  }
  const CUresult r = fn(map, elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank), const_cast<void*>(base),
                        gdim, gstride, bdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(kStatusCudaError, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  return kStatusOk;
}

// Token blocks the permutation is expected to produce: experts hit at least once (each token picks
// top_k distinct experts out of E) plus the full blocks of the busy ones. Only used to pick tile widths.
double expected_m_blocks(int numel, int top_k, int num_experts) {
  const double tokens = static_cast<double>(numel) / top_k;
  const double miss = pow(1.0 - static_cast<double>(top_k) / num_experts, tokens);
  return num_experts * (1.0 - miss) + static_cast<double>(numel) / BM;
}

// Fraction of SM-time doing work when `tiles` equal tiles are dealt round-robin to `sms` persistent CTAs.
double wave_efficiency(double tiles, int sms) {
  const double waves = ceil(tiles / sms);
  return waves > 0 ? tiles / (waves * sms) : 1.0;
}

int device_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

int launch_grouped_gemm1(const GroupedGemmArgs& a, const __nv_bfloat16* x, const __nv_bfloat16* w13,
                         const __nv_bfloat16* w13_bias, __nv_bfloat16* h_sorted, int rows_cap, cudaStream_t stream) {
  if (int st = check_common(a)) return st;
  if (a.numel == 0 || a.max_m_blocks == 0) return kStatusOk;
  const int tile_cols = pick_gate_up_tile(a.inter, expected_m_blocks(a.numel, a.top_k, a.num_experts));
  const int mma_n = 2 * tile_cols;
  if (int st = ensure_smem_attr<1, 4, 4>()) return st;

  CUtensorMap map_b;
  const uint64_t dims[3] = {static_cast<uint64_t>(a.hidden), static_cast<uint64_t>(2 * a.inter), static_cast<uint64_t>(a.num_experts)};
  const uint32_t box[3] = {BK, static_cast<uint32_t>(a.activation == 1 ? mma_n : tile_cols), 1};
  if (int st = make_map(&map_b, w13, 3, dims, box, 2)) return st;

  KernelParams p{};
  p.sorted_ids = a.sorted_ids; p.expert_ids = a.expert_ids; p.num_post_pad = a.num_post_pad;
  p.x = x; p.numel = a.numel; p.top_k = a.top_k; p.K = a.hidden;
  p.n_tiles = a.inter / tile_cols; p.tile_cols = tile_cols; p.mma_n = mma_n; p.out_cols = a.inter; p.inter = a.inter;
  p.interleaved = a.activation == 1 ? 1 : 0;
  p.out = h_sorted; p.out_ld = a.inter; p.topk_w = nullptr; p.bias = w13_bias;
  p.alpha = a.act_alpha; p.limit = a.act_limit; p.status = a.status;
  pick_ring(mma_n, 0, &p.stages, &p.stage_bytes);
  (void)rows_cap;

  long long tiles = static_cast<long long>(a.max_m_blocks) * p.n_tiles;
  const int grid = static_cast<int>(tiles < device_sm_count() ? tiles : device_sm_count());
  const int smem_bytes = kBarrierBytes + 1024 + p.stages * p.stage_bytes;
  if (int st = check_cuda(launch_pdl(grouped_gemm_kernel<1, 4, 4>, dim3(grid), dim3(role_threads(4, 4)), smem_bytes, stream, map_b, p),
                          "grouped_gemm gate_up launch"))
    return st;
  count_launches(1);
  return check_launch("grouped_gemm gate_up");
}

int launch_grouped_gemm2(const GroupedGemmArgs& a, const __nv_bfloat16* h_sorted, int rows_cap,
                         const __nv_bfloat16* w2, const __nv_bfloat16* w2_bias, const float* topk_w,
                         __nv_bfloat16* c3, cudaStream_t stream) {
  if (int st = check_common(a)) return st;
  if (a.numel == 0 || a.max_m_blocks == 0) return kStatusOk;
  if (a.hidden % 16 != 0) return set_error(kStatusInvalidArgument, "grouped GEMM down: hidden must be a multiple of 16");
  const int tile_cols = pick_down_tile(a.hidden, a.inter, expected_m_blocks(a.numel, a.top_k, a.num_experts));
  // A rank's thin slice of I (tensor parallel): the main loop of a tile is two to four K blocks and the epilogue
  // warps set the pace, so eight of them share the tile (two per TMEM lane quarter, half the columns each) and two
  // gather warps are enough for the short token rows; three operand stages then hold more than a tile.
  const bool thin = a.inter <= 256 && tile_cols == 256;
  const int epi_warps = thin ? 8 : 4;
  if (int st = thin ? ensure_smem_attr<2, 8, 2>() : ensure_smem_attr<2, 4, 4>()) return st;

  CUtensorMap map_b;
  (void)rows_cap;
  const uint64_t dims_b[3] = {static_cast<uint64_t>(a.inter), static_cast<uint64_t>(a.hidden), static_cast<uint64_t>(a.num_experts)};
  const uint32_t box_b[3] = {BK, static_cast<uint32_t>(tile_cols), 1};
  if (int st = make_map(&map_b, w2, 3, dims_b, box_b, 2)) return st;

  KernelParams p{};
  p.sorted_ids = a.sorted_ids; p.expert_ids = a.expert_ids; p.num_post_pad = a.num_post_pad;
  p.x = h_sorted; p.numel = a.numel; p.top_k = a.top_k; p.K = a.inter;
  p.n_tiles = (a.hidden + tile_cols - 1) / tile_cols; p.tile_cols = tile_cols; p.mma_n = tile_cols;
  p.out_cols = a.hidden; p.inter = a.inter; p.interleaved = 0;
  p.out = c3; p.out_ld = a.hidden; p.topk_w = topk_w; p.bias = w2_bias;
  p.alpha = 0.f; p.limit = 0.f; p.status = a.status;
  const int patch_bytes = epi_warps * kPatchesPerWarp * kPatchBytes;
  pick_ring(p.mma_n, patch_bytes, &p.stages, &p.stage_bytes);

  long long tiles = static_cast<long long>(a.max_m_blocks) * p.n_tiles;
  const int grid = static_cast<int>(tiles < device_sm_count() ? tiles : device_sm_count());
  const int smem_bytes = kBarrierBytes + 1024 + p.stages * p.stage_bytes + patch_bytes;
  const cudaError_t le = thin ? launch_pdl(grouped_gemm_kernel<2, 8, 2>, dim3(grid), dim3(role_threads(8, 2)), smem_bytes, stream, map_b, p)
                              : launch_pdl(grouped_gemm_kernel<2, 4, 4>, dim3(grid), dim3(role_threads(4, 4)), smem_bytes, stream, map_b, p);
  if (int st = check_cuda(le, "grouped_gemm down launch")) return st;
  count_launches(1);
  return check_launch("grouped_gemm down");
}

}  // namespace moe_b200
