// Block-scaled FP8 (e4m3) GEMM core for sm_100a: one persistent, warp-specialised kernel
// shared by the dense block-scaled GEMM and the two grouped GEMMs of the MoE expert layer.
//
//   C[m, n] = sum_kb ( sum_{k in kb} A[m, k] * B[n, k] ) * sfa[kb, m] * sfb[n/128, kb]
//
// Layout contract (reference: docs/adr/0023-block-scales-are-axis-relations.md:21-27,
// src/open_cake_ir/tasks/solx_fib/moe.py:13-20): A e4m3 [rows, K] row-major with fp32 scales
// stored K-block-major [K/128, rows]; B e4m3 [N, K] row-major ("N-K weights") with fp32 scales
// [N/128, K/128]; grouped problems stack B as [G, N, K] and A as expert-contiguous row
// segments described by `offsets[G+1]`.
//
// Mapping to the hardware.  A CTA owns a 128-row x 256-column output tile per work item.
// Rows are TMEM lanes (UMMA M = 128), columns are TMEM columns (UMMA N = 256).  For every
// 128-wide K block, four tcgen05.mma.kind::f8f6f4 (K = 32 each) write a FRESH partial product
// into one of two TMEM accumulator stages; eight epilogue warps read that stage back
// (tcgen05.ld), multiply it by the block's scales and add it to fp32 registers ("promotion"),
// which is what arbitrary fp32 1x128 / 128x128 scales need -- the hardware block-scaled kinds
// only take power-of-two scales per 32 elements.  While the epilogue promotes block kb the
// tensor core already works on block kb+1 in the other stage.  Operands arrive through a
// 4-stage TMA ring (128-byte swizzle, one elected producer thread); the MMA is issued by one
// elected thread of a second warp.  Work items are (group, n tile, m tile) with the m tile
// fastest, so CTAs that share a weight tile run at the same time and the second reader hits L2.
// Items either go round the CTAs in turn or are drawn from a device counter by the TMA warp, which
// hands them to the other roles through a four-slot ring (Params::queue).
#pragma once
#include "common.cuh"

namespace cake {
namespace gemm {

constexpr int kBM = 128;          // rows per tile = UMMA M = TMEM lanes
constexpr int kBN = 256;          // columns per tile = UMMA N
constexpr int kBK = 128;          // e4m3 elements (= bytes) per K block = scale granularity
constexpr int kUmmaK = 32;        // K of one tcgen05.mma for 8-bit operands
constexpr int kStages = 4;        // shared-memory ring depth
constexpr int kTmemStages = 2;    // accumulator stages in tensor memory
constexpr int kTmemColumns = kTmemStages * kBN;   // 512 = all of an SM's tensor memory
constexpr int kBytesA = kBM * kBK;                // 16 KiB
constexpr int kBytesB = kBN * kBK;                // 32 KiB
constexpr int kStageBytes = kBytesA + kBytesB;
constexpr int kTailRows = 32;                    // box rows of the small A map
constexpr int kControlWarps = 4;                  // one warpgroup: warp 0 TMA, warp 1 MMA, warps 2-3 idle
constexpr int kEpilogueWarps = 8;                 // two warpgroups: 2 column groups x 4 TMEM lane quadrants
constexpr int kThreads = (kControlWarps + kEpilogueWarps) * 32;
// Register budget moved between the warpgroups once the roles split.  The pool setmaxnreg draws on
// is what the launch allocated, 168 registers x 384 threads = 64512, not the SM's 65536: an
// increase that asks for more than the pool ever holds blocks for good.  128 x 40 + 256 x 232 = 64512.
constexpr int kControlRegs = 40;
constexpr int kEpilogueRegs = 232;
static_assert(kControlWarps * 32 * kControlRegs + kEpilogueWarps * 32 * kEpilogueRegs <= (65536 / kThreads / 8 * 8) * kThreads,
              "setmaxnreg budget exceeds the registers the launch allocates");
constexpr int kMaxGroups = 512;
constexpr int kItemSlots = 4;

enum Mode : int {
  kDense = 0,        // C bf16 [M, N]
  kGateUp = 1,       // grouped GEMM1: x1 = cols [0,128), x2 = cols [128,256) of the tile;
                     // out = e4m3(x1 * silu(x2)) + per-(row,128) scale  (optionally hi+lo split)
  kDown = 2,         // grouped GEMM2: out bf16 [rows, N] = acc * route weight of the row
};

struct Params {
  int n;                       // output columns per group (dense N; GEMM1: I; GEMM2: H)
  int k_blocks;                // K / 128 of the A operand
  int b_k_blocks;              // K / 128 of the B operand (== k_blocks unless A is hi/lo split)
  int b_rows_per_group;        // rows of B per group (dense N; GEMM1: 2I; GEMM2: H)
  int groups;                  // 1 for dense
  int row_capacity;            // rows the A buffer (and its scale rows) is allocated for
  int interleave_hi_lo;        // 1: A K-block kb -> A column block (kb&1)*(k_blocks/2) + kb/2, B block kb/2
  const int* offsets;          // [groups+1] device row offsets into A; null = one group of dense_rows rows
  int dense_rows;
  const float* sfa;            // [k_blocks, row_capacity]
  const float* sfb;            // [groups, b_rows_per_group/128, b_k_blocks]
  void* out;                   // see Mode
  float* out_scale;            // kGateUp: [out_k_blocks, row_capacity]
  const float* row_weight;     // kDown: [row_capacity] route weight per sorted row
  int split_act;               // kGateUp: 1 = also write the residual (lo) term
  int* status;                 // device status word (0 = ok)
  int* queue;                  // device counter, 0 at launch: work items are drawn from it (null: item i goes to CTA i mod grid)
  int wait_kiloclocks;         // budget of a bounded wait in units of 1024 clocks (0: the default, about a second)
  int skip_load;               // test hook: CTA 0's producer leaves out the loads of its second K block, once
};

struct Shared {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[kTmemStages];
  uint64_t tmem_empty[kTmemStages];
  uint64_t exchange_done;                                   // kGateUp: all epilogue warps have published their amax
  uint64_t item_full[kItemSlots], item_empty[kItemSlots];   // hand-over of drawn work items from the TMA warp to the other roles
  int item_q[kItemSlots];
  uint32_t tmem_base;
  WaitControl wait;
  int tile_prefix[kMaxGroups + 1];     // m tiles before group g
  float exchange[2][2][2][kBM];        // [item parity][term][column group][row] amax exchange for kGateUp
};

struct Item {
  int group, row0, rows_valid, n_tile;
};

// Work item `g` -> (group, m tile, n tile); items of one group are ordered n tile major,
// m tile minor.  Returns false past the end.
__device__ __forceinline__ bool locate(const Shared* sh, const Params& p, int n_tiles, int g, Item* it) {
  const int total = sh->tile_prefix[p.groups] * n_tiles;
  if (g >= total) return false;
  int lo = 0, hi = p.groups;            // largest group with prefix*n_tiles <= g
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (sh->tile_prefix[mid] * n_tiles <= g) lo = mid; else hi = mid;
  }
  const int m_tiles = sh->tile_prefix[lo + 1] - sh->tile_prefix[lo];
  const int idx = g - sh->tile_prefix[lo] * n_tiles;
  const int begin = p.offsets ? p.offsets[lo] : 0;
  const int end = p.offsets ? p.offsets[lo + 1] : p.dense_rows;
  const int mt = idx % m_tiles;
  it->group = lo;
  it->n_tile = idx / m_tiles;
  it->row0 = begin + mt * kBM;
  it->rows_valid = min(kBM, end - it->row0);
  return true;
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_a_tail,
                const __grid_constant__ CUtensorMap map_b, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Shared* sh = reinterpret_cast<Shared*>(tiles + kStages * kStageBytes);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tiles = (MODE == kGateUp) ? p.n / 128 : (p.n + kBN - 1) / kBN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&sh->full[s], 1); mbar_init(&sh->empty[s], 1); }
    for (int s = 0; s < kTmemStages; ++s) { mbar_init(&sh->tmem_full[s], 1); mbar_init(&sh->tmem_empty[s], kEpilogueWarps); }
    for (int s = 0; s < kItemSlots; ++s) { mbar_init(&sh->item_full[s], 1); mbar_init(&sh->item_empty[s], 1 + kEpilogueWarps); }
    mbar_init(&sh->exchange_done, kEpilogueWarps);
    sh->wait.abort_flag = 0;
    sh->wait.budget_kiloclocks = p.wait_kiloclocks;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, kTmemColumns);
    tmem_relinquish();
  }
  if (warp == kControlWarps) {   // m-tile prefix over groups (serial per lane chunk, then a warp scan)
    int running = 0;
    for (int base = 0; base < p.groups; base += 32) {
      int g = base + lane;
      int tiles_g = 0;
      if (g < p.groups) {
        int cnt = p.offsets ? p.offsets[g + 1] - p.offsets[g] : p.dense_rows;
        tiles_g = (cnt + kBM - 1) / kBM;
      }
      int incl = tiles_g;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (g < p.groups) sh->tile_prefix[g] = running + incl - tiles_g;
      running += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) sh->tile_prefix[p.groups] = running;
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  volatile int* abort_flag = &sh->wait.abort_flag;

  if (warp < kControlWarps) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kControlRegs));
  if (warp == 0) {
    // ------------------------------ TMA producer --------------------------------------
    if (elect_one()) {
      tma_prefetch_descriptor(&map_a);
      tma_prefetch_descriptor(&map_a_tail);
      tma_prefetch_descriptor(&map_b);
      const uint64_t keep = l2_policy_evict_last();    // activations: re-read by every n tile
      // Work items.  With a queue, this thread draws them (the first is the CTA's index, every later
      // one comes from the device counter, asked for one item ahead) and hands each to the MMA and
      // epilogue warps through a small ring, so that an SM that runs slower simply takes fewer
      // items; without one, item i belongs to CTA i mod grid.
      uint32_t it = 0, k = 0;
      bool ok = true;
      Item item;
      int g = blockIdx.x;
      while (ok) {
        const bool valid = locate(sh, p, n_tiles, g, &item);
        int drawn = g + int(gridDim.x);
        if (p.queue) {
          const int slot = k % kItemSlots;
          ok = mbar_wait(&sh->item_empty[slot], ((k / kItemSlots) & 1) ^ 1, abort_flag, p.status, kStatusWaitFlag);
          if (!ok) break;
          sh->item_q[slot] = valid ? g : -1;
          mbar_arrive(&sh->item_full[slot]);
          if (valid) drawn = int(gridDim.x) + atomicAdd(p.queue, 1);
        }
        if (!valid) break;
        const int b_row0 = item.group * p.b_rows_per_group;
        // A tile of at most kTailRows valid rows (the second tile of a group a little over 128 rows) brings in those
        // rows only, through a map with a smaller box: such a tile streams its weights from L2 at what one SM can
        // draw, so every byte not fetched shortens it.  Rows of the stage beyond them keep what an earlier tile left
        // there; their products land in accumulator rows that no one reads.
        const bool tail = item.rows_valid <= kTailRows;
        const uint32_t stage_tx = tail ? uint32_t(kTailRows * kBK + kBytesB) : uint32_t(kStageBytes);
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          ok = mbar_wait(&sh->empty[s], ((it / kStages) & 1) ^ 1, abort_flag, p.status, kStatusWaitSmemEmpty);
          if (!ok) break;
          if (p.skip_load && blockIdx.x == 0 && it == 1) continue;      // test hook: this ring slot is never filled
          uint8_t* a_dst = tiles + s * kStageBytes;
          uint8_t* b_dst = a_dst + kBytesA;
          int a_col = kb, b_col = kb;
          if (p.interleave_hi_lo) { a_col = (kb & 1) * (p.k_blocks >> 1) + (kb >> 1); b_col = kb >> 1; }
          mbar_arrive_expect_tx(&sh->full[s], stage_tx);
          tma_load_2d_hint(a_dst, tail ? &map_a_tail : &map_a, a_col * kBK, item.row0, &sh->full[s], keep);
          if (MODE == kGateUp) {
            // gate/up: 128 rows of the first half (x1) and the matching 128 rows of the second half (x2)
            tma_load_2d(b_dst, &map_b, b_col * kBK, b_row0 + item.n_tile * 128, &sh->full[s]);
            tma_load_2d(b_dst + 128 * kBK, &map_b, b_col * kBK, b_row0 + p.n + item.n_tile * 128, &sh->full[s]);
          } else {
            tma_load_2d(b_dst, &map_b, b_col * kBK, b_row0 + item.n_tile * kBN, &sh->full[s]);
          }
        }
        g = drawn;
        ++k;
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ----------------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc(0 /* e4m3 */, kBM, kBN);
      uint32_t it = 0, k = 0;
      bool ok = true;
      Item item;
      for (int g = blockIdx.x; ok; g += gridDim.x, ++k) {
        if (p.queue) {                 // the k-th item of this CTA, as drawn by the TMA warp
          const int slot = k % kItemSlots;
          ok = mbar_wait(&sh->item_full[slot], (k / kItemSlots) & 1, abort_flag, p.status, kStatusWaitFlag);
          if (!ok) break;
          g = sh->item_q[slot];
          mbar_arrive(&sh->item_empty[slot]);
          if (g < 0) break;
        }
        if (!locate(sh, p, n_tiles, g, &item)) break;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const int t = it % kTmemStages;
          ok = mbar_wait(&sh->full[s], (it / kStages) & 1, abort_flag, p.status, kStatusWaitSmemFull) &&
               mbar_wait(&sh->tmem_empty[t], ((it / kTmemStages) & 1) ^ 1, abort_flag, p.status, kStatusWaitTmemEmpty);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(tiles + s * kStageBytes);
          const uint64_t a_desc = umma_desc_sw128(a_addr);
          const uint64_t b_desc = umma_desc_sw128(a_addr + kBytesA);
          const uint32_t d = tmem_base + t * kBN;
#pragma unroll
          for (int j = 0; j < kBK / kUmmaK; ++j) {
            // advancing K inside the 128-byte swizzle row: +32 bytes = +2 in the 16-byte address field
            umma_f8f6f4(d, a_desc + uint64_t(j * (kUmmaK >> 4)), b_desc + uint64_t(j * (kUmmaK >> 4)), idesc, j > 0);
          }
          tcgen05_commit(&sh->empty[s]);       // the ring slot is free once these MMAs have read it
          tcgen05_commit(&sh->tmem_full[t]);   // and the partial product is complete
        }
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kEpilogueRegs));
    // ------------------------------ epilogue / promotion ------------------------------
    const int ew = warp - kControlWarps;
    const int quad = warp & 3;                 // TMEM lanes a warp may read: 32*(warp id % 4)
    const int cg = ew >> 2;                    // column group 0..1
    const int r = quad * 32 + lane;            // row inside the tile
    const uint32_t lane_base = tmem_base + (uint32_t(quad * 32) << 16);
    // Two 64-column segments per thread: gate/up takes 64 x1 columns and the matching 64 x2
    // columns; the other modes take 128 consecutive columns.
    const int seg_col0 = (MODE == kGateUp) ? cg * 64 : cg * 128;
    const int seg_col1 = (MODE == kGateUp) ? 128 + cg * 64 : cg * 128 + 64;
    const int sfb_rows = p.b_rows_per_group / 128;
    uint32_t it = 0, k = 0;
    uint32_t exchanges = 0;                    // amax exchanges so far (phase of Shared::exchange_done)
    int parity = 0;
    bool ok = true;
    Item item;
    for (int g = blockIdx.x; ok; g += gridDim.x, parity ^= 1, ++k) {
      if (p.queue) {                   // the k-th item of this CTA, as drawn by the TMA warp
        const int slot = k % kItemSlots;
        ok = mbar_wait(&sh->item_full[slot], (k / kItemSlots) & 1, abort_flag, p.status, kStatusWaitFlag);
        if (!ok) break;
        g = sh->item_q[slot];
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->item_empty[slot]);
        if (g < 0) break;
      }
      if (!locate(sh, p, n_tiles, g, &item)) break;
      const int row = item.row0 + r;
      const int row_c = min(row, p.row_capacity - 1);
      int sfb_row0, sfb_row1;
      if (MODE == kGateUp) {
        sfb_row0 = item.n_tile;
        sfb_row1 = p.n / 128 + item.n_tile;
      } else {
        sfb_row0 = sfb_row1 = min(item.n_tile * 2 + cg, sfb_rows - 1);
      }
      const float* sfb0 = p.sfb + (size_t(item.group) * sfb_rows + sfb_row0) * p.b_k_blocks;
      const float* sfb1 = p.sfb + (size_t(item.group) * sfb_rows + sfb_row1) * p.b_k_blocks;
      float acc[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) acc[i] = 0.f;
      // Scales travel kScaleAhead K blocks ahead of their use: an L2 round trip under a full TMA
      // stream is longer than one K block, and a scale that arrives late stalls the whole promotion.
      constexpr int kScaleAhead = 3;
      float sa_q[kScaleAhead], sb0_q[kScaleAhead], sb1_q[kScaleAhead];
      auto fetch = [&](int kb, float& sa, float& sb0, float& sb1) {
        int a_col = kb, b_col = kb;
        if (p.interleave_hi_lo) { a_col = (kb & 1) * (p.k_blocks >> 1) + (kb >> 1); b_col = kb >> 1; }
        sa = __ldg(p.sfa + size_t(a_col) * p.row_capacity + row_c);
        sb0 = __ldg(sfb0 + b_col);
        sb1 = __ldg(sfb1 + b_col);
      };
#pragma unroll
      for (int j = 0; j < kScaleAhead; ++j) {
        sa_q[j] = sb0_q[j] = sb1_q[j] = 0.f;
        if (j < p.k_blocks) fetch(j, sa_q[j], sb0_q[j], sb1_q[j]);
      }
      // A warp none of whose 32 rows exists (the tail tile of a group), or whose columns lie past N, only hands
      // the accumulator stages back: no tensor-memory reads, no arithmetic.  Not in the gate/up mode: there the
      // tail tile of a group runs beside the group's full tile on a neighbouring SM over the same 56 K blocks of
      // weights, and a tail tile that skips its promotion runs so far ahead that the weights it fetched have left
      // L2 again when the full tile asks for them (measured: 11 % more DRAM traffic and 10 % more time).
      const bool warp_active = MODE == kGateUp || (quad * 32 < item.rows_valid && item.n_tile * kBN + cg * 128 < p.n);
      for (int kb = 0; !warp_active && kb < p.k_blocks; ++kb, ++it) {
        const int t = it % kTmemStages;
        ok = mbar_wait(&sh->tmem_full[t], (it / kTmemStages) & 1, abort_flag, p.status, kStatusWaitTmemFull);
        if (!ok) break;
        if (lane == 0) mbar_arrive(&sh->tmem_empty[t]);
      }
      for (int kb = 0; warp_active && kb < p.k_blocks; ++kb, ++it) {
        const int t = it % kTmemStages;
        const float s0 = sa_q[0] * sb0_q[0], s1 = sa_q[0] * sb1_q[0];
#pragma unroll
        for (int j = 0; j + 1 < kScaleAhead; ++j) { sa_q[j] = sa_q[j + 1]; sb0_q[j] = sb0_q[j + 1]; sb1_q[j] = sb1_q[j + 1]; }
        if (kb + kScaleAhead < p.k_blocks) fetch(kb + kScaleAhead, sa_q[kScaleAhead - 1], sb0_q[kScaleAhead - 1], sb1_q[kScaleAhead - 1]);
        ok = mbar_wait(&sh->tmem_full[t], (it / kTmemStages) & 1, abort_flag, p.status, kStatusWaitTmemFull);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t stage_addr = lane_base + t * kBN;
        // two round trips to tensor memory per K block, 64 columns each
        float va[32], vb[32];
        tmem_ld_32x32b_x32(stage_addr + seg_col0, va);
        tmem_ld_32x32b_x32(stage_addr + seg_col0 + 32, vb);
        tcgen05_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          acc[i] = fmaf(va[i], s0, acc[i]);
          acc[32 + i] = fmaf(vb[i], s0, acc[32 + i]);
        }
        tmem_ld_32x32b_x32(stage_addr + seg_col1, va);
        tmem_ld_32x32b_x32(stage_addr + seg_col1 + 32, vb);
        tcgen05_wait_ld();
        tcgen05_fence_before();            // everything this warp needs has left tensor memory
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->tmem_empty[t]);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          acc[64 + i] = fmaf(va[i], s1, acc[64 + i]);
          acc[96 + i] = fmaf(vb[i], s1, acc[96 + i]);
        }
      }
      if (!ok) break;
      // rows past the group's end and, where N is an odd multiple of 128, the tile's second column group hold nothing
      const bool valid = r < item.rows_valid && (MODE == kGateUp || item.n_tile * kBN + cg * 128 < p.n);

      if (MODE == kDense) {
        if (valid) {
          __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + size_t(row) * p.n + item.n_tile * kBN + cg * 128;
#pragma unroll
          for (int i = 0; i < 128; i += 8) {
            uint4 w;
            w.x = pack_bf16x2(acc[i], acc[i + 1]); w.y = pack_bf16x2(acc[i + 2], acc[i + 3]);
            w.z = pack_bf16x2(acc[i + 4], acc[i + 5]); w.w = pack_bf16x2(acc[i + 6], acc[i + 7]);
            *reinterpret_cast<uint4*>(out + i) = w;
          }
        }
      } else if (MODE == kDown) {
        if (valid) {
          const float w = __ldg(p.row_weight + row);
          __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + size_t(row) * p.n + item.n_tile * kBN + cg * 128;
#pragma unroll
          for (int i = 0; i < 128; i += 8) {
            uint4 v;
            v.x = pack_bf16x2(acc[i] * w, acc[i + 1] * w); v.y = pack_bf16x2(acc[i + 2] * w, acc[i + 3] * w);
            v.z = pack_bf16x2(acc[i + 4] * w, acc[i + 5] * w); v.w = pack_bf16x2(acc[i + 6] * w, acc[i + 7] * w);
            *reinterpret_cast<uint4*>(out + i) = v;
          }
        }
      } else {
        // SwiGLU on the 64 (x1, x2) pairs this thread holds, then e4m3 quantisation of the 128-wide
        // group it shares with the thread of the same row in the other column group.
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const float gate = acc[64 + i];
          acc[i] = acc[i] * (gate / (1.f + __expf(-gate)));
          amax = fmaxf(amax, fabsf(acc[i]));
        }
        const int out_kb = p.n / 128;                      // K blocks of one term of the output
        const int terms = p.split_act ? 2 : 1;
        uint8_t* out_base = reinterpret_cast<uint8_t*>(p.out) + size_t(row) * (size_t(p.n) * terms) + item.n_tile * 128 + cg * 64;
        for (int term = 0; term < terms; ++term, ++exchanges) {
          // The two column groups of a row meet through shared memory.  The hand-over is an mbarrier wait like
          // every other wait of the kernel: bounded, and given up when another role has raised the abort flag.
          sh->exchange[parity][term][cg][r] = amax;
          __syncwarp();
          if (lane == 0) mbar_arrive(&sh->exchange_done);
          ok = mbar_wait(&sh->exchange_done, exchanges & 1, abort_flag, p.status, kStatusWaitFlag);
          if (!ok) break;
          const float group_amax = fmaxf(amax, sh->exchange[parity][term][cg ^ 1][r]);
          const float scale = group_amax > 0.f ? group_amax / 448.f : 1.f;
          const float inv = 1.f / scale;
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 64; i += 4) packed[i >> 2] = pack_e4m3x4(acc[i] * inv, acc[i + 1] * inv, acc[i + 2] * inv, acc[i + 3] * inv);
          if (valid) {
            uint4* dst = reinterpret_cast<uint4*>(out_base + size_t(term) * p.n);
#pragma unroll
            for (int i = 0; i < 4; ++i) dst[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
            if (cg == 0) p.out_scale[size_t(term * out_kb + item.n_tile) * p.row_capacity + row] = scale;
          }
          if (term + 1 < terms) {        // residual after the first term becomes the value to quantise
            amax = 0.f;
#pragma unroll
            for (int i = 0; i < 64; ++i) {
              const uint32_t word = packed[i >> 2];
              acc[i] -= e4m3_to_float(uint8_t(word >> ((i & 3) * 8))) * scale;
              amax = fmaxf(amax, fabsf(acc[i]));
            }
          }
        }
        if (!ok) break;
      }
    }
  }

  // ------------------------------ teardown ---------------------------------------------
  tcgen05_fence_before();
  __syncthreads();
  if (sh->wait.abort_flag) {
    // A wait ran out somewhere: give copies still in flight time to land before the shared
    // memory they target is released with the CTA.
    const long long start = clock64();
    while (clock64() - start < 2000000LL) { __nanosleep(1000); }
    __syncthreads();
  }
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, kTmemColumns);
  }
}

constexpr size_t kSmemBytes = size_t(kStages) * kStageBytes + sizeof(Shared) + 1024;

}  // namespace gemm
}  // namespace cake
