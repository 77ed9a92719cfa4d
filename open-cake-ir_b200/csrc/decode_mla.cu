// Paged MLA decode (absorbed form) for sm_100a: split-KV flash-decode on tcgen05 (plan + decode + reduce).
//
// Operator: src/open_cake_ir/tasks/solx_fib/attention.py:132-183, MLA branch (:164-165,
// :175-177); tensor ABI attention_specs.py:249-292.  All query heads share one latent KV row of
// 512 (ckv) + 64 (kpe) bf16 per token:  logits = (ckv . q_nope + kpe . q_pe) * scale,
// out = bf16(softmax(logits) ckv), lse base 2.
//
// At 128 heads the operator does 242 flop per byte of latent cache, which is the bf16 ridge of the
// machine, so both contractions run on the tensor core.  A CTA owns 128 heads, one HALF of the 512
// output dims and an equal share of all the tiles of the launch (a consecutive range of the list
// of tiles of all sequences, so it works through one to a few sequences in turn); the two halves
// of a range are neighbouring CTAs, so one of them reads the latent rows from L2.  The 128 heads
// are the 128 TMEM lanes:
//   S[128 x 32 tokens]  = Q[128 x 576] . KV_tile^T      Q dims 0..383 from TENSOR memory, 384..575 and
//                                                        the tile K-major from shared memory
//   O[128 x 256 dims]  += P[128 x 32] . V[32 x 256]     P from tensor memory, V = the same tile read
//                                                        MN-major (no transposed copy is made)
// Tensor memory holds O (256 columns), two S/P buffers of 32 columns (a tile's logits, which the softmax
// warps overwrite in place with the tile's weights, so that the softmax of tile i+1 need not wait for
// PV(i)) and as much of Q as fits beside them (192 columns = 384 of a row's 576 bf16: a product step
// whose A operand comes from shared memory costs four times one that takes it from tensor memory);
// the rest of Q (48 KiB) stays in shared memory.  All of Q in
// shared memory would take 147 KiB, leave room for two ring stages only, and be re-read by every
// QK (1152 clocks of shared-memory bandwidth per tile); all of Q in tensor memory leaves O only
// 128 columns, i.e. four CTAs per range that each repeat the QK product AND the softmax.  With the
// split, 144 KiB of shared memory are a four-stage ring of 32-token tiles (cp.async gather per
// token, so any page size works; a stage's barrier is arrived on by the copies themselves).
// Eight softmax warps, two per head row, read S from TMEM, keep the running max and sum in base
// 2, and write P back to TMEM as TWO bf16 terms (value + rounding residual; one term is not
// accurate enough for the contract's tolerance).  The MMA warp issues QK of the next tile before
// PV of the current one, so the tensor pipe works on QK while the softmax of the current tile
// runs.  The running max only moves when it grows by more than 2^8, so O is rescaled in TMEM
// rarely.  Every wait is bounded and reports through the status word.
#include "common.cuh"
#include "prefill.cuh"
#include "../../include/cake_b200.h"
#include <new>

namespace cake {
namespace mla {

constexpr int kCkv = 512, kKpe = 64, kRow = kCkv + kKpe;   // 576 elements per latent row
constexpr int kSlabs = kRow / 64;                          // 9 slabs of 64 columns (128 bytes per row)
constexpr int kRowChunks = kRow / 8;                       // 72 16-byte chunks per row
constexpr int kHeads = 128;                                // query heads per CTA = TMEM lanes
constexpr int kDimsPerCta = 256;                           // output dims per CTA (half of ckv)
constexpr int kDimSplit = kCkv / kDimsPerCta;              // CTAs that share a (head block, tile range)
constexpr int kQTmemSlabs = 6;                             // Q dims 0..383 live in tensor memory,
constexpr int kQSmemSlabs = kSlabs - kQTmemSlabs;          //   dims 384..575 (three slabs) in shared memory
constexpr int kQTmemCols = kQTmemSlabs * 32;               // 192 columns, two bf16 per column
constexpr int kQSlabBytes = kHeads * 128;                  // 16 KiB
constexpr int kQSmemBytes = kQSmemSlabs * kQSlabBytes;     // 48 KiB
constexpr int kQStageRow = kQTmemSlabs * 128;              // 768 bytes of a Q row pass through the staging area
constexpr int kTile = 32;                                  // tokens per tile
constexpr int kStages = 4;                                 // ring stages
constexpr int kKvSlabBytes = kTile * 128;                  // 4 KiB
constexpr int kKvStageBytes = kSlabs * kKvSlabBytes;       // 36 864
constexpr int kLoaderWarps = 4, kLoaderThreads = kLoaderWarps * 32;   // warps 0..3: eight rows of a tile each
constexpr int kMmaWarp = 4;                                // warps 5..7 only take part in the CTA-wide barriers
constexpr int kSoftmaxWarp0 = 8;                           // warps 8..15: warp % 4 = TMEM lane quadrant,
constexpr int kSoftmaxWarps = 8;                           //   (warp - 8) / 4 = which 16 tokens of a tile
constexpr int kThreads = 512;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.f;                   // log2 units
constexpr int kOutRowFloats = 36;                          // write-out: a row of 32 fp32 columns + 16 bytes of padding
static_assert(kSoftmaxWarps * 32 * kOutRowFloats * 4 <= kKvStageBytes, "the write-out blocks must fit in ring stage 0");
// tensor-memory columns: O fp32 (256); two S/P buffers of 32 (the logits of a tile as fp32, overwritten in place by its
// weights as two bf16 terms: each softmax warp owns 16 columns = its 16 tokens' logits, then 8 + 8 columns of P);
// Q dims 0..383 (192): all 512
constexpr uint32_t kColO = 0, kColSP = kColO + kDimsPerCta, kColQ = kColSP + 2 * kTile, kTmemColumns = 512;
static_assert(kColQ + kQTmemCols <= kTmemColumns, "Q does not fit in tensor memory");

struct Params {
  const __nv_bfloat16 *q_nope, *q_pe, *ckv, *kpe;
  const int *kv_indptr, *kv_indices, *kv_last_page_len;
  const float* sm_scale;
  __nv_bfloat16* out;     // [B, H, 512]
  float* lse;             // [B, H]
  float* part_o;          // [slots, H, 512]   slot = worker + sequence (see mla_plan_kernel)
  float* part_lse;        // [slots, H]
  int* tile_prefix;       // [B+1] work units (tiles + start-up shares) before sequence b, written by the plan kernel
  int* status;
  int batch, heads, page_size, workers;
  // Sparse form (DeepSeek-V3.2 sparse attention): sequence b is the `top_k` cache rows listed in
  // sparse_indices[b, :] (token-level row numbers page * page_size + offset, -1 = no entry) instead of a page list.
  const int* sparse_indices;
  int top_k;
  // Explicit sequence table (causal prefill: every query token is a sequence of its own over a prefix of its
  // segment's rows): sequence b holds seq_tokens[b] tokens whose page list starts at kv_indices[seq_start[b]].
  const int* seq_start;
  const int* seq_tokens;
  int wait_kiloclocks;    // budget of a bounded wait in units of 1024 clocks (0: the default, about a second)
  int skip_load;          // test hook: a CTA's loader warps leave out the third tile of the first sequence they work on
};

struct Shared {
  uint64_t kv_full[kStages], kv_empty[kStages];
  uint64_t s_full[2], p_ready[2], pv_done[2];     // per S/P buffer (tile i uses buffer i mod 2)
  uint64_t pair_read[4];                          // per lane quadrant: both warps of a row have read the tile's logits
  uint64_t q_placed;                              // Q dims 0..383 are in tensor memory
  uint64_t row_sums;                              // the two softmax warps of a row exchange their sums once
  uint64_t q_moved;                               // Q has left its staging area (ring stages 1..3)
  uint32_t tmem_base;
  WaitControl wait;
  float l_part[2][kHeads];
};

constexpr size_t kSmemBytes = size_t(kQSmemBytes) + size_t(kStages) * kKvStageBytes + sizeof(Shared) + 1024;
static_assert(kSmemBytes <= 232448, "the kernel's shared memory exceeds what a CTA may have on sm_100");

__device__ __forceinline__ int seq_len(const Params& p, int b) {
  if (p.sparse_indices) return p.top_k;            // listed entries, some of which may be -1
  if (p.seq_tokens) return p.seq_tokens[b];
  const int pages = p.kv_indptr[b + 1] - p.kv_indptr[b];
  return pages <= 0 ? 0 : (pages - 1) * p.page_size + p.kv_last_page_len[b];
}
// 2^x by the special-function unit alone (relative error 2^-22; results below 2^-126 become 0, which is what a
// softmax weight that small is worth).
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;      // 0 source bytes = zero fill
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
// Makes `bar` receive one (pre-counted) arrival from this thread once all its earlier cp.async copies have landed.
__device__ __forceinline__ void cp_async_arrive_on(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Byte offset of 16-byte chunk `chunk` (0..71) of row `row` in a slab-major tile whose slabs hold
// `rows` rows of 128 bytes with the 128-byte swizzle (chunk index XOR row mod 8).
__device__ __forceinline__ uint32_t slab_off(int rows, int row, int chunk) {
  return uint32_t((chunk >> 3) * rows * 128 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

// One 32-token tile of latent rows -> one ring stage, by the four loader warps.  A warp takes
// eight rows; its lanes cover consecutive 16-byte chunks of one row at a time (coalesced 512-byte
// reads).  The page of each row is looked up by one lane (`lookup_row`, issued a tile ahead so
// that the dependent load of the page table is never waited for) and passed round by shuffle.
__device__ __forceinline__ long long lookup_row(const Params& p, int page_base, int tok0, int len, int loader_tid) {
  const int tok = tok0 + (loader_tid >> 5) * 8 + (loader_tid & 7);
  if (tok >= len) return -1;
  if (p.sparse_indices) return (long long)__ldg(p.sparse_indices + page_base + tok);      // page_base = b * top_k here
  const int page = __ldg(p.kv_indices + page_base + tok / p.page_size);
  return (long long)page * p.page_size + (tok % p.page_size);
}
__device__ __forceinline__ void load_tile(const Params& p, long long my_slot, uint32_t dst, int loader_tid) {
  const int w = loader_tid >> 5, lane = loader_tid & 31;
#pragma unroll
  for (int rr = 0; rr < 8; ++rr) {
    const int row = w * 8 + rr;
    const long long slot = __shfl_sync(0xffffffffu, my_slot, rr);
    const bool valid = slot >= 0;
    const __nv_bfloat16* ckv_row = p.ckv + (valid ? slot : 0) * kCkv;
    cp_async_16(dst + slab_off(kTile, row, lane), ckv_row + lane * 8, valid);
    cp_async_16(dst + slab_off(kTile, row, 32 + lane), ckv_row + (32 + lane) * 8, valid);
    if (lane < kKpe / 8) cp_async_16(dst + slab_off(kTile, row, kCkv / 8 + lane), p.kpe + (valid ? slot : 0) * kKpe + lane * 8, valid);
  }
}

// The work of all sequences, in order, forms one list of units: kSeqCost units for a sequence's
// start-up and write-out (Q into tensor memory, the partial result out: about ten tiles' worth of
// time), then one unit per 32-token tile.  Worker w (of `workers`) takes the w-th of `workers` equal
// consecutive ranges of the list, so every SM has the same amount of work whatever the lengths
// are, and a sequence is cut only where a range ends.  A (worker, sequence) pair that meets over at
// least one tile writes one partial result; along the list both indices only grow, so worker +
// sequence numbers the pairs uniquely and at most workers + batch - 1 slots are needed.
constexpr int kSeqCost = 14;
__device__ __forceinline__ int units_per_worker(const Params& p) {
  const int total = p.tile_prefix[p.batch];
  return total > 0 ? (total + p.workers - 1) / p.workers : 1;
}

// One CTA: tile_prefix[b] = units before sequence b (exclusive scan), tile_prefix[B] = all units.
__global__ void __launch_bounds__(1024)
mla_plan_kernel(const Params p) {
  __shared__ int sums[32];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");      // the decode grid may become resident now; it waits for this grid's end
  if (threadIdx.x == 0) *p.status = 0;
  int before = 0;
  for (int base = 0; base < p.batch; base += 1024) {
    const int b = base + threadIdx.x;
    const int tiles = b < p.batch ? (seq_len(p, b) + kTile - 1) / kTile : 0;
    const int n = tiles > 0 ? tiles + kSeqCost : 0;
    int batch_total;
    const int mine = before + cta1024_exclusive_scan(n, sums, batch_total);
    if (b < p.batch) p.tile_prefix[b] = mine;
    before += batch_total;
  }
  if (threadIdx.x == 0) p.tile_prefix[p.batch] = before;
}

template <bool SPARSE>
__global__ void __launch_bounds__(kThreads, 1)
mla_decode_kernel(const Params p) {
  extern __shared__ uint8_t smem_raw[];
  // launched as a programmatic dependent of the plan kernel: resident early, reads the plan after that grid has completed
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int head_blocks = (p.heads + kHeads - 1) / kHeads;
  const int dq = blockIdx.x % kDimSplit, hb = (blockIdx.x / kDimSplit) % head_blocks, worker = blockIdx.x / (kDimSplit * head_blocks);
  const int per_worker = units_per_worker(p);
  const int range_begin = worker * per_worker, range_end = min(p.tile_prefix[p.batch], range_begin + per_worker);
  if (range_begin >= range_end) return;            // the whole CTA leaves together
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t q_tail_addr = smem_u32(base);                      // Q dims 384..575, slab-major, 128-byte swizzle
  const uint32_t kv_addr = q_tail_addr + kQSmemBytes;
  Shared* sh = reinterpret_cast<Shared*>(base + kQSmemBytes + kStages * kKvStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head0 = hb * kHeads;
  if (threadIdx.x == 0) { sh->wait.abort_flag = 0; sh->wait.budget_kiloclocks = p.wait_kiloclocks; }
  if (warp == kMmaWarp) {
    tmem_alloc(&sh->tmem_base, kTmemColumns);
    tmem_relinquish();
  }

  // One pass of the loop below per sequence this worker's range touches.
  for (int at = range_begin; at < range_end;) {
  int b = 0;
  for (int lo = 0, hi = p.batch; hi - lo > 1;) {   // the sequence tile `at` belongs to: largest b with prefix[b] <= at
    const int mid = (lo + hi) >> 1;
    if (p.tile_prefix[mid] <= at) lo = mid; else hi = mid;
    b = lo;
  }
  const int upto = min(p.tile_prefix[b + 1], range_end);        // this range holds units [at, upto) of sequence b
  const int first_tile = max(at - p.tile_prefix[b] - kSeqCost, 0);
  const int tiles = upto - p.tile_prefix[b] - kSeqCost - first_tile;
  const bool first_pass = at == range_begin;      // (test hook below)
  at = upto;
  if (tiles <= 0) continue;                        // only (part of) the sequence's start-up share fell into this range
  const int len = seq_len(p, b);
  const int begin = first_tile * kTile;
  const int end = min(len, begin + tiles * kTile);
  const int slot_index = worker + b;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&sh->kv_full[s], kLoaderThreads); mbar_init(&sh->kv_empty[s], 1); }
    for (int k = 0; k < 2; ++k) { mbar_init(&sh->s_full[k], 1); mbar_init(&sh->p_ready[k], kSoftmaxWarps); mbar_init(&sh->pv_done[k], 1); }
    for (int k = 0; k < 4; ++k) mbar_init(&sh->pair_read[k], 2);
    mbar_init(&sh->q_placed, kSoftmaxWarps);
    mbar_init(&sh->row_sums, kSoftmaxWarps);
    mbar_init(&sh->q_moved, kSoftmaxWarps);
    fence_barrier_init();
  }
  // Q block, coalesced: the first 768 bytes of every row -> a staging area in ring stages 1..3 (the
  // 16-byte chunk index XORed with the row's low bits, so that a thread reading its own row later
  // meets no bank conflicts; from there each softmax thread moves its row to tensor memory); the
  // last 384 bytes -> their final place, three K-major slabs laid out as a 128-byte-swizzled TMA box
  // would leave them.
  const uint32_t q_stage = kv_addr + kKvStageBytes;
  static_assert((kStages - 1) * kKvStageBytes >= kHeads * kQStageRow, "the Q staging area must fit behind ring stage 0");
  for (int idx = threadIdx.x; idx < kHeads * kRowChunks; idx += kThreads) {
    const int r = idx / kRowChunks, chunk = idx % kRowChunks;
    const int head = head0 + r;
    const bool valid = head < p.heads;
    const size_t hrow = size_t(b) * p.heads + (valid ? head : 0);
    const __nv_bfloat16* src = chunk < kCkv / 8 ? p.q_nope + hrow * kCkv + chunk * 8 : p.q_pe + hrow * kKpe + (chunk - kCkv / 8) * 8;
    const uint32_t dst = chunk < kQTmemSlabs * 8 ? q_stage + r * kQStageRow + ((chunk ^ (r & 7)) << 4)
                                                 : q_tail_addr + slab_off(kHeads, r, chunk - kQTmemSlabs * 8);
    cp_async_16(dst, src, valid);
  }
  cp_async_commit();
  // The first tile goes out while the Q block is in flight (its page lookup is two dependent loads);
  // it is a copy group of its own, so that the barrier below waits for Q only.
  const int page_base = SPARSE ? b * p.top_k : (p.seq_start ? p.seq_start[b] : p.kv_indptr[b]);
  if (warp < kLoaderWarps) load_tile(p, lookup_row(p, page_base, begin, end, threadIdx.x), kv_addr, threadIdx.x);
  cp_async_commit();
  cp_async_wait<1>();
  fence_proxy_async_smem();
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  volatile int* abort_flag = &sh->wait.abort_flag;

  if (warp < kLoaderWarps) {
    // ------------------------------ loader --------------------------------------------
    // A stage is announced by the copies themselves: each thread's arrival on the stage's barrier
    // is tied to the completion of the copies it has just issued, so nothing here waits for data
    // and as many tiles are in flight as the ring has free stages.
    bool ok = true;
    long long my_slot = tiles > 1 ? lookup_row(p, page_base, begin + kTile, end, threadIdx.x) : -1;
    cp_async_arrive_on(&sh->kv_full[0]);            // tile 0 went out before the CTA's barrier
    for (int i = 1; ok && i < tiles; ++i) {
      const int s = i % kStages;
      const long long next_slot = i + 1 < tiles ? lookup_row(p, page_base, begin + (i + 1) * kTile, end, threadIdx.x) : -1;
      ok = mbar_wait(&sh->kv_empty[s], ((i / kStages) & 1) ^ 1, abort_flag, p.status, kStatusWaitSmemEmpty);
      // stages 1..3 hold the Q block until the softmax warps have moved it to tensor memory
      if (ok && i == 1) ok = mbar_wait(&sh->q_moved, 0, abort_flag, p.status, kStatusWaitFlag);
      if (!ok) break;
      if (p.skip_load && i == 2 && first_pass) { my_slot = next_slot; continue; }   // test hook: never filled
      load_tile(p, my_slot, kv_addr + s * kKvStageBytes, threadIdx.x);
      cp_async_arrive_on(&sh->kv_full[s]);
      my_slot = next_slot;
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------ MMA issuer ----------------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc_qk = umma_idesc_ex(1 /* bf16 */, kHeads, kTile, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_ex(1 /* bf16 */, kHeads, kDimsPerCta, 0, 1 /* V is MN-major */);
      bool ok = true;
      // S(i) = Q . tile(i)^T, Q from tensor memory: 36 steps of 16 elements, 8 columns of Q each
      auto issue_qk = [&](int i) {
        const int s = i % kStages;
        // S/P buffer i mod 2 needs no wait: its last reader, PV(i-2), was issued before this product and the tensor
        // pipe runs the products of one thread in order
        ok = mbar_wait(&sh->kv_full[s], (i / kStages) & 1, abort_flag, p.status, kStatusWaitSmemFull);
        if (!ok) return;
        fence_proxy_async_smem();               // the tile was written by cp.async (generic proxy), the MMA reads it through the async proxy
        tcgen05_fence_after();
        // One descriptor per tile; the 36 steps differ by constants in its 16-byte address field
        // (a slab further every four steps, 32 bytes inside the swizzled row otherwise), so the
        // single issuing thread spends a few instructions per MMA, not a descriptor build.
        const uint64_t b_base = umma_desc_sw128(kv_addr + s * kKvStageBytes);
        const uint64_t a_base = umma_desc_sw128(q_tail_addr);
#pragma unroll
        for (int step = 0; step < kRow / 16; ++step) {
          const uint64_t b_desc = b_base + uint64_t(((step >> 2) * kKvSlabBytes + (step & 3) * 32) >> 4);
          if (step < kQTmemSlabs * 4) {         // Q dims 0..383 from tensor memory
            umma_f16_a_tmem(tmem_base + kColSP + (i & 1) * kTile, tmem_base + kColQ + step * 8, b_desc, idesc_qk, step != 0);
          } else {                              // dims 384..575 from shared memory
            const uint64_t a_desc = a_base + uint64_t((((step >> 2) - kQTmemSlabs) * kQSlabBytes + (step & 3) * 32) >> 4);
            umma_f16(tmem_base + kColSP + (i & 1) * kTile, a_desc, b_desc, idesc_qk, 1);
          }
        }
        tcgen05_commit(&sh->s_full[i & 1]);
      };
      ok = mbar_wait(&sh->q_placed, 0, abort_flag, p.status, kStatusWaitTmemEmpty);
      if (ok) issue_qk(0);
      for (int i = 0; ok && i < tiles; ++i) {
        // QK of the next tile first: the tensor pipe works on it while the softmax of tile i runs
        if (i + 1 < tiles) issue_qk(i + 1);
        if (!ok) break;
        // O += P(i) . V(i), P as two bf16 terms
        const int s = i % kStages;
        ok = mbar_wait(&sh->p_ready[i & 1], (i >> 1) & 1, abort_flag, p.status, kStatusWaitFlag);
        if (!ok) break;
        tcgen05_fence_after();
        // 16 tokens = two 8-row groups of 1024 bytes; the next 64 dims are one slab further
        const uint64_t v_base = umma_desc_sw128_ex(kv_addr + s * kKvStageBytes + dq * (kDimsPerCta / 64) * kKvSlabBytes, kKvSlabBytes, 1024);
#pragma unroll
        for (int term = 0; term < 2; ++term) {
#pragma unroll
          for (int ks = 0; ks < kTile / 16; ++ks) {
            const uint32_t a_tmem = tmem_base + kColSP + (i & 1) * kTile + ks * 16 + term * 8;    // warp ks's columns
            umma_f16_a_tmem(tmem_base + kColO, a_tmem, v_base + uint64_t((ks * 2048) >> 4), idesc_pv, (i | term | ks) != 0);
          }
        }
        tcgen05_commit(&sh->pv_done[i & 1]);
        tcgen05_commit(&sh->kv_empty[s]);
      }
    }
  } else if (warp >= kSoftmaxWarp0) {
    // ------------------------------ softmax / epilogue --------------------------------
    // Two warps per head row: both read the tile's 32 logits and agree on the running maximum;
    // warp group g exponentiates tokens 16g..16g+15, keeps the sum over them, and owns half of
    // the O columns when O is rescaled or written out.
    const int quad = warp & 3;
    const int grp = (warp - kSoftmaxWarp0) >> 2;
    const int r = quad * 32 + lane;                 // head row of this thread
    const uint32_t lane_base = tmem_base + (uint32_t(quad * 32) << 16);
    const float scale2 = __ldg(p.sm_scale) * kLog2e;
    const bool scale_positive = scale2 > 0.f;      // the contract's scales are; any other is applied to the logits first
    const float pre = scale_positive ? 1.f : scale2, post = scale_positive ? scale2 : 1.f;
    constexpr int kOwnCols = kDimsPerCta / 2;       // O columns per warp group
    bool ok = true;
    {
      // Q rows, staging area -> tensor memory: dims 0..383 = 192 columns, two elements per column;
      // group 0 stores columns 0..95, group 1 the rest.  Heads past the end are rows of zeros.
#pragma unroll 1
      for (int c = grp * (kQTmemCols / 2); c < (grp + 1) * (kQTmemCols / 2); c += 32) {       // 32 columns = 8 x 16 bytes per store
        uint32_t w[32];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int chunk = c / 4 + k;                // 16-byte chunk of the staged 768 bytes of the row
          const uint4 x = *reinterpret_cast<const uint4*>(base + kQSmemBytes + kKvStageBytes + r * kQStageRow + ((chunk ^ (r & 7)) << 4));
          w[4 * k] = x.x; w[4 * k + 1] = x.y; w[4 * k + 2] = x.z; w[4 * k + 3] = x.w;
        }
        tmem_st_32x32b_x32(lane_base + kColQ + c, reinterpret_cast<const float*>(w));
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->q_moved);     // the staging area has been read
      tcgen05_wait_st();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->q_placed);
    }
    float m_ref = -INFINITY, l = 0.f;               // l: this group's share of the row sum
    for (int i = 0; ok && i < tiles; ++i) {
      ok = mbar_wait(&sh->s_full[i & 1], (i >> 1) & 1, abort_flag, p.status, kStatusWaitTmemFull);
      if (!ok) break;
      tcgen05_fence_after();
      float sc[kTile];
      tmem_ld_32x32b_x32(lane_base + kColSP + (i & 1) * kTile, sc);
      tcgen05_wait_ld();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->pair_read[quad]);    // this warp has the logits: its partner may write P over its own half
      // The softmax of a tile sits between QK(i) and PV(i): four-way partial maxima and sums keep
      // its dependent chains short.
      const int tok0 = begin + i * kTile;
      float t4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (SPARSE) {                                  // entries of the list may be absent anywhere
        const int tok = tok0 + lane;
        const uint32_t present = __ballot_sync(0xffffffffu, tok < end && __ldg(p.sparse_indices + page_base + tok) >= 0);
#pragma unroll
        for (int c = 0; c < kTile; ++c) {
          sc[c] = ((present >> c) & 1u) ? sc[c] * pre : -INFINITY;
          t4[c & 3] = fmaxf(t4[c & 3], sc[c]);
        }
      } else if (tok0 + kTile <= end) {              // all but a chunk's last tile
#pragma unroll
        for (int c = 0; c < kTile; ++c) {
          if (!scale_positive) sc[c] *= pre;
          t4[c & 3] = fmaxf(t4[c & 3], sc[c]);
        }
      } else {
#pragma unroll
        for (int c = 0; c < kTile; ++c) {
          sc[c] = tok0 + c < end ? sc[c] * pre : -INFINITY;
          t4[c & 3] = fmaxf(t4[c & 3], sc[c]);
        }
      }
      // the maximum of the scaled logits; with a positive scale the logits themselves stay unscaled and the scale
      // rides in the multiply-add in front of the exponential
      const float tmax = fmaxf(fmaxf(t4[0], t4[1]), fmaxf(t4[2], t4[3])) * post;
      if (i >= 2) {              // this tile's P buffer is free once PV(i-2), which read it, has completed
        ok = mbar_wait(&sh->pv_done[i & 1], ((i - 2) >> 1) & 1, abort_flag, p.status, kStatusWaitFlag);
        if (!ok) break;
        tcgen05_fence_after();
      }
      if (i == 0) {
        m_ref = tmax;                                // finite: the first tile holds a valid token (sparse: may be -inf)
      } else {
        const bool need = tmax > m_ref + kRescaleThreshold;
        if (__any_sync(0xffffffffu, need)) {         // both warps of a row see the same logits and decide alike
          // O is about to be rescaled in tensor memory: PV(i-1) must have landed
          ok = mbar_wait(&sh->pv_done[(i - 1) & 1], ((i - 1) >> 1) & 1, abort_flag, p.status, kStatusWaitFlag);
          if (!ok) break;
          tcgen05_fence_after();
          const float alpha = need ? exp2f(m_ref - tmax) : 1.f;      // m_ref = -inf (sparse: nothing present so far) gives 0
          if (need) { m_ref = tmax; l *= alpha; }
#pragma unroll 1
          for (int c = grp * kOwnCols; c < (grp + 1) * kOwnCols; c += 32) {
            float o[32];
            tmem_ld_32x32b_x32(lane_base + kColO + c, o);
            tcgen05_wait_ld();
#pragma unroll
            for (int k = 0; k < 32; ++k) o[k] *= alpha;
            tmem_st_32x32b_x32(lane_base + kColO + c, o);
          }
          tcgen05_wait_st();
        }
      }
      uint32_t hi[kTile / 4], lo[kTile / 4];
      float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < kTile / 2; c += 2) {
        const float x0 = grp == 0 ? sc[c] : sc[kTile / 2 + c], x1 = grp == 0 ? sc[c + 1] : sc[kTile / 2 + c + 1];
        // sparse: while no entry has been present m_ref is -inf and every logit is -inf: the weights are 0, not NaN
        const float m_use = (SPARSE && m_ref == -INFINITY) ? 0.f : m_ref;
        const float p0 = ex2_approx(fmaf(x0, post, -m_use)), p1 = ex2_approx(fmaf(x1, post, -m_use));
        s4[(c >> 1) & 3] += p0 + p1;
        split_bf16x2(p0, p1, hi[c >> 1], lo[c >> 1]);
      }
      l += (s4[0] + s4[1]) + (s4[2] + s4[3]);
      // P goes over the logits of this warp's own 16 tokens, once the row's other warp has read them too
      ok = mbar_wait(&sh->pair_read[quad], i & 1, abort_flag, p.status, kStatusWaitFlag);
      if (!ok) break;
      tmem_st_32x32b_x8(lane_base + kColSP + (i & 1) * kTile + grp * (kTile / 2), hi);
      tmem_st_32x32b_x8(lane_base + kColSP + (i & 1) * kTile + grp * (kTile / 2) + kTile / 4, lo);
      tcgen05_wait_st();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->p_ready[i & 1]);
    }
    // the row sum is the two groups' sums; exchanged once through shared memory
    if (ok) {
      sh->l_part[grp][r] = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->row_sums);
      ok = mbar_wait(&sh->row_sums, 0, abort_flag, p.status, kStatusWaitFlag);
    }
    if (ok) ok = mbar_wait(&sh->pv_done[(tiles - 1) & 1], ((tiles - 1) >> 1) & 1, abort_flag, p.status, kStatusWaitFlag);
    if (ok) {
      tcgen05_fence_after();
      const int head = head0 + r;
      const float total = sh->l_part[0][r] + sh->l_part[1][r];
      const float inv = (SPARSE && total == 0.f) ? 0.f : 1.f / total;        // sparse: no entry present in this range
      const size_t slot = size_t(slot_index) * p.heads + (head < p.heads ? head : 0);
      // O leaves through shared memory (ring stage 0: every product of the pass has completed), so that a store
      // instruction of a warp writes four whole 128-byte lines instead of 16 bytes of each of 32 rows: a warp
      // transposes 32 rows x 32 columns at a time in a block of its own (rows 144 bytes apart: 16-byte accesses of
      // eight consecutive rows, and of eight consecutive chunks of one row, meet no bank conflict).
      float* scratch = reinterpret_cast<float*>(base + kQSmemBytes) + (warp - kSoftmaxWarp0) * (32 * kOutRowFloats);
      const int first_head = head0 + quad * 32;                      // head of this warp's row 0
      float* dst = p.part_o + (size_t(slot_index) * p.heads + first_head) * kCkv + dq * kDimsPerCta;
#pragma unroll 1
      for (int c = grp * kOwnCols; c < (grp + 1) * kOwnCols; c += 32) {
        float o[32];
        tmem_ld_32x32b_x32(lane_base + kColO + c, o);
        tcgen05_wait_ld();
#pragma unroll
        for (int k = 0; k < 32; k += 4)
          *reinterpret_cast<float4*>(scratch + lane * kOutRowFloats + k) = make_float4(o[k] * inv, o[k + 1] * inv, o[k + 2] * inv, o[k + 3] * inv);
        __syncwarp();
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int rr = it * 4 + (lane >> 3), cc = (lane & 7) * 4;
          const float4 v = *reinterpret_cast<const float4*>(scratch + rr * kOutRowFloats + cc);
          if (first_head + rr < p.heads) *reinterpret_cast<float4*>(dst + size_t(rr) * kCkv + c + cc) = v;
        }
        __syncwarp();
      }
      if (dq == 0 && grp == 0 && head < p.heads) p.part_lse[slot] = (SPARSE && total == 0.f) ? -INFINITY : m_ref + log2f(total);
    }
  }

  cp_async_wait<0>();
  tcgen05_fence_before();
  __syncthreads();                                 // every role is done with this sequence's barriers and tiles
  tcgen05_fence_after();
  if (sh->wait.abort_flag) break;
  }
  if (warp == kMmaWarp) tmem_dealloc(sh->tmem_base, kTmemColumns);
}

// One CTA per (sequence, head): merges the chunks.  128 threads x 4 dims.
__global__ void __launch_bounds__(128)
mla_reduce_kernel(const Params p) {
  // launched as a programmatic dependent of the decode kernel: resident early, reads after it has completed
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int head = blockIdx.x, b = blockIdx.y;
  const int d = threadIdx.x * 4;
  const int len = seq_len(p, b);
  __nv_bfloat16* out = p.out + (size_t(b) * p.heads + head) * kCkv + d;
  if (len == 0) {
    *reinterpret_cast<uint2*>(out) = make_uint2(0u, 0u);
    if (threadIdx.x == 0 && p.lse) p.lse[size_t(b) * p.heads + head] = -INFINITY;
    return;
  }
  // the partial results of sequence b: one per worker whose range holds some of its tiles
  const int per_worker = units_per_worker(p);
  const int first_worker = (p.tile_prefix[b] + kSeqCost) / per_worker, last_worker = (p.tile_prefix[b + 1] - 1) / per_worker;
  float mm = -INFINITY;
  for (int w = first_worker; w <= last_worker; ++w) mm = fmaxf(mm, p.part_lse[size_t(w + b) * p.heads + head]);
  if (mm == -INFINITY) {                           // sparse form: every listed entry of the row was absent
    *reinterpret_cast<uint2*>(out) = make_uint2(0u, 0u);
    if (threadIdx.x == 0 && p.lse) p.lse[size_t(b) * p.heads + head] = -INFINITY;
    return;
  }
  float total = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int w = first_worker; w <= last_worker; ++w) {
    const size_t slot = size_t(w + b) * p.heads + head;
    const float wt = exp2f(p.part_lse[slot] - mm);
    const float4 v = *reinterpret_cast<const float4*>(p.part_o + slot * kCkv + d);
    total += wt;
    acc.x += wt * v.x; acc.y += wt * v.y; acc.z += wt * v.z; acc.w += wt * v.w;
  }
  const float inv = 1.f / total;
  *reinterpret_cast<uint2*>(out) = make_uint2(pack_bf16x2(acc.x * inv, acc.y * inv), pack_bf16x2(acc.z * inv, acc.w * inv));
  if (threadIdx.x == 0 && p.lse) p.lse[size_t(b) * p.heads + head] = mm + log2f(total);
}

struct Handle {
  int device;
  Params p;
  float sm_scale;            // sparse form: the scale is a configuration number, copied into the workspace at launch
};

constexpr int kMaxWorkers = 128;                           // workers the scratch is sized for (SMs / 2 per head block)

// Workspace behind the 256-byte status block: tile_prefix [B+1] int | part_o [slots, H, 512] f32 | part_lse [slots, H] f32
inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }
inline size_t slots_for(const cake_b200_mla_decode_config& c) { return size_t(kMaxWorkers) + size_t(c.batch); }

}  // namespace mla
}  // namespace cake

int cake::mla_decode_plan_view(void* handle, int which, void** device_pointer_out, int* count_out) {
  auto* h = static_cast<mla::Handle*>(handle);
  switch (which) {
    case 0: *device_pointer_out = h->p.tile_prefix; *count_out = h->p.batch + 1; return 0;
    case 1: *device_pointer_out = nullptr; *count_out = h->p.workers; return 0;         // ranges the unit list is cut into
    default: return kErrBadArgument;
  }
}

void cake::mla_decode_launch_facts(int* threads, int* dynamic_shared_bytes) {
  *threads = cake::mla::kThreads;
  *dynamic_shared_bytes = int(cake::mla::kSmemBytes);
}

static bool mla_config_ok(const cake_b200_mla_decode_config& c) {
  return c.batch >= 0 && c.batch <= 65535 && c.num_qo_heads > 0 && c.num_qo_heads <= 65535 * 64 &&
         c.head_dim_ckv == cake::mla::kCkv && c.head_dim_kpe == cake::mla::kKpe && c.page_size > 0 && c.max_kv_len >= 0;
}

extern "C" size_t cake_b200_mla_decode_workspace_bytes(const cake_b200_mla_decode_config* c) {
  if (!c || !mla_config_ok(*c)) return 0;
  const size_t slots = cake::mla::slots_for(*c);
  return 256 + cake::mla::align256((size_t(c->batch) + 1) * sizeof(int)) +
         slots * c->num_qo_heads * (cake::mla::kCkv + 1) * sizeof(float) + 256;
}

extern "C" int cake_b200_mla_decode_create(void** buffers, const cake_b200_mla_decode_config* config, void** handle_out) {
  using namespace cake;
  if (!buffers || !config || !handle_out) return kErrBadArgument;
  *handle_out = nullptr;
  int device = 0;
  if (int rc = require_blackwell(&device)) return rc;
  if (!mla_config_ok(*config)) return kErrBadArgument;
  for (int i = 0; i < 11; ++i) {
    if (!buffers[i]) return kErrBadArgument;
    if (i <= 3 && (reinterpret_cast<uintptr_t>(buffers[i]) & 15)) return kErrBadArgument;
  }
  auto* h = new (std::nothrow) mla::Handle;
  if (!h) return int(cudaErrorMemoryAllocation);
  h->device = device;
  mla::Params& p = h->p;
  p.q_nope = static_cast<const __nv_bfloat16*>(buffers[0]);
  p.q_pe = static_cast<const __nv_bfloat16*>(buffers[1]);
  p.ckv = static_cast<const __nv_bfloat16*>(buffers[2]);
  p.kpe = static_cast<const __nv_bfloat16*>(buffers[3]);
  p.kv_indptr = static_cast<const int*>(buffers[4]);
  p.kv_indices = static_cast<const int*>(buffers[5]);
  p.kv_last_page_len = static_cast<const int*>(buffers[6]);
  p.sm_scale = static_cast<const float*>(buffers[7]);
  p.out = static_cast<__nv_bfloat16*>(buffers[8]);
  p.lse = static_cast<float*>(buffers[9]);
  p.batch = int(config->batch);
  p.heads = config->num_qo_heads;
  p.page_size = config->page_size;
  p.sparse_indices = nullptr;
  p.top_k = 0;
  p.seq_start = nullptr;
  p.seq_tokens = nullptr;
  if (reinterpret_cast<uintptr_t>(buffers[10]) & 3) { delete h; return kErrBadArgument; }
  p.status = static_cast<int*>(buffers[10]);              // first word of the workspace
  // what follows the status block starts at the next 256-byte boundary (the size query allows for the slack):
  // the partial results are read and written sixteen bytes at a time
  uint8_t* ws = static_cast<uint8_t*>(buffers[10]) + 256;
  ws += (256 - (reinterpret_cast<uintptr_t>(ws) & 255)) & 255;
  p.tile_prefix = reinterpret_cast<int*>(ws);
  ws += mla::align256((size_t(p.batch) + 1) * sizeof(int));
  p.part_o = reinterpret_cast<float*>(ws);
  p.part_lse = p.part_o + mla::slots_for(*config) * p.heads * mla::kCkv;
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) { delete h; return kErrBadArgument; }
  const int head_blocks = (p.heads + mla::kHeads - 1) / mla::kHeads;
  p.workers = sms / (mla::kDimSplit * head_blocks);          // one CTA per SM
  p.workers = p.workers < 1 ? 1 : (p.workers > mla::kMaxWorkers ? mla::kMaxWorkers : p.workers);
  int rc = int(cudaFuncSetAttribute(mla::mla_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(mla::kSmemBytes)));
  if (rc) { delete h; return rc; }
  *handle_out = h;
  return 0;
}

extern "C" int cake_b200_mla_decode_launch(void* handle, void* cuda_stream) {
  using namespace cake;
  if (!handle) return kErrBadArgument;
  auto* h = static_cast<mla::Handle*>(handle);
  int device = -1;
  CAKE_CUDA_OK(cudaGetDevice(&device));
  if (device != h->device) return kErrWrongDevice;
  mla::Params p = h->p;
  p.wait_kiloclocks = test_hooks().budget_kiloclocks;
  p.skip_load = test_hooks().skip_load;
  if (p.batch == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(cuda_stream);
  const int head_blocks = (p.heads + mla::kHeads - 1) / mla::kHeads;
  mla::mla_plan_kernel<<<1, 1024, 0, s>>>(p);
  // The decode grid is a programmatic dependent of the plan grid and the reduce grid one of the decode grid: each
  // is resident (and past its launch latency) when the grid before it ends.
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t config = {};
  config.stream = s;
  config.attrs = attribute;
  config.numAttrs = 1;
  config.gridDim = dim3(p.workers * mla::kDimSplit * head_blocks);
  config.blockDim = dim3(mla::kThreads);
  config.dynamicSmemBytes = mla::kSmemBytes;
  cudaError_t err = p.sparse_indices ? cudaLaunchKernelEx(&config, mla::mla_decode_kernel<true>, p)
                                     : cudaLaunchKernelEx(&config, mla::mla_decode_kernel<false>, p);
  if (err != cudaSuccess) return int(err);
  config.gridDim = dim3(p.heads, p.batch);
  config.blockDim = dim3(128);
  config.dynamicSmemBytes = 0;
  err = cudaLaunchKernelEx(&config, mla::mla_reduce_kernel, p);
  if (err != cudaSuccess) return int(err);
  return int(cudaGetLastError());
}

extern "C" int cake_b200_mla_decode_destroy(void* handle) {
  delete static_cast<cake::mla::Handle*>(handle);
  return 0;
}

// ---- sparse form -------------------------------------------------------------------------------
static bool sparse_mla_config_ok(const cake_b200_sparse_mla_decode_config& c) {
  return c.num_tokens >= 0 && c.num_tokens <= 65535 && c.num_qo_heads > 0 && c.num_qo_heads <= 65535 * 64 &&
         c.head_dim_ckv == cake::mla::kCkv && c.head_dim_kpe == cake::mla::kKpe && c.top_k > 0 && c.top_k <= (1 << 20) &&
         c.num_cache_rows >= 0;
}
static cake_b200_mla_decode_config as_dense(const cake_b200_sparse_mla_decode_config& c) {
  cake_b200_mla_decode_config d{};
  d.batch = c.num_tokens;
  d.num_qo_heads = c.num_qo_heads;
  d.head_dim_ckv = c.head_dim_ckv;
  d.head_dim_kpe = c.head_dim_kpe;
  d.page_size = 1;
  d.max_kv_len = c.top_k;
  return d;
}

extern "C" size_t cake_b200_sparse_mla_decode_workspace_bytes(const cake_b200_sparse_mla_decode_config* c) {
  if (!c || !sparse_mla_config_ok(*c)) return 0;
  const cake_b200_mla_decode_config d = as_dense(*c);
  return cake_b200_mla_decode_workspace_bytes(&d) + 256;           // + the sm_scale word the kernel reads
}

extern "C" int cake_b200_sparse_mla_decode_create(void** buffers, const cake_b200_sparse_mla_decode_config* config, void** handle_out) {
  using namespace cake;
  if (!buffers || !config || !handle_out) return kErrBadArgument;
  *handle_out = nullptr;
  int device = 0;
  if (int rc = require_blackwell(&device)) return rc;
  if (!sparse_mla_config_ok(*config)) return kErrBadArgument;
  for (int i = 0; i < 7; ++i) {
    if (!buffers[i] && !(config->num_tokens == 0 && (i == 0 || i == 1 || i == 4 || i == 5))) return kErrBadArgument;
    if (i <= 3 && (reinterpret_cast<uintptr_t>(buffers[i]) & 15)) return kErrBadArgument;
  }
  if (reinterpret_cast<uintptr_t>(buffers[6]) & 3) return kErrBadArgument;
  auto* h = new (std::nothrow) mla::Handle;
  if (!h) return int(cudaErrorMemoryAllocation);
  h->device = device;
  mla::Params& p = h->p;
  p = mla::Params{};
  p.q_nope = static_cast<const __nv_bfloat16*>(buffers[0]);
  p.q_pe = static_cast<const __nv_bfloat16*>(buffers[1]);
  p.ckv = static_cast<const __nv_bfloat16*>(buffers[2]);
  p.kpe = static_cast<const __nv_bfloat16*>(buffers[3]);
  p.sparse_indices = static_cast<const int*>(buffers[4]);
  p.top_k = config->top_k;
  p.out = static_cast<__nv_bfloat16*>(buffers[5]);
  p.lse = nullptr;                                         // the contract returns the output only
  p.batch = int(config->num_tokens);
  p.heads = config->num_qo_heads;
  p.page_size = 1;
  p.status = static_cast<int*>(buffers[6]);                // first word of the workspace
  // words 16.. of the status block hold the scale, which the contract fixes as a number, not a tensor
  p.sm_scale = reinterpret_cast<const float*>(p.status + 16);
  h->sm_scale = config->sm_scale;
  uint8_t* ws = static_cast<uint8_t*>(buffers[6]) + 256;
  ws += (256 - (reinterpret_cast<uintptr_t>(ws) & 255)) & 255;
  p.tile_prefix = reinterpret_cast<int*>(ws);
  ws += mla::align256((size_t(p.batch) + 1) * sizeof(int));
  p.part_o = reinterpret_cast<float*>(ws);
  const cake_b200_mla_decode_config d = as_dense(*config);
  p.part_lse = p.part_o + mla::slots_for(d) * p.heads * mla::kCkv;
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) { delete h; return kErrBadArgument; }
  const int head_blocks = (p.heads + mla::kHeads - 1) / mla::kHeads;
  p.workers = sms / (mla::kDimSplit * head_blocks);
  p.workers = p.workers < 1 ? 1 : (p.workers > mla::kMaxWorkers ? mla::kMaxWorkers : p.workers);
  int rc = int(cudaFuncSetAttribute(mla::mla_decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(mla::kSmemBytes)));
  if (rc) { delete h; return rc; }
  *handle_out = h;
  return 0;
}

extern "C" int cake_b200_sparse_mla_decode_launch(void* handle, void* cuda_stream) {
  using namespace cake;
  if (!handle) return kErrBadArgument;
  auto* h = static_cast<mla::Handle*>(handle);
  if (!h->p.sparse_indices && h->p.batch != 0) return kErrBadArgument;
  if (h->p.batch == 0) return 0;
  // the scale travels as a kernel-readable word; the plan kernel clears word 0 of the block only
  CAKE_CUDA_OK(cudaMemcpyAsync(h->p.status + 16, &h->sm_scale, sizeof(float), cudaMemcpyHostToDevice,
                               reinterpret_cast<cudaStream_t>(cuda_stream)));
  return cake_b200_mla_decode_launch(handle, cuda_stream);
}

extern "C" int cake_b200_sparse_mla_decode_destroy(void* handle) {
  delete static_cast<cake::mla::Handle*>(handle);
  return 0;
}

// ---- causal prefill (see prefill.cuh) -------------------------------------------------------------
namespace cake {
namespace mla {
struct PrefillHandle {
  Handle decode;             // first member: the decode launch path takes it as a Handle
  const int *qo_indptr, *kv_indptr_segments, *last_page_len;
  int *seq_start, *seq_tokens, *masked;
  int segments, total_q, kv_unit, nan_for_masked;
};
}  // namespace mla
}  // namespace cake

static bool mla_prefill_config_ok(const cake_b200_mla_prefill_config& c, cake_b200_mla_decode_config* as_decode) {
  if (c.total_q < 0 || c.total_q > 65535 || c.segments <= 0 || c.segments > 65535) return false;
  cake_b200_mla_decode_config d{};
  d.batch = c.total_q;
  d.num_qo_heads = c.num_qo_heads;
  d.head_dim_ckv = c.head_dim_ckv;
  d.head_dim_kpe = c.head_dim_kpe;
  d.page_size = c.page_size;
  d.max_kv_len = c.max_kv_len;
  *as_decode = d;
  return mla_config_ok(d);
}

extern "C" size_t cake_b200_mla_prefill_workspace_bytes(const cake_b200_mla_prefill_config* c) {
  cake_b200_mla_decode_config d;
  if (!c || !mla_prefill_config_ok(*c, &d)) return 0;
  return cake_b200_mla_decode_workspace_bytes(&d) + cake::prefill::table_bytes(c->total_q) + 512;      // + this operator's own status block and its alignment slack
}

extern "C" int cake_b200_mla_prefill_create(void** buffers, const cake_b200_mla_prefill_config* config, void** handle_out) {
  using namespace cake;
  if (!buffers || !config || !handle_out) return kErrBadArgument;
  *handle_out = nullptr;
  cake_b200_mla_decode_config d;
  if (!mla_prefill_config_ok(*config, &d)) return kErrBadArgument;
  // buffers: q_nope, q_pe, ckv_cache, kpe_cache, qo_indptr, kv_indptr, kv_indices, kv_last_page_len (may be null),
  //          sm_scale, output, lse, workspace
  for (int i = 0; i < 12; ++i) if (!buffers[i] && i != 7) return kErrBadArgument;
  if (reinterpret_cast<uintptr_t>(buffers[11]) & 3) return kErrBadArgument;
  const size_t tables = prefill::table_bytes(config->total_q);
  // the decode part of the workspace follows the three per-token tables; its own status block leads it
  uint8_t* ws = static_cast<uint8_t*>(buffers[11]);
  uint8_t* table_base = ws + 256;
  table_base += (256 - (reinterpret_cast<uintptr_t>(table_base) & 255)) & 255;
  uint8_t* decode_ws = table_base + tables;
  void* as_decode[11] = {buffers[0], buffers[1], buffers[2], buffers[3], buffers[5], buffers[6], buffers[7] ? buffers[7] : buffers[5],
                         buffers[8], buffers[9], buffers[10], decode_ws};
  void* inner = nullptr;
  if (int rc = cake_b200_mla_decode_create(as_decode, &d, &inner)) return rc;
  auto* h = new (std::nothrow) mla::PrefillHandle;
  if (!h) { cake_b200_mla_decode_destroy(inner); return int(cudaErrorMemoryAllocation); }
  h->decode = *static_cast<mla::Handle*>(inner);
  cake_b200_mla_decode_destroy(inner);
  h->decode.p.status = reinterpret_cast<int*>(ws);                // one status word for the operator, at the start
  h->seq_start = reinterpret_cast<int*>(table_base);
  h->seq_tokens = reinterpret_cast<int*>(table_base + tables / 3);
  h->masked = reinterpret_cast<int*>(table_base + 2 * (tables / 3));
  h->decode.p.seq_start = h->seq_start;
  h->decode.p.seq_tokens = h->seq_tokens;
  h->decode.p.kv_last_page_len = nullptr;
  h->qo_indptr = static_cast<const int*>(buffers[4]);
  h->kv_indptr_segments = static_cast<const int*>(buffers[5]);
  h->last_page_len = static_cast<const int*>(buffers[7]);
  h->segments = config->segments;
  h->total_q = int(config->total_q);
  h->kv_unit = config->page_size;
  h->nan_for_masked = config->nan_for_masked;
  *handle_out = h;
  return 0;
}

extern "C" int cake_b200_mla_prefill_launch(void* handle, void* cuda_stream) {
  using namespace cake;
  if (!handle) return kErrBadArgument;
  auto* h = static_cast<mla::PrefillHandle*>(handle);
  int device = -1;
  CAKE_CUDA_OK(cudaGetDevice(&device));
  if (device != h->decode.device) return kErrWrongDevice;
  if (h->total_q == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(cuda_stream);
  prefill::prefill_plan_kernel<<<(h->total_q + 255) / 256, 256, 0, s>>>(h->qo_indptr, h->kv_indptr_segments, h->last_page_len, h->segments,
                                                                       h->kv_unit, h->total_q, h->seq_start, h->seq_tokens, h->masked);
  if (int rc = cake_b200_mla_decode_launch(&h->decode, cuda_stream)) return rc;
  if (h->nan_for_masked)
    prefill::prefill_mark_kernel<<<(h->total_q + 7) / 8, 256, 0, s>>>(h->masked, h->total_q, h->decode.p.out, h->decode.p.heads * mla::kCkv);
  return int(cudaGetLastError());
}

extern "C" int cake_b200_mla_prefill_destroy(void* handle) {
  delete static_cast<cake::mla::PrefillHandle*>(handle);
  return 0;
}
