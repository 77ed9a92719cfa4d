// Paged GQA decode for sm_100a: split-KV flash-decode + reduce.
//
// Operator: src/open_cake_ir/tasks/solx_fib/attention.py:132-183 (decode branch), tensor ABI
// attention_specs.py:44-84.  One query token per sequence; out = bf16(softmax(K q * scale) V),
// lse = logsumexp / ln 2; an empty sequence gives zeros and -inf.
//
// The kernel is bound by the HBM stream of K and V (2 * Hkv * D * 2 bytes per token) and never
// writes logits or probabilities to memory.  The tokens of all sequences, in order, form one list,
// and it is cut into as many equal consecutive ranges as there are SMs (a one-CTA plan kernel
// lists the pieces of sequences each range holds).  The decode kernel is persistent, one CTA of
// sixteen warps per SM: the CTA takes one range and each PAIR of warps (w, w+8) one KV head of it,
// so the eight pairs stream whole pages (page_size * Hkv * 256 B contiguous) and every SM moves
// the same number of bytes whatever the sequence lengths are.  The two warps of a pair take
// alternate 16-token tiles and run their own cp.async rings (128-bit copies, one 256-byte row per
// token and head, XOR-swizzled in shared memory, K and V halves of a tile in separate slots);
// there is no CTA-wide barrier, and a ring does not drain where a range passes from one sequence
// to the next.  The G = Hq/Hkv query heads that share a KV head are the rows of an m16n8k16 bf16
// MMA for S = Q K^T (ldmatrix on the K tile; rows beyond G are zero) and the columns of
// O^T += V^T P^T (ldmatrix.trans on the V tile; P as two bf16 terms, so the weights keep ~16
// significant bits); the online softmax runs in base 2 with warp shuffles.  The pair merges through
// shared memory and writes one partial result per piece; the pair that finishes the last piece of
// a (sequence, KV head) merges the pieces and writes the output, so there is no reduce launch.
#include "common.cuh"
#include "prefill.cuh"
#include "../../include/cake_b200.h"
#include <mutex>
#include <new>

namespace cake {
namespace gqa {

constexpr int kD = 128;                 // head dimension
constexpr int kTile = 16;               // tokens per warp tile
constexpr int kHeads = 8;               // KV heads per CTA
constexpr int kParts = 2;               // warps per KV head; warp part p takes tiles p, p+2, ...
constexpr int kWarps = kHeads * kParts;
constexpr int kSlots = 3;               // cp.async slots per warp, each one K or V half of a tile
constexpr int kTileBytes = kTile * kD * 2;          // 4 KiB: 16 tokens of K (or of V) of one head
constexpr int kWarpSmem = kSlots * kTileBytes;       // 12 KiB
constexpr int kRingBytes = kWarps * kWarpSmem;       // 192 KiB per CTA, one CTA per SM
constexpr int kParkBytes = 34 * 32 * 4;               // a warp's O^T (32 registers), m and l
constexpr int kSmemBytes = kRingBytes + kHeads * kParkBytes;          // + per pair: the second warp's parked state
constexpr float kLog2e = 1.4426950408889634f;

struct Params {
  const __nv_bfloat16* q;        // [B, Hq, D]
  const __nv_bfloat16* k_cache;  // [pages, page_size, Hkv, D]
  const __nv_bfloat16* v_cache;
  const int* kv_indptr;          // [B+1] in pages
  const int* kv_indices;
  const int* kv_last_page_len;   // [B]
  const float* sm_scale;         // [1]
  __nv_bfloat16* out;            // [B, Hq, D]
  float* lse;                    // [B, Hq]
  float* part_o;                 // [capacity, Hq, D] normalised partial outputs, one slot per entry of `items`
  float* part_lse;               // [capacity, Hq]    base-2 partial log-sum-exp
  int4* items;                   // [capacity] pieces of sequences in token order, written by the plan kernel:
                                 //   x = b | (pieces of b << 16), y = first token, z = list index of b's first piece, w = end token
  int* item_page;                // [capacity] kv_indptr[b] of the piece
  int* range_first;              // [ranges] list index of the first piece of each range
  int* range_count;              // [ranges] pieces of each range
  int* done;                     // [B, Hkv] finished items
  int* status;                   // library status word (may be null)
  int batch, hq, hkv, page_size, capacity, ranges;
  // Explicit sequence table (causal prefill, where every query token is a sequence of its own over a prefix of its
  // segment's rows): sequence b holds seq_tokens[b] tokens whose page list starts at kv_indices[seq_start[b]];
  // null = sequences come from kv_indptr / kv_last_page_len.  With kv_indices null the page list is the
  // identity (ragged K/V: row r of the cache is token r).
  const int* seq_start;
  const int* seq_tokens;
};

__device__ __forceinline__ int seq_len(const Params& p, int b) {
  if (p.seq_tokens) return p.seq_tokens[b];
  const int pages = p.kv_indptr[b + 1] - p.kv_indptr[b];
  return pages <= 0 ? 0 : (pages - 1) * p.page_size + p.kv_last_page_len[b];
}

// K and V are read exactly once: their lines are marked evict-first in L2, and the partial
// results evict-last, so that the stream does not push the partial results out to DRAM before
// they are merged.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid, uint64_t policy) {
  const int bytes = valid ? 16 : 0;     // 0 source bytes = zero fill
  asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2, %3;" ::"r"(dst), "l"(src), "r"(bytes), "l"(policy)
               : "memory");
}
__device__ __forceinline__ void store_keep(float* dst, float value, uint64_t policy) {
  asm volatile("st.global.L2::cache_hint.f32 [%0], %1, %2;" ::"l"(dst), "f"(value), "l"(policy) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Byte offset of (token row, 16-byte chunk) inside a swizzled [16][256 B] tile.
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) { return uint32_t(row * 256 + ((chunk ^ (row & 7)) << 4)); }

// Lane r (and r+16) looks up the page of token tok0+r once: the result is the index of that token's
// 256-byte (token, head) row in the cache, or -1 beyond the sequence, so the page-table arithmetic
// (an integer division by the run-time page size) is done once per token, not once per copy.
__device__ __forceinline__ int lookup_rows(const Params& p, int page_base, int kvh, int tok0, int len, int lane) {
  const int tok = tok0 + (lane & 15);
  if (tok >= len) return -1;
  const int page = p.kv_indices ? __ldg(p.kv_indices + page_base + tok / p.page_size) : page_base + tok / p.page_size;
  return (page * p.page_size + (tok % p.page_size)) * p.hkv + kvh;   // < 2^31 rows = 512 GiB per cache
}

// Issues the copies of the K (or V) half of a tile: 16 rows of 256 bytes, 16 lanes per row.
__device__ __forceinline__ void load_half(const __nv_bfloat16* __restrict__ cache, int my_row, uint32_t dst, int lane,
                                          uint64_t policy) {
  const int chunk = lane & 15;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = (lane >> 4) + 2 * i;
    const int idx = __shfl_sync(0xffffffffu, my_row, row);
    cp_async_16(dst + tile_off(row, chunk), cache + (size_t(idx < 0 ? 0 : idx) * kD + chunk * 8), idx >= 0, policy);
  }
}

// One CTA: cuts the work of the launch into p.ranges equal ranges and lists the pieces of
// sequences they hold, in order, so that the pieces of a range, and the pieces of a sequence, are
// consecutive entries.  Work is counted in token units: kPieceCost units for the start of a sequence
// (a range that holds the start of another sequence pays one more merge of its two warps, partial
// result, fence and counter: about 4 us, the time of ~32 tokens), then one unit per token.  Also
// resets the counters and writes the results of empty sequences (zeros, lse = -inf), which no
// piece covers.
constexpr int kPieceCost = 32;
__global__ void __launch_bounds__(1024)
gqa_plan_kernel(const Params p) {
  __shared__ long long sums64[32];
  __shared__ int sums32[32];
  const int tid = threadIdx.x;
  if (tid == 0 && p.status) *p.status = 0;
  for (int r = tid; r < p.ranges; r += 1024) { p.range_first[r] = 0x7fffffff; p.range_count[r] = 0; }
  const int len0 = tid < p.batch ? seq_len(p, tid) : 0;              // the first 1024 lengths stay in registers
  long long mine = len0 > 0 ? len0 + kPieceCost : 0, all_units = 0;
  for (int b = tid + 1024; b < p.batch; b += 1024) { const int n = seq_len(p, b); mine += n > 0 ? n + kPieceCost : 0; }
  cta1024_exclusive_scan(mine, sums64, all_units);                    // (its barriers also publish the defaults above)
  const long long per = max(16LL, (((all_units + p.ranges - 1) / p.ranges) + 15) & ~15LL);

  long long units_before = 0;
  int entries_before = 0;
  for (int base = 0; base < p.batch; base += 1024) {
    const int b = base + tid;
    const int len = base == 0 ? len0 : (b < p.batch ? seq_len(p, b) : 0);
    long long batch_units;
    const long long start = units_before + cta1024_exclusive_scan((long long)(len > 0 ? len + kPieceCost : 0), sums64, batch_units) + kPieceCost;
    const int first_range = int(start / per);                          // `start`: where the sequence's tokens begin
    const int n = len > 0 ? int((start + len - 1) / per) - first_range + 1 : 0;
    int batch_entries;
    const int first = entries_before + cta1024_exclusive_scan(n, sums32, batch_entries);
    if (b < p.batch) {
      const int page_base = p.seq_start ? p.seq_start[b] : p.kv_indptr[b];
      for (int k = 0; k < n; ++k) {
        const long long range_start = (long long)(first_range + k) * per;
        const long long piece_begin = max(start, range_start), piece_end = min(start + len, range_start + per);
        p.items[first + k] = make_int4(b | (n << 16), int(piece_begin - start), first, int(piece_end - start));
        p.item_page[first + k] = page_base;
        atomicMin(p.range_first + first_range + k, first + k);
        atomicAdd(p.range_count + first_range + k, 1);
      }
      for (int h = 0; h < p.hkv; ++h) p.done[size_t(b) * p.hkv + h] = 0;
      if (len == 0) {
        for (int h = 0; h < p.hq; ++h) {
          p.lse[size_t(b) * p.hq + h] = -INFINITY;
          for (int d = 0; d < kD; ++d) p.out[(size_t(b) * p.hq + h) * kD + d] = __float2bfloat16(0.f);
        }
      }
    }
    units_before += batch_units;
    entries_before += batch_entries;
  }
}

__device__ __forceinline__ void pair_barrier(int pair) { asm volatile("bar.sync %0, 64;" ::"r"(pair + 1) : "memory"); }

// Merges the chunks of (sequence b, KV head kvh): out = sum_s w_s o_s / sum_s w_s with
// w_s = 2^(lse_s - max lse).  One warp works on all heads of the group at once: L lanes per head,
// each owning 32/L float4 of the head's 128 dims, sixteen 16-byte loads in flight per lane, so
// the merge costs a few memory round trips however many heads there are.  The partial results
// were written by other SMs during this launch, so they are read past L1.
template <int L>
__device__ __forceinline__ void merge_chunks_t(const Params& p, int b, int kvh, int first, int chunks, int group, int lane) {
  constexpr int NF = 32 / L;            // float4 per lane
  constexpr int BATCH = 16 / NF;        // chunks in flight
  const int hs = lane / L, sub = lane % L;
  const bool have = hs < group;
  const int head = kvh * group + (have ? hs : 0);
  const size_t slot0 = size_t(first) * p.hq + head;                  // + s * hq
  float mm = -INFINITY, total = 0.f;    // running maximum and sum of weights relative to it
  float4 acc[NF];
#pragma unroll
  for (int k = 0; k < NF; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s0 = 0; s0 < chunks; s0 += BATCH) {
    float ls[BATCH];
    float4 v[BATCH][NF];
#pragma unroll
    for (int i = 0; i < BATCH; ++i) {
      const int s = min(s0 + i, chunks - 1);            // past the end: the last row again, weight 0
      ls[i] = __ldcg(p.part_lse + slot0 + size_t(s) * p.hq);
      const float4* src = reinterpret_cast<const float4*>(p.part_o + (slot0 + size_t(s) * p.hq) * kD);
#pragma unroll
      for (int k = 0; k < NF; ++k) v[i][k] = __ldcg(src + sub + L * k);
    }
    float m_new = mm;                   // every piece holds a token, so its lse is finite
#pragma unroll
    for (int i = 0; i < BATCH; ++i) m_new = fmaxf(m_new, ls[i]);
    const float rescale = exp2f(mm - m_new);            // 0 on the first batch
    mm = m_new;
    total *= rescale;
#pragma unroll
    for (int k = 0; k < NF; ++k) { acc[k].x *= rescale; acc[k].y *= rescale; acc[k].z *= rescale; acc[k].w *= rescale; }
#pragma unroll
    for (int i = 0; i < BATCH; ++i) {
      const float w = s0 + i < chunks ? exp2f(ls[i] - mm) : 0.f;
      total += w;
#pragma unroll
      for (int k = 0; k < NF; ++k) {
        acc[k].x += w * v[i][k].x; acc[k].y += w * v[i][k].y; acc[k].z += w * v[i][k].z; acc[k].w += w * v[i][k].w;
      }
    }
  }
  if (!have) return;
  const float inv = 1.f / total;
#pragma unroll
  for (int k = 0; k < NF; ++k) {
    uint2 packed;
    packed.x = pack_bf16x2(acc[k].x * inv, acc[k].y * inv);
    packed.y = pack_bf16x2(acc[k].z * inv, acc[k].w * inv);
    *reinterpret_cast<uint2*>(p.out + (size_t(b) * p.hq + head) * kD + (sub + L * k) * 4) = packed;
  }
  if (sub == 0) p.lse[size_t(b) * p.hq + head] = mm + log2f(total);
}

__device__ __forceinline__ void merge_chunks(const Params& p, int b, int kvh, int first, int chunks, int group, int lane) {
  if (group == 1) merge_chunks_t<32>(p, b, kvh, first, chunks, group, lane);
  else if (group == 2) merge_chunks_t<16>(p, b, kvh, first, chunks, group, lane);
  else if (group <= 4) merge_chunks_t<8>(p, b, kvh, first, chunks, group, lane);
  else merge_chunks_t<4>(p, b, kvh, first, chunks, group, lane);
}

__global__ void __launch_bounds__(kWarps * 32, 1)
gqa_decode_kernel(const Params p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pair = warp % kHeads, part = warp / kHeads;
  const int group = p.hq / p.hkv;
  const int row = lane >> 2;            // query head inside the group held by this lane's rows of S
  const int quad = lane & 3;
  const float scale2 = __ldg(p.sm_scale) * kLog2e;
  const uint32_t ring = smem_u32(smem) + warp * kWarpSmem;
  float* park = reinterpret_cast<float*>(smem + kRingBytes + pair * kParkBytes);

  const uint64_t stream_policy = l2_policy_evict_first(), keep_policy = l2_policy_evict_last();
  // Which token range and which KV head this pair works on.  With eight or more KV heads a CTA
  // takes one range and eight heads of it; with 1, 2 or 4 the CTA's pairs share 8 / Hkv ranges.
  int range_id, kvh_mine;
  bool active;
  if (p.hkv >= kHeads) {
    const int head_blocks = (p.hkv + kHeads - 1) / kHeads;
    range_id = blockIdx.x / head_blocks;
    kvh_mine = (blockIdx.x % head_blocks) * kHeads + pair;
    active = kvh_mine < p.hkv && range_id < p.ranges;
  } else if (kHeads % p.hkv == 0) {
    range_id = blockIdx.x * (kHeads / p.hkv) + pair / p.hkv;
    kvh_mine = pair % p.hkv;
    active = range_id < p.ranges;
  } else {
    range_id = blockIdx.x;
    kvh_mine = pair;
    active = pair < p.hkv && range_id < p.ranges;
  }
  // Launched as a programmatic dependent of the plan kernel: everything above overlaps it, the
  // list and the counters are read only after it has completed.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // Items are numbered piece * Hkv + KV head; this pair's run from idx up to (not including) total.
  int idx = 0, total = 0;
  if (active && p.range_count[range_id] > 0) {
    idx = p.range_first[range_id] * p.hkv + kvh_mine;
    total = (p.range_first[range_id] + p.range_count[range_id]) * p.hkv;
  }
  int4 rec = make_int4(0, 0, 0, 0);
  int page_base = 0;
  if (idx < total) {
    rec = __ldg(p.items + idx / p.hkv);
    page_base = __ldg(p.item_page + idx / p.hkv);
  }
  auto tiles_of = [&](int item, const int4& r) {    // tiles of an item that fall to this warp
    return item < total ? ((r.w - r.y + kTile - 1) / kTile - part + kParts - 1) / kParts : 0;
  };
  // Q fragments (A operand of S = Q K^T): rows = heads of the group, zero beyond it.
  uint32_t qa[8][2];
  auto load_q = [&](int item, const int4& r) {
    const bool have = row < group && item < total;
    const __nv_bfloat16* qrow = p.q + (size_t(r.x & 0xffff) * p.hq + (have ? (item % p.hkv) * group + row : 0)) * kD;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qa[ks][0] = have ? __ldg(reinterpret_cast<const uint32_t*>(qrow + ks * 16 + quad * 2)) : 0u;
      qa[ks][1] = have ? __ldg(reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + quad * 2)) : 0u;
    }
  };
  load_q(idx, rec);

  // A warp's tiles form one stream across its items.  Copy groups alternate K(t), V(t), K(t+1),
  // ... through three 4 KiB slots: two are in flight while the third is being consumed, also
  // across the boundary between two items (`primed`: the first tile of the coming item is on
  // its way already).
  int k_slot = 0;
  int next_row = -1;
  bool primed = false;

  while (idx < total) {
    const int kvh = idx % p.hkv;
    const int b = rec.x & 0xffff, chunks = int(unsigned(rec.x) >> 16);
    const int begin = rec.y, end = rec.w;
    const int my_tiles = tiles_of(idx, rec);
    // The next piece of the range (same KV head): its record is asked for now and needed at this
    // item's last tile, where the first copies of the next item go out.
    const int nxt_idx = idx + p.hkv;
    int4 nxt_rec = make_int4(0, 0, 0, 0);
    int nxt_page = 0;
    if (nxt_idx < total) {
      nxt_rec = __ldg(p.items + nxt_idx / p.hkv);
      nxt_page = __ldg(p.item_page + nxt_idx / p.hkv);
    }
    if (my_tiles > 0 && !primed) {      // cold start: nothing of this item is in flight yet
      const int v_slot = k_slot == 2 ? 0 : k_slot + 1;
      next_row = lookup_rows(p, page_base, kvh, begin + part * kTile, end, lane);
      load_half(p.k_cache, next_row, ring + k_slot * kTileBytes, lane, stream_policy);
      cp_async_commit();
      load_half(p.v_cache, next_row, ring + v_slot * kTileBytes, lane, stream_policy);
      cp_async_commit();
    }
    primed = false;

    // O is kept transposed, O^T[dim][head] = V^T P^T, so that all four accumulator registers of
    // an MMA are live (dims are the 16 rows, the group's heads the 8 columns): o[n] covers dims
    // n*16 + lane/4 (+8 for registers 2, 3) and heads quad*2 (+1 for registers 1, 3).
    float o[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m = -INFINITY, l = 0.f;       // running max (base 2) and sum of head `row`

    for (int j = 0; j < my_tiles; ++j) {
      const int v_slot = k_slot == 2 ? 0 : k_slot + 1;
      const int free_slot = v_slot == 2 ? 0 : v_slot + 1;     // held the V half of the previous tile
      const int tok0 = begin + (part + j * kParts) * kTile;
      // the tile after this one in the stream: the item's next, or the first of the coming item
      const bool last = j + 1 == my_tiles;
      const int nxt_tiles = tiles_of(nxt_idx, nxt_rec);
      const bool follows = !last || nxt_tiles > 0;
      cp_async_wait<1>();
      __syncwarp();                     // K(t) has landed; every lane is done with V(t-1)
      if (follows) {
        next_row = last ? lookup_rows(p, nxt_page, kvh, nxt_rec.y + part * kTile, nxt_rec.w, lane)
                        : lookup_rows(p, page_base, kvh, tok0 + kParts * kTile, end, lane);
        load_half(p.k_cache, next_row, ring + free_slot * kTileBytes, lane, stream_policy);
      }
      cp_async_commit();
      const uint32_t k_smem = ring + k_slot * kTileBytes, v_smem = ring + v_slot * kTileBytes;

      // S = Q K^T : two n-tiles of 8 tokens
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t b0, b1, b2, b3;
        const int mi = lane >> 3;                       // which 8x8 matrix this lane addresses
        const int trow = (mi >> 1) * 8 + (lane & 7);
        ldmatrix_x4(k_smem + tile_off(trow, ks * 2 + (mi & 1)), b0, b1, b2, b3);
        mma_bf16_16816(s0, qa[ks][0], 0u, qa[ks][1], 0u, b0, b1);
        mma_bf16_16816(s1, qa[ks][0], 0u, qa[ks][1], 0u, b2, b3);
      }
      // this lane: head `row`, tokens tok0 + quad*2 + {0,1} (s0) and + 8 (s1)
      float v[4];
      v[0] = s0[0] * scale2; v[1] = s0[1] * scale2; v[2] = s1[0] * scale2; v[3] = s1[1] * scale2;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int tok = tok0 + quad * 2 + (i & 1) + (i >> 1) * 8;
        if (tok >= end) v[i] = -INFINITY;
      }
      float tmax = fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3]));
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
      const float m_new = fmaxf(m, tmax);            // finite: every tile holds at least one valid token
      const float alpha = exp2f(m - m_new);
      float pr[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) pr[i] = exp2f(v[i] - m_new);
      float psum = pr[0] + pr[1] + pr[2] + pr[3];
      psum += __shfl_xor_sync(0xffffffffu, psum, 1);
      psum += __shfl_xor_sync(0xffffffffu, psum, 2);
      l = l * alpha + psum;
      m = m_new;
      // P enters the tensor core as two bf16 terms (value + rounding residual): a single bf16
      // term would put 2^-9 relative error on every weight, more than the contract's tolerance
      // allows once the weighted values cancel.  As the B operand of O^T += V^T P^T the fragment
      // layout of P^T (tokens quad*2.. of head lane/4) is exactly the accumulator layout of S.
      uint32_t p_hi0, p_hi1, p_lo0, p_lo1;
      split_bf16x2(pr[0], pr[1], p_hi0, p_lo0);       // tokens 0..7 of the tile
      split_bf16x2(pr[2], pr[3], p_hi1, p_lo1);       // tokens 8..15
      const float alpha0 = __shfl_sync(0xffffffffu, alpha, quad * 8);       // head quad*2
      const float alpha1 = __shfl_sync(0xffffffffu, alpha, quad * 8 + 4);   // head quad*2 + 1

      cp_async_wait<1>();
      __syncwarp();                     // V(t) has landed; every lane is done with K(t)
      if (follows) load_half(p.v_cache, next_row, ring + k_slot * kTileBytes, lane, stream_policy);
      cp_async_commit();
#pragma unroll
      for (int n = 0; n < 8; ++n) { o[n][0] *= alpha0; o[n][1] *= alpha1; o[n][2] *= alpha0; o[n][3] *= alpha1; }
      // V^T fragments through ldmatrix.trans: 16 dims x 16 tokens per instruction
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        uint32_t a0, a1, a2, a3;
        const int mi = lane >> 3;
        const int trow = (mi >> 1) * 8 + (lane & 7);    // matrices 0/1: tokens 0-7, dims +0/+8; 2/3: tokens 8-15
        ldmatrix_x4_trans(v_smem + tile_off(trow, n * 2 + (mi & 1)), a0, a1, a2, a3);
        mma_bf16_16816(o[n], a0, a1, a2, a3, p_hi0, p_hi1);
        mma_bf16_16816(o[n], a0, a1, a2, a3, p_lo0, p_lo1);
      }
      k_slot = free_slot;
      primed = last && follows;
    }
    load_q(nxt_idx, nxt_rec);           // the Q registers are free: fetch the coming item's

    if (part == 1) {                    // the second warp parks its state for the first
#pragma unroll
      for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int r = 0; r < 4; ++r) park[(n * 4 + r) * 32 + lane] = o[n][r];
      park[32 * 32 + lane] = m;
      park[33 * 32 + lane] = l;
    }
    pair_barrier(pair);                 // the parked state is written
    float f00 = 0.f, f01 = 0.f, f10 = 0.f, f11 = 0.f;
    if (part == 0) {                    // fold the partner's state into the registers
      const float m1 = park[32 * 32 + lane], l1 = park[33 * 32 + lane];
      const float m_all = fmaxf(m, m1);            // m is finite: the first warp always has a tile
      const float w0 = exp2f(m - m_all), w1 = exp2f(m1 - m_all);
      l = l * w0 + l1 * w1;
      m = m_all;
      const float inv = 1.f / l;
      f00 = __shfl_sync(0xffffffffu, w0 * inv, quad * 8); f01 = __shfl_sync(0xffffffffu, w0 * inv, quad * 8 + 4);
      f10 = __shfl_sync(0xffffffffu, w1 * inv, quad * 8); f11 = __shfl_sync(0xffffffffu, w1 * inv, quad * 8 + 4);
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        o[n][0] = o[n][0] * f00 + park[(n * 4 + 0) * 32 + lane] * f10;
        o[n][1] = o[n][1] * f01 + park[(n * 4 + 1) * 32 + lane] * f11;
        o[n][2] = o[n][2] * f00 + park[(n * 4 + 2) * 32 + lane] * f10;
        o[n][3] = o[n][3] * f01 + park[(n * 4 + 3) * 32 + lane] * f11;
      }
    }
    pair_barrier(pair);                 // the parked state has been read
    if (part == 0) {
      // partial result of this item: normalised rows and base-2 log-sum-exp
      const size_t slot0 = size_t(idx / p.hkv) * p.hq + kvh * group;
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const int dim = n * 16 + row;
        if (quad * 2 < group) {
          store_keep(p.part_o + (slot0 + quad * 2) * kD + dim, o[n][0], keep_policy);
          store_keep(p.part_o + (slot0 + quad * 2) * kD + dim + 8, o[n][2], keep_policy);
        }
        if (quad * 2 + 1 < group) {
          store_keep(p.part_o + (slot0 + quad * 2 + 1) * kD + dim, o[n][1], keep_policy);
          store_keep(p.part_o + (slot0 + quad * 2 + 1) * kD + dim + 8, o[n][3], keep_policy);
        }
      }
      if (row < group && quad == 0) store_keep(p.part_lse + slot0 + row, m + log2f(l), keep_policy);
      // The pair that completes the last item of (b, kvh) merges the chunks.
      __threadfence();
      __syncwarp();
      int last_item = 0;
      if (lane == 0) last_item = atomicAdd(p.done + size_t(b) * p.hkv + kvh, 1) == chunks - 1;
      if (__shfl_sync(0xffffffffu, last_item, 0)) {
        __threadfence();
        merge_chunks(p, b, kvh, rec.z, chunks, group, lane);
      }
    }
    idx = nxt_idx; rec = nxt_rec; page_base = nxt_page;
  }
  cp_async_wait<0>();
}

struct Handle {
  int device;
  int sms;
  Params p;
};

// Token ranges and CTAs for `sms` SMs: with eight or more KV heads a CTA takes one range and a block
// of eight heads; with 1, 2 or 4 its eight warp pairs share 8 / Hkv ranges; otherwise a CTA takes
// one range and leaves the pairs beyond Hkv idle.
inline void geometry(int hkv, int sms, int* ranges, int* grid) {
  if (hkv >= kHeads) {
    const int head_blocks = (hkv + kHeads - 1) / kHeads;
    *ranges = sms / head_blocks > 0 ? sms / head_blocks : 1;
    *grid = *ranges * head_blocks;
  } else {
    *ranges = kHeads % hkv == 0 ? sms * (kHeads / hkv) : sms;
    *grid = sms;
  }
}
constexpr int kMaxSms = 192;             // SM count the workspace is sized for

// A range holds a piece of every sequence it touches: at most ranges + batch pieces in all.
inline size_t entries_for(const cake_b200_gqa_decode_config& c, int sms) {
  int ranges, grid;
  geometry(c.num_kv_heads, sms, &ranges, &grid);
  return size_t(ranges) + size_t(c.batch);
}

// Scratch layout shared by the two entry points (offsets from a 256-byte aligned base):
//   done [B*Hkv] int | items [entries] int4 | item_page [entries] int | range_first [ranges] int | range_count [ranges] int |
//   part_o [entries*Hq*D] f32 | part_lse [entries*Hq] f32
inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }
inline size_t scratch_bytes(const cake_b200_gqa_decode_config& c, size_t entries) {
  return align256(size_t(c.batch) * c.num_kv_heads * sizeof(int)) + align256(entries * sizeof(int4)) + 3 * align256((entries + 1) * sizeof(int)) +
         align256(entries * c.num_qo_heads * kD * sizeof(float)) + align256(entries * c.num_qo_heads * sizeof(float));
}
inline void carve_scratch(Params& p, uint8_t* base) {
  const size_t entries = size_t(p.capacity);
  p.done = reinterpret_cast<int*>(base);
  base += align256(size_t(p.batch) * p.hkv * sizeof(int));
  p.items = reinterpret_cast<int4*>(base);
  base += align256(entries * sizeof(int4));
  p.item_page = reinterpret_cast<int*>(base);
  base += align256((entries + 1) * sizeof(int));
  p.range_first = reinterpret_cast<int*>(base);          // ranges <= entries
  base += align256((entries + 1) * sizeof(int));
  p.range_count = reinterpret_cast<int*>(base);
  base += align256((entries + 1) * sizeof(int));
  p.part_o = reinterpret_cast<float*>(base);
  base += align256(entries * p.hq * kD * sizeof(float));
  p.part_lse = reinterpret_cast<float*>(base);
}

inline int fill_params(Params& p, void** buffers, const cake_b200_gqa_decode_config& c) {
  for (int i = 0; i < 9; ++i) {
    if (!buffers[i]) return kErrBadArgument;
    if (i <= 2 && (reinterpret_cast<uintptr_t>(buffers[i]) & 15)) return kErrBadArgument;
  }
  p.q = static_cast<const __nv_bfloat16*>(buffers[0]);
  p.k_cache = static_cast<const __nv_bfloat16*>(buffers[1]);
  p.v_cache = static_cast<const __nv_bfloat16*>(buffers[2]);
  p.kv_indptr = static_cast<const int*>(buffers[3]);
  p.kv_indices = static_cast<const int*>(buffers[4]);
  p.kv_last_page_len = static_cast<const int*>(buffers[5]);
  p.sm_scale = static_cast<const float*>(buffers[6]);
  p.out = static_cast<__nv_bfloat16*>(buffers[7]);
  p.lse = static_cast<float*>(buffers[8]);
  p.batch = int(c.batch);
  p.hq = c.num_qo_heads;
  p.hkv = c.num_kv_heads;
  p.page_size = c.page_size;
  p.status = nullptr;
  p.seq_start = nullptr;
  p.seq_tokens = nullptr;
  return 0;
}

inline int launch(Params& p, int sms, cudaStream_t s) {
  int grid;
  geometry(p.hkv, sms, &p.ranges, &grid);
  gqa_plan_kernel<<<1, 1024, 0, s>>>(p);
  // The decode grid is a programmatic dependent: it may start while the plan kernel runs and waits
  // for it on the device, which takes the second launch latency off the critical path.
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid);
  config.blockDim = dim3(kWarps * 32);
  config.dynamicSmemBytes = kSmemBytes;
  config.stream = s;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  const cudaError_t err = cudaLaunchKernelEx(&config, gqa_decode_kernel, p);
  return int(err != cudaSuccess ? err : cudaGetLastError());
}

}  // namespace gqa
}  // namespace cake

int cake::gqa_decode_plan_view(void* handle, int which, void** device_pointer_out, int* count_out) {
  auto* h = static_cast<gqa::Handle*>(handle);
  const gqa::Params& p = h->p;
  int ranges = 0, grid = 0;
  gqa::geometry(p.hkv, h->sms, &ranges, &grid);       // what a launch of this handle uses
  switch (which) {
    case 0: *device_pointer_out = p.items; *count_out = p.capacity; return 0;          // int4 per piece
    case 1: *device_pointer_out = p.range_first; *count_out = ranges; return 0;
    case 2: *device_pointer_out = p.range_count; *count_out = ranges; return 0;
    default: return kErrBadArgument;
  }
}

void cake::gqa_decode_launch_facts(int* threads, int* dynamic_shared_bytes) {
  *threads = cake::gqa::kWarps * 32;
  *dynamic_shared_bytes = int(cake::gqa::kSmemBytes);
}

static bool gqa_config_ok(const cake_b200_gqa_decode_config& c) {
  if (c.batch < 0 || c.batch > 65535 || c.head_dim != cake::gqa::kD || c.page_size <= 0 || c.max_kv_len < 0) return false;
  if (c.max_kv_len > (1 << 21) || c.batch * c.max_kv_len >= (1LL << 40)) return false;
  if (c.num_kv_heads <= 0 || c.num_kv_heads > 65535 || c.num_qo_heads % c.num_kv_heads) return false;
  const int g = c.num_qo_heads / c.num_kv_heads;
  return g >= 1 && g <= 8;
}

static int gqa_sm_count(int device, int* sms) {
  CAKE_CUDA_OK(cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, device));
  return 0;
}

extern "C" size_t cake_b200_gqa_decode_workspace_bytes(const cake_b200_gqa_decode_config* c) {
  if (!c || !gqa_config_ok(*c)) return 0;
  return 256 + cake::gqa::scratch_bytes(*c, cake::gqa::entries_for(*c, cake::gqa::kMaxSms)) + 256;
}

extern "C" int cake_b200_gqa_decode_create(void** buffers, const cake_b200_gqa_decode_config* config, void** handle_out) {
  using namespace cake;
  if (!buffers || !config || !handle_out) return kErrBadArgument;
  *handle_out = nullptr;
  int device = 0;
  if (int rc = require_blackwell(&device)) return rc;
  if (!gqa_config_ok(*config) || !buffers[9] || (reinterpret_cast<uintptr_t>(buffers[9]) & 3)) return kErrBadArgument;
  auto* h = new (std::nothrow) gqa::Handle;
  if (!h) return int(cudaErrorMemoryAllocation);
  h->device = device;
  gqa::Params& p = h->p;
  if (int rc = gqa::fill_params(p, buffers, *config)) { delete h; return rc; }
  p.capacity = int(gqa::entries_for(*config, gqa::kMaxSms));
  p.status = static_cast<int*>(buffers[9]);               // first word of the workspace
  uint8_t* ws = static_cast<uint8_t*>(buffers[9]) + 256;
  ws += (256 - (reinterpret_cast<uintptr_t>(ws) & 255)) & 255;
  gqa::carve_scratch(p, ws);
  int sms = 0;
  int rc = gqa_sm_count(device, &sms);
  if (!rc) rc = int(cudaFuncSetAttribute(gqa::gqa_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gqa::kSmemBytes));
  if (rc) { delete h; return rc; }
  h->sms = sms < gqa::kMaxSms ? sms : gqa::kMaxSms;
  *handle_out = h;
  return 0;
}

extern "C" int cake_b200_gqa_decode_launch(void* handle, void* cuda_stream) {
  using namespace cake;
  if (!handle) return kErrBadArgument;
  auto* h = static_cast<gqa::Handle*>(handle);
  int device = -1;
  CAKE_CUDA_OK(cudaGetDevice(&device));
  if (device != h->device) return kErrWrongDevice;
  if (h->p.batch == 0) return 0;
  gqa::Params p = h->p;
  return gqa::launch(p, h->sms, reinterpret_cast<cudaStream_t>(cuda_stream));
}

extern "C" int cake_b200_gqa_decode_destroy(void* handle) {
  delete static_cast<cake::gqa::Handle*>(handle);
  return 0;
}

// ------------------------------------------------------------------------------------------
// Paged GQA decode without any allocation.
//
// Some hosts of this library may not call the CUDA allocator at all: a serving process whose own
// pool already owns the whole of device memory (a cudaMalloc there fails or fragments the pool),
// a plug-in sandbox that forbids allocator calls from plug-in code, or a latency-critical loop that
// cannot afford the device-wide synchronisation an allocation may imply.  They also cannot hand us
// a workspace they do not have.  For them the work list, the counters and the split-KV partial
// results live in the fixed array below, which is part of the library image: every GPU that loads
// the library carries these 16 MiB until the process exits, whether or not the entry point is ever
// called.
//
// All calls share the array and nothing clears it between calls: the plan kernel of a call
// rewrites the counters and the work list before the decode kernel of the same call
// reads them, and a partial result is read only after the same call has written it, so stale
// contents are never consumed and nothing needs to start at zero.  Two calls that overlap on the
// GPU (different streams, or different host threads) race on it -- serialise them.
// ------------------------------------------------------------------------------------------
namespace cake {
namespace gqa {

constexpr size_t kNoAllocScratchBytes = size_t(16) << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

constexpr int kMaxDevices = 64;
static std::mutex g_noalloc_mutex;
static void* g_noalloc_address[kMaxDevices];     // DEVICE address of g_noalloc_scratch on each device
static bool g_noalloc_ready[kMaxDevices];

// In host code the name `g_noalloc_scratch` is only a handle for the runtime, not an address a
// kernel can use; the device address is asked for once per device, with that device current.
static int noalloc_setup(int device, void** address) {
  if (device < 0 || device >= kMaxDevices) return kErrBadArgument;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_ready[device]) {
    void* ptr = nullptr;
    cudaError_t err = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (err != cudaSuccess) return int(err);
    if (!ptr) return int(cudaErrorInvalidSymbol);
    err = cudaFuncSetAttribute(gqa_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (err != cudaSuccess) return int(err);
    g_noalloc_address[device] = ptr;
    g_noalloc_ready[device] = true;
  }
  *address = g_noalloc_address[device];
  return 0;
}

}  // namespace gqa
}  // namespace cake

extern "C" size_t cake_b200_gqa_decode_noalloc_scratch_limit(void) { return cake::gqa::kNoAllocScratchBytes; }

extern "C" int cake_b200_gqa_decode_noalloc(void** buffers, const cake_b200_gqa_decode_config* config, void* cuda_stream) {
  using namespace cake;
  if (!buffers || !config) return kErrBadArgument;
  int device = 0;
  if (int rc = require_blackwell(&device)) return rc;
  if (!gqa_config_ok(*config)) return kErrBadArgument;
  gqa::Params p;
  if (int rc = gqa::fill_params(p, buffers, *config)) return rc;
  if (p.batch == 0) return 0;
  int sms = 0;
  if (int rc = gqa_sm_count(device, &sms)) return rc;
  if (sms > gqa::kMaxSms) sms = gqa::kMaxSms;
  // The work list, the counters and one partial result per (token range, sequence) piece must fit.
  const size_t entries = gqa::entries_for(*config, sms);
  if (gqa::scratch_bytes(*config, entries) > gqa::kNoAllocScratchBytes) return kErrWorkspace;   // batch * heads too large for 16 MiB
  p.capacity = int(entries);
  void* scratch = nullptr;
  if (int rc = gqa::noalloc_setup(device, &scratch)) return rc;
  gqa::carve_scratch(p, static_cast<uint8_t*>(scratch));
  return gqa::launch(p, sms, reinterpret_cast<cudaStream_t>(cuda_stream));
}

// ------------------------------------------------------------------------------------------
// Causal prefill (paged or ragged K/V): see prefill.cuh.
namespace cake {
namespace gqa {
struct PrefillHandle {
  int device, sms;
  Params p;
  const int *qo_indptr, *kv_indptr_segments, *last_page_len;
  int *seq_start, *seq_tokens, *masked;
  int segments, total_q, kv_unit, nan_for_masked;
};
}  // namespace gqa
}  // namespace cake

static bool gqa_prefill_config_ok(const cake_b200_gqa_prefill_config& c, cake_b200_gqa_decode_config* as_decode) {
  if (c.total_q < 0 || c.total_q > 65535 || c.segments <= 0 || c.segments > 65535) return false;
  cake_b200_gqa_decode_config d{};
  d.batch = c.total_q;
  d.num_qo_heads = c.num_qo_heads;
  d.num_kv_heads = c.num_kv_heads;
  d.head_dim = c.head_dim;
  d.page_size = c.ragged ? 1 : c.page_size;
  d.max_kv_len = c.max_kv_len;
  *as_decode = d;
  return gqa_config_ok(d);
}

extern "C" size_t cake_b200_gqa_prefill_workspace_bytes(const cake_b200_gqa_prefill_config* c) {
  cake_b200_gqa_decode_config d;
  if (!c || !gqa_prefill_config_ok(*c, &d)) return 0;
  return cake_b200_gqa_decode_workspace_bytes(&d) + cake::prefill::table_bytes(c->total_q);
}

extern "C" int cake_b200_gqa_prefill_create(void** buffers, const cake_b200_gqa_prefill_config* config, void** handle_out) {
  using namespace cake;
  if (!buffers || !config || !handle_out) return kErrBadArgument;
  *handle_out = nullptr;
  int device = 0;
  if (int rc = require_blackwell(&device)) return rc;
  cake_b200_gqa_decode_config d;
  if (!gqa_prefill_config_ok(*config, &d)) return kErrBadArgument;
  // buffers: q, k, v, qo_indptr, kv_indptr, kv_indices, kv_last_page_len, sm_scale, output, lse, workspace;
  // ragged K/V: kv_indices and kv_last_page_len are null
  for (int i = 0; i < 11; ++i) {
    const bool optional = i == 6 || (config->ragged && i == 5);
    if (!buffers[i] && !optional) return kErrBadArgument;
    if (i <= 2 && (reinterpret_cast<uintptr_t>(buffers[i]) & 15)) return kErrBadArgument;
  }
  if (config->ragged && (buffers[5] || buffers[6])) return kErrBadArgument;
  if (reinterpret_cast<uintptr_t>(buffers[10]) & 3) return kErrBadArgument;
  auto* h = new (std::nothrow) gqa::PrefillHandle;
  if (!h) return int(cudaErrorMemoryAllocation);
  h->device = device;
  gqa::Params& p = h->p;
  void* as_decode[9] = {buffers[0], buffers[1], buffers[2], buffers[4], buffers[5] ? buffers[5] : buffers[4], buffers[6] ? buffers[6] : buffers[4],
                        buffers[7], buffers[8], buffers[9]};
  if (int rc = gqa::fill_params(p, as_decode, d)) { delete h; return rc; }
  p.kv_indices = static_cast<const int*>(buffers[5]);              // null: identity page list (ragged)
  p.kv_last_page_len = nullptr;                                    // lengths come from the sequence table
  p.capacity = int(gqa::entries_for(d, gqa::kMaxSms));
  p.status = static_cast<int*>(buffers[10]);
  uint8_t* ws = static_cast<uint8_t*>(buffers[10]) + 256;
  ws += (256 - (reinterpret_cast<uintptr_t>(ws) & 255)) & 255;
  const size_t table = prefill::table_bytes(config->total_q) / 3;
  h->seq_start = reinterpret_cast<int*>(ws);
  h->seq_tokens = reinterpret_cast<int*>(ws + table);
  h->masked = reinterpret_cast<int*>(ws + 2 * table);
  gqa::carve_scratch(p, ws + 3 * table);
  p.seq_start = h->seq_start;
  p.seq_tokens = h->seq_tokens;
  h->qo_indptr = static_cast<const int*>(buffers[3]);
  h->kv_indptr_segments = static_cast<const int*>(buffers[4]);
  h->last_page_len = static_cast<const int*>(buffers[6]);
  h->segments = config->segments;
  h->total_q = int(config->total_q);
  h->kv_unit = d.page_size;
  h->nan_for_masked = config->nan_for_masked;
  int sms = 0;
  int rc = gqa_sm_count(device, &sms);
  if (!rc) rc = int(cudaFuncSetAttribute(gqa::gqa_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gqa::kSmemBytes));
  if (rc) { delete h; return rc; }
  h->sms = sms < gqa::kMaxSms ? sms : gqa::kMaxSms;
  *handle_out = h;
  return 0;
}

extern "C" int cake_b200_gqa_prefill_launch(void* handle, void* cuda_stream) {
  using namespace cake;
  if (!handle) return kErrBadArgument;
  auto* h = static_cast<gqa::PrefillHandle*>(handle);
  int device = -1;
  CAKE_CUDA_OK(cudaGetDevice(&device));
  if (device != h->device) return kErrWrongDevice;
  if (h->total_q == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(cuda_stream);
  prefill::prefill_plan_kernel<<<(h->total_q + 255) / 256, 256, 0, s>>>(h->qo_indptr, h->kv_indptr_segments, h->last_page_len, h->segments,
                                                                       h->kv_unit, h->total_q, h->seq_start, h->seq_tokens, h->masked);
  gqa::Params p = h->p;
  if (int rc = gqa::launch(p, h->sms, s)) return rc;
  if (h->nan_for_masked)
    prefill::prefill_mark_kernel<<<(h->total_q + 7) / 8, 256, 0, s>>>(h->masked, h->total_q, p.out, p.hq * gqa::kD);
  return int(cudaGetLastError());
}

extern "C" int cake_b200_gqa_prefill_destroy(void* handle) {
  delete static_cast<cake::gqa::PrefillHandle*>(handle);
  return 0;
}
