// Paged MLA decode (absorbed form) for sm_100a: split-KV flash-decode on tcgen05 + reduce.
//
// Operator: src/open_cake_ir/tasks/solx_fib/attention.py:132-183, MLA branch (:164-165,
// :175-177); tensor ABI attention_specs.py:249-292.  All query heads share one latent KV row of
// 512 (ckv) + 64 (kpe) bf16 per token:  logits = (ckv . q_nope + kpe . q_pe) * scale,
// out = bf16(softmax(logits) ckv), lse base 2.
//
// At 128 heads the operator does 242 flop per byte of latent cache, which is the bf16 ridge of the
// machine, so both contractions run on the tensor core.  A CTA owns (128 heads, one half of the 512
// output dims, sequence, KV chunk); the two halves of a chunk are neighbouring CTAs, so the second
// reads the latent rows from L2.  The 128 heads are the 128 TMEM lanes:
//   S[128 x 32 tokens]  = Q[128 x 576] . KV_tile^T      Q and the tile K-major in shared memory
//   O[128 x 256 dims]  += P[128 x 32] . V[32 x 256]     P from tensor memory, V = the same tile read
//                                                        MN-major (no transposed copy is made)
// Q (147 KiB, nine 64-column slabs of 128-byte rows, 128-byte swizzle) stays in shared memory for
// the whole CTA (its size is what limits the ring to two stages); 32-token tiles stream through a
// two-stage cp.async ring in the same slab layout
// (the gather is per token, so any page size works).  Four softmax warps own one head row each per
// thread: they read S from TMEM, keep the running max and sum in base 2, and write P back to TMEM
// as TWO bf16 terms (value + rounding residual; one term is not accurate enough for the
// contract's tolerance).  The running max only moves when it grows by more than 2^8, so O is
// rescaled in TMEM rarely.  Every wait is bounded and reports through the status word.
#include "common.cuh"
#include "../../include/cake_b200.h"
#include <new>

namespace cake {
namespace mla {

constexpr int kCkv = 512, kKpe = 64, kRow = kCkv + kKpe;   // 576 elements per latent row
constexpr int kSlabs = kRow / 64;                          // 9 slabs of 64 columns (128 bytes per row)
constexpr int kRowChunks = kRow / 8;                       // 72 16-byte chunks per row
constexpr int kHeads = 128;                                // query heads per CTA = TMEM lanes
constexpr int kDimsPerCta = 256;                           // output dims per CTA (half of ckv)
constexpr int kTile = 32;                                  // tokens per tile
constexpr int kStages = 2;
constexpr int kQSlabBytes = kHeads * 128;                  // 16 KiB
constexpr int kQBytes = kSlabs * kQSlabBytes;              // 147 456
constexpr int kKvSlabBytes = kTile * 128;                  // 4 KiB
constexpr int kKvStageBytes = kSlabs * kKvSlabBytes;       // 36 864
constexpr int kLoaderWarps = 2, kLoaderThreads = kLoaderWarps * 32;
constexpr int kMmaWarp = 2;
constexpr int kSoftmaxWarp0 = 4;                           // warps 4..7: warp % 4 = TMEM lane quadrant
constexpr int kThreads = 256;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.f;                   // log2 units
// tensor-memory columns
constexpr uint32_t kColO = 0, kColS = 256, kColP = 320, kTmemColumns = 512;

struct Params {
  const __nv_bfloat16 *q_nope, *q_pe, *ckv, *kpe;
  const int *kv_indptr, *kv_indices, *kv_last_page_len;
  const float* sm_scale;
  __nv_bfloat16* out;     // [B, H, 512]
  float* lse;             // [B, H]
  float* part_o;          // [B, splits, H, 512]
  float* part_lse;        // [B, splits, H]
  int* status;
  int batch, heads, page_size, chunk, max_splits;
};

struct Shared {
  uint64_t kv_full[kStages], kv_empty[kStages];
  uint64_t s_full[2], s_free[2], p_ready[2], pv_done[2];
  uint32_t tmem_base;
  int abort_flag;
};

constexpr size_t kSmemBytes = size_t(kQBytes) + kStages * kKvStageBytes + sizeof(Shared) + 1024;

__device__ __forceinline__ int seq_len(const Params& p, int b) {
  const int pages = p.kv_indptr[b + 1] - p.kv_indptr[b];
  return pages <= 0 ? 0 : (pages - 1) * p.page_size + p.kv_last_page_len[b];
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;      // 0 source bytes = zero fill
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Byte offset of 16-byte chunk `chunk` (0..71) of row `row` in a slab-major tile whose slabs hold
// `rows` rows of 128 bytes with the 128-byte swizzle (chunk index XOR row mod 8).
__device__ __forceinline__ uint32_t slab_off(int rows, int row, int chunk) {
  return uint32_t((chunk >> 3) * rows * 128 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

// One 32-token tile of latent rows -> one ring stage, by the two loader warps.  A warp takes 16
// rows; its lanes cover consecutive 16-byte chunks of one row at a time (coalesced 512-byte reads),
// and the page of each row is looked up once per tile by one lane and passed round by shuffle.
__device__ __forceinline__ void load_tile(const Params& p, int b, int tok0, int len, uint32_t dst, int loader_tid) {
  const int w = loader_tid >> 5, lane = loader_tid & 31;
  const int my_tok = tok0 + w * 16 + (lane & 15);
  const bool my_valid = my_tok < len;
  const int t = my_valid ? my_tok : 0;
  const int page = __ldg(p.kv_indices + p.kv_indptr[b] + t / p.page_size);
  const long long my_slot = (long long)page * p.page_size + (t % p.page_size);
#pragma unroll
  for (int rr = 0; rr < 16; ++rr) {
    const int row = w * 16 + rr;
    const long long slot = __shfl_sync(0xffffffffu, my_slot, rr);
    const bool valid = __shfl_sync(0xffffffffu, int(my_valid), rr) != 0;
    const __nv_bfloat16* ckv_row = p.ckv + slot * kCkv;
    cp_async_16(dst + slab_off(kTile, row, lane), ckv_row + lane * 8, valid);
    cp_async_16(dst + slab_off(kTile, row, 32 + lane), ckv_row + (32 + lane) * 8, valid);
    if (lane < kKpe / 8) cp_async_16(dst + slab_off(kTile, row, kCkv / 8 + lane), p.kpe + slot * kKpe + lane * 8, valid);
  }
}

__global__ void __launch_bounds__(kThreads, 1)
mla_decode_kernel(const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const int dh = blockIdx.x & 1, hb = blockIdx.x >> 1, split = blockIdx.y, b = blockIdx.z;
  const int len = seq_len(p, b);
  const int begin = split * p.chunk;
  if (begin >= len) return;
  const int end = min(len, begin + p.chunk);
  const int tiles = (end - begin + kTile - 1) / kTile;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t q_addr = smem_u32(base);
  const uint32_t kv_addr = q_addr + kQBytes;
  Shared* sh = reinterpret_cast<Shared*>(base + kQBytes + kStages * kKvStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head0 = hb * kHeads;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&sh->kv_full[s], kLoaderThreads); mbar_init(&sh->kv_empty[s], 1); }
    for (int j = 0; j < 2; ++j) {
      mbar_init(&sh->s_full[j], 1); mbar_init(&sh->s_free[j], 4);
      mbar_init(&sh->p_ready[j], 4); mbar_init(&sh->pv_done[j], 1);
    }
    sh->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(&sh->tmem_base, kTmemColumns);
    tmem_relinquish();
  }
  // the loader warps start the first tile before anything else so that it travels with the Q block
  if (warp < kLoaderWarps) load_tile(p, b, begin, end, kv_addr, threadIdx.x);
  // Q block -> shared memory, slab-major and swizzled like a TMA box would leave it
  for (int idx = threadIdx.x; idx < kHeads * kRowChunks; idx += kThreads) {
    const int r = idx / kRowChunks, chunk = idx % kRowChunks;
    const int head = head0 + r;
    const bool valid = head < p.heads;
    const size_t hrow = size_t(b) * p.heads + (valid ? head : 0);
    const __nv_bfloat16* src = chunk < kCkv / 8 ? p.q_nope + hrow * kCkv + chunk * 8 : p.q_pe + hrow * kKpe + (chunk - kCkv / 8) * 8;
    cp_async_16(q_addr + slab_off(kHeads, r, chunk), src, valid);
  }
  cp_async_commit();
  cp_async_wait<0>();
  fence_proxy_async_smem();
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  volatile int* abort_flag = &sh->abort_flag;

  if (warp < kLoaderWarps) {
    // ------------------------------ loader --------------------------------------------
    bool ok = true;
    for (int i = 0; ok && i < tiles; ++i) {
      const int s = i % kStages;
      ok = mbar_wait(&sh->kv_empty[s], ((i / kStages) & 1) ^ 1, abort_flag, p.status, kStatusWaitSmemEmpty);
      if (!ok) break;
      if (i > 0) {               // tile 0 was issued, and has landed, with the Q block
        load_tile(p, b, begin + i * kTile, end, kv_addr + s * kKvStageBytes, threadIdx.x);
        cp_async_commit();
        cp_async_wait<0>();
      }
      fence_proxy_async_smem();
      mbar_arrive(&sh->kv_full[s]);
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------ MMA issuer ----------------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc_qk = umma_idesc_ex(1 /* bf16 */, kHeads, kTile, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_ex(1 /* bf16 */, kHeads, kDimsPerCta, 0, 1 /* V is MN-major */);
      bool ok = true;
      for (int i = 0; ok && i <= tiles; ++i) {
        // PV of the previous tile goes first: it is what releases that tile's ring stage, and with
        // two stages the loader needs it back before it can fetch tile i+1.
        if (i >= 1) {             // O += P(i-1) . V(i-1), P as two bf16 terms
          const int t = i - 1, s = t % kStages, j = t & 1;
          ok = mbar_wait(&sh->p_ready[j], (t >> 1) & 1, abort_flag, p.status, kStatusWaitFlag);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t v_addr = kv_addr + s * kKvStageBytes + dh * (kDimsPerCta / 64) * kKvSlabBytes;
#pragma unroll
          for (int term = 0; term < 2; ++term) {
#pragma unroll
            for (int ks = 0; ks < kTile / 16; ++ks) {
              const uint32_t a_tmem = tmem_base + kColP + j * kTile + term * (kTile / 2) + ks * 8;
              // 16 tokens = two 8-row groups of 1024 bytes; the next 64 dims are one slab further
              const uint64_t b_desc = umma_desc_sw128_ex(v_addr + ks * 2048, kKvSlabBytes, 1024);
              umma_f16_a_tmem(tmem_base + kColO, a_tmem, b_desc, idesc_pv, (t | term | ks) != 0);
            }
          }
          tcgen05_commit(&sh->pv_done[j]);
          tcgen05_commit(&sh->kv_empty[s]);
        }
        if (i < tiles) {          // S(i) = Q . tile(i)^T
          const int s = i % kStages, j = i & 1;
          ok = mbar_wait(&sh->kv_full[s], (i / kStages) & 1, abort_flag, p.status, kStatusWaitSmemFull) &&
               mbar_wait(&sh->s_free[j], ((i >> 1) & 1) ^ 1, abort_flag, p.status, kStatusWaitTmemEmpty);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t tile_addr = kv_addr + s * kKvStageBytes;
#pragma unroll 1
          for (int slab = 0; slab < kSlabs; ++slab) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const uint64_t a_desc = umma_desc_sw128(q_addr + slab * kQSlabBytes + kk * 32);
              const uint64_t b_desc = umma_desc_sw128(tile_addr + slab * kKvSlabBytes + kk * 32);
              umma_f16(tmem_base + kColS + j * kTile, a_desc, b_desc, idesc_qk, (slab | kk) != 0);
            }
          }
          tcgen05_commit(&sh->s_full[j]);
        }
      }
    }
  } else if (warp >= kSoftmaxWarp0) {
    // ------------------------------ softmax / epilogue --------------------------------
    const int quad = warp & 3;
    const int r = quad * 32 + lane;                 // head row of this thread
    const uint32_t lane_base = tmem_base + (uint32_t(quad * 32) << 16);
    const float scale2 = __ldg(p.sm_scale) * kLog2e;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int i = 0; ok && i < tiles; ++i) {
      const int j = i & 1;
      ok = mbar_wait(&sh->s_full[j], (i >> 1) & 1, abort_flag, p.status, kStatusWaitTmemFull);
      if (!ok) break;
      tcgen05_fence_after();
      float sc[kTile];
      tmem_ld_32x32b_x32(lane_base + kColS + j * kTile, sc);
      tcgen05_wait_ld();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->s_free[j]);
      const int tok0 = begin + i * kTile;
      float tmax = -INFINITY;
#pragma unroll
      for (int c = 0; c < kTile; ++c) {
        sc[c] = tok0 + c < end ? sc[c] * scale2 : -INFINITY;
        tmax = fmaxf(tmax, sc[c]);
      }
      if (i == 0) {
        m_ref = tmax;                                // finite: the first tile holds a valid token
      } else {
        const bool need = tmax > m_ref + kRescaleThreshold;
        if (__any_sync(0xffffffffu, need)) {
          // O is about to be rescaled in tensor memory: the PV of the previous tile must have landed
          ok = mbar_wait(&sh->pv_done[(i - 1) & 1], ((i - 1) >> 1) & 1, abort_flag, p.status, kStatusWaitFlag);
          if (!ok) break;
          tcgen05_fence_after();
          const float alpha = need ? exp2f(m_ref - tmax) : 1.f;
          if (need) { m_ref = tmax; l *= alpha; }
#pragma unroll 1
          for (int c = 0; c < kDimsPerCta; c += 32) {
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
      if (i >= 2) {              // the P buffer is free once the PV that read it has completed
        ok = mbar_wait(&sh->pv_done[j], ((i - 2) >> 1) & 1, abort_flag, p.status, kStatusWaitFlag);
        if (!ok) break;
      }
      uint32_t hi[kTile / 2], lo[kTile / 2];
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < kTile; c += 2) {
        const float p0 = exp2f(sc[c] - m_ref), p1 = exp2f(sc[c + 1] - m_ref);
        sum += p0 + p1;
        split_bf16x2(p0, p1, hi[c >> 1], lo[c >> 1]);
      }
      l += sum;
      tmem_st_32x32b_x16(lane_base + kColP + j * kTile, hi);
      tmem_st_32x32b_x16(lane_base + kColP + j * kTile + kTile / 2, lo);
      tcgen05_wait_st();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->p_ready[j]);
    }
    if (ok) ok = mbar_wait(&sh->pv_done[(tiles - 1) & 1], ((tiles - 1) >> 1) & 1, abort_flag, p.status, kStatusWaitFlag);
    if (ok) {
      tcgen05_fence_after();
      const int head = head0 + r;
      const float inv = 1.f / l;
      const size_t slot = (size_t(b) * p.max_splits + split) * p.heads + (head < p.heads ? head : 0);
      float* dst = p.part_o + slot * kCkv + dh * kDimsPerCta;
#pragma unroll 1
      for (int c = 0; c < kDimsPerCta; c += 32) {
        float o[32];
        tmem_ld_32x32b_x32(lane_base + kColO + c, o);
        tcgen05_wait_ld();
        if (head < p.heads) {
#pragma unroll
          for (int k = 0; k < 32; k += 4)
            *reinterpret_cast<float4*>(dst + c + k) = make_float4(o[k] * inv, o[k + 1] * inv, o[k + 2] * inv, o[k + 3] * inv);
        }
      }
      if (dh == 0 && head < p.heads) p.part_lse[slot] = m_ref + log2f(l);
    }
  }

  cp_async_wait<0>();
  tcgen05_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, kTmemColumns);
  }
}

// One CTA per (sequence, head): merges the chunks.  128 threads x 4 dims.
__global__ void __launch_bounds__(128)
mla_reduce_kernel(const Params p) {
  const int head = blockIdx.x, b = blockIdx.y;
  const int d = threadIdx.x * 4;
  const int len = seq_len(p, b);
  __nv_bfloat16* out = p.out + (size_t(b) * p.heads + head) * kCkv + d;
  if (len == 0) {
    *reinterpret_cast<uint2*>(out) = make_uint2(0u, 0u);
    if (threadIdx.x == 0) p.lse[size_t(b) * p.heads + head] = -INFINITY;
    return;
  }
  const int splits = (len + p.chunk - 1) / p.chunk;
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, p.part_lse[(size_t(b) * p.max_splits + s) * p.heads + head]);
  float total = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < splits; ++s) {
    const size_t slot = (size_t(b) * p.max_splits + s) * p.heads + head;
    const float w = exp2f(p.part_lse[slot] - mm);
    const float4 v = *reinterpret_cast<const float4*>(p.part_o + slot * kCkv + d);
    total += w;
    acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
  }
  const float inv = 1.f / total;
  *reinterpret_cast<uint2*>(out) = make_uint2(pack_bf16x2(acc.x * inv, acc.y * inv), pack_bf16x2(acc.z * inv, acc.w * inv));
  if (threadIdx.x == 0) p.lse[size_t(b) * p.heads + head] = mm + log2f(total);
}

struct Handle {
  int device;
  Params p;
};

inline int pick_chunk(const cake_b200_mla_decode_config& c, int sms) {
  // Few, long chunks keep the partial-output traffic (heads * 512 fp32 per chunk) small next to
  // the latent rows a chunk reads (1152 B per token); enough of them to fill the SMs.
  const long long head_blocks = 2LL * ((c.num_qo_heads + kHeads - 1) / kHeads);     // two dim halves per 128 heads
  const long long max_len = c.max_kv_len > 0 ? c.max_kv_len : 1;
  int chunk = 4096;
  while (chunk > 128 && c.batch * head_blocks * ((max_len * 5 / 8 + chunk - 1) / chunk) < 3LL * sms) chunk >>= 1;
  return chunk;
}

}  // namespace mla
}  // namespace cake

static bool mla_config_ok(const cake_b200_mla_decode_config& c) {
  return c.batch >= 0 && c.batch <= 65535 && c.num_qo_heads > 0 && c.num_qo_heads <= 65535 * 64 &&
         c.head_dim_ckv == cake::mla::kCkv && c.head_dim_kpe == cake::mla::kKpe && c.page_size > 0 && c.max_kv_len >= 0;
}

extern "C" size_t cake_b200_mla_decode_workspace_bytes(const cake_b200_mla_decode_config* c) {
  if (!c || !mla_config_ok(*c)) return 0;
  const int chunk = cake::mla::pick_chunk(*c, 148);
  const size_t splits = size_t((c->max_kv_len + chunk - 1) / chunk) + 1;
  const size_t slots = size_t(c->batch) * splits * c->num_qo_heads;
  return 256 + slots * (cake::mla::kCkv + 1) * sizeof(float) + 256;
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
  p.chunk = mla::pick_chunk(*config, 148);
  p.max_splits = int((config->max_kv_len + p.chunk - 1) / p.chunk) + 1;
  p.status = static_cast<int*>(buffers[10]);
  uint8_t* ws = static_cast<uint8_t*>(buffers[10]) + 256;
  p.part_o = reinterpret_cast<float*>(ws);
  p.part_lse = p.part_o + size_t(p.batch) * p.max_splits * p.heads * mla::kCkv;
  int rc = int(cudaFuncSetAttribute(mla::mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(mla::kSmemBytes)));
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
  const mla::Params& p = h->p;
  if (p.batch == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(cuda_stream);
  CAKE_CUDA_OK(cudaMemsetAsync(p.status, 0, sizeof(int), s));
  const int head_blocks = (p.heads + mla::kHeads - 1) / mla::kHeads;
  mla::mla_decode_kernel<<<dim3(2 * head_blocks, p.max_splits, p.batch), mla::kThreads, mla::kSmemBytes, s>>>(p);
  mla::mla_reduce_kernel<<<dim3(p.heads, p.batch), 128, 0, s>>>(p);
  return int(cudaGetLastError());
}

extern "C" int cake_b200_mla_decode_destroy(void* handle) {
  delete static_cast<cake::mla::Handle*>(handle);
  return 0;
}
