// Paged MLA decode (absorbed form) for sm_100a: split-KV flash-decode + reduce.
//
// Operator: src/open_cake_ir/tasks/solx_fib/attention.py:132-183, MLA branch (:164-165,
// :175-177); tensor ABI attention_specs.py:249-292.  All query heads share one latent KV row of
// 512 (ckv) + 64 (kpe) bf16 per token:  logits = (ckv . q_nope + kpe . q_pe) * scale,
// out = bf16(softmax(logits) ckv), lse base 2.
//
// A CTA owns (64 query heads, sequence, KV chunk) and streams the chunk's latent rows once
// through a three-stage cp.async ring of 32-token tiles (576 bf16 per row, XOR-swizzled);
// the two head blocks of a sequence are adjacent CTAs, so the second reads the rows from L2.
// Eight warps: warp w works on heads 16*(w%4).. and on output dims 256*(w/4)...  Q stays in
// shared memory for the whole CTA; S = Q K^T and O += P V are m16n8k16 bf16 MMAs fed by
// ldmatrix, with the online softmax (base 2) in registers between them.
#include "common.cuh"
#include "../../include/cake_b200.h"
#include <new>

namespace cake {
namespace mla {

constexpr int kCkv = 512, kKpe = 64, kRow = kCkv + kKpe;   // 576 elements per latent row
constexpr int kRowBytes = kRow * 2;                        // 1152
constexpr int kRowChunks = kRowBytes / 16;                 // 72
constexpr int kHeads = 64;                                 // query heads per CTA
constexpr int kTile = 32;                                  // tokens per tile
constexpr int kRing = 3;
constexpr int kThreads = 256;
constexpr int kQBytes = kHeads * kRowBytes;                // 73 728
constexpr int kTileBytes = kTile * kRowBytes;              // 36 864
constexpr int kSmemBytes = kQBytes + kRing * kTileBytes;   // 184 320
constexpr float kLog2e = 1.4426950408889634f;

struct Params {
  const __nv_bfloat16 *q_nope, *q_pe, *ckv, *kpe;
  const int *kv_indptr, *kv_indices, *kv_last_page_len;
  const float* sm_scale;
  __nv_bfloat16* out;     // [B, H, 512]
  float* lse;             // [B, H]
  float* part_o;          // [B, splits, H, 512]
  float* part_lse;        // [B, splits, H]
  int batch, heads, page_size, chunk, max_splits;
};

__device__ __forceinline__ int seq_len(const Params& p, int b) {
  const int pages = p.kv_indptr[b + 1] - p.kv_indptr[b];
  return pages <= 0 ? 0 : (pages - 1) * p.page_size + p.kv_last_page_len[b];
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
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
// Byte offset of (row, 16-byte chunk) in a swizzled tile of 1152-byte rows (72 chunks; the XOR
// stays inside a group of eight chunks).
__device__ __forceinline__ uint32_t row_off(int row, int chunk) {
  return uint32_t(row * kRowBytes + ((chunk ^ (row & 7)) << 4));
}

__device__ __forceinline__ void load_tile(const Params& p, int b, int tok0, int len, uint32_t dst) {
  const int page_base = p.kv_indptr[b];
  for (int idx = threadIdx.x; idx < kTile * kRowChunks; idx += kThreads) {
    const int row = idx / kRowChunks, chunk = idx % kRowChunks;
    const int tok = tok0 + row;
    const bool valid = tok < len;
    const int t = valid ? tok : 0;
    const int page = __ldg(p.kv_indices + page_base + t / p.page_size);
    const size_t slot = size_t(page) * p.page_size + (t % p.page_size);
    const __nv_bfloat16* src = chunk < kCkv / 8 ? p.ckv + slot * kCkv + chunk * 8 : p.kpe + slot * kKpe + (chunk - kCkv / 8) * 8;
    cp_async_16(dst + row_off(row, chunk), src, valid);
  }
}

__global__ void __launch_bounds__(kThreads, 1)
mla_decode_kernel(const Params p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int hb = blockIdx.x, split = blockIdx.y, b = blockIdx.z;
  const int len = seq_len(p, b);
  const int begin = split * p.chunk;
  if (begin >= len) return;
  const int end = min(len, begin + p.chunk);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hg = warp & 3, dh = warp >> 2;
  const int row = lane >> 2, quad = lane & 3;
  const float scale2 = __ldg(p.sm_scale) * kLog2e;
  const uint32_t q_smem = smem_u32(smem);
  const uint32_t ring = q_smem + kQBytes;
  const int head0 = hb * kHeads;

  // Q block -> shared memory (rows beyond the head count are zero-filled)
  for (int idx = threadIdx.x; idx < kHeads * kRowChunks; idx += kThreads) {
    const int r = idx / kRowChunks, chunk = idx % kRowChunks;
    const int head = head0 + r;
    const bool valid = head < p.heads;
    const size_t hrow = size_t(b) * p.heads + (valid ? head : 0);
    const __nv_bfloat16* src = chunk < kCkv / 8 ? p.q_nope + hrow * kCkv + chunk * 8 : p.q_pe + hrow * kKpe + (chunk - kCkv / 8) * 8;
    cp_async_16(q_smem + row_off(r, chunk), src, valid);
  }
  const int tiles = (end - begin + kTile - 1) / kTile;
#pragma unroll
  for (int s = 0; s < kRing - 1; ++s) {
    if (s < tiles) load_tile(p, b, begin + s * kTile, end, ring + s * kTileBytes);
    cp_async_commit();      // the first group also carries Q
  }

  float o[32][4];
#pragma unroll
  for (int n = 0; n < 32; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // rows `row` and `row + 8` of this warp's 16 heads
  const int mi = lane >> 3, lr = lane & 7;

  for (int i = 0; i < tiles; ++i) {
    cp_async_wait<kRing - 2>();
    __syncthreads();                 // tile i visible to all; everyone is done with tile i-1
    {
      const int next = i + kRing - 1;
      if (next < tiles) load_tile(p, b, begin + next * kTile, end, ring + (next % kRing) * kTileBytes);
      cp_async_commit();
    }
    const uint32_t kv = ring + (i % kRing) * kTileBytes;
    const int tok0 = begin + i * kTile;

    // S[16 heads x 32 tokens] over the 576-wide latent row
    float s[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll 4
    for (int ks = 0; ks < kRow / 16; ++ks) {
      uint32_t a0, a1, a2, a3;
      // A: matrices (rows 0-7 | 8-15) x (k 0-7 | 8-15) of this warp's 16 heads
      ldmatrix_x4(q_smem + row_off(hg * 16 + (mi & 1) * 8 + lr, ks * 2 + (mi >> 1)), a0, a1, a2, a3);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(kv + row_off(half * 16 + (mi >> 1) * 8 + lr, ks * 2 + (mi & 1)), b0, b1, b2, b3);
        mma_bf16_16816(s[half * 2], a0, a1, a2, a3, b0, b1);
        mma_bf16_16816(s[half * 2 + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    // online softmax; lane holds tokens tok0 + n*8 + quad*2 + {0,1} of rows `row` (c0,c1) and `row+8` (c2,c3)
    float tmax0 = -INFINITY, tmax1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < 4; ++n) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const bool valid = tok0 + n * 8 + quad * 2 + j < end;
        s[n][j] = valid ? s[n][j] * scale2 : -INFINITY;
        s[n][2 + j] = valid ? s[n][2 + j] * scale2 : -INFINITY;
        tmax0 = fmaxf(tmax0, s[n][j]);
        tmax1 = fmaxf(tmax1, s[n][2 + j]);
      }
    }
    tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 1));
    tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 2));
    tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 1));
    tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 2));
    const float n0 = fmaxf(m0, tmax0), n1 = fmaxf(m1, tmax1);
    const float alpha0 = exp2f(m0 - n0), alpha1 = exp2f(m1 - n1);
    m0 = n0; m1 = n1;
    float sum0 = 0.f, sum1 = 0.f;
    uint32_t pa[4][2], pb[4][2];   // P as bf16 pairs, value and rounding residual: [n-tile][row | row+8]
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const float p0 = exp2f(s[n][0] - n0), p1 = exp2f(s[n][1] - n0);
      const float p2 = exp2f(s[n][2] - n1), p3 = exp2f(s[n][3] - n1);
      sum0 += p0 + p1; sum1 += p2 + p3;
      split_bf16x2(p0, p1, pa[n][0], pb[n][0]);
      split_bf16x2(p2, p3, pa[n][1], pb[n][1]);
    }
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1); sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1); sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
    l0 = l0 * alpha0 + sum0;
    l1 = l1 * alpha1 + sum1;
#pragma unroll
    for (int n = 0; n < 32; ++n) { o[n][0] *= alpha0; o[n][1] *= alpha0; o[n][2] *= alpha1; o[n][3] *= alpha1; }
    // O[16 heads x 256 dims] += P[16 x 32] V[32 x 256]; V = the ckv part of the same tile
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
      for (int np = 0; np < 16; ++np) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(kv + row_off(ks * 16 + (mi & 1) * 8 + lr, dh * 32 + np * 2 + (mi >> 1)), b0, b1, b2, b3);
        mma_bf16_16816(o[np * 2], pa[ks * 2][0], pa[ks * 2][1], pa[ks * 2 + 1][0], pa[ks * 2 + 1][1], b0, b1);
        mma_bf16_16816(o[np * 2], pb[ks * 2][0], pb[ks * 2][1], pb[ks * 2 + 1][0], pb[ks * 2 + 1][1], b0, b1);
        mma_bf16_16816(o[np * 2 + 1], pa[ks * 2][0], pa[ks * 2][1], pa[ks * 2 + 1][0], pa[ks * 2 + 1][1], b2, b3);
        mma_bf16_16816(o[np * 2 + 1], pb[ks * 2][0], pb[ks * 2][1], pb[ks * 2 + 1][0], pb[ks * 2 + 1][1], b2, b3);
      }
    }
  }
  cp_async_wait<0>();

  // partial results: normalised output and base-2 log-sum-exp of this chunk
  const float inv0 = 1.f / l0, inv1 = 1.f / l1;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int head = head0 + hg * 16 + row + half * 8;
    if (head < p.heads) {
      const size_t slot = (size_t(b) * p.max_splits + split) * p.heads + head;
      float* dst = p.part_o + slot * kCkv + dh * 256 + quad * 2;
      const float inv = half ? inv1 : inv0;
#pragma unroll
      for (int n = 0; n < 32; ++n)
        *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][half * 2] * inv, o[n][half * 2 + 1] * inv);
      if (dh == 0 && quad == 0) p.part_lse[slot] = (half ? m1 : m0) + log2f(half ? l1 : l0);
    }
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
  const long long head_blocks = (c.num_qo_heads + kHeads - 1) / kHeads;
  const long long max_len = c.max_kv_len > 0 ? c.max_kv_len : 1;
  int chunk = 4096;
  while (chunk > 128 && c.batch * head_blocks * ((max_len * 5 / 8 + chunk - 1) / chunk) < 2LL * sms) chunk >>= 1;
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
  uint8_t* ws = static_cast<uint8_t*>(buffers[10]) + 256;
  p.part_o = reinterpret_cast<float*>(ws);
  p.part_lse = p.part_o + size_t(p.batch) * p.max_splits * p.heads * mla::kCkv;
  int rc = int(cudaFuncSetAttribute(mla::mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, mla::kSmemBytes));
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
  const int head_blocks = (p.heads + mla::kHeads - 1) / mla::kHeads;
  mla::mla_decode_kernel<<<dim3(head_blocks, p.max_splits, p.batch), mla::kThreads, mla::kSmemBytes, s>>>(p);
  mla::mla_reduce_kernel<<<dim3(p.heads, p.batch), 128, 0, s>>>(p);
  return int(cudaGetLastError());
}

extern "C" int cake_b200_mla_decode_destroy(void* handle) {
  delete static_cast<cake::mla::Handle*>(handle);
  return 0;
}
