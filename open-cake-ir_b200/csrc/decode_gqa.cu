// Paged GQA decode for sm_100a: split-KV flash-decode + reduce.
//
// Operator: src/open_cake_ir/tasks/solx_fib/attention.py:132-183 (decode branch), tensor ABI
// attention_specs.py:44-84.  One query token per sequence; out = bf16(softmax(K q * scale) V),
// lse = logsumexp / ln 2; an empty sequence gives zeros and -inf.
//
// The kernel is bound by the HBM stream of K and V (2 * Hkv * D * 2 bytes per token) and never
// writes logits or probabilities to memory.  A CTA owns (sequence, KV chunk); each of its eight warps
// owns one KV head and runs its own cp.async ring over the chunk's 16-token tiles (128-bit copies, one 256-byte
// row per token and head, XOR-swizzled in shared memory), so there is no CTA-wide barrier in
// the main loop.  The G = Hq/Hkv query heads that share a KV head are the rows of an
// m16n8k16 bf16 MMA (rows beyond G are zero): S = Q K^T via ldmatrix on the K tile, online
// softmax in base 2 with warp shuffles, O += P V via ldmatrix.trans on the V tile (P as two bf16
// terms, so the weights keep ~16 significant bits).  Chunks are merged by a second small kernel.
#include "common.cuh"
#include "../../include/cake_b200.h"
#include <mutex>
#include <new>

namespace cake {
namespace gqa {

constexpr int kD = 128;                 // head dimension
constexpr int kTile = 16;               // tokens per warp tile
constexpr int kWarps = 8;                // one KV head per warp
constexpr int kRing = 3;                // cp.async stages per warp
constexpr int kTileBytes = kTile * kD * 2;          // 4 KiB for K, same for V
constexpr int kWarpSmem = kRing * 2 * kTileBytes;    // 24 KiB
constexpr int kSmemBytes = kWarps * kWarpSmem;       // 192 KiB per CTA, one CTA per SM
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
  float* part_o;                 // [B, splits, Hq, D] normalised partial outputs
  float* part_lse;               // [B, splits, Hq]   base-2 partial log-sum-exp
  int batch, hq, hkv, page_size, chunk, max_splits;
};

__device__ __forceinline__ int seq_len(const Params& p, int b) {
  const int pages = p.kv_indptr[b + 1] - p.kv_indptr[b];
  return pages <= 0 ? 0 : (pages - 1) * p.page_size + p.kv_last_page_len[b];
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;     // 0 source bytes = zero fill
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

// Byte offset of (token row, 16-byte chunk) inside a swizzled [16][256 B] tile.
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) { return uint32_t(row * 256 + ((chunk ^ (row & 7)) << 4)); }

// Issues the copies of one 16-token tile of K and V for one KV head.  Lane r (< 16) looks up the
// page of token r once and passes the row's element offset round by shuffle, so the page-table
// arithmetic (an integer division by the run-time page size) is done once per token, not per copy.
__device__ __forceinline__ void load_tile(const Params& p, int b, int kvh, int tok0, int len, uint32_t k_smem,
                                          uint32_t v_smem, int lane) {
  const int my_tok = tok0 + (lane & 15);
  const bool my_valid = my_tok < len;
  const int t = my_valid ? my_tok : 0;
  const int page = __ldg(p.kv_indices + p.kv_indptr[b] + t / p.page_size);
  const long long my_elem = (((long long)page * p.page_size + (t % p.page_size)) * p.hkv + kvh) * kD;
  const int chunk = lane & 15;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = (lane >> 4) + 2 * i;
    const long long elem = __shfl_sync(0xffffffffu, my_elem, row) + chunk * 8;
    const bool valid = __shfl_sync(0xffffffffu, int(my_valid), row) != 0;
    cp_async_16(k_smem + tile_off(row, chunk), p.k_cache + elem, valid);
    cp_async_16(v_smem + tile_off(row, chunk), p.v_cache + elem, valid);
  }
}

__global__ void __launch_bounds__(kWarps * 32, 1)
gqa_decode_kernel(const Params p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int split = blockIdx.x, b = blockIdx.z;
  const int len = seq_len(p, b);
  const int begin = split * p.chunk;
  if (begin >= len) return;
  const int end = min(len, begin + p.chunk);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Warp w of the CTA owns KV head blockIdx.y*8 + w and walks the whole chunk: the eight warps read
  // the eight heads' 256-byte pieces of the same tokens at about the same time, so the CTA streams
  // whole pages (page_size * Hkv * 256 B contiguous) instead of scattered 256-byte pieces.
  const int kvh = blockIdx.y * kWarps + warp;
  if (kvh >= p.hkv) return;
  const int group = p.hq / p.hkv;
  const int row = lane >> 2;          // query head inside the group held by this lane's MMA rows
  const int quad = lane & 3;
  const float scale2 = __ldg(p.sm_scale) * kLog2e;

  // Q fragments (A operand): rows = heads of the group, zero beyond it.
  uint32_t qa[8][2];
  {
    const __nv_bfloat16* qrow = p.q + (size_t(b) * p.hq + kvh * group + row) * kD;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qa[ks][0] = row < group ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + quad * 2) : 0u;
      qa[ks][1] = row < group ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + quad * 2) : 0u;
    }
  }
  float o[16][4];
#pragma unroll
  for (int n = 0; n < 16; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  float m = -INFINITY, l = 0.f;       // running max (base 2) and sum of this lane's head row

  const uint32_t ring = smem_u32(smem) + warp * kWarpSmem;
  const int my_tiles = (end - begin + kTile - 1) / kTile;
#pragma unroll
  for (int s = 0; s < kRing - 1; ++s) {
    if (s < my_tiles)
      load_tile(p, b, kvh, begin + s * kTile, end, ring + s * 2 * kTileBytes,
                ring + s * 2 * kTileBytes + kTileBytes, lane);
    cp_async_commit();
  }
  for (int i = 0; i < my_tiles; ++i) {
    cp_async_wait<kRing - 2>();
    __syncwarp();                     // tile i has landed; every lane is done with tile i-1
    {
      // the stage tile i-1 used is free: start the load that keeps kRing-1 tiles in flight
      const int next = i + kRing - 1;
      if (next < my_tiles)
        load_tile(p, b, kvh, begin + next * kTile, end, ring + (next % kRing) * 2 * kTileBytes,
                  ring + (next % kRing) * 2 * kTileBytes + kTileBytes, lane);
      cp_async_commit();
    }
    const int stage = i % kRing;
    const uint32_t k_smem = ring + stage * 2 * kTileBytes, v_smem = k_smem + kTileBytes;
    const int tok0 = begin + i * kTile;

    // S = Q K^T : two n-tiles of 8 tokens
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      uint32_t b0, b1, b2, b3;
      const int mi = lane >> 3;                         // which 8x8 matrix this lane addresses
      const int trow = (mi >> 1) * 8 + (lane & 7);
      ldmatrix_x4(k_smem + tile_off(trow, ks * 2 + (mi & 1)), b0, b1, b2, b3);
      mma_bf16_16816(s0, qa[ks][0], 0u, qa[ks][1], 0u, b0, b1);
      mma_bf16_16816(s1, qa[ks][0], 0u, qa[ks][1], 0u, b2, b3);
    }
    // this lane: row `row`, tokens tok0 + quad*2 + {0,1} (s0) and + 8 (s1)
    float v[4];
    v[0] = s0[0] * scale2; v[1] = s0[1] * scale2; v[2] = s1[0] * scale2; v[3] = s1[1] * scale2;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int tok = tok0 + quad * 2 + (j & 1) + (j >> 1) * 8;
      if (tok >= end) v[j] = -INFINITY;
    }
    float tmax = fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3]));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
    const float m_new = fmaxf(m, tmax);              // finite: every tile holds at least one valid token
    const float alpha = exp2f(m - m_new);
    float pr[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) pr[j] = exp2f(v[j] - m_new);
    float psum = pr[0] + pr[1] + pr[2] + pr[3];
    psum += __shfl_xor_sync(0xffffffffu, psum, 1);
    psum += __shfl_xor_sync(0xffffffffu, psum, 2);
    l = l * alpha + psum;
    m = m_new;
    // P enters the tensor core as two bf16 terms (value + rounding residual): a single bf16 term
    // would put 2^-9 relative error on every weight, more than the contract's tolerance allows
    // once the weighted values cancel.
    uint32_t pa0, pa2, pb0, pb2;
    split_bf16x2(pr[0], pr[1], pa0, pb0);             // tokens 0..7 of the tile  (A cols k..k+1)
    split_bf16x2(pr[2], pr[3], pa2, pb2);             // tokens 8..15             (A cols k+8..)
#pragma unroll
    for (int n = 0; n < 16; ++n) { o[n][0] *= alpha; o[n][1] *= alpha; }
    // O += P V : V^T fragments through ldmatrix.trans, 16 dims per instruction
#pragma unroll
    for (int np = 0; np < 8; ++np) {
      uint32_t b0, b1, b2, b3;
      const int mi = lane >> 3;
      const int trow = (mi & 1) * 8 + (lane & 7);       // matrices 0/1: tokens 0-7 / 8-15; 2/3: next 8 dims
      ldmatrix_x4_trans(v_smem + tile_off(trow, np * 2 + (mi >> 1)), b0, b1, b2, b3);
      mma_bf16_16816(o[np * 2], pa0, 0u, pa2, 0u, b0, b1);
      mma_bf16_16816(o[np * 2], pb0, 0u, pb2, 0u, b0, b1);
      mma_bf16_16816(o[np * 2 + 1], pa0, 0u, pa2, 0u, b2, b3);
      mma_bf16_16816(o[np * 2 + 1], pb0, 0u, pb2, 0u, b2, b3);
    }
  }
  cp_async_wait<0>();

  // partial result of this (sequence, KV head, chunk): normalised rows and base-2 log-sum-exp
  if (row < group) {
    const int head = kvh * group + row;
    const size_t slot = (size_t(b) * p.max_splits + split) * p.hq + head;
    const float inv = 1.f / l;
    float* dst = p.part_o + slot * kD + quad * 2;
#pragma unroll
    for (int n = 0; n < 16; ++n) *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][0] * inv, o[n][1] * inv);
    if (quad == 0) p.part_lse[slot] = m + log2f(l);
  }
}

// One CTA per (sequence, query head): merges the chunks' partial results.
__global__ void __launch_bounds__(kD)
gqa_reduce_kernel(const Params p) {
  const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const int len = seq_len(p, b);
  const size_t o_idx = (size_t(b) * p.hq + head) * kD + d;
  if (len == 0) {
    p.out[o_idx] = __float2bfloat16(0.f);
    if (d == 0) p.lse[size_t(b) * p.hq + head] = -INFINITY;
    return;
  }
  const int splits = (len + p.chunk - 1) / p.chunk;
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, p.part_lse[(size_t(b) * p.max_splits + s) * p.hq + head]);
  float total = 0.f, acc = 0.f;
  for (int s = 0; s < splits; ++s) {
    const size_t slot = (size_t(b) * p.max_splits + s) * p.hq + head;
    const float w = exp2f(p.part_lse[slot] - mm);
    total += w;
    acc += w * p.part_o[slot * kD + d];
  }
  p.out[o_idx] = __float2bfloat16(acc / total);
  if (d == 0) p.lse[size_t(b) * p.hq + head] = mm + log2f(total);
}

struct Handle {
  int device;
  Params p;
  int* status;      // first word of the workspace; this operator has no device-side waits, it stays 0
};

inline int pick_chunk(const cake_b200_gqa_decode_config& c, int sms) {
  // One CTA per SM; aim for several rounds of CTAs so that unequal sequence lengths even out.  A
  // chunk is a multiple of the 16-token tile.
  int chunk = 1024;
  const long long max_len = c.max_kv_len > 0 ? c.max_kv_len : 1;
  const long long head_blocks = (c.num_kv_heads + kWarps - 1) / kWarps;
  while (chunk > 64 && (long long)c.batch * head_blocks * ((max_len / 2 + chunk - 1) / chunk) < 3LL * sms) chunk >>= 1;
  return chunk;
}

}  // namespace gqa
}  // namespace cake

static bool gqa_config_ok(const cake_b200_gqa_decode_config& c) {
  if (c.batch < 0 || c.batch > 65535 || c.head_dim != cake::gqa::kD || c.page_size <= 0 || c.max_kv_len < 0) return false;
  if (c.num_kv_heads <= 0 || c.num_kv_heads > 65535 || c.num_qo_heads % c.num_kv_heads) return false;
  const int g = c.num_qo_heads / c.num_kv_heads;
  return g >= 1 && g <= 8;
}

extern "C" size_t cake_b200_gqa_decode_workspace_bytes(const cake_b200_gqa_decode_config* c) {
  if (!c || !gqa_config_ok(*c)) return 0;
  const int chunk = cake::gqa::pick_chunk(*c, 148);
  const size_t splits = size_t((c->max_kv_len + chunk - 1) / chunk) + 1;
  const size_t slots = size_t(c->batch) * splits * c->num_qo_heads;
  return 256 + slots * (cake::gqa::kD + 1) * sizeof(float) + 256;
}

extern "C" int cake_b200_gqa_decode_create(void** buffers, const cake_b200_gqa_decode_config* config, void** handle_out) {
  using namespace cake;
  if (!buffers || !config || !handle_out) return kErrBadArgument;
  *handle_out = nullptr;
  int device = 0;
  if (int rc = require_blackwell(&device)) return rc;
  if (!gqa_config_ok(*config)) return kErrBadArgument;
  for (int i = 0; i < 10; ++i) {
    if (!buffers[i]) return kErrBadArgument;
    if (i <= 2 && (reinterpret_cast<uintptr_t>(buffers[i]) & 15)) return kErrBadArgument;
  }
  auto* h = new (std::nothrow) gqa::Handle;
  if (!h) return int(cudaErrorMemoryAllocation);
  h->device = device;
  gqa::Params& p = h->p;
  p.q = static_cast<const __nv_bfloat16*>(buffers[0]);
  p.k_cache = static_cast<const __nv_bfloat16*>(buffers[1]);
  p.v_cache = static_cast<const __nv_bfloat16*>(buffers[2]);
  p.kv_indptr = static_cast<const int*>(buffers[3]);
  p.kv_indices = static_cast<const int*>(buffers[4]);
  p.kv_last_page_len = static_cast<const int*>(buffers[5]);
  p.sm_scale = static_cast<const float*>(buffers[6]);
  p.out = static_cast<__nv_bfloat16*>(buffers[7]);
  p.lse = static_cast<float*>(buffers[8]);
  p.batch = int(config->batch);
  p.hq = config->num_qo_heads;
  p.hkv = config->num_kv_heads;
  p.page_size = config->page_size;
  p.chunk = gqa::pick_chunk(*config, 148);
  p.max_splits = int((config->max_kv_len + p.chunk - 1) / p.chunk) + 1;
  h->status = static_cast<int*>(buffers[9]);
  uint8_t* ws = static_cast<uint8_t*>(buffers[9]) + 256;
  p.part_o = reinterpret_cast<float*>(ws);
  p.part_lse = p.part_o + size_t(p.batch) * p.max_splits * p.hq * gqa::kD;
  int rc = int(cudaFuncSetAttribute(gqa::gqa_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gqa::kSmemBytes));
  if (rc) { delete h; return rc; }
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
  const gqa::Params& p = h->p;
  if (p.batch == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(cuda_stream);
  CAKE_CUDA_OK(cudaMemsetAsync(h->status, 0, sizeof(int), s));
  gqa::gqa_decode_kernel<<<dim3(p.max_splits, (p.hkv + gqa::kWarps - 1) / gqa::kWarps, p.batch), gqa::kWarps * 32, gqa::kSmemBytes, s>>>(p);
  gqa::gqa_reduce_kernel<<<dim3(p.hq, p.batch), gqa::kD, 0, s>>>(p);
  return int(cudaGetLastError());
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
// a workspace they do not have.  For them the split-KV partial results live in the fixed array
// below, which is part of the library image: every GPU that loads the library carries these
// 16 MiB until the process exits, whether or not the entry point is ever called.
//
// All calls share the array and nothing clears it between calls: the reduce kernel reads only
// the slots the decode kernel of the same call has just written, so stale contents are never
// consumed and nothing needs to start at zero.  Two calls that overlap on the GPU (different
// streams, or different host threads) race on it -- serialise them.
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
  for (int i = 0; i < 9; ++i) {
    if (!buffers[i]) return kErrBadArgument;
    if (i <= 2 && (reinterpret_cast<uintptr_t>(buffers[i]) & 15)) return kErrBadArgument;
  }
  gqa::Params p;
  p.q = static_cast<const __nv_bfloat16*>(buffers[0]);
  p.k_cache = static_cast<const __nv_bfloat16*>(buffers[1]);
  p.v_cache = static_cast<const __nv_bfloat16*>(buffers[2]);
  p.kv_indptr = static_cast<const int*>(buffers[3]);
  p.kv_indices = static_cast<const int*>(buffers[4]);
  p.kv_last_page_len = static_cast<const int*>(buffers[5]);
  p.sm_scale = static_cast<const float*>(buffers[6]);
  p.out = static_cast<__nv_bfloat16*>(buffers[7]);
  p.lse = static_cast<float*>(buffers[8]);
  p.batch = int(config->batch);
  p.hq = config->num_qo_heads;
  p.hkv = config->num_kv_heads;
  p.page_size = config->page_size;
  if (p.batch == 0) return 0;
  // Same chunking as the workspace variant; longer chunks (fewer partial results) if that is what
  // it takes to fit the fixed scratch, and a refusal if even two chunks per sequence do not fit.
  p.chunk = gqa::pick_chunk(*config, 148);
  auto bytes_needed = [&](int chunk) {
    const size_t splits = size_t((config->max_kv_len + chunk - 1) / chunk) + 1;
    return size_t(p.batch) * splits * p.hq * (gqa::kD + 1) * sizeof(float);
  };
  while (bytes_needed(p.chunk) > gqa::kNoAllocScratchBytes && p.chunk < config->max_kv_len) p.chunk *= 2;
  if (bytes_needed(p.chunk) > gqa::kNoAllocScratchBytes) return kErrWorkspace;   // batch * heads too large for 16 MiB
  p.max_splits = int((config->max_kv_len + p.chunk - 1) / p.chunk) + 1;
  void* scratch = nullptr;
  if (int rc = gqa::noalloc_setup(device, &scratch)) return rc;
  p.part_o = static_cast<float*>(scratch);
  p.part_lse = p.part_o + size_t(p.batch) * p.max_splits * p.hq * gqa::kD;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(cuda_stream);
  gqa::gqa_decode_kernel<<<dim3(p.max_splits, (p.hkv + gqa::kWarps - 1) / gqa::kWarps, p.batch), gqa::kWarps * 32, gqa::kSmemBytes, s>>>(p);
  gqa::gqa_reduce_kernel<<<dim3(p.hq, p.batch), gqa::kD, 0, s>>>(p);
  return int(cudaGetLastError());
}
