// FP8 block-scaled MoE expert layer for sm_100a (rank-local): routing, token permute, grouped
// GEMM1 + SwiGLU (+ e4m3 requantisation), grouped GEMM2 * route weight, weighted combine.
//
// Operator and layouts: src/open_cake_ir/tasks/solx_fib/moe.py:13-20 (tensor ABI), :122-155
// (oracle), :275-287 (routing).  The grouped GEMMs run on the tcgen05 core in gemm_fp8.cuh; the
// small integer kernels here are warp-level (top-k by 64-bit ordered keys, ballot prefix scans).
#include "gemm_fp8.cuh"
#include "../../include/cake_b200.h"
#include <new>

namespace cake {
namespace moe {

constexpr int kMaxExpertsPerLane = 16;   // experts <= 512

// fp32 -> unsigned key with the same order; -0.0 is folded onto +0.0 so that the two tie
// (compiler/backends/triton.py:2428-2460 builds the same key for the reference's top-k).
__device__ __forceinline__ uint32_t ordered_bits(float v) {
  uint32_t b = __float_as_uint(v);
  if ((b << 1) == 0) b = 0;
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ unsigned long long make_key(float score, int id) {
  return (static_cast<unsigned long long>(ordered_bits(score)) << 32) | (0xffffffffu - uint32_t(id));
}
__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
    v = other > v ? other : v;
  }
  return v;
}

// One warp per token.  Lane l holds experts j*32 + l.
template <int EPL>
__global__ void __launch_bounds__(128)
routing_kernel(const float* __restrict__ logits, const __nv_bfloat16* __restrict__ bias,
               const float* __restrict__ factor_ptr, int* __restrict__ expert_ids,
               float* __restrict__ route_weights, int tokens, int experts, int top_k, int n_group,
               int topk_group, int mode) {
  __shared__ float group_scores[4][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int token = blockIdx.x * 4 + warp;
  if (token >= tokens) return;
  const float factor = __ldg(factor_ptr);
  float raw[EPL], choice[EPL];   // raw = value the weight is made from; choice = value ranked
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    const int id = j * 32 + lane;
    float x = id < experts ? __ldg(logits + size_t(token) * experts + id) : -INFINITY;
    if (mode == 0) {
      const float s = id < experts ? 1.f / (1.f + expf(-x)) : -INFINITY;
      raw[j] = s;
      choice[j] = id < experts ? s + __bfloat162float(bias[id]) : -INFINITY;
    } else {
      raw[j] = x;
      choice[j] = x;
    }
  }
  if (mode == 0 && n_group > 1) {
    const int group_size = experts / n_group;
    for (int g = 0; g < n_group; ++g) {
      float m1 = -INFINITY, m2 = -INFINITY;      // this lane's two best of group g
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        const int id = j * 32 + lane;
        if (id < experts && id / group_size == g) {
          const float v = choice[j];
          if (v > m1) { m2 = m1; m1 = v; } else if (v > m2) { m2 = v; }
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {          // disjoint halves: merging two top-2 sets is exact
        const float p1 = __shfl_xor_sync(0xffffffffu, m1, o);
        const float p2 = __shfl_xor_sync(0xffffffffu, m2, o);
        const float hi = fmaxf(m1, p1);
        const float lo = fmaxf(fminf(m1, p1), fmaxf(m2, p2));
        m1 = hi; m2 = lo;
      }
      if (lane == 0) group_scores[warp][g] = m1 + m2;
    }
    __syncwarp();
    bool keep = false;
    if (lane < n_group) {
      const float mine = group_scores[warp][lane];
      int rank = 0;
      for (int g = 0; g < n_group; ++g) {
        const float other = group_scores[warp][g];
        rank += (other > mine) || (other == mine && g < lane);
      }
      keep = rank < topk_group;
    }
    const uint32_t kept = __ballot_sync(0xffffffffu, keep);
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const int id = j * 32 + lane;
      if (id < experts && !((kept >> (id / group_size)) & 1u)) choice[j] = -INFINITY;
    }
  }
  unsigned long long keys[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    const int id = j * 32 + lane;
    keys[j] = id < experts ? make_key(choice[j], id) : 0ull;
  }
  float picked = 0.f;      // lane k keeps the raw value of the k-th selection
  int picked_id = 0;
  for (int k = 0; k < top_k; ++k) {
    unsigned long long best = 0ull;
#pragma unroll
    for (int j = 0; j < EPL; ++j) best = keys[j] > best ? keys[j] : best;
    best = warp_max_u64(best);
    const int id = int(0xffffffffu - uint32_t(best & 0xffffffffull));
    const int owner = id & 31, slot = id >> 5;
    float value = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j)
      if (j == slot) { value = raw[j]; if (lane == owner) keys[j] = 0ull; }
    value = __shfl_sync(0xffffffffu, value, owner);
    if (lane == k) { picked = value; picked_id = id; }
  }
  // weights over the selected experts, in selection order
  float weight;
  if (mode == 0) {
    float total = 0.f;
    for (int k = 0; k < top_k; ++k) total += __shfl_sync(0xffffffffu, picked, k);
    weight = picked / (total + 1e-20f) * factor;
  } else {
    const float top = __shfl_sync(0xffffffffu, picked, 0);
    const float e = expf(picked - top);
    float total = 0.f;
    for (int k = 0; k < top_k; ++k) total += __shfl_sync(0xffffffffu, e, k);
    weight = e / total * factor;
  }
  if (lane < top_k) {
    expert_ids[size_t(token) * top_k + lane] = picked_id;
    route_weights[size_t(token) * top_k + lane] = weight;
  }
}

// ---- permute: histogram, scan, stable placement -------------------------------------------
__global__ void histogram_kernel(const int* __restrict__ expert_ids, const int* __restrict__ offset_ptr,
                                 int* __restrict__ counts, int* __restrict__ inv_perm, int pairs, int local_experts) {
  const int offset = __ldg(offset_ptr);
  for (int p = blockIdx.x * blockDim.x + threadIdx.x; p < pairs; p += gridDim.x * blockDim.x) {
    const int e = expert_ids[p] - offset;
    if (e >= 0 && e < local_experts) atomicAdd(counts + e, 1);
    else inv_perm[p] = -1;
  }
}

__global__ void __launch_bounds__(1024)
scan_kernel(const int* __restrict__ counts, int* __restrict__ offsets, int local_experts) {
  __shared__ int warp_totals[32];
  __shared__ int carry;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < local_experts; base += blockDim.x) {
    const int e = base + threadIdx.x;
    const int c = e < local_experts ? counts[e] : 0;
    int incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) warp_totals[warp] = incl;
    __syncthreads();
    int before = carry;
    for (int w = 0; w < warp; ++w) before += warp_totals[w];
    if (e < local_experts) offsets[e] = before + incl - c;
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) carry = before + incl;
    __syncthreads();
  }
  if (threadIdx.x == 0) offsets[local_experts] = carry;
}

// One CTA of eight warps per local expert.  Each warp owns a contiguous eighth of the pairs: a first
// pass counts its matches, a prefix over the eight warps gives every warp its starting position, a
// second pass places the pairs by ballot rank -- ascending pair order inside the expert, so the
// permutation is the stable sort by expert.  Eight loads per lane are in flight per step.
constexpr int kPlaceWarps = 8;
constexpr int kPlaceStep = 256;      // pairs one warp looks at per step
__global__ void __launch_bounds__(kPlaceWarps * 32)
place_kernel(const int* __restrict__ expert_ids, const int* __restrict__ offset_ptr,
             const int* __restrict__ offsets, int* __restrict__ sorted_pairs, int* __restrict__ inv_perm,
             int pairs, int local_experts) {
  __shared__ int warp_count[kPlaceWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int e = blockIdx.x;
  const int want = e + __ldg(offset_ptr);
  const int first = offsets[e];
  if (offsets[e + 1] == first) return;
  const int per_warp = ((pairs + kPlaceWarps - 1) / kPlaceWarps + kPlaceStep - 1) / kPlaceStep * kPlaceStep;
  const int begin = warp * per_warp, end = min(pairs, begin + per_warp);
  const uint32_t below = (1u << lane) - 1u;
  int count = 0;
  for (int base = begin; base < end; base += kPlaceStep) {
    int ids[kPlaceStep / 32];
#pragma unroll
    for (int i = 0; i < kPlaceStep / 32; ++i) {
      const int p = base + 32 * i + lane;
      ids[i] = p < end ? __ldg(expert_ids + p) : -1;
    }
#pragma unroll
    for (int i = 0; i < kPlaceStep / 32; ++i) count += __popc(__ballot_sync(0xffffffffu, ids[i] == want));
  }
  if (lane == 0) warp_count[warp] = count;
  __syncthreads();
  int cursor = first;
  for (int w = 0; w < warp; ++w) cursor += warp_count[w];
  for (int base = begin; base < end; base += kPlaceStep) {
    int ids[kPlaceStep / 32];
#pragma unroll
    for (int i = 0; i < kPlaceStep / 32; ++i) {
      const int p = base + 32 * i + lane;      // lane-contiguous loads keep ballots in ascending pair order
      ids[i] = p < end ? __ldg(expert_ids + p) : -1;
    }
#pragma unroll
    for (int i = 0; i < kPlaceStep / 32; ++i) {
      const bool hit = ids[i] == want;
      const uint32_t mask = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        const int pos = cursor + __popc(mask & below);
        const int p = base + 32 * i + lane;
        sorted_pairs[pos] = p;
        inv_perm[p] = pos;
      }
      cursor += __popc(mask);
    }
  }
}

// Copies each routed row (e4m3 hidden state + its K-block scales + its route weight) to its
// sorted position.  One warp per destination row.
__global__ void __launch_bounds__(256)
gather_kernel(const uint8_t* __restrict__ hidden, const float* __restrict__ hidden_scale,
              const float* __restrict__ route_weights, const int* __restrict__ sorted_pairs,
              const int* __restrict__ offsets, uint8_t* __restrict__ x_perm, float* __restrict__ sx_perm,
              float* __restrict__ row_weight, int tokens, int hidden_width, int top_k, int local_experts,
              int capacity) {
  const int lane = threadIdx.x & 31;
  const int n_local = __ldg(offsets + local_experts);
  for (int pos = blockIdx.x * 8 + (threadIdx.x >> 5); pos < n_local; pos += gridDim.x * 8) {
    const int pair = __ldg(sorted_pairs + pos);
    const int token = pair / top_k;
    const uint4* src = reinterpret_cast<const uint4*>(hidden + size_t(token) * hidden_width);
    uint4* dst = reinterpret_cast<uint4*>(x_perm + size_t(pos) * hidden_width);
    for (int i = lane; i < hidden_width / 16; i += 32) dst[i] = __ldg(src + i);
    for (int kb = lane; kb < hidden_width / 128; kb += 32)
      sx_perm[size_t(kb) * capacity + pos] = __ldg(hidden_scale + size_t(kb) * tokens + token);
    if (lane == 0) row_weight[pos] = __ldg(route_weights + pair);
  }
}

// out[t,:] = bf16( fp32 sum over the token's local slots, in slot order, of the bf16 rows y[inv_perm[t,slot],:] ).
__global__ void __launch_bounds__(256)
combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ inv_perm, __nv_bfloat16* __restrict__ out,
               int hidden_width, int top_k) {
  const int token = blockIdx.x;
  __shared__ int rows[32];
  if (threadIdx.x < top_k) rows[threadIdx.x] = inv_perm[size_t(token) * top_k + threadIdx.x];
  __syncthreads();
  for (int c = threadIdx.x * 8; c < hidden_width; c += blockDim.x * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < top_k; ++s) {
      const int row = rows[s];
      if (row >= 0) {
        const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(y + size_t(row) * hidden_width + c));
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h[i]);
          acc[2 * i] += f.x;
          acc[2 * i + 1] += f.y;
        }
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + size_t(token) * hidden_width + c) = o;
  }
}

template <int EPL>
void launch_routing_t(const float* logits, const __nv_bfloat16* bias, const float* factor, int* ids, float* w,
                      int tokens, int experts, int top_k, int n_group, int topk_group, int mode, cudaStream_t s) {
  routing_kernel<EPL><<<(tokens + 3) / 4, 128, 0, s>>>(logits, bias, factor, ids, w, tokens, experts, top_k, n_group,
                                                      topk_group, mode);
}
inline void launch_routing(const float* logits, const __nv_bfloat16* bias, const float* factor, int* ids, float* w,
                           int tokens, int experts, int top_k, int n_group, int topk_group, int mode, cudaStream_t s) {
  const int epl = (experts + 31) / 32;
  if (epl <= 2) launch_routing_t<2>(logits, bias, factor, ids, w, tokens, experts, top_k, n_group, topk_group, mode, s);
  else if (epl <= 4) launch_routing_t<4>(logits, bias, factor, ids, w, tokens, experts, top_k, n_group, topk_group, mode, s);
  else if (epl <= 8) launch_routing_t<8>(logits, bias, factor, ids, w, tokens, experts, top_k, n_group, topk_group, mode, s);
  else launch_routing_t<16>(logits, bias, factor, ids, w, tokens, experts, top_k, n_group, topk_group, mode, s);
}

inline bool routing_config_ok(int64_t tokens, int experts, int top_k, int n_group, int topk_group, int mode) {
  if (tokens < 0 || tokens > (1 << 24) || experts <= 0 || experts > 32 * kMaxExpertsPerLane) return false;
  if (top_k <= 0 || top_k > 32 || top_k > experts) return false;
  if (mode != 0 && mode != 1) return false;
  if (mode == 0 && (n_group <= 0 || n_group > 32 || experts % n_group || topk_group <= 0 || topk_group > n_group)) return false;
  return true;
}

struct PermuteArgs {
  const int* expert_ids; const int* local_offset;
  int *counts, *offsets, *sorted_pairs, *inv_perm;
  int pairs, local_experts;
};
inline int launch_permute(const PermuteArgs& a, cudaStream_t s) {
  CAKE_CUDA_OK(cudaMemsetAsync(a.counts, 0, sizeof(int) * a.local_experts, s));
  if (a.pairs > 0) {
    const int blocks = (a.pairs + 255) / 256;
    histogram_kernel<<<blocks < 1024 ? blocks : 1024, 256, 0, s>>>(a.expert_ids, a.local_offset, a.counts, a.inv_perm,
                                                                  a.pairs, a.local_experts);
  }
  const int scan_threads = a.local_experts >= 1024 ? 1024 : ((a.local_experts + 31) / 32) * 32;
  scan_kernel<<<1, scan_threads, 0, s>>>(a.counts, a.offsets, a.local_experts);
  if (a.pairs > 0)
    place_kernel<<<a.local_experts, kPlaceWarps * 32, 0, s>>>(a.expert_ids, a.local_offset, a.offsets, a.sorted_pairs,
                                                          a.inv_perm, a.pairs, a.local_experts);
  return int(cudaGetLastError());
}

struct RoutingHandle {
  int device;
  const float* logits; const __nv_bfloat16* bias; const float* factor; int* ids; float* weights;
  cake_b200_routing_config cfg;
};
struct PermuteHandle {
  int device;
  PermuteArgs args;
};

inline size_t align_up(size_t v, size_t a = 256) { return (v + a - 1) / a * a; }

struct Layout {     // byte offsets inside the workspace
  size_t status, expert_ids, route_weights, counts, offsets, sorted_pairs, inv_perm, row_weight, x_perm, sx_perm,
      act, act_scale, y, total;
  int capacity, terms;
};
inline Layout make_layout(const cake_b200_moe_config& c) {
  Layout l{};
  const size_t pairs = size_t(c.tokens) * c.top_k;
  l.capacity = int(pairs < 1 ? 1 : pairs);
  l.terms = c.act_mode == 1 ? 2 : 1;
  size_t at = 0;
  auto take = [&](size_t bytes) { size_t here = at; at += align_up(bytes); return here; };
  l.status = take(256);
  l.expert_ids = take(pairs * 4);
  l.route_weights = take(pairs * 4);
  l.counts = take(size_t(c.local_experts) * 4);
  l.offsets = take(size_t(c.local_experts + 1) * 4);
  l.sorted_pairs = take(pairs * 4);
  l.inv_perm = take(pairs * 4);
  l.row_weight = take(size_t(l.capacity) * 4);
  l.x_perm = take(size_t(l.capacity) * c.hidden);
  l.sx_perm = take(size_t(c.hidden / 128) * l.capacity * 4);
  l.act = take(size_t(l.capacity) * c.intermediate * l.terms);
  l.act_scale = take(size_t(c.intermediate / 128) * l.terms * l.capacity * 4);
  l.y = take(size_t(l.capacity) * c.hidden * 2);
  l.total = at;
  return l;
}

struct MoeHandle {
  int device;
  cake_b200_moe_config cfg;
  Layout layout;
  uint8_t* ws;
  const float* logits; const __nv_bfloat16* bias; const uint8_t* hidden; const float* hidden_scale;
  const int* local_offset; const float* factor;
  __nv_bfloat16* output;
  int* expert_ids; float* route_weights;       // in the workspace, or the caller's when routing is external
  CUtensorMap map_a1, map_a1_tail, map_b1, map_a2, map_a2_tail, map_b2;
  gemm::Params p1, p2;
  int grid;
};

}  // namespace moe
}  // namespace cake

// ------------------------------------------------------------------------------------------
extern "C" int cake_b200_moe_routing_create(void** buffers, const cake_b200_routing_config* config, void** handle_out) {
  using namespace cake;
  if (!buffers || !config || !handle_out) return kErrBadArgument;
  *handle_out = nullptr;
  int device = 0;
  if (int rc = require_blackwell(&device)) return rc;
  for (int i = 0; i < 5; ++i) if (!buffers[i]) return kErrBadArgument;
  if (!moe::routing_config_ok(config->tokens, config->experts, config->top_k, config->n_group, config->topk_group, config->mode))
    return kErrBadArgument;
  auto* h = new (std::nothrow) moe::RoutingHandle;
  if (!h) return int(cudaErrorMemoryAllocation);
  h->device = device;
  h->logits = static_cast<const float*>(buffers[0]);
  h->bias = static_cast<const __nv_bfloat16*>(buffers[1]);
  h->factor = static_cast<const float*>(buffers[2]);
  h->ids = static_cast<int*>(buffers[3]);
  h->weights = static_cast<float*>(buffers[4]);
  h->cfg = *config;
  *handle_out = h;
  return 0;
}
extern "C" int cake_b200_moe_routing_launch(void* handle, void* cuda_stream) {
  using namespace cake;
  if (!handle) return kErrBadArgument;
  auto* h = static_cast<moe::RoutingHandle*>(handle);
  int device = -1;
  CAKE_CUDA_OK(cudaGetDevice(&device));
  if (device != h->device) return kErrWrongDevice;
  if (h->cfg.tokens == 0) return 0;
  moe::launch_routing(h->logits, h->bias, h->factor, h->ids, h->weights, int(h->cfg.tokens), h->cfg.experts, h->cfg.top_k,
                      h->cfg.n_group, h->cfg.topk_group, h->cfg.mode, reinterpret_cast<cudaStream_t>(cuda_stream));
  return int(cudaGetLastError());
}
extern "C" int cake_b200_moe_routing_destroy(void* handle) {
  delete static_cast<cake::moe::RoutingHandle*>(handle);
  return 0;
}

extern "C" int cake_b200_moe_permute_create(void** buffers, const cake_b200_permute_config* config, void** handle_out) {
  using namespace cake;
  if (!buffers || !config || !handle_out) return kErrBadArgument;
  *handle_out = nullptr;
  int device = 0;
  if (int rc = require_blackwell(&device)) return rc;
  for (int i = 0; i < 6; ++i) if (!buffers[i]) return kErrBadArgument;
  if (config->tokens < 0 || config->top_k <= 0 || config->local_experts <= 0 ||
      config->tokens * config->top_k > (int64_t(1) << 30))
    return kErrBadArgument;
  auto* h = new (std::nothrow) moe::PermuteHandle;
  if (!h) return int(cudaErrorMemoryAllocation);
  h->device = device;
  h->args = moe::PermuteArgs{static_cast<const int*>(buffers[0]), static_cast<const int*>(buffers[1]),
                             static_cast<int*>(buffers[2]), static_cast<int*>(buffers[3]), static_cast<int*>(buffers[4]),
                             static_cast<int*>(buffers[5]), int(config->tokens * config->top_k), config->local_experts};
  *handle_out = h;
  return 0;
}
extern "C" int cake_b200_moe_permute_launch(void* handle, void* cuda_stream) {
  using namespace cake;
  if (!handle) return kErrBadArgument;
  auto* h = static_cast<moe::PermuteHandle*>(handle);
  int device = -1;
  CAKE_CUDA_OK(cudaGetDevice(&device));
  if (device != h->device) return kErrWrongDevice;
  return moe::launch_permute(h->args, reinterpret_cast<cudaStream_t>(cuda_stream));
}
extern "C" int cake_b200_moe_permute_destroy(void* handle) {
  delete static_cast<cake::moe::PermuteHandle*>(handle);
  return 0;
}

// ------------------------------------------------------------------------------------------
static bool moe_config_ok(const cake_b200_moe_config& c) {
  if (c.tokens < 0 || c.tokens * int64_t(c.top_k > 0 ? c.top_k : 1) > (int64_t(1) << 28)) return false;
  if (c.hidden <= 0 || c.hidden % 128 || c.intermediate <= 0 || c.intermediate % 128) return false;
  if (c.local_experts <= 0 || c.local_experts > cake::gemm::kMaxGroups || c.local_experts > c.experts) return false;
  if (c.act_mode != 0 && c.act_mode != 1) return false;
  if (c.top_k <= 0 || c.top_k > 32) return false;
  if (!c.external_routing &&
      !cake::moe::routing_config_ok(c.tokens, c.experts, c.top_k, c.n_group, c.topk_group, c.routing_mode))
    return false;
  return true;
}

extern "C" size_t cake_b200_moe_workspace_bytes(const cake_b200_moe_config* config) {
  if (!config || !moe_config_ok(*config)) return 0;
  return cake::moe::make_layout(*config).total;
}

extern "C" int cake_b200_moe_create(void** buffers, const cake_b200_moe_config* config, void** handle_out) {
  using namespace cake;
  if (!buffers || !config || !handle_out) return kErrBadArgument;
  *handle_out = nullptr;
  int device = 0;
  if (int rc = require_blackwell(&device)) return rc;
  if (!moe_config_ok(*config)) return kErrBadArgument;
  for (int i = 0; i < 12; ++i)
    if (!buffers[i] || (reinterpret_cast<uintptr_t>(buffers[i]) & (i >= 2 && i <= 7 ? 15 : 3))) return kErrBadArgument;
  if (reinterpret_cast<uintptr_t>(buffers[11]) & 255) return kErrBadArgument;
  auto* h = new (std::nothrow) moe::MoeHandle;
  if (!h) return int(cudaErrorMemoryAllocation);
  const cake_b200_moe_config& c = *config;
  h->device = device;
  h->cfg = c;
  h->layout = moe::make_layout(c);
  const moe::Layout& l = h->layout;
  h->ws = static_cast<uint8_t*>(buffers[11]);
  h->logits = static_cast<const float*>(buffers[0]);
  h->bias = static_cast<const __nv_bfloat16*>(buffers[1]);
  h->hidden = static_cast<const uint8_t*>(buffers[2]);
  h->hidden_scale = static_cast<const float*>(buffers[3]);
  h->local_offset = static_cast<const int*>(buffers[8]);
  h->factor = static_cast<const float*>(buffers[9]);
  h->output = static_cast<__nv_bfloat16*>(buffers[10]);
  if (c.external_routing) {
    h->expert_ids = static_cast<int*>(buffers[0]);
    h->route_weights = static_cast<float*>(buffers[1]);
  } else {
    h->expert_ids = reinterpret_cast<int*>(h->ws + l.expert_ids);
    h->route_weights = reinterpret_cast<float*>(h->ws + l.route_weights);
  }
  const int inter = c.intermediate, hidden = c.hidden;
  int rc = make_tensor_map_u8_sw128(&h->map_a1, h->ws + l.x_perm, uint64_t(l.capacity), uint64_t(hidden), gemm::kBM);
  if (!rc) rc = make_tensor_map_u8_sw128(&h->map_a1_tail, h->ws + l.x_perm, uint64_t(l.capacity), uint64_t(hidden), gemm::kTailRows);
  if (!rc) rc = make_tensor_map_u8_sw128(&h->map_a2_tail, h->ws + l.act, uint64_t(l.capacity), uint64_t(inter) * l.terms, gemm::kTailRows);
  if (!rc) rc = make_tensor_map_u8_sw128(&h->map_b1, buffers[4], uint64_t(c.local_experts) * 2 * inter, uint64_t(hidden), 128);
  if (!rc) rc = make_tensor_map_u8_sw128(&h->map_a2, h->ws + l.act, uint64_t(l.capacity), uint64_t(inter) * l.terms, gemm::kBM);
  if (!rc) rc = make_tensor_map_u8_sw128(&h->map_b2, buffers[6], uint64_t(c.local_experts) * hidden, uint64_t(inter), gemm::kBN);
  if (!rc) rc = int(cudaFuncSetAttribute(gemm::gemm_fp8_kernel<gemm::kGateUp>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(gemm::kSmemBytes)));
  if (!rc) rc = int(cudaFuncSetAttribute(gemm::gemm_fp8_kernel<gemm::kDown>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(gemm::kSmemBytes)));
  if (rc) { delete h; return rc; }
  int* status = reinterpret_cast<int*>(h->ws + l.status);
  const int* offsets = reinterpret_cast<const int*>(h->ws + l.offsets);
  gemm::Params& p1 = h->p1;
  p1 = gemm::Params{};
  p1.n = inter;
  p1.k_blocks = p1.b_k_blocks = hidden / 128;
  p1.b_rows_per_group = 2 * inter;
  p1.groups = c.local_experts;
  p1.row_capacity = l.capacity;
  p1.offsets = offsets;
  p1.sfa = reinterpret_cast<const float*>(h->ws + l.sx_perm);
  p1.sfb = static_cast<const float*>(buffers[5]);
  p1.out = h->ws + l.act;
  p1.out_scale = reinterpret_cast<float*>(h->ws + l.act_scale);
  p1.split_act = l.terms == 2;
  p1.status = status;
  p1.queue = status + 9;                 // GEMM1: items drawn from a counter too: the two row tiles of an expert then start together on two SMs
                                         // and the second reads the weights from L2 (DRAM reads 1.12 -> 1.00 x algorithmic, 2 % less time)
  gemm::Params& p2 = h->p2;
  p2 = gemm::Params{};
  p2.n = hidden;
  p2.k_blocks = inter / 128 * l.terms;
  p2.b_k_blocks = inter / 128;
  p2.interleave_hi_lo = l.terms == 2;
  p2.b_rows_per_group = hidden;
  p2.groups = c.local_experts;
  p2.row_capacity = l.capacity;
  p2.offsets = offsets;
  p2.sfa = reinterpret_cast<const float*>(h->ws + l.act_scale);
  p2.sfb = static_cast<const float*>(buffers[7]);
  p2.out = h->ws + l.y;
  p2.row_weight = reinterpret_cast<const float*>(h->ws + l.row_weight);
  p2.status = status;
  p2.queue = status + 8;                 // GEMM2: items are drawn from a counter inside the 256-byte status block (12 % faster: short
                                         // items, 16 K blocks each, so an SM that runs slower should simply take fewer)
  h->grid = sm_count(device);
  *handle_out = h;
  return 0;
}

// stage 0: routing + permute + gather; 1: grouped GEMM1 + SwiGLU; 2: grouped GEMM2; 3: combine
static int moe_launch_stage(cake::moe::MoeHandle* h, int stage, cudaStream_t s) {
  using namespace cake;
  const cake_b200_moe_config& c = h->cfg;
  const moe::Layout& l = h->layout;
  const int tokens = int(c.tokens);
  moe::PermuteArgs pa{h->expert_ids, h->local_offset, reinterpret_cast<int*>(h->ws + l.counts),
                      reinterpret_cast<int*>(h->ws + l.offsets), reinterpret_cast<int*>(h->ws + l.sorted_pairs),
                      reinterpret_cast<int*>(h->ws + l.inv_perm), tokens * c.top_k, c.local_experts};
  switch (stage) {
    case 0: {
      CAKE_CUDA_OK(cudaMemsetAsync(h->ws + l.status, 0, 256, s));
      if (!c.external_routing)
        moe::launch_routing(h->logits, h->bias, h->factor, h->expert_ids, h->route_weights, tokens, c.experts, c.top_k,
                            c.n_group, c.topk_group, c.routing_mode, s);
      if (int rc = moe::launch_permute(pa, s)) return rc;
      const int gather_blocks = (l.capacity + 7) / 8;
      moe::gather_kernel<<<gather_blocks < 4096 ? gather_blocks : 4096, 256, 0, s>>>(
          h->hidden, h->hidden_scale, h->route_weights, pa.sorted_pairs, pa.offsets, h->ws + l.x_perm,
          reinterpret_cast<float*>(h->ws + l.sx_perm), reinterpret_cast<float*>(h->ws + l.row_weight), tokens, c.hidden,
          c.top_k, c.local_experts, l.capacity);
      break;
    }
    case 1: {
      if (h->p1.queue) CAKE_CUDA_OK(cudaMemsetAsync(h->p1.queue, 0, sizeof(int), s));     // the work-item counter starts at 0
      gemm::Params p = h->p1;
      p.wait_kiloclocks = test_hooks().budget_kiloclocks;
      gemm::gemm_fp8_kernel<gemm::kGateUp><<<h->grid, gemm::kThreads, gemm::kSmemBytes, s>>>(h->map_a1, h->map_a1_tail, h->map_b1, p);
      break;
    }
    case 2: {
      if (h->p2.queue) CAKE_CUDA_OK(cudaMemsetAsync(h->p2.queue, 0, sizeof(int), s));
      gemm::Params p = h->p2;
      p.wait_kiloclocks = test_hooks().budget_kiloclocks;
      gemm::gemm_fp8_kernel<gemm::kDown><<<h->grid, gemm::kThreads, gemm::kSmemBytes, s>>>(h->map_a2, h->map_a2_tail, h->map_b2, p);
      break;
    }
    case 3:
      moe::combine_kernel<<<tokens, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(h->ws + l.y), pa.inv_perm, h->output,
                                                 c.hidden, c.top_k);
      break;
    default:
      return kErrBadArgument;
  }
  return int(cudaGetLastError());
}

extern "C" int cake_b200_moe_launch_stage(void* handle, int stage, void* cuda_stream) {
  using namespace cake;
  if (!handle) return kErrBadArgument;
  auto* h = static_cast<moe::MoeHandle*>(handle);
  int device = -1;
  CAKE_CUDA_OK(cudaGetDevice(&device));
  if (device != h->device) return kErrWrongDevice;
  if (h->cfg.tokens == 0) return stage >= 0 && stage <= 3 ? 0 : kErrBadArgument;
  return moe_launch_stage(h, stage, reinterpret_cast<cudaStream_t>(cuda_stream));
}

extern "C" int cake_b200_moe_launch(void* handle, void* cuda_stream) {
  for (int stage = 0; stage < 4; ++stage)
    if (int rc = cake_b200_moe_launch_stage(handle, stage, cuda_stream)) return rc;
  return 0;
}

extern "C" int cake_b200_moe_destroy(void* handle) {
  delete static_cast<cake::moe::MoeHandle*>(handle);
  return 0;
}

extern "C" int cake_b200_moe_intermediate(void* handle, int which, void** out) {
  using namespace cake;
  if (!handle || !out) return kErrBadArgument;
  auto* h = static_cast<moe::MoeHandle*>(handle);
  const moe::Layout& l = h->layout;
  switch (which) {
    case 0: *out = h->expert_ids; break;
    case 1: *out = h->route_weights; break;
    case 2: *out = h->ws + l.counts; break;
    case 3: *out = h->ws + l.offsets; break;
    case 4: *out = h->ws + l.sorted_pairs; break;
    case 5: *out = h->ws + l.inv_perm; break;
    case 6: *out = h->ws + l.y; break;
    default: return kErrBadArgument;
  }
  return 0;
}
