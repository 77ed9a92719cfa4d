// Expert-parallel exchange kernels for the FP8 MoE layer: everything around the two all-to-alls
// that is not the collective itself.  All shapes are static (each rank exchanges `capacity` rows
// with every peer, unused rows are marked by expert id -1), so a layer needs no host
// synchronisation: plan + pack -> all-to-all -> unpack -> rank-local layer -> all-to-all -> reduce.
//
// The reference has no distributed layer; what it fixes is the rank-local view -- a rank owns the
// experts [local_expert_offset, +local_experts) and pairs routed elsewhere contribute nothing
// (src/open_cake_ir/tasks/solx_fib/moe.py:139-146).  A token is sent ONCE to each rank that owns at
// least one of its experts, as one packed byte row:
//   H e4m3 bytes | H/128 fp32 scales | K int32 expert ids | K fp32 route weights.
#include "common.cuh"
#include "../../include/cake_b200.h"
#include <new>

namespace cake {
namespace ep {

__host__ __device__ inline int row_bytes(int hidden, int top_k) { return hidden + 4 * (hidden / 128) + 8 * top_k; }

// One warp per destination rank walks the tokens in order; ballots give each needed token its
// slot in that rank's send block (stable: ascending token).  Rows past the count get id -1.
__global__ void __launch_bounds__(32)
plan_kernel(const int* __restrict__ expert_ids, int* __restrict__ slot_of, uint8_t* __restrict__ send, int tokens,
            int top_k, int world, int experts_per_rank, int capacity, int hidden) {
  const int r = blockIdx.x, lane = threadIdx.x;
  const uint32_t below = (1u << lane) - 1u;
  int cursor = 0;
  for (int base = 0; base < tokens; base += 32) {
    const int t = base + lane;
    bool need = false;
    if (t < tokens) {
      for (int k = 0; k < top_k; ++k) {
        const int e = expert_ids[size_t(t) * top_k + k];
        need |= (e >= 0 && e / experts_per_rank == r);
      }
    }
    const uint32_t mask = __ballot_sync(0xffffffffu, need);
    if (t < tokens) slot_of[size_t(t) * world + r] = need ? cursor + __popc(mask & below) : -1;
    cursor += __popc(mask);
  }
  // mark the unused rows of this rank's send block: every expert id -1
  const int w = row_bytes(hidden, top_k);
  const int id_off = hidden + 4 * (hidden / 128);
  for (int row = cursor + lane; row < capacity; row += 32) {
    int* ids = reinterpret_cast<int*>(send + (size_t(r) * capacity + row) * w + id_off);
    for (int k = 0; k < top_k; ++k) ids[k] = -1;
  }
}

// One warp per (token, rank) with a slot: copies the packed row.
__global__ void __launch_bounds__(256)
pack_kernel(const uint8_t* __restrict__ hidden_states, const float* __restrict__ hidden_scale,
            const int* __restrict__ expert_ids, const float* __restrict__ route_weights,
            const int* __restrict__ slot_of, uint8_t* __restrict__ send, int tokens, int top_k, int world,
            int capacity, int hidden) {
  const int lane = threadIdx.x & 31;
  const int w = row_bytes(hidden, top_k);
  const int kb = hidden / 128;
  for (int item = blockIdx.x * 8 + (threadIdx.x >> 5); item < tokens * world; item += gridDim.x * 8) {
    const int t = item / world, r = item % world;
    const int slot = slot_of[item];
    if (slot < 0) continue;
    uint8_t* dst = send + (size_t(r) * capacity + slot) * w;
    const uint4* src = reinterpret_cast<const uint4*>(hidden_states + size_t(t) * hidden);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (int i = lane; i < hidden / 16; i += 32) d4[i] = __ldg(src + i);
    float* ds = reinterpret_cast<float*>(dst + hidden);
    for (int i = lane; i < kb; i += 32) ds[i] = __ldg(hidden_scale + size_t(i) * tokens + t);
    int* di = reinterpret_cast<int*>(dst + hidden + 4 * kb);
    float* dw = reinterpret_cast<float*>(dst + hidden + 4 * kb + 4 * top_k);
    if (lane < top_k) {
      di[lane] = expert_ids[size_t(t) * top_k + lane];
      dw[lane] = route_weights[size_t(t) * top_k + lane];
    }
  }
}

// One warp per received row: splits the packed row into the rank-local layer's input tensors
// (the scales go back to K-block-major).
__global__ void __launch_bounds__(256)
unpack_kernel(const uint8_t* __restrict__ recv, uint8_t* __restrict__ hidden_states, float* __restrict__ hidden_scale,
              int* __restrict__ expert_ids, float* __restrict__ route_weights, int rows, int top_k, int hidden) {
  const int lane = threadIdx.x & 31;
  const int w = row_bytes(hidden, top_k);
  const int kb = hidden / 128;
  for (int row = blockIdx.x * 8 + (threadIdx.x >> 5); row < rows; row += gridDim.x * 8) {
    const uint8_t* src = recv + size_t(row) * w;
    const int* si = reinterpret_cast<const int*>(src + hidden + 4 * kb);
    const float* sw = reinterpret_cast<const float*>(src + hidden + 4 * kb + 4 * top_k);
    const bool used = si[0] >= 0;          // a used row has all of its ids >= 0, an unused one all -1
    if (lane < top_k) {
      expert_ids[size_t(row) * top_k + lane] = si[lane];
      route_weights[size_t(row) * top_k + lane] = used ? sw[lane] : 0.f;
    }
    if (!used) continue;                   // the layer never reads the data of a row no expert owns
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(hidden_states + size_t(row) * hidden);
    for (int i = lane; i < hidden / 16; i += 32) d4[i] = s4[i];
    const float* ss = reinterpret_cast<const float*>(src + hidden);
    for (int i = lane; i < kb; i += 32) hidden_scale[size_t(i) * rows + row] = ss[i];
  }
}

// out[t,:] = bf16( sum over ranks r with a slot, in rank order, of returned[r, slot_of[t,r], :] ) in fp32.
__global__ void __launch_bounds__(256)
reduce_kernel(const __nv_bfloat16* __restrict__ returned, const int* __restrict__ slot_of, __nv_bfloat16* __restrict__ out,
              int world, int capacity, int hidden) {
  const int t = blockIdx.x;
  __shared__ int slots[64];
  if (threadIdx.x < world) slots[threadIdx.x] = slot_of[size_t(t) * world + threadIdx.x];
  __syncthreads();
  for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; ++r) {
      const int slot = slots[r];
      if (slot < 0) continue;
      const uint4 raw = *reinterpret_cast<const uint4*>(returned + (size_t(r) * capacity + slot) * hidden + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + size_t(t) * hidden + c) = o;
  }
}

struct Handle {
  int device;
  cake_b200_ep_config cfg;
  void* b[13];
};

}  // namespace ep
}  // namespace cake

static bool ep_config_ok(const cake_b200_ep_config& c) {
  // pack and unpack move rows with 16-byte loads and stores, so every row of a send or receive block must start
  // on a 16-byte boundary: H + 4*H/128 is a multiple of 16 when H % 512 == 0, and 8*top_k when top_k is even
  return c.tokens >= 0 && c.tokens <= (1 << 22) && c.hidden > 0 && c.hidden % 512 == 0 && c.top_k > 0 && c.top_k <= 32 &&
         c.top_k % 2 == 0 && cake::ep::row_bytes(c.hidden, c.top_k) % 16 == 0 &&
         c.world > 0 && c.world <= 64 && c.experts > 0 && c.experts % c.world == 0 && c.capacity >= c.tokens;
}

extern "C" size_t cake_b200_ep_row_bytes(const cake_b200_ep_config* c) {
  return c && ep_config_ok(*c) ? size_t(cake::ep::row_bytes(c->hidden, c->top_k)) : 0;
}

extern "C" int cake_b200_ep_exchange_create(void** buffers, const cake_b200_ep_config* config, void** handle_out) {
  using namespace cake;
  if (!buffers || !config || !handle_out) return kErrBadArgument;
  *handle_out = nullptr;
  int device = 0;
  if (int rc = require_blackwell(&device)) return rc;
  if (!ep_config_ok(*config)) return kErrBadArgument;
  for (int i = 0; i < 13; ++i)
    if (!buffers[i] || (reinterpret_cast<uintptr_t>(buffers[i]) & 15)) return kErrBadArgument;
  auto* h = new (std::nothrow) ep::Handle;
  if (!h) return int(cudaErrorMemoryAllocation);
  h->device = device;
  h->cfg = *config;
  for (int i = 0; i < 13; ++i) h->b[i] = buffers[i];
  *handle_out = h;
  return 0;
}

extern "C" int cake_b200_ep_exchange_launch_stage(void* handle, int stage, void* cuda_stream) {
  using namespace cake;
  if (!handle) return kErrBadArgument;
  auto* h = static_cast<ep::Handle*>(handle);
  int device = -1;
  CAKE_CUDA_OK(cudaGetDevice(&device));
  if (device != h->device) return kErrWrongDevice;
  const cake_b200_ep_config& c = h->cfg;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(cuda_stream);
  const int tokens = int(c.tokens), cap = int(c.capacity), rows = c.world * cap;
  auto* ids = static_cast<const int*>(h->b[0]);
  auto* weights = static_cast<const float*>(h->b[1]);
  auto* hidden = static_cast<const uint8_t*>(h->b[2]);
  auto* scale = static_cast<const float*>(h->b[3]);
  auto* slot_of = static_cast<int*>(h->b[4]);
  auto* send = static_cast<uint8_t*>(h->b[5]);
  auto* recv = static_cast<const uint8_t*>(h->b[6]);
  switch (stage) {
    case 0:   // plan + pack: local routing results -> send blocks
      ep::plan_kernel<<<c.world, 32, 0, s>>>(ids, slot_of, send, tokens, c.top_k, c.world, c.experts / c.world, cap, c.hidden);
      if (tokens > 0) {
        const int blocks = (tokens * c.world + 7) / 8;
        ep::pack_kernel<<<blocks < 2048 ? blocks : 2048, 256, 0, s>>>(hidden, scale, ids, weights, slot_of, send, tokens,
                                                                    c.top_k, c.world, cap, c.hidden);
      }
      break;
    case 1: { // unpack: received blocks -> inputs of the rank-local layer
      const int blocks = (rows + 7) / 8;
      ep::unpack_kernel<<<blocks < 2048 ? blocks : 2048, 256, 0, s>>>(recv, static_cast<uint8_t*>(h->b[7]),
                                                                    static_cast<float*>(h->b[8]), static_cast<int*>(h->b[9]),
                                                                    static_cast<float*>(h->b[10]), rows, c.top_k, c.hidden);
      break;
    }
    case 2:   // reduce: partial rows returned by the owners of the experts -> this rank's output
      if (tokens > 0)
        ep::reduce_kernel<<<tokens, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(h->b[11]), slot_of,
                                                 static_cast<__nv_bfloat16*>(h->b[12]), c.world, cap, c.hidden);
      break;
    default:
      return kErrBadArgument;
  }
  return int(cudaGetLastError());
}

extern "C" int cake_b200_ep_exchange_destroy(void* handle) {
  delete static_cast<cake::ep::Handle*>(handle);
  return 0;
}
