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

// ------------------------------------------------------------------------------------------
// The same exchange without a collective library: ranks write straight into each other's memory.
//
// Every rank owns one SYMMETRIC buffer (the same layout on every rank, each mapped into every other rank's
// address space by the host: torch.distributed._symmetric_memory, or any other peer mapping):
//   flags block | recv [world, capacity, row_bytes] | returned [world, capacity, H] bf16
// Dispatch: the rank that routed a token writes its packed row into the receive block of every rank that owns
// one of its experts, with plain 16-byte stores over NVLink -- only the rows that are needed travel -- and,
// once all of its rows are out, publishes the row count and a step number (the "epoch") in that rank's flags
// block with a system-scope release.  The receiver waits for the epoch of every source (bounded: on expiry it
// records a status and goes on with what it has), then compacts the rows it received into the rank-local
// layer's inputs.  The way back is the mirror image: the owner of the experts adds a received row's local
// contributions (slot order, fp32), rounds to bf16 and writes the row into the token owner's `returned`
// block; the token owner waits for every rank's epoch and adds the partial rows in rank order.
// No load or store here uses a cluster or multicast form; a peer's memory is only ever the target of plain
// stores, and every wait is on a flag in the waiting GPU's own memory.
namespace cake {
namespace ep {

constexpr int kMaxWorld = 64;
constexpr size_t kFlagBytes = 1024;      // dispatch_flag[64] | dispatch_count[64] | return_flag[64] | spare
__host__ __device__ inline size_t align256(size_t v) { return (v + 255) & ~size_t(255); }
__host__ __device__ inline size_t recv_offset() { return kFlagBytes; }
__host__ __device__ inline size_t returned_offset(int world, int cap, int hidden, int top_k) {
  return kFlagBytes + align256(size_t(world) * cap * row_bytes(hidden, top_k));
}

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(int* p, int v) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

struct PushScratch {       // ints in the rank's own (non-symmetric) scratch, after the 256-byte status block
  int* status;
  int* epoch;              // [1] step number, bumped by the plan kernel
  int* done;               // [2] CTA completion counters of the two push kernels
  int* send_count;         // [world]
  int* recv_total;         // [1] rows received this step
  int* row_src;            // [rows] source rank of compacted row c
  int* row_slot;           // [rows] its slot in that rank's block
  int* slot_of;            // [T, world]
  long long wait_clocks;   // budget of a wait for another rank (set at launch: the default, or the test hook's)
};

// One CTA of 1024 threads per destination rank: slots of the tokens that rank needs, in token order (a block-wide
// exclusive scan per 1024 tokens); the row count; and the epoch.
__global__ void __launch_bounds__(1024)
push_plan_kernel(const int* __restrict__ expert_ids, PushScratch sc, int tokens, int top_k, int world, int experts_per_rank) {
  __shared__ int warp_sums[32];
  const int r = blockIdx.x;
  int cursor = 0;
  for (int base = 0; base < tokens; base += 1024) {
    const int t = base + threadIdx.x;
    int need = 0;
    if (t < tokens) {
      const int* row = expert_ids + size_t(t) * top_k;
      for (int k = 0; k < top_k; k += 2) {                 // top_k is even (checked at create): 8-byte loads
        const int2 e = *reinterpret_cast<const int2*>(row + k);
        need |= (e.x >= 0 && e.x / experts_per_rank == r) || (e.y >= 0 && e.y / experts_per_rank == r);
      }
    }
    int total;
    const int before = cta1024_exclusive_scan(need, warp_sums, total);
    if (t < tokens) sc.slot_of[size_t(t) * world + r] = need ? cursor + before : -1;
    cursor += total;
  }
  if (threadIdx.x == 0) {
    sc.send_count[r] = cursor;
    if (r == 0) *sc.epoch = *sc.epoch + 1;
  }
}

// After its own stores a CTA fences at system scope and counts itself; the last one publishes `values[r]`
// (may be null) and the epoch in every peer's flags block.  Every thread of the CTA must call.
__device__ __forceinline__ void publish_when_last(int* done, const unsigned long long* peer_bases, int world, int me, int epoch,
                                                  const int* values, size_t count_off, size_t flag_off) {
  __shared__ int is_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(done, 1) == int(gridDim.x) - 1;
  __syncthreads();
  if (!is_last) return;
  if (threadIdx.x < world) {
    uint8_t* peer = reinterpret_cast<uint8_t*>(peer_bases[threadIdx.x]);
    if (values) st_relaxed_sys(reinterpret_cast<int*>(peer + count_off) + me, values[threadIdx.x]);
    __threadfence_system();
    st_release_sys(reinterpret_cast<int*>(peer + flag_off) + me, epoch);
  }
  if (threadIdx.x == 0) *done = 0;               // ready for the next step
}

// One warp per (token, destination rank) with a slot: the packed row goes straight into that rank's receive block.
__global__ void __launch_bounds__(256)
push_dispatch_kernel(const uint8_t* __restrict__ hidden_states, const float* __restrict__ hidden_scale,
                     const int* __restrict__ expert_ids, const float* __restrict__ route_weights, PushScratch sc,
                     const unsigned long long* __restrict__ peer_bases, int tokens, int top_k, int world, int me, int capacity,
                     int hidden) {
  const int lane = threadIdx.x & 31;
  const int w = row_bytes(hidden, top_k);
  const int kb = hidden / 128;
  for (int item = blockIdx.x * 8 + (threadIdx.x >> 5); item < tokens * world; item += gridDim.x * 8) {
    const int t = item / world, r = item % world;
    const int slot = sc.slot_of[item];
    if (slot < 0) continue;
    uint8_t* dst = reinterpret_cast<uint8_t*>(peer_bases[r]) + recv_offset() + (size_t(me) * capacity + slot) * w;
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
  publish_when_last(sc.done, peer_bases, world, me, *sc.epoch, sc.send_count, 64 * sizeof(int), 0);
}

// Waits (bounded) until every source's flag has reached this step's epoch; returns the counts in shared memory.
// A wait for another RANK covers whatever keeps that rank's host from launching its step on time (a collective a
// few lines earlier, a pause of its process), not just kernel latencies, so its budget is longer than that of the
// waits inside one kernel: about ten seconds of clocks instead of one.  It is still a bound: a rank that never
// arrives makes this rank report through the status word and go on.
constexpr long long kPeerWaitClockBudget = 20000000000LL;

__device__ __forceinline__ void wait_for_sources(const int* flags, const int* counts, int world, int epoch, int* status,
                                                 long long budget, int* cnt /* shared [kMaxWorld] */) {
  if (threadIdx.x < world) {
    const long long start = clock64();
    bool ok = true;
    while (ld_acquire_sys(flags + threadIdx.x) < epoch) {
      if (clock64() - start > budget) { ok = false; if (status) atomicCAS(status, 0, kStatusWaitFlag); break; }
      __nanosleep(64);
    }
    cnt[threadIdx.x] = ok && counts ? counts[threadIdx.x] : 0;
  }
  __syncthreads();
}

// One warp per row of the rank-local layer's inputs: row c < total is the c-th received row (sources in rank
// order, slots in order), anything beyond carries expert id -1.
__global__ void __launch_bounds__(256)
push_unpack_kernel(const uint8_t* __restrict__ own_base, PushScratch sc, uint8_t* __restrict__ hidden_states,
                   float* __restrict__ hidden_scale, int* __restrict__ expert_ids, float* __restrict__ route_weights,
                   int rows, int top_k, int world, int capacity, int hidden) {
  __shared__ int cnt[kMaxWorld];
  __shared__ int pre[kMaxWorld + 1];
  const int lane = threadIdx.x & 31;
  const int epoch = *sc.epoch;
  wait_for_sources(reinterpret_cast<const int*>(own_base), reinterpret_cast<const int*>(own_base) + 64, world, epoch, sc.status, sc.wait_clocks, cnt);
  if (threadIdx.x == 0) {
    int run = 0;
    for (int r = 0; r < world; ++r) { pre[r] = run; run += min(cnt[r], capacity); }
    pre[world] = run;
    if (blockIdx.x == 0) *sc.recv_total = run;
  }
  __syncthreads();
  const int total = pre[world];
  const int w = row_bytes(hidden, top_k);
  const int kb = hidden / 128;
  for (int c = blockIdx.x * 8 + (threadIdx.x >> 5); c < rows; c += gridDim.x * 8) {
    if (c >= total) {
      if (lane < top_k) { expert_ids[size_t(c) * top_k + lane] = -1; route_weights[size_t(c) * top_k + lane] = 0.f; }
      continue;
    }
    int src = 0;
    while (src + 1 < world && c >= pre[src + 1]) ++src;
    const int slot = c - pre[src];
    const uint8_t* row = own_base + recv_offset() + (size_t(src) * capacity + slot) * w;
    const int* si = reinterpret_cast<const int*>(row + hidden + 4 * kb);
    const float* sw = reinterpret_cast<const float*>(row + hidden + 4 * kb + 4 * top_k);
    if (lane < top_k) {
      expert_ids[size_t(c) * top_k + lane] = si[lane];
      route_weights[size_t(c) * top_k + lane] = sw[lane];
    }
    if (lane == 0) { sc.row_src[c] = src; sc.row_slot[c] = slot; }
    const uint4* s4 = reinterpret_cast<const uint4*>(row);
    uint4* d4 = reinterpret_cast<uint4*>(hidden_states + size_t(c) * hidden);
    for (int i = lane; i < hidden / 16; i += 32) d4[i] = s4[i];
    const float* ss = reinterpret_cast<const float*>(row + hidden);
    for (int i = lane; i < kb; i += 32) hidden_scale[size_t(i) * rows + c] = ss[i];
  }
}

// One CTA per received row: its local contributions (rows of y by inv_perm) added in slot order in fp32, rounded to
// bf16 and written into the token owner's `returned` block.
__global__ void __launch_bounds__(256)
push_return_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ inv_perm, PushScratch sc,
                   const unsigned long long* __restrict__ peer_bases, int world, int me, int capacity, int hidden, int top_k) {
  __shared__ int rows_of[32];
  __shared__ int valid_rows;
  const int c = blockIdx.x;
  const int total = *sc.recv_total;
  if (c < total) {
    if (threadIdx.x < 32) {              // the row's local contributions, compacted, still in slot order
      const int row = threadIdx.x < top_k ? inv_perm[size_t(c) * top_k + threadIdx.x] : -1;
      const uint32_t have = __ballot_sync(0xffffffffu, row >= 0);
      if (row >= 0) rows_of[__popc(have & ((1u << threadIdx.x) - 1u))] = row;
      if (threadIdx.x == 0) valid_rows = __popc(have);
    }
    __syncthreads();
    const int n = valid_rows;
    const int src = sc.row_src[c], slot = sc.row_slot[c];
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<uint8_t*>(peer_bases[src]) +
                                                          returned_offset(world, capacity, hidden, top_k)) +
                         (size_t(me) * capacity + slot) * hidden;
    for (int col = threadIdx.x * 8; col < hidden; col += blockDim.x * 8) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s0 = 0; s0 < n; s0 += 4) {          // four loads in flight, added in slot order
        uint4 raw[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          raw[j] = s0 + j < n ? __ldcs(reinterpret_cast<const uint4*>(y + size_t(rows_of[s0 + j]) * hidden + col)) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (s0 + j >= n) break;
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[j]);
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
      *reinterpret_cast<uint4*>(dst + col) = o;
    }
  }
  publish_when_last(sc.done + 1, peer_bases, world, me, *sc.epoch, nullptr, 0, 128 * sizeof(int));
}

// out[t,:] = bf16( sum over ranks r with a slot, in rank order, of returned[r, slot_of[t,r], :] ), once every rank's
// partial rows of this step have landed.
__global__ void __launch_bounds__(256)
push_reduce_kernel(const uint8_t* __restrict__ own_base, PushScratch sc, __nv_bfloat16* __restrict__ out, int world, int capacity,
                   int hidden, int top_k) {
  __shared__ int cnt[kMaxWorld];
  __shared__ int slots[kMaxWorld];
  wait_for_sources(reinterpret_cast<const int*>(own_base) + 128, nullptr, world, *sc.epoch, sc.status, sc.wait_clocks, cnt);
  const int t = blockIdx.x;
  if (threadIdx.x < world) slots[threadIdx.x] = sc.slot_of[size_t(t) * world + threadIdx.x];
  __syncthreads();
  const __nv_bfloat16* returned = reinterpret_cast<const __nv_bfloat16*>(own_base + returned_offset(world, capacity, hidden, top_k));
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

struct PushHandle {
  int device;
  cake_b200_ep_push_config cfg;
  void* b[14];
  PushScratch sc;
};

inline size_t push_scratch_bytes(const cake_b200_ep_push_config& c) {
  const size_t rows = size_t(c.world) * c.capacity;
  return 256 + align256(sizeof(int) * (8 + kMaxWorld)) + 2 * align256(rows * sizeof(int)) + align256(size_t(c.tokens) * c.world * sizeof(int));
}

}  // namespace ep
}  // namespace cake

static bool ep_push_config_ok(const cake_b200_ep_push_config& c) {
  cake_b200_ep_config base{c.tokens, c.capacity, c.hidden, c.top_k, c.world, c.experts};
  return ep_config_ok(base) && c.rank >= 0 && c.rank < c.world && c.world <= cake::ep::kMaxWorld && c.capacity <= (1 << 22);
}

extern "C" size_t cake_b200_ep_push_symmetric_bytes(const cake_b200_ep_push_config* c) {
  if (!c || !ep_push_config_ok(*c)) return 0;
  return cake::ep::returned_offset(c->world, int(c->capacity), c->hidden, c->top_k) + size_t(c->world) * c->capacity * c->hidden * 2;
}

extern "C" size_t cake_b200_ep_push_scratch_bytes(const cake_b200_ep_push_config* c) {
  return c && ep_push_config_ok(*c) ? cake::ep::push_scratch_bytes(*c) : 0;
}

extern "C" int cake_b200_ep_push_create(void** buffers, const cake_b200_ep_push_config* config, void** handle_out) {
  using namespace cake;
  if (!buffers || !config || !handle_out) return kErrBadArgument;
  *handle_out = nullptr;
  int device = 0;
  if (int rc = require_blackwell(&device)) return rc;
  if (!ep_push_config_ok(*config)) return kErrBadArgument;
  for (int i = 0; i < 14; ++i)
    if (!buffers[i] || (reinterpret_cast<uintptr_t>(buffers[i]) & 15)) return kErrBadArgument;
  if (reinterpret_cast<uintptr_t>(buffers[5]) & 255) return kErrBadArgument;     // the symmetric buffer and the scratch are 256-byte aligned
  if (reinterpret_cast<uintptr_t>(buffers[6]) & 255) return kErrBadArgument;
  auto* h = new (std::nothrow) ep::PushHandle;
  if (!h) return int(cudaErrorMemoryAllocation);
  h->device = device;
  h->cfg = *config;
  for (int i = 0; i < 14; ++i) h->b[i] = buffers[i];
  uint8_t* s = static_cast<uint8_t*>(buffers[6]);
  const size_t rows = size_t(config->world) * config->capacity;
  ep::PushScratch& sc = h->sc;
  sc.status = reinterpret_cast<int*>(s);
  int* words = reinterpret_cast<int*>(s + 256);
  sc.epoch = words;
  sc.done = words + 1;
  sc.recv_total = words + 3;
  sc.send_count = words + 8;
  s += 256 + ep::align256(sizeof(int) * (8 + ep::kMaxWorld));
  sc.row_src = reinterpret_cast<int*>(s);
  s += ep::align256(rows * sizeof(int));
  sc.row_slot = reinterpret_cast<int*>(s);
  s += ep::align256(rows * sizeof(int));
  sc.slot_of = reinterpret_cast<int*>(s);
  *handle_out = h;
  return 0;
}

extern "C" int cake_b200_ep_push_launch_stage(void* handle, int stage, void* cuda_stream) {
  using namespace cake;
  if (!handle) return kErrBadArgument;
  auto* h = static_cast<ep::PushHandle*>(handle);
  int device = -1;
  CAKE_CUDA_OK(cudaGetDevice(&device));
  if (device != h->device) return kErrWrongDevice;
  const cake_b200_ep_push_config& c = h->cfg;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(cuda_stream);
  const int tokens = int(c.tokens), cap = int(c.capacity), rows = c.world * cap;
  auto* ids = static_cast<const int*>(h->b[0]);
  auto* weights = static_cast<const float*>(h->b[1]);
  auto* hidden = static_cast<const uint8_t*>(h->b[2]);
  auto* scale = static_cast<const float*>(h->b[3]);
  auto* peers = static_cast<const unsigned long long*>(h->b[4]);
  auto* own = static_cast<const uint8_t*>(h->b[5]);
  ep::PushScratch scratch = h->sc;
  const int hook_kiloclocks = test_hooks().budget_kiloclocks;          // failure-path tests shorten the waits
  scratch.wait_clocks = hook_kiloclocks > 0 ? (long long)hook_kiloclocks << 10 : ep::kPeerWaitClockBudget;
  switch (stage) {
    case 0: {  // plan + dispatch: this rank's rows go into their owners' receive blocks
      ep::push_plan_kernel<<<c.world, 1024, 0, s>>>(ids, scratch, tokens, c.top_k, c.world, c.experts / c.world);
      const int blocks = tokens > 0 ? (tokens * c.world + 7) / 8 : 1;
      ep::push_dispatch_kernel<<<blocks < 1184 ? blocks : 1184, 256, 0, s>>>(hidden, scale, ids, weights, scratch, peers, tokens, c.top_k,
                                                                           c.world, c.rank, cap, c.hidden);
      break;
    }
    case 1: {  // wait for every source, then compact the received rows into the rank-local layer's inputs
      const int blocks = (rows + 7) / 8;
      ep::push_unpack_kernel<<<blocks < 1184 ? blocks : 1184, 256, 0, s>>>(own, scratch, static_cast<uint8_t*>(h->b[7]),
                                                                         static_cast<float*>(h->b[8]), static_cast<int*>(h->b[9]),
                                                                         static_cast<float*>(h->b[10]), rows, c.top_k, c.world, cap, c.hidden);
      break;
    }
    case 2:    // combine the local contributions of every received row and write it back to the token's owner
      ep::push_return_kernel<<<rows, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(h->b[11]), static_cast<const int*>(h->b[12]), scratch,
                                                  peers, c.world, c.rank, cap, c.hidden, c.top_k);
      break;
    case 3:    // wait for every rank's partial rows, then add them in rank order
      if (tokens > 0)
        ep::push_reduce_kernel<<<tokens, 256, 0, s>>>(own, scratch, static_cast<__nv_bfloat16*>(h->b[13]), c.world, cap, c.hidden, c.top_k);
      break;
    default:
      return kErrBadArgument;
  }
  return int(cudaGetLastError());
}

extern "C" int cake_b200_ep_push_destroy(void* handle) {
  delete static_cast<cake::ep::PushHandle*>(handle);
  return 0;
}
