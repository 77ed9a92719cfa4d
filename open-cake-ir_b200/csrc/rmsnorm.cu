// RMSNorm for sm_100a, fp32 arithmetic, one bf16 rounding of the result.
//
// Operators:
//   out[r,c] = bf16( z[r,c] * weight[c] / sqrt(mean_j z[r,j]^2 + eps) ),  z = x or fp32(x + residual)
//     (src/open_cake_ir/tasks/solx_fib/workload.py:214-218, oracle :334-358), and the two-output form
//   z = bf16(delta + residual); residual_out = z; out = bf16( fp32(z) * rsqrt(mean z^2 + eps) * weight )
//     (src/open_cake_ir/tasks/add_rmsnorm.py:66, oracle :131-143): the sum is rounded to bf16 FIRST, the
//     rounded row is what is written back and what is normalised.
// Both are bound by HBM traffic (2 bytes in and 2 out per element and operand), so what matters is how
// many bytes an SM keeps in flight.  Rows of up to 16 KiB go through `rmsnorm_ring_kernel`: small
// persistent CTAs whose rows arrive by untiled bulk copies (cp.async.bulk, one elected thread) in a ring
// of shared-memory slots, several rows ahead of the one being reduced, so that the loads in flight do
// not depend on registers or on the row's reduction.  Wider rows use `rmsnorm_kernel`, which holds the row
// in registers (one CTA per row, next row prefetched).
#include "common.cuh"
#include "../../include/cake_b200.h"
#include <new>

namespace cake {
namespace {

constexpr int kMaxThreads = 512;

__device__ __forceinline__ void unpack8(const uint4& raw, float* v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {   // read once: do not keep in L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream(uint4* p, const uint4& v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ float sum_squares8(const uint4& raw) {
  float v[8];
  unpack8(raw, v);
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) ss = fmaf(v[j], v[j], ss);
  return ss;
}

// VPT = 16-byte vectors per thread; a row has width/8 vectors, at most VPT*kThreads.  The row and
// the weights stay in registers as the packed bf16 they arrived as (4 registers per vector) and
// are unpacked where they are used; with one vector per thread the kernel fits 40 registers, so an
// SM holds 1536 threads, each with the next row's vector already in flight (48 KiB of loads per SM).
template <int kThreads, int VPT, bool RESIDUAL>
__global__ void __launch_bounds__(kThreads, VPT == 1 ? 1536 / kThreads : ((2048 / kThreads) / VPT > 0 ? (2048 / kThreads) / VPT : 1))
rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
               const __nv_bfloat16* __restrict__ weight, __nv_bfloat16* __restrict__ out,
               int rows, int width, float eps) {
  __shared__ float partial[2][kThreads / 32];
  const int vectors = width >> 3;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint4 w[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * kThreads;
    w[i] = idx < vectors ? __ldg(reinterpret_cast<const uint4*>(weight) + idx) : make_uint4(0, 0, 0, 0);
  }
  const float inv_width = 1.f / float(width);
  int flip = 0;
  // The next row's loads are issued before the current row is reduced and stored, so a CTA
  // always has a row in flight while it works on another.
  uint4 ahead[VPT];
  if (blockIdx.x < rows) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * kThreads;
      ahead[i] = idx < vectors ? ld_stream(reinterpret_cast<const uint4*>(x + size_t(blockIdx.x) * width) + idx)
                               : make_uint4(0, 0, 0, 0);
    }
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x, flip ^= 1) {
    uint4 raw[VPT];
    float z[RESIDUAL ? VPT : 1][8];        // the fused variant must keep fp32(x + residual)
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) raw[i] = ahead[i];
    const int next = row + gridDim.x;
    if (next < rows) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int idx = threadIdx.x + i * kThreads;
        if (idx < vectors) ahead[i] = ld_stream(reinterpret_cast<const uint4*>(x + size_t(next) * width) + idx);
      }
    }
    if (RESIDUAL) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int idx = threadIdx.x + i * kThreads;
        float r[8];
        unpack8(raw[i], z[RESIDUAL ? i : 0]);
        unpack8(idx < vectors ? ld_stream(reinterpret_cast<const uint4*>(residual + size_t(row) * width) + idx)
                              : make_uint4(0, 0, 0, 0), r);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          z[RESIDUAL ? i : 0][j] += r[j];
          ss = fmaf(z[RESIDUAL ? i : 0][j], z[RESIDUAL ? i : 0][j], ss);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < VPT; ++i) ss += sum_squares8(raw[i]);
    }
    ss = warp_sum(ss);
    if (lane == 0) partial[flip][warp] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < kThreads / 32; ++i) total += partial[flip][i];
    const float inverse = 1.f / sqrtf(total * inv_width + eps);
    uint4* dst = reinterpret_cast<uint4*>(out + size_t(row) * width);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * kThreads;
      if (idx < vectors) {
        float v[8], wf[8];
        if (RESIDUAL) {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = z[RESIDUAL ? i : 0][j];
        } else {
          unpack8(raw[i], v);
        }
        unpack8(w[i], wf);
        uint4 o;
        o.x = pack_bf16x2(v[0] * inverse * wf[0], v[1] * inverse * wf[1]);
        o.y = pack_bf16x2(v[2] * inverse * wf[2], v[3] * inverse * wf[3]);
        o.z = pack_bf16x2(v[4] * inverse * wf[4], v[5] * inverse * wf[5]);
        o.w = pack_bf16x2(v[6] * inverse * wf[6], v[7] * inverse * wf[7]);
        st_stream(dst + idx, o);
      }
    }
  }
}

// ---- bulk-copy ring ------------------------------------------------------------------------
constexpr int kRingThreads = 128;
constexpr int kRingMaxSlots = 8;
enum RingMode : int { kPlain = 0, kFusedResidual = 1, kAddTwoOutputs = 2 };

// Set when a wait for a row's bulk copy ran out (never in correct operation); read by
// cake_b200_rmsnorm_last_status.
__device__ int g_rmsnorm_status = 0;

struct RingParams {
  const __nv_bfloat16 *x, *residual, *weight;
  __nv_bfloat16 *out, *residual_out;
  int rows, width, slots;
  float eps;
};

// Dynamic shared memory: weight row | slots x (x row [| residual row]) ; static: barriers, partial sums.
template <int MODE>
__global__ void __launch_bounds__(kRingThreads)
rmsnorm_ring_kernel(const RingParams p) {
  extern __shared__ __align__(128) uint8_t ring_smem[];
  __shared__ uint64_t full[kRingMaxSlots];
  __shared__ float partial[2][kRingThreads / 32];
  __shared__ int give_up;
  constexpr int kOperands = MODE == kPlain ? 1 : 2;
  const int vectors = p.width >> 3;
  const uint32_t row_bytes = uint32_t(p.width) * 2u;
  const uint32_t slot_bytes = row_bytes * kOperands;
  uint8_t* w_smem = ring_smem;
  uint8_t* slots = ring_smem + row_bytes;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int my_rows = p.rows > int(blockIdx.x) ? (p.rows - 1 - int(blockIdx.x)) / int(gridDim.x) + 1 : 0;
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.slots; ++s) mbar_init(&full[s], 1);
    give_up = 0;
    fence_barrier_init();
  }
  for (int i = threadIdx.x; i < vectors; i += kRingThreads)
    reinterpret_cast<uint4*>(w_smem)[i] = __ldg(reinterpret_cast<const uint4*>(p.weight) + i);
  __syncthreads();
  const uint64_t once = l2_policy_evict_first();
  auto request = [&](int k) {            // the CTA's k-th row -> slot k mod slots (one thread)
    const int s = k % p.slots;
    const size_t row = size_t(blockIdx.x) + size_t(k) * gridDim.x;
    uint8_t* dst = slots + size_t(s) * slot_bytes;
    mbar_arrive_expect_tx(&full[s], slot_bytes);
    bulk_load_1d(dst, p.x + row * p.width, row_bytes, &full[s], once);
    if (kOperands == 2) bulk_load_1d(dst + row_bytes, p.residual + row * p.width, row_bytes, &full[s], once);
  };
  if (threadIdx.x == 0)
    for (int k = 0; k < p.slots && k < my_rows; ++k) request(k);
  const float inv_width = 1.f / float(p.width);
  for (int k = 0; k < my_rows; ++k) {
    const int s = k % p.slots;
    const uint32_t phase = uint32_t(k / p.slots) & 1u;
    if (!mbar_try_wait(&full[s], phase)) {           // bounded: about a second, then the CTA gives the launch up
      const long long start = clock64();
      while (!mbar_try_wait(&full[s], phase)) {
        if (clock64() - start > kWaitClockBudget) { give_up = 1; atomicCAS(&g_rmsnorm_status, 0, kStatusWaitSmemFull); break; }
      }
    }
    __syncthreads();
    if (give_up) break;
    const size_t row = size_t(blockIdx.x) + size_t(k) * gridDim.x;
    const uint4* xs = reinterpret_cast<const uint4*>(slots + size_t(s) * slot_bytes);
    const uint4* rs = reinterpret_cast<const uint4*>(slots + size_t(s) * slot_bytes + row_bytes);
    // z of one 16-byte vector, as the operator defines it
    auto load_z = [&](int idx, float* z, uint4* rounded) {
      unpack8(xs[idx], z);
      if (MODE != kPlain) {
        float r[8];
        unpack8(rs[idx], r);
#pragma unroll
        for (int j = 0; j < 8; ++j) z[j] += r[j];
      }
      if (MODE == kAddTwoOutputs) {                  // the rounding seam: z = bf16(delta + residual)
        uint4 q;
        q.x = pack_bf16x2(z[0], z[1]); q.y = pack_bf16x2(z[2], z[3]); q.z = pack_bf16x2(z[4], z[5]); q.w = pack_bf16x2(z[6], z[7]);
        unpack8(q, z);
        *rounded = q;
      }
    };
    float ss = 0.f;
    for (int idx = threadIdx.x; idx < vectors; idx += kRingThreads) {
      float z[8];
      uint4 q;
      load_z(idx, z, &q);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(z[j], z[j], ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) partial[k & 1][warp] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < kRingThreads / 32; ++i) total += partial[k & 1][i];
    const float inverse = 1.f / sqrtf(total * inv_width + p.eps);
    uint4* dst = reinterpret_cast<uint4*>(p.out + row * p.width);
    for (int idx = threadIdx.x; idx < vectors; idx += kRingThreads) {
      float z[8], wf[8];
      uint4 q;
      load_z(idx, z, &q);
      unpack8(reinterpret_cast<const uint4*>(w_smem)[idx], wf);
      uint4 o;
      o.x = pack_bf16x2(z[0] * inverse * wf[0], z[1] * inverse * wf[1]);
      o.y = pack_bf16x2(z[2] * inverse * wf[2], z[3] * inverse * wf[3]);
      o.z = pack_bf16x2(z[4] * inverse * wf[4], z[5] * inverse * wf[5]);
      o.w = pack_bf16x2(z[6] * inverse * wf[6], z[7] * inverse * wf[7]);
      st_stream(dst + idx, o);
      if (MODE == kAddTwoOutputs) st_stream(reinterpret_cast<uint4*>(p.residual_out + row * p.width) + idx, q);
    }
    __syncthreads();                                 // every thread has read the slot for the last time
    if (threadIdx.x == 0 && k + p.slots < my_rows) {
      fence_proxy_async_smem();                      // generic-proxy reads of the slot before the async-proxy refill
      request(k + p.slots);
    }
  }
  if (give_up) {                                     // copies may still be in flight into this CTA's shared memory
    const long long start = clock64();
    while (clock64() - start < 2000000LL) __nanosleep(1000);
  }
}

// Resident CTAs per SM and ring depth for `rows` rows of `row_bytes` x `operands`: the CTA count per SM
// (2..6) that leaves the least idle time in the last round of rows, with at least two slots each.
inline bool ring_plan(int rows, uint32_t row_bytes, int operands, int sms, int* grid, int* slots, size_t* smem) {
  const size_t budget = 216 * 1024;
  int best_c = 0, best_slots = 0;
  double best_eff = 0.0;
  for (int c = 6; c >= 2; --c) {
    const size_t per_cta = budget / c;
    if (per_cta < row_bytes + 2 * size_t(row_bytes) * operands) continue;
    int sl = int((per_cta - row_bytes) / (size_t(row_bytes) * operands));
    sl = sl > kRingMaxSlots ? kRingMaxSlots : sl;
    const int ctas = sms * c;
    const int rounds = (rows + ctas - 1) / ctas;
    const double eff = rows >= ctas ? double(rows) / (double(rounds) * ctas) : 1.0;
    if (eff > best_eff + 1e-9) { best_eff = eff; best_c = c; best_slots = sl; }
  }
  if (!best_c) return false;
  const int ctas = sms * best_c;
  *grid = rows < ctas ? (rows < 1 ? 1 : rows) : ctas;
  *slots = best_slots;
  *smem = row_bytes + size_t(best_slots) * row_bytes * operands;
  return true;
}

struct Handle {
  int device;
  const __nv_bfloat16 *x, *residual, *weight;
  __nv_bfloat16* out;
  int rows, width;
  float eps;
  int vpt;
  int grid;
  bool ring;                 // rows go through the bulk-copy ring
  int ring_mode, ring_grid, ring_slots;
  size_t ring_smem;
  __nv_bfloat16* residual_out;
};

template <int MODE>
int launch_ring(const Handle* h, cudaStream_t stream) {
  RingParams p{h->x, h->residual, h->weight, h->out, h->residual_out, h->rows, h->width, h->ring_slots, h->eps};
  rmsnorm_ring_kernel<MODE><<<h->ring_grid, kRingThreads, h->ring_smem, stream>>>(p);
  return int(cudaGetLastError());
}

template <int MODE>
int prepare_ring(Handle* h, int device, int operands) {
  h->ring = ring_plan(h->rows, uint32_t(h->width) * 2u, operands, sm_count(device), &h->ring_grid, &h->ring_slots, &h->ring_smem);
  h->ring_mode = MODE;
  if (!h->ring) return 0;
  return int(cudaFuncSetAttribute(rmsnorm_ring_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(h->ring_smem)));
}

template <int kThreads, int VPT>
void launch(const Handle* h, cudaStream_t stream) {
  if (h->residual)
    rmsnorm_kernel<kThreads, VPT, true><<<h->grid, kThreads, 0, stream>>>(h->x, h->residual, h->weight, h->out, h->rows, h->width, h->eps);
  else
    rmsnorm_kernel<kThreads, VPT, false><<<h->grid, kThreads, 0, stream>>>(h->x, nullptr, h->weight, h->out, h->rows, h->width, h->eps);
}

}  // namespace
}  // namespace cake

extern "C" int cake_b200_rmsnorm_create(void** buffers, const cake_b200_rmsnorm_config* config, void** handle_out) {
  using namespace cake;
  if (!buffers || !config || !handle_out) return kErrBadArgument;
  *handle_out = nullptr;
  int device = 0;
  if (int rc = require_blackwell(&device)) return rc;
  const int count = config->fused_residual ? 4 : 3;
  for (int i = 0; i < count; ++i) {
    const bool may_be_empty = config->rows == 0 && i != count - 2;      // only the weight row exists then
    if ((!buffers[i] && !may_be_empty) || (reinterpret_cast<uintptr_t>(buffers[i]) & 15)) return kErrBadArgument;
  }
  if (config->rows < 0 || config->rows > INT32_MAX || config->width <= 0 || (config->width & 7) ||
      config->width > 8 * 8 * kMaxThreads || !(config->epsilon >= 0.f))
    return kErrBadArgument;
  auto* h = new (std::nothrow) Handle;
  if (!h) return int(cudaErrorMemoryAllocation);
  h->device = device;
  int i = 0;
  h->x = static_cast<const __nv_bfloat16*>(buffers[i++]);
  h->residual = config->fused_residual ? static_cast<const __nv_bfloat16*>(buffers[i++]) : nullptr;
  h->weight = static_cast<const __nv_bfloat16*>(buffers[i++]);
  h->out = static_cast<__nv_bfloat16*>(buffers[i++]);
  h->rows = int(config->rows);
  h->width = int(config->width);
  h->eps = config->epsilon;
  const int vectors = h->width / 8;
  // shape class: 0 = 256 threads x 1 vector; 1..4 = 512 threads x 1, 2, 4, 8 vectors
  h->vpt = vectors <= 256 ? 0 : vectors <= 512 ? 1 : vectors <= 1024 ? 2 : vectors <= 2048 ? 3 : 4;
  // persistent CTAs: as many as are resident at once, each walking rows with a stride of the grid
  const int resident = sm_count(device) * (h->vpt == 0 ? 6 : h->vpt == 1 ? 3 : h->vpt == 2 ? 2 : 1);
  h->grid = h->rows < 1 ? 1 : (h->rows < resident ? h->rows : resident);
  h->residual_out = nullptr;
  // rows of up to 16 KiB go through the bulk-copy ring; wider rows stay with the register kernel
  h->ring = false;
  if (h->width <= 8192) {
    const int rc = h->residual ? prepare_ring<kFusedResidual>(h, device, 2) : prepare_ring<kPlain>(h, device, 1);
    if (rc) { delete h; return rc; }
  }
  *handle_out = h;
  return 0;
}

extern "C" int cake_b200_rmsnorm_launch(void* handle, void* cuda_stream) {
  using namespace cake;
  if (!handle) return kErrBadArgument;
  auto* h = static_cast<Handle*>(handle);
  int device = -1;
  CAKE_CUDA_OK(cudaGetDevice(&device));
  if (device != h->device) return kErrWrongDevice;
  if (h->rows == 0) return 0;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
  if (h->ring) return h->residual ? launch_ring<kFusedResidual>(h, stream) : launch_ring<kPlain>(h, stream);
  switch (h->vpt) {
    case 0: launch<256, 1>(h, stream); break;
    case 1: launch<512, 1>(h, stream); break;
    case 2: launch<512, 2>(h, stream); break;
    case 3: launch<512, 4>(h, stream); break;
    default: launch<512, 8>(h, stream); break;
  }
  return int(cudaGetLastError());
}

extern "C" int cake_b200_rmsnorm_destroy(void* handle) {
  delete static_cast<cake::Handle*>(handle);
  return 0;
}

// ---- two-output add + RMSNorm ----------------------------------------------------------------
extern "C" int cake_b200_add_rmsnorm_create(void** buffers, const cake_b200_add_rmsnorm_config* config, void** handle_out) {
  using namespace cake;
  if (!buffers || !config || !handle_out) return kErrBadArgument;
  *handle_out = nullptr;
  int device = 0;
  if (int rc = require_blackwell(&device)) return rc;
  for (int i = 0; i < 5; ++i) {
    const bool may_be_empty = config->rows == 0 && i != 2;              // only the weight row exists then
    if ((!buffers[i] && !may_be_empty) || (reinterpret_cast<uintptr_t>(buffers[i]) & 15)) return kErrBadArgument;
  }
  // the reference bounds a row at 16384 columns (src/open_cake_ir/tasks/add_rmsnorm.py:44); the ring holds two
  // operand rows per slot, which fits up to 8192 columns
  if (config->rows < 0 || config->rows > INT32_MAX || config->width <= 0 || (config->width & 7) || config->width > 8192 ||
      !(config->epsilon >= 0.f))
    return kErrBadArgument;
  auto* h = new (std::nothrow) Handle;
  if (!h) return int(cudaErrorMemoryAllocation);
  *h = Handle{};
  h->device = device;
  h->x = static_cast<const __nv_bfloat16*>(buffers[0]);               // delta
  h->residual = static_cast<const __nv_bfloat16*>(buffers[1]);
  h->weight = static_cast<const __nv_bfloat16*>(buffers[2]);
  h->out = static_cast<__nv_bfloat16*>(buffers[3]);
  h->residual_out = static_cast<__nv_bfloat16*>(buffers[4]);
  h->rows = int(config->rows);
  h->width = int(config->width);
  h->eps = config->epsilon;
  const int rc = prepare_ring<kAddTwoOutputs>(h, device, 2);
  if (rc || !h->ring) { delete h; return rc ? rc : kErrBadArgument; }
  *handle_out = h;
  return 0;
}

extern "C" int cake_b200_add_rmsnorm_launch(void* handle, void* cuda_stream) {
  using namespace cake;
  if (!handle) return kErrBadArgument;
  auto* h = static_cast<Handle*>(handle);
  int device = -1;
  CAKE_CUDA_OK(cudaGetDevice(&device));
  if (device != h->device) return kErrWrongDevice;
  if (h->rows == 0) return 0;
  return launch_ring<kAddTwoOutputs>(h, reinterpret_cast<cudaStream_t>(cuda_stream));
}

extern "C" int cake_b200_add_rmsnorm_destroy(void* handle) {
  delete static_cast<cake::Handle*>(handle);
  return 0;
}

// 0, or the code of a bulk-copy wait that ran out in any RMSNorm launch on the current device since the
// library was loaded (synchronises `cuda_stream`).
extern "C" int cake_b200_rmsnorm_last_status(void* cuda_stream, int* status_out) {
  using namespace cake;
  if (!status_out) return kErrBadArgument;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(cuda_stream);
  CAKE_CUDA_OK(cudaMemcpyFromSymbolAsync(status_out, g_rmsnorm_status, sizeof(int), 0, cudaMemcpyDeviceToHost, s));
  CAKE_CUDA_OK(cudaStreamSynchronize(s));
  return 0;
}
