// RMSNorm for sm_100a: one CTA per row, the row held in registers between the reduction and the
// scaling, 128-bit loads and stores, fp32 arithmetic, one bf16 rounding of the result.
//
// Operators:
//   out[r,c] = bf16( z[r,c] * weight[c] / sqrt(mean_j z[r,j]^2 + eps) ),  z = x or fp32(x + residual)
//     (src/open_cake_ir/tasks/solx_fib/workload.py:214-218, oracle :334-358), and the two-output form
//   z = bf16(delta + residual); residual_out = z; out = bf16( fp32(z) * rsqrt(mean z^2 + eps) * weight )
//     (src/open_cake_ir/tasks/add_rmsnorm.py:66, oracle :131-143): the sum is rounded to bf16 FIRST, and the
//     rounded row is both what is written back and what is normalised.
// The kernel is bound by HBM traffic: 2 bytes in and 2 out per element and operand, plus the weight row.
// (A variant that staged rows in shared memory through a ring of bulk copies, several rows ahead, was built
// and measured: 18.4 to 25.5 us on 4096 x 4096 against 15.9 us for this kernel and 14.3 us for a plain copy of
// the same bytes -- a row's wait -> reduce -> write chain per CTA costs more than the deeper prefetch gains.)
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
// MODE: 0 = x only; 1 = z = fp32(x + residual); 2 = z = bf16(x + residual), also written to residual_out.
template <int kThreads, int VPT, int MODE>
__global__ void __launch_bounds__(kThreads, VPT == 1 ? 1536 / kThreads : ((2048 / kThreads) / VPT > 0 ? (2048 / kThreads) / VPT : 1))
rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
               const __nv_bfloat16* __restrict__ weight, __nv_bfloat16* __restrict__ out,
               __nv_bfloat16* __restrict__ residual_out, int rows, int width, float eps) {
  constexpr bool RESIDUAL = MODE != 0;
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
        for (int j = 0; j < 8; ++j) z[RESIDUAL ? i : 0][j] += r[j];
        if (MODE == 2) {                     // the rounding seam: the bf16 sum is returned and normalised
          float* zz = z[RESIDUAL ? i : 0];
          uint4 q;
          q.x = pack_bf16x2(zz[0], zz[1]); q.y = pack_bf16x2(zz[2], zz[3]); q.z = pack_bf16x2(zz[4], zz[5]); q.w = pack_bf16x2(zz[6], zz[7]);
          unpack8(q, zz);
          if (idx < vectors) st_stream(reinterpret_cast<uint4*>(residual_out + size_t(row) * width) + idx, q);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(z[RESIDUAL ? i : 0][j], z[RESIDUAL ? i : 0][j], ss);
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

struct Handle {
  int device;
  const __nv_bfloat16 *x, *residual, *weight;
  __nv_bfloat16 *out, *residual_out;
  int rows, width;
  float eps;
  int vpt;
  int grid;
};

inline void choose_shape(Handle* h, int device) {
  const int vectors = h->width / 8;
  // shape class: 0 = 256 threads x 1 vector; 1..4 = 512 threads x 1, 2, 4, 8 vectors
  h->vpt = vectors <= 256 ? 0 : vectors <= 512 ? 1 : vectors <= 1024 ? 2 : vectors <= 2048 ? 3 : 4;
  // persistent CTAs: as many as are resident at once, each walking rows with a stride of the grid
  const int resident = sm_count(device) * (h->vpt == 0 ? 6 : h->vpt == 1 ? 3 : h->vpt == 2 ? 2 : 1);
  h->grid = h->rows < 1 ? 1 : (h->rows < resident ? h->rows : resident);
}

template <int kThreads, int VPT>
void launch(const Handle* h, cudaStream_t stream) {
  if (h->residual_out)
    rmsnorm_kernel<kThreads, VPT, 2><<<h->grid, kThreads, 0, stream>>>(h->x, h->residual, h->weight, h->out, h->residual_out, h->rows, h->width, h->eps);
  else if (h->residual)
    rmsnorm_kernel<kThreads, VPT, 1><<<h->grid, kThreads, 0, stream>>>(h->x, h->residual, h->weight, h->out, nullptr, h->rows, h->width, h->eps);
  else
    rmsnorm_kernel<kThreads, VPT, 0><<<h->grid, kThreads, 0, stream>>>(h->x, nullptr, h->weight, h->out, nullptr, h->rows, h->width, h->eps);
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
  h->residual_out = nullptr;
  h->rows = int(config->rows);
  h->width = int(config->width);
  h->eps = config->epsilon;
  choose_shape(h, device);
  *handle_out = h;
  return 0;
}

static int rmsnorm_launch_any(void* handle, void* cuda_stream) {
  using namespace cake;
  if (!handle) return kErrBadArgument;
  auto* h = static_cast<Handle*>(handle);
  int device = -1;
  CAKE_CUDA_OK(cudaGetDevice(&device));
  if (device != h->device) return kErrWrongDevice;
  if (h->rows == 0) return 0;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
  switch (h->vpt) {
    case 0: launch<256, 1>(h, stream); break;
    case 1: launch<512, 1>(h, stream); break;
    case 2: launch<512, 2>(h, stream); break;
    case 3: launch<512, 4>(h, stream); break;
    default: launch<512, 8>(h, stream); break;
  }
  return int(cudaGetLastError());
}

extern "C" int cake_b200_rmsnorm_launch(void* handle, void* cuda_stream) { return rmsnorm_launch_any(handle, cuda_stream); }

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
  // the reference bounds a row at 16384 columns (src/open_cake_ir/tasks/add_rmsnorm.py:44)
  if (config->rows < 0 || config->rows > INT32_MAX || config->width <= 0 || (config->width & 7) ||
      config->width > 8 * 8 * kMaxThreads || !(config->epsilon >= 0.f))
    return kErrBadArgument;
  auto* h = new (std::nothrow) Handle;
  if (!h) return int(cudaErrorMemoryAllocation);
  h->device = device;
  h->x = static_cast<const __nv_bfloat16*>(buffers[0]);               // delta
  h->residual = static_cast<const __nv_bfloat16*>(buffers[1]);
  h->weight = static_cast<const __nv_bfloat16*>(buffers[2]);
  h->out = static_cast<__nv_bfloat16*>(buffers[3]);
  h->residual_out = static_cast<__nv_bfloat16*>(buffers[4]);
  h->rows = int(config->rows);
  h->width = int(config->width);
  h->eps = config->epsilon;
  choose_shape(h, device);
  *handle_out = h;
  return 0;
}

extern "C" int cake_b200_add_rmsnorm_launch(void* handle, void* cuda_stream) { return rmsnorm_launch_any(handle, cuda_stream); }

extern "C" int cake_b200_add_rmsnorm_destroy(void* handle) {
  delete static_cast<cake::Handle*>(handle);
  return 0;
}
