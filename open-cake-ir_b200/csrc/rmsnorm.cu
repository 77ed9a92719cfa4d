// RMSNorm for sm_100a: one CTA per row, the row held in registers between the reduction and the
// scaling, 128-bit loads and stores, fp32 arithmetic, one bf16 rounding.
//
// Operator (src/open_cake_ir/tasks/solx_fib/workload.py:214-218, oracle :334-358):
//   out[r,c] = bf16( z[r,c] * weight[c] / sqrt(mean_j z[r,j]^2 + eps) ),  z = x or fp32(x + residual).
// The kernel is bound by HBM traffic: 2*rows*width*2 bytes + the weight row.
#include "common.cuh"
#include "../../include/cake_b200.h"
#include <new>

namespace cake {
namespace {

constexpr int kThreads = 256;

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

// VPT = 16-byte vectors per thread; a row has width/8 vectors, at most VPT*kThreads.
template <int VPT, bool RESIDUAL>
__global__ void __launch_bounds__(kThreads)
rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
               const __nv_bfloat16* __restrict__ weight, __nv_bfloat16* __restrict__ out,
               int rows, int width, float eps) {
  __shared__ float partial[2][kThreads / 32];
  const int vectors = width >> 3;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float w[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * kThreads;
    if (idx < vectors) unpack8(__ldg(reinterpret_cast<const uint4*>(weight) + idx), w[i]);
  }
  const float inv_width = 1.f / float(width);
  int flip = 0;
  for (int row = blockIdx.x; row < rows; row += gridDim.x, flip ^= 1) {
    const uint4* src = reinterpret_cast<const uint4*>(x + size_t(row) * width);
    float v[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * kThreads;
      if (idx < vectors) {
        unpack8(ld_stream(src + idx), v[i]);
        if (RESIDUAL) {
          float r[8];
          unpack8(ld_stream(reinterpret_cast<const uint4*>(residual + size_t(row) * width) + idx), r);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] += r[j];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(v[i][j], v[i][j], ss);
      }
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
        uint4 o;
        o.x = pack_bf16x2(v[i][0] * inverse * w[i][0], v[i][1] * inverse * w[i][1]);
        o.y = pack_bf16x2(v[i][2] * inverse * w[i][2], v[i][3] * inverse * w[i][3]);
        o.z = pack_bf16x2(v[i][4] * inverse * w[i][4], v[i][5] * inverse * w[i][5]);
        o.w = pack_bf16x2(v[i][6] * inverse * w[i][6], v[i][7] * inverse * w[i][7]);
        st_stream(dst + idx, o);
      }
    }
  }
}

struct Handle {
  int device;
  const __nv_bfloat16 *x, *residual, *weight;
  __nv_bfloat16* out;
  int rows, width;
  float eps;
  int vpt;
  int grid;
};

template <int VPT>
void launch(const Handle* h, cudaStream_t stream) {
  if (h->residual)
    rmsnorm_kernel<VPT, true><<<h->grid, kThreads, 0, stream>>>(h->x, h->residual, h->weight, h->out, h->rows, h->width, h->eps);
  else
    rmsnorm_kernel<VPT, false><<<h->grid, kThreads, 0, stream>>>(h->x, nullptr, h->weight, h->out, h->rows, h->width, h->eps);
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
      config->width > 8 * 8 * kThreads || !(config->epsilon >= 0.f))
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
  const int need = (vectors + kThreads - 1) / kThreads;
  h->vpt = need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 8;
  h->grid = h->rows < 1 ? 1 : (h->rows < sm_count(device) * 64 ? h->rows : sm_count(device) * 64);
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
  switch (h->vpt) {
    case 1: launch<1>(h, stream); break;
    case 2: launch<2>(h, stream); break;
    case 4: launch<4>(h, stream); break;
    default: launch<8>(h, stream); break;
  }
  return int(cudaGetLastError());
}

extern "C" int cake_b200_rmsnorm_destroy(void* handle) {
  delete static_cast<cake::Handle*>(handle);
  return 0;
}
