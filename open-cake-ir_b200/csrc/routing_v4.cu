// DeepSeek-V4 routing stages for sm_100a: the MoE gate (sqrt-softplus scores, 384 experts, top-6) and the
// CSA indexer top-k (the 1024 best of 2048 scores, in descending order).
//
// Operators: src/open_cake_ir/tasks/deepseek_v4/workload.py:46-108 (contracts), oracle :184-202.
//   gate:    score = fp32(sqrt(log1p(exp(x)))); expert_ids = top_k of (score + selection_bias), descending;
//            weights = fp32(route_scale * score[ids] / sum(score[ids]))
//   indexer: indices[q, :] = positions of the top_k largest index_scores[q, :], descending
// Indices are compared bit for bit by the contract, so every order decision is made on exactly the numbers
// the oracle ranks: the gate evaluates the score in double and rounds it to fp32 as the oracle does, and
// ranks the DOUBLE sum score + bias (two fp32 values: exact); both kernels break ties, which the contract
// excludes, towards the lower index.  Both are small integer/compare kernels: a warp per token for the
// gate (lane-strided experts, warp-shuffle arg-max per selection), a CTA per row for the indexer (bitonic
// sort of 64-bit keys in shared memory).
#include "common.cuh"
#include "../../include/cake_b200.h"
#include <new>

namespace cake {
namespace v4 {

constexpr int kMaxExpertsPerLane = 16;     // experts <= 512

// double -> unsigned key with the same order (-0.0 folded onto +0.0)
__device__ __forceinline__ unsigned long long ordered_bits64(double v) {
  unsigned long long b = (unsigned long long)__double_as_longlong(v);
  if ((b << 1) == 0) b = 0;
  return (b >> 63) ? ~b : (b | 0x8000000000000000ull);
}

// One warp per token; lane l holds experts j*32 + l.
__global__ void __launch_bounds__(128)
gate_kernel(const float* __restrict__ logits, const float* __restrict__ bias, float* __restrict__ weights,
            int* __restrict__ expert_ids, int tokens, int experts, int top_k, float route_scale) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int token = blockIdx.x * 4 + warp;
  if (token >= tokens) return;
  float score[kMaxExpertsPerLane];
  unsigned long long key[kMaxExpertsPerLane];      // 0 = absent or already taken
#pragma unroll
  for (int j = 0; j < kMaxExpertsPerLane; ++j) {
    const int id = j * 32 + lane;
    score[j] = 0.f;
    key[j] = 0ull;
    if (id < experts) {
      const double x = double(__ldg(logits + size_t(token) * experts + id));
      score[j] = float(sqrt(log1p(exp(x))));
      key[j] = ordered_bits64(double(score[j]) + double(__ldg(bias + id)));
    }
  }
  double picked = 0.0;       // lane k keeps the score of the k-th selection
  int picked_id = 0;
  for (int k = 0; k < top_k; ++k) {
    unsigned long long best = 0ull;
    int best_id = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kMaxExpertsPerLane; ++j)
      if (key[j] > best) { best = key[j]; best_id = j * 32 + lane; }     // ascending j: the lane's lowest id wins its ties
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
      const int other_id = __shfl_xor_sync(0xffffffffu, best_id, o);
      if (other > best || (other == best && other_id < best_id)) { best = other; best_id = other_id; }
    }
    const int owner = best_id & 31, slot = best_id >> 5;
    float value = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxExpertsPerLane; ++j)
      if (j == slot) { value = score[j]; if (lane == owner) key[j] = 0ull; }
    value = __shfl_sync(0xffffffffu, value, owner);
    if (lane == k) { picked = double(value); picked_id = best_id; }
  }
  double total = 0.0;        // six fp32 values of similar size: the double sum is exact, as the oracle's fsum is
  for (int k = 0; k < top_k; ++k) total += __shfl_sync(0xffffffffu, picked, k);
  if (lane < top_k) {
    weights[size_t(token) * top_k + lane] = float(double(route_scale) * picked / total);
    expert_ids[size_t(token) * top_k + lane] = picked_id;
  }
}

// fp32 -> unsigned key with the same order (-0.0 folded onto +0.0), index in the low half so that equal
// scores order by ascending index when keys are sorted descending.
__device__ __forceinline__ unsigned long long score_key(float v, int id) {
  uint32_t b = __float_as_uint(v);
  if ((b << 1) == 0) b = 0;
  b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  return (static_cast<unsigned long long>(b) << 32) | (0xffffffffu - uint32_t(id));
}

// One CTA per row: bitonic sort (descending) of kSortWidth keys in shared memory, two keys per thread.
constexpr int kSortWidth = 2048;
__global__ void __launch_bounds__(kSortWidth / 2)
topk_sort_kernel(const float* __restrict__ scores, int* __restrict__ indices, int candidates, int top_k) {
  __shared__ unsigned long long keys[kSortWidth];
  const size_t row = blockIdx.x;
  for (int i = threadIdx.x; i < kSortWidth; i += blockDim.x)
    keys[i] = i < candidates ? score_key(__ldg(scores + row * candidates + i), i) : 0ull;    // padding sorts last
  __syncthreads();
  for (int size = 2; size <= kSortWidth; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      const int t = threadIdx.x;
      const int lo = 2 * t - (t & (stride - 1));         // index with the `stride` bit clear
      const int hi = lo + stride;
      const bool descending = (lo & size) == 0;
      const unsigned long long a = keys[lo], b = keys[hi];
      if ((a < b) == descending) { keys[lo] = b; keys[hi] = a; }
      __syncthreads();
    }
  }
  for (int i = threadIdx.x; i < top_k; i += blockDim.x)
    indices[row * top_k + i] = int(0xffffffffu - uint32_t(keys[i] & 0xffffffffull));
}

struct GateHandle {
  int device;
  const float *logits, *bias;
  float* weights;
  int* ids;
  cake_b200_v4_gate_config cfg;
};
struct TopkHandle {
  int device;
  const float* scores;
  int* indices;
  cake_b200_topk_config cfg;
};

}  // namespace v4
}  // namespace cake

extern "C" int cake_b200_v4_moe_gate_create(void** buffers, const cake_b200_v4_gate_config* config, void** handle_out) {
  using namespace cake;
  if (!buffers || !config || !handle_out) return kErrBadArgument;
  *handle_out = nullptr;
  int device = 0;
  if (int rc = require_blackwell(&device)) return rc;
  for (int i = 0; i < 4; ++i) {
    const bool may_be_empty = config->tokens == 0 && i != 1;            // only the bias exists then
    if ((!buffers[i] && !may_be_empty) || (reinterpret_cast<uintptr_t>(buffers[i]) & 3)) return kErrBadArgument;
  }
  if (config->tokens < 0 || config->tokens > (1 << 24) || config->experts <= 0 || config->experts > 32 * v4::kMaxExpertsPerLane ||
      config->top_k <= 0 || config->top_k > 32 || config->top_k > config->experts || !(config->route_scale > 0.f))
    return kErrBadArgument;
  auto* h = new (std::nothrow) v4::GateHandle;
  if (!h) return int(cudaErrorMemoryAllocation);
  h->device = device;
  h->logits = static_cast<const float*>(buffers[0]);
  h->bias = static_cast<const float*>(buffers[1]);
  h->weights = static_cast<float*>(buffers[2]);
  h->ids = static_cast<int*>(buffers[3]);
  h->cfg = *config;
  *handle_out = h;
  return 0;
}
extern "C" int cake_b200_v4_moe_gate_launch(void* handle, void* cuda_stream) {
  using namespace cake;
  if (!handle) return kErrBadArgument;
  auto* h = static_cast<v4::GateHandle*>(handle);
  int device = -1;
  CAKE_CUDA_OK(cudaGetDevice(&device));
  if (device != h->device) return kErrWrongDevice;
  if (h->cfg.tokens == 0) return 0;
  const int tokens = int(h->cfg.tokens);
  v4::gate_kernel<<<(tokens + 3) / 4, 128, 0, reinterpret_cast<cudaStream_t>(cuda_stream)>>>(
      h->logits, h->bias, h->weights, h->ids, tokens, h->cfg.experts, h->cfg.top_k, h->cfg.route_scale);
  return int(cudaGetLastError());
}
extern "C" int cake_b200_v4_moe_gate_destroy(void* handle) {
  delete static_cast<cake::v4::GateHandle*>(handle);
  return 0;
}

extern "C" int cake_b200_csa_topk_create(void** buffers, const cake_b200_topk_config* config, void** handle_out) {
  using namespace cake;
  if (!buffers || !config || !handle_out) return kErrBadArgument;
  *handle_out = nullptr;
  int device = 0;
  if (int rc = require_blackwell(&device)) return rc;
  for (int i = 0; i < 2; ++i) if ((!buffers[i] && config->rows != 0) || (reinterpret_cast<uintptr_t>(buffers[i]) & 3)) return kErrBadArgument;
  if (config->rows < 0 || config->rows > (1 << 24) || config->candidates <= 0 || config->candidates > v4::kSortWidth ||
      config->top_k <= 0 || config->top_k > config->candidates)
    return kErrBadArgument;
  auto* h = new (std::nothrow) v4::TopkHandle;
  if (!h) return int(cudaErrorMemoryAllocation);
  h->device = device;
  h->scores = static_cast<const float*>(buffers[0]);
  h->indices = static_cast<int*>(buffers[1]);
  h->cfg = *config;
  *handle_out = h;
  return 0;
}
extern "C" int cake_b200_csa_topk_launch(void* handle, void* cuda_stream) {
  using namespace cake;
  if (!handle) return kErrBadArgument;
  auto* h = static_cast<v4::TopkHandle*>(handle);
  int device = -1;
  CAKE_CUDA_OK(cudaGetDevice(&device));
  if (device != h->device) return kErrWrongDevice;
  if (h->cfg.rows == 0) return 0;
  v4::topk_sort_kernel<<<int(h->cfg.rows), v4::kSortWidth / 2, 0, reinterpret_cast<cudaStream_t>(cuda_stream)>>>(
      h->scores, h->indices, h->cfg.candidates, h->cfg.top_k);
  return int(cudaGetLastError());
}
extern "C" int cake_b200_csa_topk_destroy(void* handle) {
  delete static_cast<cake::v4::TopkHandle*>(handle);
  return 0;
}
