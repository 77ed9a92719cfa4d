// Dense block-scaled FP8 GEMM entry points (C ABI) on top of the shared tcgen05 core.
#include "gemm_fp8.cuh"
#include "../../include/cake_b200.h"
#include <new>

namespace cake {
namespace {

struct DenseHandle {
  int device;
  CUtensorMap map_a, map_a_tail, map_b;
  gemm::Params params;
  int grid;
  int* status;
};

}  // namespace
}  // namespace cake

void cake::gemm_launch_facts(int* threads, int* dynamic_shared_bytes) {
  *threads = cake::gemm::kThreads;
  *dynamic_shared_bytes = int(cake::gemm::kSmemBytes);
}

extern "C" size_t cake_b200_block_scaled_gemm_workspace_bytes(const cake_b200_gemm_config*) { return 256; }

extern "C" int cake_b200_block_scaled_gemm_create(void** buffers, const cake_b200_gemm_config* config,
                                                  void** handle_out) {
  using namespace cake;
  if (!buffers || !config || !handle_out) return kErrBadArgument;
  *handle_out = nullptr;
  int device = 0;
  if (int rc = require_blackwell(&device)) return rc;
  for (int i = 0; i < 6; ++i)
    if (!buffers[i] || (reinterpret_cast<uintptr_t>(buffers[i]) & 15)) return kErrBadArgument;
  const int64_t m = config->m, n = config->n, k = config->k;
  if (m <= 0 || n <= 0 || k <= 0 || (k % gemm::kBK) || (n % 128) || m > INT32_MAX / 2 || n > INT32_MAX / 2)
    return kErrBadArgument;
  auto* h = new (std::nothrow) DenseHandle;
  if (!h) return int(cudaErrorMemoryAllocation);
  h->device = device;
  int rc = make_tensor_map_u8_sw128(&h->map_a, buffers[0], uint64_t(m), uint64_t(k), gemm::kBM);
  if (!rc) rc = make_tensor_map_u8_sw128(&h->map_a_tail, buffers[0], uint64_t(m), uint64_t(k), gemm::kTailRows);
  if (!rc) rc = make_tensor_map_u8_sw128(&h->map_b, buffers[2], uint64_t(n), uint64_t(k), gemm::kBN);
  if (!rc) rc = int(cudaFuncSetAttribute(gemm::gemm_fp8_kernel<gemm::kDense>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, int(gemm::kSmemBytes)));
  if (rc) { delete h; return rc; }
  gemm::Params& p = h->params;
  p = gemm::Params{};
  p.n = int(n);
  p.k_blocks = p.b_k_blocks = int(k / gemm::kBK);
  p.b_rows_per_group = int(n);
  p.groups = 1;
  p.row_capacity = int(m);
  p.offsets = nullptr;
  p.dense_rows = int(m);
  p.sfa = static_cast<const float*>(buffers[1]);
  p.sfb = static_cast<const float*>(buffers[3]);
  p.out = buffers[4];
  h->status = static_cast<int*>(buffers[5]);
  p.status = h->status;
  p.queue = h->status + 4;               // work-item counter, inside the 256-byte status block
  const long long items = ((m + gemm::kBM - 1) / gemm::kBM) * ((n + gemm::kBN - 1) / gemm::kBN);
  const int sms = sm_count(device);
  h->grid = int(items < sms ? items : sms);
  *handle_out = h;
  return 0;
}

extern "C" int cake_b200_block_scaled_gemm_launch(void* handle, void* cuda_stream) {
  using namespace cake;
  if (!handle) return kErrBadArgument;
  auto* h = static_cast<DenseHandle*>(handle);
  int device = -1;
  CAKE_CUDA_OK(cudaGetDevice(&device));
  if (device != h->device) return kErrWrongDevice;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
  CAKE_CUDA_OK(cudaMemsetAsync(h->status, 0, 8 * sizeof(int), stream));     // status word and work-item counter
  gemm::Params p = h->params;
  p.wait_kiloclocks = test_hooks().budget_kiloclocks;
  p.skip_load = test_hooks().skip_load;
  gemm::gemm_fp8_kernel<gemm::kDense><<<h->grid, gemm::kThreads, gemm::kSmemBytes, stream>>>(h->map_a, h->map_a_tail, h->map_b, p);
  return int(cudaGetLastError());
}

extern "C" int cake_b200_block_scaled_gemm_destroy(void* handle) {
  delete static_cast<cake::DenseHandle*>(handle);
  return 0;
}
