// Library identification and the status-word reader of the C ABI.
#include "common.cuh"
#include <string>
#include "../../include/cake_b200.h"

extern "C" int cake_b200_abi_version(void) { return 1; }

extern "C" int cake_b200_launch_facts(const char* kernel, int* threads_per_cta, int* dynamic_shared_bytes) {
  if (!kernel || !threads_per_cta || !dynamic_shared_bytes) return cake::kErrBadArgument;
  const std::string name(kernel);
  if (name == "gemm_fp8_kernel") cake::gemm_launch_facts(threads_per_cta, dynamic_shared_bytes);
  else if (name == "gqa_decode_kernel") cake::gqa_decode_launch_facts(threads_per_cta, dynamic_shared_bytes);
  else if (name == "mla_decode_kernel") cake::mla_decode_launch_facts(threads_per_cta, dynamic_shared_bytes);
  else return cake::kErrBadArgument;
  return 0;
}

extern "C" int cake_b200_decode_plan_view(const char* kind, void* handle, int which, void** device_pointer_out, int* count_out) {
  if (!kind || !handle || !device_pointer_out || !count_out) return cake::kErrBadArgument;
  const std::string name(kind);
  if (name == "gqa_decode") return cake::gqa_decode_plan_view(handle, which, device_pointer_out, count_out);
  if (name == "mla_decode") return cake::mla_decode_plan_view(handle, which, device_pointer_out, count_out);
  return cake::kErrBadArgument;
}

extern "C" int cake_b200_test_hooks(int wait_budget_kiloclocks, int skip_load) {
  if (wait_budget_kiloclocks < 0) return cake::kErrBadArgument;
  cake::test_hooks().budget_kiloclocks = wait_budget_kiloclocks;
  cake::test_hooks().skip_load = skip_load ? 1 : 0;
  return 0;
}

extern "C" int cake_b200_read_status(const void* workspace, void* cuda_stream, int* status_out) {
  if (!workspace || !status_out) return cake::kErrBadArgument;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(cuda_stream);
  CAKE_CUDA_OK(cudaMemcpyAsync(status_out, workspace, sizeof(int), cudaMemcpyDeviceToHost, s));
  CAKE_CUDA_OK(cudaStreamSynchronize(s));
  return 0;
}
