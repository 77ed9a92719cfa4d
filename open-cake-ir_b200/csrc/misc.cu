// Library identification and the status-word reader of the C ABI.
#include "common.cuh"
#include "../../include/cake_b200.h"

extern "C" int cake_b200_abi_version(void) { return 1; }

extern "C" int cake_b200_read_status(const void* workspace, void* cuda_stream, int* status_out) {
  if (!workspace || !status_out) return cake::kErrBadArgument;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(cuda_stream);
  CAKE_CUDA_OK(cudaMemcpyAsync(status_out, workspace, sizeof(int), cudaMemcpyDeviceToHost, s));
  CAKE_CUDA_OK(cudaStreamSynchronize(s));
  return 0;
}
