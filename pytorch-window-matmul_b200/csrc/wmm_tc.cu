// tcgen05 / TMA kernels for the banded contractions (16-bit inputs).  Placeholder until the kernels land:
// nothing is eligible, so every problem takes the CUDA-core family.
#include "wmm_common.cuh"

namespace wmm {

__device__ unsigned long long g_device_status = 0ull;

cudaError_t read_device_status(unsigned long long *word, bool clear) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(word, g_device_status, sizeof(*word));
  if (e == cudaSuccess && clear && *word) {
    const unsigned long long zero = 0;
    e = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(zero));
  }
  return e;
}

bool tensor_eligible(Primitive, const Problem &) { return false; }

cudaError_t launch_tensor(Primitive, const Problem &, cudaStream_t, int *) { return cudaErrorNotSupported; }

}  // namespace wmm
