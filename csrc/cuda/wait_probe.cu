// A one-thread kernel that performs the same bounded flag wait the communication kernels use, with a
// caller-chosen budget.  Tests point it at a flag that nobody raises and check that the kernel returns
// with a kPeerTimeout status instead of spinning: the CUDA context stays usable.
#include "common.cuh"

__global__ void wait_probe_kernel(const unsigned long long* flag, unsigned long long want,
                                  unsigned long long budget_ns, int* status, int detail, int* result) {
  if (blockIdx.x == 0 && threadIdx.x == 0)
    *result = recml::wait_flag_ge(flag, want, budget_ns, status, detail) ? 1 : 0;
}

extern "C" int recml_wait_probe(const unsigned long long* flag, unsigned long long want, unsigned long long budget_ns,
                                int* status, int detail, int* result, cudaStream_t stream) {
  wait_probe_kernel<<<1, 32, 0, stream>>>(flag, want, budget_ns, status, detail, result);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
