// Shared device helpers for the sm_100a kernels of this library.
//
// Conventions used by every kernel here:
//  * every spin-wait (mbarrier, peer flag) is bounded by a wall-clock budget read from
//    %globaltimer; when it runs out the kernel records a status code and returns
//    normally, so the CUDA context stays usable and the host raises an error;
//  * status word layout: [0] = first error code (0 = ok), [1] = detail (peer / phase).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace recml {

enum StatusCode : int {
  kOk = 0,
  kMbarTimeout = 1,      // an mbarrier phase never completed
  kPeerTimeout = 2,      // a peer rank never raised its flag
  kBadArgument = 3,
  kCapacity = 4,         // a fixed-capacity buffer overflowed
  kBadIndex = 5,         // an input id lies outside its table (the access is skipped)
};

constexpr unsigned long long kDefaultWaitNs = 2000000000ull;  // 2 s

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void report(int* status, int code, int detail) {
  if (status != nullptr && atomicCAS(status, 0, code) == 0) status[1] = detail;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- system-scope flags used between GPUs -----------------------------------------------
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Waits until *flag >= want.  Returns false (and reports) when the budget runs out.
__device__ __forceinline__ bool wait_flag_ge(const unsigned long long* flag, unsigned long long want,
                                             unsigned long long budget_ns, int* status, int detail) {
  if (ld_acquire_sys(flag) >= want) return true;
  const unsigned long long t0 = global_ns();
  for (;;) {
    for (int i = 0; i < 64; ++i) {
      if (ld_acquire_sys(flag) >= want) return true;
      __nanosleep(64);
    }
    if (global_ns() - t0 > budget_ns) {
      report(status, kPeerTimeout, detail);
      return false;
    }
  }
}

// Sequence numbers of peer flags can come from device memory (so that a captured CUDA graph sees a
// new value on every replay): effective = *ptr * mul + add when ptr is set, else the literal.
struct SeqRef {
  const unsigned long long* ptr;
  unsigned long long mul, add, literal;
};
__device__ __forceinline__ unsigned long long seq_of(const SeqRef& s) {
  return s.ptr != nullptr ? (*s.ptr) * s.mul + s.add : s.literal;
}

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Kernels meant to share the SMs with a tensor-core GEMM of another stream ask for the largest shared-memory
// carve-out although they need little of it: an SM keeps one L1 / shared-memory split for all the blocks
// resident on it, so a kernel that configured it for a large L1 would keep the GEMM's CTAs (which need
// ~210 KB of shared memory) off that SM until it has drained.
template <typename Kernel>
inline void prefer_max_shared_carveout(Kernel kernel) {
  cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

}  // namespace recml
