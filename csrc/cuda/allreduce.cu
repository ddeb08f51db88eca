// Dense-gradient all-reduce over NVLink peer memory with the bf16 cast and the 1/W (and loss-scale)
// factor fused in.  Two-shot algorithm on symmetric buffers:
//   pack    fp32 gradients of a bucket -> bf16 in this rank's `in` buffer; flag A to all peers
//   reduce  rank r owns slice r of the bucket: waits for flag A from every peer, loads that slice
//           from all W ranks with peer loads, sums in fp32, scales, and stores the bf16 result
//           into every rank's `out` buffer with peer stores; flag B to all peers
//   unpack  waits for flag B from every peer, converts `out` back into the fp32 gradient tensors
// Traffic per rank: (W-1)/W of the bucket in and the same out — the two-shot optimum, at full
// NVSwitch bandwidth to all peers at once.  Flags are sequence numbers; waits are bounded.
// When the symmetric buffers are bound to an NVLink multicast object the reduce step instead issues
// `multimem.ld_reduce` (the switch sums the W copies of the slice, fp32 accumulation) and
// `multimem.st` (the switch stores the result into every rank's `out`), so each rank moves only
// 1/W of the bucket in and out over its own links.
#include "common.cuh"

namespace recml {
namespace ar {

constexpr int kMaxWorld = 8;
constexpr int kMaxTensors = 64;

struct Bucket {
  float* grad[kMaxTensors];
  long long numel[kMaxTensors];
  long long offset[kMaxTensors];       // element offset of the tensor inside the bucket (multiple of 8)
  long long block_start[kMaxTensors + 1];  // prefix of 2048-element blocks
  int n;
};

struct Comm {
  __nv_bfloat16* in[kMaxWorld];        // every rank's input buffer (peer addresses)
  __nv_bfloat16* out[kMaxWorld];
  unsigned long long* flag_a[kMaxWorld];  // address of flagA[me] on rank r
  unsigned long long* flag_b[kMaxWorld];
  const unsigned long long* my_flag_a;    // flagA[0..W) on this rank
  const unsigned long long* my_flag_b;
  unsigned int* done_counter;
  int W, me;
  SeqRef seq;
  long long total;                     // bucket elements, multiple of 8*W
  float scale;
  int* status;
  __nv_bfloat16* mc_in;                // multicast address of `in` (nullptr: plain peer loads / stores)
  __nv_bfloat16* mc_out;
};

__device__ __forceinline__ void signal_all(unsigned int* done_counter, unsigned long long* const* flags, int W,
                                           unsigned long long seq) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(done_counter, 1u) == gridDim.x - 1) {
      *done_counter = 0;
      __threadfence_system();
      for (int r = 0; r < W; ++r) st_release_sys(flags[r], seq);
    }
  }
}

__device__ __forceinline__ bool wait_all(const unsigned long long* flags, int W, unsigned long long seq, int* status,
                                         int chan) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < W && !wait_flag_ge(flags + threadIdx.x, seq, kDefaultWaitNs, status, chan * 16 + threadIdx.x)) ok = 0;
  __syncthreads();
  return ok != 0;
}

__global__ void __launch_bounds__(256) pack_kernel(const Bucket b, const Comm c) {
  int t = 0;
  while (t + 1 < b.n && static_cast<long long>(blockIdx.x) >= b.block_start[t + 1]) ++t;
  const long long base = (blockIdx.x - b.block_start[t]) * 2048LL;
  const float* g = b.grad[t];
  __nv_bfloat16* dst = c.in[c.me] + b.offset[t];
  const long long n = b.numel[t];
  for (int i = threadIdx.x * 8; i < 2048; i += blockDim.x * 8) {
    const long long j = base + i;
    if (j >= n) break;
    float x[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] = (j + e < n) ? g[j + e] : 0.f;
    *reinterpret_cast<uint4*>(dst + j) = make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]),
                                                    pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
  }
  signal_all(c.done_counter, c.flag_a, c.W, seq_of(c.seq));
}

// In-switch reduction of one 16-byte vector of bf16 pairs over all ranks bound to the multicast object.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
// One 16-byte store that the switch replicates into every bound rank's copy.
__device__ __forceinline__ void multimem_st_16(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               :: "l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__global__ void __launch_bounds__(256) reduce_nvls_kernel(const Comm c) {
  const unsigned long long seq = seq_of(c.seq);
  if (!wait_all(c.my_flag_a, c.W, seq, c.status, 8)) return;
  const long long slice = c.total / c.W;
  const long long lo = slice * c.me;
  const long long nvec = slice / 8;
  for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < nvec;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = lo + v * 8;
    const uint4 t = multimem_ld_reduce_bf16x8(c.mc_in + e);
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = pack_bf16(bf16_lo(w[j]) * c.scale, bf16_hi(w[j]) * c.scale);
    multimem_st_16(c.mc_out + e, make_uint4(o[0], o[1], o[2], o[3]));
  }
  signal_all(c.done_counter + 1, c.flag_b, c.W, seq);
}

__global__ void __launch_bounds__(256) reduce_kernel(const Comm c) {
  const unsigned long long seq = seq_of(c.seq);
  if (!wait_all(c.my_flag_a, c.W, seq, c.status, 8)) return;
  const long long slice = c.total / c.W;
  const long long lo = slice * c.me;
  const long long nvec = slice / 8;
  for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < nvec;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = lo + v * 8;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int r = 0; r < c.W; ++r) {
      const int src = (c.me + r) % c.W;   // stagger peers so the ranks do not all hit the same one
      const uint4 t = __ldcg(reinterpret_cast<const uint4*>(c.in[src] + e));
      const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) { acc[2 * j] += bf16_lo(w[j]); acc[2 * j + 1] += bf16_hi(w[j]); }
    }
    const uint4 o = make_uint4(pack_bf16(acc[0] * c.scale, acc[1] * c.scale), pack_bf16(acc[2] * c.scale, acc[3] * c.scale),
                               pack_bf16(acc[4] * c.scale, acc[5] * c.scale), pack_bf16(acc[6] * c.scale, acc[7] * c.scale));
    for (int r = 0; r < c.W; ++r) {
      const int dst = (c.me + r) % c.W;
      *reinterpret_cast<uint4*>(c.out[dst] + e) = o;
    }
  }
  signal_all(c.done_counter + 1, c.flag_b, c.W, seq);
}

__global__ void __launch_bounds__(256) unpack_kernel(const Bucket b, const Comm c) {
  if (!wait_all(c.my_flag_b, c.W, seq_of(c.seq), c.status, 9)) return;
  int t = 0;
  while (t + 1 < b.n && static_cast<long long>(blockIdx.x) >= b.block_start[t + 1]) ++t;
  const long long base = (blockIdx.x - b.block_start[t]) * 2048LL;
  float* g = b.grad[t];
  const __nv_bfloat16* src = c.out[c.me] + b.offset[t];
  const long long n = b.numel[t];
  for (int i = threadIdx.x * 8; i < 2048; i += blockDim.x * 8) {
    const long long j = base + i;
    if (j >= n) break;
    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(src + j));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (j + 2 * e < n) g[j + 2 * e] = bf16_lo(w[e]);
      if (j + 2 * e + 1 < n) g[j + 2 * e + 1] = bf16_hi(w[e]);
    }
  }
}

}  // namespace ar
}  // namespace recml

using namespace recml::ar;

extern "C" int recml_ar_struct_sizes(int* out) { out[0] = sizeof(Bucket); out[1] = sizeof(Comm); return 0; }

// Runs pack -> reduce -> unpack for one bucket on `stream`.
extern "C" int recml_allreduce_bucket(const Bucket* b, const Comm* c, cudaStream_t stream) {
  const long long blocks = b->block_start[b->n];
  if (blocks <= 0) return 0;
  pack_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(*b, *c);
  const long long nvec = c->total / c->W / 8;
  int rb = static_cast<int>((nvec + 255) / 256);
  rb = rb < 1 ? 1 : (rb > 592 ? 592 : rb);
  if (c->mc_in != nullptr && c->mc_out != nullptr && c->W > 1)
    reduce_nvls_kernel<<<rb, 256, 0, stream>>>(*c);
  else
    reduce_kernel<<<rb, 256, 0, stream>>>(*c);
  unpack_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(*b, *c);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
