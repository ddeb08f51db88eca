// Fused multi-tensor dense optimizer: global-norm clipping, Adam / RSS-Adagrad / SGD scaling,
// masked weight decay and the learning-rate step in ONE launch over a list of tensors, also
// refreshing the bf16 compute copy of every parameter.  A separate reduction kernel produces the
// squared gradient norm when clipping is on.
#include "common.cuh"

namespace recml {
namespace optim {

constexpr int kMaxTensors = 64;
struct TensorList {
  float* param[kMaxTensors];
  const float* grad[kMaxTensors];
  float* s0[kMaxTensors];            // adam: mu; rss: sum of squares
  float* s1[kMaxTensors];            // adam: nu
  __nv_bfloat16* copy[kMaxTensors];  // optional bf16 copy of the updated parameter
  long long numel[kMaxTensors];
  long long block_start[kMaxTensors + 1];  // prefix of blocks (each block = 1024 elements)
  int decay[kMaxTensors];
  int n;
};

struct Hyper {
  int kind;  // 0 identity, 1 adam, 2 rss
  float lr, b1, b2, eps, bc1, bc2, weight_decay, clip_norm;
  const float* sqnorm;  // device scalar: Σ g² (null: no clipping)
};

__global__ void sqnorm_kernel(const TensorList tl, float* out) {
  int t = 0;
  while (t + 1 < tl.n && static_cast<long long>(blockIdx.x) >= tl.block_start[t + 1]) ++t;
  const long long base = (blockIdx.x - tl.block_start[t]) * 1024LL;
  const float* g = tl.grad[t];
  float s = 0.f;
  for (int i = threadIdx.x; i < 1024; i += blockDim.x) {
    const long long j = base + i;
    if (j < tl.numel[t]) { const float v = g[j]; s += v * v; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  __shared__ float sh[8];
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) tot += sh[w];
    atomicAdd(out, tot);
  }
}

__global__ void step_kernel(const TensorList tl, const Hyper h_val, const Hyper* __restrict__ h_dev) {
  const Hyper h = h_dev != nullptr ? *h_dev : h_val;   // device copy: refreshed per replay of a CUDA graph
  int t = 0;
  while (t + 1 < tl.n && static_cast<long long>(blockIdx.x) >= tl.block_start[t + 1]) ++t;
  const long long base = (blockIdx.x - tl.block_start[t]) * 1024LL;
  float factor = 1.f;
  if (h.sqnorm != nullptr) {
    const float norm = sqrtf(*h.sqnorm);
    factor = h.clip_norm / fmaxf(norm, h.clip_norm);
  }
  float* p = tl.param[t];
  const float* g = tl.grad[t];
  for (int i = threadIdx.x; i < 1024; i += blockDim.x) {
    const long long j = base + i;
    if (j >= tl.numel[t]) break;
    const float gi = g[j] * factor;
    float w = p[j], u;
    if (h.kind == 1) {
      const float m = h.b1 * tl.s0[t][j] + (1.f - h.b1) * gi;
      const float v = h.b2 * tl.s1[t][j] + (1.f - h.b2) * gi * gi;
      tl.s0[t][j] = m; tl.s1[t][j] = v;
      u = (m / h.bc1) / (sqrtf(v / h.bc2) + h.eps);
    } else if (h.kind == 2) {
      const float a = tl.s0[t][j] + gi * gi;
      tl.s0[t][j] = a;
      u = a > 0.f ? gi * rsqrtf(a + h.eps) : 0.f;
    } else {
      u = gi;
    }
    if (tl.decay[t]) u += h.weight_decay * w;
    w -= h.lr * u;
    p[j] = w;
    if (tl.copy[t] != nullptr) tl.copy[t][j] = __float2bfloat16(w);
  }
}

}  // namespace optim
}  // namespace recml

using namespace recml::optim;

extern "C" int recml_optim_struct_sizes(int* out) { out[0] = sizeof(TensorList); out[1] = sizeof(Hyper); return 0; }

extern "C" int recml_optim_sqnorm(const TensorList* tl, float* out, cudaStream_t stream) {
  const long long blocks = tl->block_start[tl->n];
  if (blocks <= 0) return 0;
  sqnorm_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(*tl, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int recml_optim_step(const TensorList* tl, const Hyper* h, const Hyper* h_dev, cudaStream_t stream) {
  const long long blocks = tl->block_start[tl->n];
  if (blocks <= 0) return 0;
  step_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(*tl, *h, h_dev);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
