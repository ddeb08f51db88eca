// Sampled-softmax loss over [positive | C shared candidates] logits, forward and gradient in one pass.
//
//   l_0 = pos[t] / temp,   l_j = neg[t, j] / temp  (j = 1..C),   candidate j is dropped for row t when
//   cand_ids[j] == target_ids[t] (an accidental hit: the "negative" is the positive item)
//   nll_t = logsumexp(l) - l_0;   loss = sum_t w_t nll_t / max(sum_t w_t, 1);   hit_t = [l_0 >= max_j l_j]
//
// One warp per row reads the bf16 candidate logits twice (row maximum, then exponent sum) and writes
// the gradient of the UNNORMALISED loss sum  d(sum_t w_t nll_t)  as bf16 in the same layout, so the
// [T, 1 + C] fp32 logits, the mask, the softmax and their gradients never exist as separate tensors.
// stats[0] += sum w nll, stats[1] += sum w, stats[2] += sum w hit   (pre-zeroed by the caller).
#include "common.cuh"

namespace recml {
namespace ssm {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_add(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(256) sampled_softmax_kernel(
    const float* pos, const __nv_bfloat16* neg, long long ld_neg, const long long* cand_ids, const long long* target_ids,
    const float* weights, int T, int C, float inv_temp, float* stats, float* dpos, __nv_bfloat16* dneg) {
  __shared__ float part[8][3];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  float s_loss = 0.f, s_w = 0.f, s_hit = 0.f;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
    const float w = weights != nullptr ? weights[t] : 1.f;
    const long long tgt = target_ids[t];
    const __nv_bfloat16* row = neg + static_cast<long long>(t) * ld_neg;
    const float l0 = pos[t] * inv_temp;
    float m = -INFINITY;
    for (int j = lane; j < C; j += 32)
      if (cand_ids[j] != tgt) m = fmaxf(m, __bfloat162float(row[j]) * inv_temp);
    m = warp_max(m);
    const bool hit = l0 >= m;
    const float top = fmaxf(m, l0);
    float sum = 0.f;
    for (int j = lane; j < C; j += 32)
      if (cand_ids[j] != tgt) sum += __expf(__bfloat162float(row[j]) * inv_temp - top);
    sum = warp_add(sum) + __expf(l0 - top);
    const float lse = top + logf(sum);
    const float inv_sum = 1.f / sum;
    // gradient of w * nll w.r.t. the raw (un-tempered) logits
    const float gscale = w * inv_temp;
    __nv_bfloat16* drow = dneg + static_cast<long long>(t) * ld_neg;
    for (int j = lane; j < C; j += 32) {
      const float pj = cand_ids[j] != tgt ? __expf(__bfloat162float(row[j]) * inv_temp - top) * inv_sum : 0.f;
      drow[j] = __float2bfloat16(pj * gscale);
    }
    if (lane == 0) {
      dpos[t] = (__expf(l0 - top) * inv_sum - 1.f) * gscale;
      s_loss += w * (lse - l0);
      s_w += w;
      s_hit += hit ? w : 0.f;
    }
  }
  if (lane == 0) { part[wib][0] = s_loss; part[wib][1] = s_w; part[wib][2] = s_hit; }
  __syncthreads();
  if (threadIdx.x < 3) {
    float acc = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) acc += part[i][threadIdx.x];
    if (acc != 0.f) atomicAdd(stats + threadIdx.x, acc);
  }
}

}  // namespace ssm
}  // namespace recml

extern "C" int recml_sampled_softmax(const float* pos, const void* neg, long long ld_neg, const long long* cand_ids,
                                     const long long* target_ids, const float* weights, int T, int C, float inv_temp,
                                     float* stats, float* dpos, void* dneg, cudaStream_t stream) {
  if (T <= 0 || C <= 0) return 0;
  int blocks = (T + 7) / 8;
  blocks = blocks > 148 * 8 ? 148 * 8 : blocks;
  recml::ssm::sampled_softmax_kernel<<<blocks, 256, 0, stream>>>(
      pos, static_cast<const __nv_bfloat16*>(neg), ld_neg, cand_ids, target_ids, weights, T, C, inv_temp, stats, dpos,
      static_cast<__nv_bfloat16*>(dneg));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
