// Sampled-softmax loss over [positive | C shared candidates] logits, forward and gradient in one pass.
//
//   l_0 = pos[t] / temp,   l_j = neg[t, j] / temp  (j = 1..C),   candidate j is dropped for row t when
//   cand_ids[j] == target_ids[t] (an accidental hit: the "negative" is the positive item)
//   nll_t = logsumexp(l) - l_0;   loss = sum_t w_t nll_t / max(sum_t w_t, 1);   hit_t = [l_0 >= max_j l_j]
//
// One warp per row writes the gradient of the MEAN loss  d(sum_t w_t nll_t / den)  as bf16 in the layout of the
// logits (den = max(sum_t w_t, 1) comes in through a device pointer), so the [T, 1 + C] fp32 logits, the mask,
// the softmax and their gradients never exist as separate tensors.  With C = 256, 512 or 1024 the warp holds
// the whole row in registers (16-byte loads, the next row in flight while this one is reduced): the logits are
// read once and the gradient written once.  The low words of the lane's candidate ids stay in registers, so
// the accidental-hit test costs no memory traffic unless a low word matches.  Other C: three strided passes.
// stats[0] += sum w nll, stats[1] += sum w, stats[2] += sum w hit   (pre-zeroed by the caller).
// `scale_rows_kernel` multiplies the stored gradient by the incoming loss gradient and leaves at once when
// that is exactly 1 (the usual `loss.backward()`).
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
    const float* weights, int T, int C, float inv_temp, const float* den, float* stats, float* dpos,
    __nv_bfloat16* dneg) {
  __shared__ float part[8][3];
  const float inv_den = 1.f / __ldg(den);
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
    const float gscale = w * inv_temp * inv_den;
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

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// C = 256 * NV: lane owns the 16-byte chunks i * 32 + lane (i < NV) of a row, i.e. columns (i * 32 + lane) * 8 + e.
template <int NV>
__global__ void __launch_bounds__(256) sampled_softmax_vec_kernel(
    const float* pos, const __nv_bfloat16* neg, long long ld_neg, const long long* cand_ids, const long long* target_ids,
    const float* weights, int T, float inv_temp, const float* den, float* stats, float* dpos, __nv_bfloat16* dneg) {
  __shared__ float part[8][3];
  constexpr int NE = NV * 8;
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const float inv_den = 1.f / __ldg(den);
  uint32_t cl[NE];
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) cl[i * 8 + e] = static_cast<uint32_t>(cand_ids[(i * 32 + lane) * 8 + e]);
  float s_loss = 0.f, s_w = 0.f, s_hit = 0.f;
  int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  uint4 v[NV];
  if (t < T) {
    const uint4* row4 = reinterpret_cast<const uint4*>(neg + static_cast<long long>(t) * ld_neg);
#pragma unroll
    for (int i = 0; i < NV; ++i) v[i] = ld_stream(row4 + i * 32 + lane);
  }
  while (t < T) {
    const int tn = t + warps;
    uint4 vn[NV];
    if (tn < T) {
      const uint4* row4 = reinterpret_cast<const uint4*>(neg + static_cast<long long>(tn) * ld_neg);
#pragma unroll
      for (int i = 0; i < NV; ++i) vn[i] = ld_stream(row4 + i * 32 + lane);
    }
    const float w = weights != nullptr ? weights[t] : 1.f;
    const long long tgt = target_ids[t];
    const uint32_t tgt_lo = static_cast<uint32_t>(tgt);
    const float l0 = pos[t] * inv_temp;
    float x[NE];
    bool low_match = false;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const uint32_t wds[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        x[i * 8 + 2 * k] = __uint_as_float(wds[k] << 16) * inv_temp;
        x[i * 8 + 2 * k + 1] = __uint_as_float(wds[k] & 0xffff0000u) * inv_temp;
      }
    }
#pragma unroll
    for (int k = 0; k < NE; ++k) low_match |= cl[k] == tgt_lo;
    if (__any_sync(0xffffffffu, low_match)) {            // rare: confirm with the full ids
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (cl[i * 8 + e] == tgt_lo && cand_ids[(i * 32 + lane) * 8 + e] == tgt) x[i * 8 + e] = -INFINITY;
    }
    float m = -INFINITY;
#pragma unroll
    for (int k = 0; k < NE; ++k) m = fmaxf(m, x[k]);
    m = warp_max(m);
    const bool hit = l0 >= m;
    const float top = fmaxf(m, l0);
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < NE; ++k) {
      x[k] = __expf(x[k] - top);                          // exp(-inf) = 0 for a dropped candidate
      sum += x[k];
    }
    const float e0 = __expf(l0 - top);
    sum = warp_add(sum) + e0;
    const float inv_sum = 1.f / sum;
    const float gscale = w * inv_temp * inv_den;
    const float gs = gscale * inv_sum;
    uint4* drow4 = reinterpret_cast<uint4*>(dneg + static_cast<long long>(t) * ld_neg);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      uint4 o;
      o.x = pack2(x[i * 8 + 0] * gs, x[i * 8 + 1] * gs);
      o.y = pack2(x[i * 8 + 2] * gs, x[i * 8 + 3] * gs);
      o.z = pack2(x[i * 8 + 4] * gs, x[i * 8 + 5] * gs);
      o.w = pack2(x[i * 8 + 6] * gs, x[i * 8 + 7] * gs);
      drow4[i * 32 + lane] = o;
    }
    if (lane == 0) {
      dpos[t] = (e0 * inv_sum - 1.f) * gscale;
      s_loss += w * (top + logf(sum) - l0);
      s_w += w;
      s_hit += hit ? w : 0.f;
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) v[i] = vn[i];
    t = tn;
  }
  if (lane == 0) { part[wib][0] = s_loss; part[wib][1] = s_w; part[wib][2] = s_hit; }
  __syncthreads();
  if (threadIdx.x < 3) {
    float acc = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) acc += part[i][threadIdx.x];
    if (acc != 0.f) atomicAdd(stats + threadIdx.x, acc);
  }
}

// rows[t, 0..C) *= *g   unless *g == 1
__global__ void __launch_bounds__(256) scale_rows_kernel(__nv_bfloat16* rows, long long ld, int T, int C, const float* g) {
  const float s = __ldg(g);
  if (s == 1.f) return;
  const long long n = static_cast<long long>(T) * C;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    __nv_bfloat16* p = rows + (i / C) * ld + (i % C);
    *p = __float2bfloat16(__bfloat162float(*p) * s);
  }
}

}  // namespace ssm
}  // namespace recml

extern "C" int recml_sampled_softmax(const float* pos, const void* neg, long long ld_neg, const long long* cand_ids,
                                     const long long* target_ids, const float* weights, int T, int C, float inv_temp,
                                     const float* den, float* stats, float* dpos, void* dneg, cudaStream_t stream) {
  if (T <= 0 || C <= 0) return 0;
  int blocks = (T + 7) / 8;
  blocks = blocks > 148 * 8 ? 148 * 8 : blocks;
  const __nv_bfloat16* n = static_cast<const __nv_bfloat16*>(neg);
  __nv_bfloat16* d = static_cast<__nv_bfloat16*>(dneg);
  const bool vec = (C == 256 || C == 512 || C == 1024) && ld_neg % 8 == 0 &&
                   reinterpret_cast<uintptr_t>(neg) % 16 == 0 && reinterpret_cast<uintptr_t>(dneg) % 16 == 0;
  using namespace recml::ssm;
  if (vec && C == 1024)
    sampled_softmax_vec_kernel<4><<<blocks, 256, 0, stream>>>(pos, n, ld_neg, cand_ids, target_ids, weights, T, inv_temp,
                                                                den, stats, dpos, d);
  else if (vec && C == 512)
    sampled_softmax_vec_kernel<2><<<blocks, 256, 0, stream>>>(pos, n, ld_neg, cand_ids, target_ids, weights, T, inv_temp,
                                                                den, stats, dpos, d);
  else if (vec)
    sampled_softmax_vec_kernel<1><<<blocks, 256, 0, stream>>>(pos, n, ld_neg, cand_ids, target_ids, weights, T, inv_temp,
                                                                den, stats, dpos, d);
  else
    sampled_softmax_kernel<<<blocks, 256, 0, stream>>>(pos, n, ld_neg, cand_ids, target_ids, weights, T, C, inv_temp, den,
                                                       stats, dpos, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// In place: rows [T, C] (row pitch ld) times the scalar at `g`; nothing is read or written when it is 1.
extern "C" int recml_scale_rows_bf16(void* rows, long long ld, int T, int C, const float* g, cudaStream_t stream) {
  if (T <= 0 || C <= 0) return 0;
  recml::ssm::scale_rows_kernel<<<148 * 4, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(rows), ld, T, C, g);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
