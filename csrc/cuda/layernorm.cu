// Row-wise LayerNorm / RMS-norm forward and backward with an optional fused output gate:
//   y = gate * ((x - mean) * rstd * w + b)          (rms: mean := 0, rstd = rsqrt(mean(x^2)+eps))
// One warp per row, values kept in registers between the statistics pass and the output pass;
// bf16 or fp32 io, fp32 math.  dw / db are accumulated with one atomic per column per block.
#include "common.cuh"

namespace recml {
namespace ln {

constexpr int kMaxPerLane = 8192 / 32;   // D <= 8192

__device__ __forceinline__ float wsum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

template <typename T> __device__ __forceinline__ float ld(const T* p, long long i);
template <> __device__ __forceinline__ float ld<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ld<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T> __device__ __forceinline__ void st(T* p, long long i, float v);
template <> __device__ __forceinline__ void st<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void st<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16(v); }

template <typename T>
__global__ void __launch_bounds__(256) ln_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gate,
                                                     const float* __restrict__ w, const float* __restrict__ b,
                                                     T* __restrict__ y, float* __restrict__ stats, long long M,
                                                     int D, float eps, int rms) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  const T* xr = x + row * D;
  float s = 0.f, ss = 0.f;
  for (int i = lane; i < D; i += 32) { const float v = ld<T>(xr, i); s += v; ss += v * v; }
  s = wsum(s); ss = wsum(ss);
  const float mean = rms ? 0.f : s / D;
  const float var = rms ? ss / D : fmaxf(ss / D - mean * mean, 0.f);
  const float rstd = rsqrtf(var + eps);
  if (lane == 0) { stats[2 * row] = mean; stats[2 * row + 1] = rstd; }
  for (int i = lane; i < D; i += 32) {
    float v = (ld<T>(xr, i) - mean) * rstd * w[i] + (b != nullptr ? b[i] : 0.f);
    if (gate != nullptr) v *= ld<T>(gate, row * D + i);
    st<T>(y, row * D + i, v);
  }
}

// dx for y = g * (xhat * w + b):  let dyh = dy * g * w ;  dx = rstd * (dyh - mean(dyh) - xhat * mean(dyh * xhat))
// (rms: the mean(dyh) term drops).  dgate = dy * (xhat * w + b).  Each warp walks `rows_per_warp`
// rows and keeps its dw / db partial sums in registers (NPL columns per lane), so the global
// atomics are one per column per warp instead of one per element.
template <typename T, int NPL>
__global__ void __launch_bounds__(256) ln_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                     const T* __restrict__ gate, const float* __restrict__ w,
                                                     const float* __restrict__ b, const float* __restrict__ stats,
                                                     T* __restrict__ dx, T* __restrict__ dgate,
                                                     float* __restrict__ dw, float* __restrict__ db, long long M,
                                                     int D, int rms, int rows_per_warp) {
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long r0 = warp * rows_per_warp;
  if (r0 >= M) return;
  float aw[NPL], ab[NPL], wv[NPL], bv[NPL];
#pragma unroll
  for (int k = 0; k < NPL; ++k) {
    const int i = lane + 32 * k;
    aw[k] = 0.f; ab[k] = 0.f;
    wv[k] = i < D ? w[i] : 0.f;
    bv[k] = (i < D && b != nullptr) ? b[i] : 0.f;
  }
  for (long long row = r0; row < min(M, r0 + rows_per_warp); ++row) {
    const float mean = stats[2 * row], rstd = stats[2 * row + 1];
    float xh[NPL], d[NPL], d0[NPL];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < NPL; ++k) {
      const int i = lane + 32 * k;
      xh[k] = 0.f; d[k] = 0.f; d0[k] = 0.f;
      if (i < D) {
        xh[k] = (ld<T>(x, row * D + i) - mean) * rstd;
        d0[k] = ld<T>(dy, row * D + i);
        d[k] = gate != nullptr ? d0[k] * ld<T>(gate, row * D + i) : d0[k];
        const float dyh = d[k] * wv[k];
        s1 += dyh; s2 += dyh * xh[k];
      }
    }
    s1 = wsum(s1) / D; s2 = wsum(s2) / D;
    if (rms) s1 = 0.f;
#pragma unroll
    for (int k = 0; k < NPL; ++k) {
      const int i = lane + 32 * k;
      if (i < D) {
        st<T>(dx, row * D + i, rstd * (d[k] * wv[k] - s1 - xh[k] * s2));
        if (dgate != nullptr) st<T>(dgate, row * D + i, d0[k] * (xh[k] * wv[k] + bv[k]));
        aw[k] += d[k] * xh[k];
        ab[k] += d[k];
      }
    }
  }
#pragma unroll
  for (int k = 0; k < NPL; ++k) {
    const int i = lane + 32 * k;
    if (i < D) { atomicAdd(dw + i, aw[k]); atomicAdd(db + i, ab[k]); }
  }
}

}  // namespace ln
}  // namespace recml

using namespace recml::ln;

extern "C" int recml_layernorm_fwd(const void* x, const void* gate, const float* w, const float* b, void* y,
                                   float* stats, long long M, int D, float eps, int rms, int is_bf16,
                                   cudaStream_t stream) {
  if (M <= 0) return 0;
  const int blocks = static_cast<int>((M * 32 + 255) / 256);
  if (is_bf16)
    ln_fwd_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x),
        static_cast<const __nv_bfloat16*>(gate), w, b, static_cast<__nv_bfloat16*>(y), stats, M, D, eps, rms);
  else
    ln_fwd_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<const float*>(x), static_cast<const float*>(gate), w, b,
                                                     static_cast<float*>(y), stats, M, D, eps, rms);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

template <typename T>
static void launch_bwd(const void* dy, const void* x, const void* gate, const float* w, const float* b,
                       const float* stats, void* dx, void* dgate, float* dw, float* db, long long M, int D, int rms,
                       cudaStream_t stream) {
  const int rows_per_warp = M > 148LL * 64 * 4 ? 16 : 4;
  const long long warps = (M + rows_per_warp - 1) / rows_per_warp;
  const int blocks = static_cast<int>((warps * 32 + 255) / 256);
#define RECML_LN(N) ln_bwd_kernel<T, N><<<blocks, 256, 0, stream>>>(static_cast<const T*>(dy), static_cast<const T*>(x), \
      static_cast<const T*>(gate), w, b, stats, static_cast<T*>(dx), static_cast<T*>(dgate), dw, db, M, D, rms, rows_per_warp)
  if (D <= 128) RECML_LN(4);
  else if (D <= 256) RECML_LN(8);
  else if (D <= 512) RECML_LN(16);
  else RECML_LN(32);
#undef RECML_LN
}

// D <= 1024 for the backward pass.
extern "C" int recml_layernorm_bwd(const void* dy, const void* x, const void* gate, const float* w, const float* b,
                                   const float* stats, void* dx, void* dgate, float* dw, float* db, long long M,
                                   int D, int rms, int is_bf16, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (D > 1024) return -10;
  if (is_bf16) launch_bwd<__nv_bfloat16>(dy, x, gate, w, b, stats, dx, dgate, dw, db, M, D, rms, stream);
  else launch_bwd<float>(dy, x, gate, w, b, stats, dx, dgate, dw, db, M, D, rms, stream);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
