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

// bf16 forward with 16-byte accesses for D % 8 == 0, D <= 256 * NCH: the row stays in registers between the
// statistics and the output, lane l owning columns [c * 256 + 8 l, + 8) of chunk c.
template <int NCH>
__global__ void __launch_bounds__(256) ln_fwd_vec_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gate,
                                                         const float* __restrict__ w, const float* __restrict__ b,
                                                         __nv_bfloat16* __restrict__ y, float* __restrict__ stats, long long M,
                                                         int D, float eps, int rms) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  float v[NCH][8];
  float s = 0.f, ss = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = c * 256 + lane * 8;
    if (col < D) {
      const uint4 t = __ldg(reinterpret_cast<const uint4*>(x + row * D + col));
      const uint32_t tw[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) { v[c][2 * j] = bf16_lo(tw[j]); v[c][2 * j + 1] = bf16_hi(tw[j]); }
#pragma unroll
      for (int j = 0; j < 8; ++j) { s += v[c][j]; ss += v[c][j] * v[c][j]; }
    }
  }
  s = wsum(s); ss = wsum(ss);
  const float mean = rms ? 0.f : s / D;
  const float var = rms ? ss / D : fmaxf(ss / D - mean * mean, 0.f);
  const float rstd = rsqrtf(var + eps);
  if (lane == 0) { stats[2 * row] = mean; stats[2 * row + 1] = rstd; }
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = c * 256 + lane * 8;
    if (col < D) {
      const float4 w0 = __ldg(reinterpret_cast<const float4*>(w + col)), w1 = __ldg(reinterpret_cast<const float4*>(w + col + 4));
      const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (v[c][j] - mean) * rstd * wv[j];
      if (b != nullptr) {
        const float4 b0 = __ldg(reinterpret_cast<const float4*>(b + col)), b1 = __ldg(reinterpret_cast<const float4*>(b + col + 4));
        o[0] += b0.x; o[1] += b0.y; o[2] += b0.z; o[3] += b0.w; o[4] += b1.x; o[5] += b1.y; o[6] += b1.z; o[7] += b1.w;
      }
      if (gate != nullptr) {
        const uint4 g = __ldg(reinterpret_cast<const uint4*>(gate + row * D + col));
        const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { o[2 * j] *= bf16_lo(gw[j]); o[2 * j + 1] *= bf16_hi(gw[j]); }
      }
      *reinterpret_cast<uint4*>(y + row * D + col) =
          make_uint4(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]), pack_bf16(o[4], o[5]), pack_bf16(o[6], o[7]));
    }
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

// bf16 backward with 16-byte accesses for D % 8 == 0, D <= 256 * NCH: lane l owns columns
// [c * 256 + 8 l, c * 256 + 8 l + 8) of chunk c.  The dw / db partial sums of a block's 8 warps meet in
// shared memory, so the global atomics are one per column per block.
template <int NCH>
__global__ void __launch_bounds__(256) ln_bwd_vec_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                         const __nv_bfloat16* __restrict__ gate, const float* __restrict__ w,
                                                         const float* __restrict__ b, const float* __restrict__ stats,
                                                         __nv_bfloat16* __restrict__ dx, __nv_bfloat16* __restrict__ dgate,
                                                         float* __restrict__ dw, float* __restrict__ db, long long M, int D,
                                                         int rms, int rows_per_warp) {
  __shared__ float red[8][2][NCH * 256];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long r0 = warp * rows_per_warp;
  float aw[NCH][8], ab[NCH][8], wv[NCH][8], bv[NCH][8];
  bool act[NCH];
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = c * 256 + lane * 8;
    act[c] = col < D;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      aw[c][j] = 0.f; ab[c][j] = 0.f;
      wv[c][j] = act[c] ? w[col + j] : 0.f;
      bv[c][j] = (act[c] && b != nullptr) ? b[col + j] : 0.f;
    }
  }
  const float inv_d = 1.f / D;
  for (long long row = r0; row < min(M, r0 + rows_per_warp); ++row) {
    const float mean = stats[2 * row], rstd = stats[2 * row + 1];
    float xh[NCH][8], d[NCH][8], d0[NCH][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      if (!act[c]) continue;
      const long long off = row * D + c * 256 + lane * 8;
      const uint4 xv = __ldg(reinterpret_cast<const uint4*>(x + off));
      const uint4 dv = __ldg(reinterpret_cast<const uint4*>(dy + off));
      const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w}, dwv[4] = {dv.x, dv.y, dv.z, dv.w};
      uint32_t gw[4] = {0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u};   // bf16 ones
      if (gate != nullptr) {
        const uint4 gv = __ldg(reinterpret_cast<const uint4*>(gate + off));
        gw[0] = gv.x; gw[1] = gv.y; gw[2] = gv.z; gw[3] = gv.w;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        xh[c][2 * j] = (bf16_lo(xw[j]) - mean) * rstd;
        xh[c][2 * j + 1] = (bf16_hi(xw[j]) - mean) * rstd;
        d0[c][2 * j] = bf16_lo(dwv[j]);
        d0[c][2 * j + 1] = bf16_hi(dwv[j]);
        d[c][2 * j] = d0[c][2 * j] * bf16_lo(gw[j]);
        d[c][2 * j + 1] = d0[c][2 * j + 1] * bf16_hi(gw[j]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float dyh = d[c][j] * wv[c][j];
        s1 += dyh; s2 += dyh * xh[c][j];
      }
    }
    s1 = wsum(s1) * inv_d; s2 = wsum(s2) * inv_d;
    if (rms) s1 = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      if (!act[c]) continue;
      const long long off = row * D + c * 256 + lane * 8;
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[j] = rstd * (d[c][j] * wv[c][j] - s1 - xh[c][j] * s2);
        aw[c][j] += d[c][j] * xh[c][j];
        ab[c][j] += d[c][j];
      }
      *reinterpret_cast<uint4*>(dx + off) =
          make_uint4(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]), pack_bf16(o[4], o[5]), pack_bf16(o[6], o[7]));
      if (dgate != nullptr) {
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = d0[c][j] * (xh[c][j] * wv[c][j] + bv[c][j]);
        *reinterpret_cast<uint4*>(dgate + off) =
            make_uint4(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]), pack_bf16(o[4], o[5]), pack_bf16(o[6], o[7]));
      }
    }
  }
#pragma unroll
  for (int c = 0; c < NCH; ++c)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      red[wib][0][c * 256 + lane * 8 + j] = aw[c][j];
      red[wib][1][c * 256 + lane * 8 + j] = ab[c][j];
    }
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float sw = 0.f, sb = 0.f;
#pragma unroll
    for (int q = 0; q < 8; ++q) { sw += red[q][0][i]; sb += red[q][1][i]; }
    atomicAdd(dw + i, sw);
    atomicAdd(db + i, sb);
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
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(y) |
                         reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(b)) & 15) == 0;
  if (is_bf16 && D % 8 == 0 && D <= 1024 && aligned) {
    using B = __nv_bfloat16;
#define RECML_LNF(N) ln_fwd_vec_kernel<N><<<blocks, 256, 0, stream>>>(static_cast<const B*>(x), static_cast<const B*>(gate), w, b, \
                                                                      static_cast<B*>(y), stats, M, D, eps, rms)
    if (D <= 256) RECML_LNF(1);
    else if (D <= 512) RECML_LNF(2);
    else RECML_LNF(4);
#undef RECML_LNF
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
  }
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
  const bool aligned = ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(gate) |
                         reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(dgate)) & 15) == 0;
  if (is_bf16 && D % 8 == 0 && D <= 512 && aligned) {
    using B = __nv_bfloat16;
    const int rows_per_warp = M > 148LL * 64 * 4 ? 8 : 2;
    const long long warps = (M + rows_per_warp - 1) / rows_per_warp;
    const int blocks = static_cast<int>((warps + 7) / 8);
    if (D <= 256)
      ln_bwd_vec_kernel<1><<<blocks, 256, 0, stream>>>(static_cast<const B*>(dy), static_cast<const B*>(x), static_cast<const B*>(gate),
                                                       w, b, stats, static_cast<B*>(dx), static_cast<B*>(dgate), dw, db, M, D, rms,
                                                       rows_per_warp);
    else
      ln_bwd_vec_kernel<2><<<blocks, 256, 0, stream>>>(static_cast<const B*>(dy), static_cast<const B*>(x), static_cast<const B*>(gate),
                                                       w, b, stats, static_cast<B*>(dx), static_cast<B*>(dgate), dw, db, M, D, rms,
                                                       rows_per_warp);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
  }
  if (is_bf16) launch_bwd<__nv_bfloat16>(dy, x, gate, w, b, stats, dx, dgate, dw, db, M, D, rms, stream);
  else launch_bwd<float>(dy, x, gate, w, b, stats, dx, dgate, dw, db, M, D, rms, stream);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
