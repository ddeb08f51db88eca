// Memory-bound helper kernels of the dense path: fused BCE-with-logits loss + gradient + metric
// statistics, casts, bias-gradient column sums, DCN backward element-wise pieces, and the
// 1-column output layer (GEMV) forward / backward.
#include "common.cuh"

namespace recml {
namespace ew {

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// ---- BCE with logits ---------------------------------------------------------------------------
// stats[0]=Σ loss·w, [1]=Σ w, [2]=Σ label·w, [3]=Σ sigmoid·w, [4]=Σ correct·w (logit>0 == label)
// hist_pos / hist_neg: [T+1] weighted histograms of sigmoid(logit) over the default AUC thresholds
// (-1e-7, 1/(T-1), ..., (T-2)/(T-1), 1+1e-7); bin = number of thresholds strictly below p.
__device__ __forceinline__ int auc_bin(float p, int T) {
  const float scale = static_cast<float>(T - 1);
  int k = static_cast<int>(ceilf(p * scale)) - 1;          // candidate: thresholds 1..k are below p
  k = max(0, min(k, T - 2));
  while (k + 1 <= T - 2 && static_cast<float>(static_cast<double>(k + 1) / (T - 1)) < p) ++k;
  while (k >= 1 && !(static_cast<float>(static_cast<double>(k) / (T - 1)) < p)) --k;
  int bin = 1 + k;                                          // threshold 0 (-1e-7) is always below p >= 0
  if (p > 1.0f + 1e-7f) bin = T;
  return bin;
}

template <typename TIn>
__global__ void bce_kernel(const TIn* __restrict__ logits, const float* __restrict__ labels,
                           const float* __restrict__ weights, long long n, float grad_scale,
                           float* __restrict__ dlogits_f32, __nv_bfloat16* __restrict__ dlogits_bf16,
                           float* __restrict__ stats, float* __restrict__ hist_pos,
                           float* __restrict__ hist_neg, int T) {
  extern __shared__ float sh[];  // [2*(T+1)] histograms
  const int nb = T > 0 ? 2 * (T + 1) : 0;
  for (int i = threadIdx.x; i < nb; i += blockDim.x) sh[i] = 0.f;
  __syncthreads();
  float s_loss = 0.f, s_w = 0.f, s_y = 0.f, s_p = 0.f, s_c = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float x = static_cast<float>(logits[i]);
    const float y = labels[i];
    const float w = weights != nullptr ? weights[i] : 1.f;
    const float p = 1.f / (1.f + __expf(-x));
    const float loss = fmaxf(x, 0.f) - x * y + log1pf(__expf(-fabsf(x)));
    s_loss += loss * w; s_w += w; s_y += y * w; s_p += p * w;
    s_c += ((x > 0.f) == (y > 0.5f)) ? w : 0.f;
    const float g = (p - y) * w * grad_scale;
    if (dlogits_f32 != nullptr) dlogits_f32[i] = g;
    if (dlogits_bf16 != nullptr) dlogits_bf16[i] = __float2bfloat16(g);
    if (T > 0) atomicAdd(&sh[(y > 0.5f ? 0 : T + 1) + auc_bin(p, T)], w);
  }
  s_loss = warp_sum(s_loss); s_w = warp_sum(s_w); s_y = warp_sum(s_y); s_p = warp_sum(s_p); s_c = warp_sum(s_c);
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(stats + 0, s_loss); atomicAdd(stats + 1, s_w); atomicAdd(stats + 2, s_y);
    atomicAdd(stats + 3, s_p); atomicAdd(stats + 4, s_c);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nb; i += blockDim.x) {
    const float v = sh[i];
    if (v != 0.f) atomicAdd((i <= T ? hist_pos + i : hist_neg + (i - T - 1)), v);
  }
}

// ---- casts ----------------------------------------------------------------------------------------
__global__ void cast_f32_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long long n) {
  const long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 4;
  if (i + 3 < n) {
    const float4 v = *reinterpret_cast<const float4*>(in + i);
    *reinterpret_cast<uint2*>(out + i) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
  } else {
    for (long long j = i; j < n; ++j) out[j] = __float2bfloat16(in[j]);
  }
}

// rows [M, cols_in] fp32 -> [M, ld_out] bf16 with zero padding of columns cols_in..cols_out
__global__ void cast_pad_rows_kernel(const float* __restrict__ in, int cols_in, __nv_bfloat16* __restrict__ out,
                                     int cols_out, long long ld_out, long long M) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= M * cols_out) return;
  const long long r = i / cols_out;
  const int c = static_cast<int>(i % cols_out);
  out[r * ld_out + c] = __float2bfloat16(c < cols_in ? in[r * cols_in + c] : 0.f);
}

// ---- column sums: out[n] (+)= Σ_m x[m, n]  (bias gradients) ----------------------------------------
__global__ void colsum_kernel(const __nv_bfloat16* __restrict__ x, long long M, int N, long long ld,
                              float* __restrict__ out, int rows_per_block) {
  // block covers 64 columns (32 lanes x bf16x2) x rows_per_block rows; 8 warps stride the rows
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 64 + lane * 2;
  const long long r0 = static_cast<long long>(blockIdx.y) * rows_per_block;
  const long long r1 = min(M, r0 + rows_per_block);
  float a = 0.f, b = 0.f;
  if (col < N) {
    for (long long r = r0 + warp; r < r1; r += 8) {
      const uint32_t t = *reinterpret_cast<const uint32_t*>(x + r * ld + col);
      a += bf16_lo(t); b += bf16_hi(t);
    }
  }
  __shared__ float sh[8][64];
  sh[warp][lane * 2] = a; sh[warp][lane * 2 + 1] = b;
  __syncthreads();
  if (warp == 0 && col < N) {
    float sa = 0.f, sb = 0.f;
    for (int w = 0; w < 8; ++w) { sa += sh[w][lane * 2]; sb += sh[w][lane * 2 + 1]; }
    atomicAdd(out + col, sa);
    if (col + 1 < N) atomicAdd(out + col + 1, sb);
  }
}

// Same sums with 16-byte loads: a block covers 256 columns (32 lanes x 8 bf16) x rows_per_block rows, its 8 warps
// stride the rows and keep four row loads in flight.  Needs N % 8 == 0, ld % 8 == 0 and a 16-byte aligned base.
__global__ void __launch_bounds__(256) colsum8_kernel(const __nv_bfloat16* __restrict__ x, long long M, int N,
                                                      long long ld, float* __restrict__ out, int rows_per_block) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 256 + lane * 8;
  const long long r0 = static_cast<long long>(blockIdx.y) * rows_per_block;
  const long long r1 = min(M, r0 + rows_per_block);
  float cs[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) cs[j] = 0.f;
  if (col < N) {
    const __nv_bfloat16* base = x + col;
    long long r = r0 + warp;
    for (; r + 24 < r1; r += 32) {
      uint4 t[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) t[u] = __ldg(reinterpret_cast<const uint4*>(base + (r + 8 * u) * ld));
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t w[4] = {t[u].x, t[u].y, t[u].z, t[u].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { cs[2 * j] += bf16_lo(w[j]); cs[2 * j + 1] += bf16_hi(w[j]); }
      }
    }
    for (; r < r1; r += 8) {
      const uint4 t = __ldg(reinterpret_cast<const uint4*>(base + r * ld));
      const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) { cs[2 * j] += bf16_lo(w[j]); cs[2 * j + 1] += bf16_hi(w[j]); }
    }
  }
  __shared__ float sh[8][256];
#pragma unroll
  for (int j = 0; j < 8; ++j) sh[warp][lane * 8 + j] = cs[j];
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < N) {
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) a += sh[w][threadIdx.x];
    atomicAdd(out + c, a);
  }
}

// ---- DCN cross backward, element-wise part ----------------------------------------------------------
// dv = g * x0 ; dx0 (+)= g * v        (all [M, N] bf16 with leading dim ld; dx0 fp32 accumulate or bf16)
// A block covers 256 columns (32 lanes x 8 bf16) x rows_per_block rows, its 8 warps striding the rows, and also
// reduces the column sums of dv (= the gradient of the layer's bias) so that dv is not read again for them.
__global__ void __launch_bounds__(256) cross_bwd_ew_kernel(
    const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ x0, const __nv_bfloat16* __restrict__ v,
    __nv_bfloat16* __restrict__ dv, __nv_bfloat16* __restrict__ dx0, int accumulate, long long M, int N, long long ld,
    float* __restrict__ colsum_dv, int rows_per_block) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 256 + lane * 8;
  const long long r0 = static_cast<long long>(blockIdx.y) * rows_per_block;
  const long long r1 = min(M, r0 + rows_per_block);
  float cs[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) cs[j] = 0.f;
  if (col < N) {        // N % 8 == 0
    for (long long r = r0 + warp; r < r1; r += 8) {
      const long long off = r * ld + col;
      const uint4 G = *reinterpret_cast<const uint4*>(g + off);
      const uint4 X = *reinterpret_cast<const uint4*>(x0 + off);
      const uint4 V = *reinterpret_cast<const uint4*>(v + off);
      uint4 D = make_uint4(0, 0, 0, 0);
      if (accumulate) D = *reinterpret_cast<const uint4*>(dx0 + off);
      const uint32_t gw[4] = {G.x, G.y, G.z, G.w}, xw[4] = {X.x, X.y, X.z, X.w}, vw[4] = {V.x, V.y, V.z, V.w};
      uint32_t dw[4] = {D.x, D.y, D.z, D.w}, ow[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float g0 = bf16_lo(gw[j]), g1 = bf16_hi(gw[j]);
        ow[j] = pack_bf16(g0 * bf16_lo(xw[j]), g1 * bf16_hi(xw[j]));
        cs[2 * j] += bf16_lo(ow[j]);          // sums of the ROUNDED values, i.e. exactly what a later pass over dv would add
        cs[2 * j + 1] += bf16_hi(ow[j]);
        dw[j] = pack_bf16(bf16_lo(dw[j]) + g0 * bf16_lo(vw[j]), bf16_hi(dw[j]) + g1 * bf16_hi(vw[j]));
      }
      *reinterpret_cast<uint4*>(dv + off) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
      *reinterpret_cast<uint4*>(dx0 + off) = make_uint4(dw[0], dw[1], dw[2], dw[3]);
    }
  }
  if (colsum_dv == nullptr) return;
  __shared__ float sh[8][256];
#pragma unroll
  for (int j = 0; j < 8; ++j) sh[warp][lane * 8 + j] = cs[j];
  __syncthreads();
  const int c = threadIdx.x;
  if (blockIdx.x * 256 + c < N) {
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) acc += sh[w][c];
    atomicAdd(colsum_dv + blockIdx.x * 256 + c, acc);
  }
}

// out = a + b (bf16, [M,N] with leading dims)
__global__ void add_bf16_kernel(const __nv_bfloat16* __restrict__ a, long long lda,
                                const __nv_bfloat16* __restrict__ b, long long ldb,
                                __nv_bfloat16* __restrict__ out, long long ldo, long long M, int N) {
  const long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 8;
  if (i >= M * N) return;
  const long long r = i / N;
  const long long c = i - r * N;
  const uint4 A = *reinterpret_cast<const uint4*>(a + r * lda + c);
  const uint4 B = *reinterpret_cast<const uint4*>(b + r * ldb + c);
  const uint32_t aw[4] = {A.x, A.y, A.z, A.w}, bw[4] = {B.x, B.y, B.z, B.w};
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
    o[j] = pack_bf16(bf16_lo(aw[j]) + bf16_lo(bw[j]), bf16_hi(aw[j]) + bf16_hi(bw[j]));
  *reinterpret_cast<uint4*>(out + r * ldo + c) = make_uint4(o[0], o[1], o[2], o[3]);
}

// dy * (y > 0)   (ReLU backward for an activation whose consumer did not fuse the mask)
__global__ void relu_mask_kernel(const __nv_bfloat16* __restrict__ dy, long long lddy,
                                 const __nv_bfloat16* __restrict__ y, long long ldy,
                                 __nv_bfloat16* __restrict__ out, long long ldo, long long M, int N) {
  const long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 8;
  if (i >= M * N) return;
  const long long r = i / N;
  const long long c = i - r * N;
  const uint4 A = *reinterpret_cast<const uint4*>(dy + r * lddy + c);
  const uint4 B = *reinterpret_cast<const uint4*>(y + r * ldy + c);
  const uint32_t aw[4] = {A.x, A.y, A.z, A.w}, bw[4] = {B.x, B.y, B.z, B.w};
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
    o[j] = pack_bf16(bf16_lo(bw[j]) > 0.f ? bf16_lo(aw[j]) : 0.f, bf16_hi(bw[j]) > 0.f ? bf16_hi(aw[j]) : 0.f);
  *reinterpret_cast<uint4*>(out + r * ldo + c) = make_uint4(o[0], o[1], o[2], o[3]);
}

// ---- SiLU over a bf16 matrix, and its backward fused with the gathering of the four gradient blocks ------
// h = z * sigmoid(z), evaluated as t * tanh(t) + t with t = z / 2 (one special-function op per element)
__device__ __forceinline__ float tanh_approx(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
  return t;
}
__device__ __forceinline__ float silu_of(float z) {
  const float t = 0.5f * z;
  return fmaf(t, tanh_approx(t), t);
}
// d silu / dz = sig + z sig (1 - sig), sig = (tanh(z / 2) + 1) / 2
__device__ __forceinline__ float silu_grad_of(float z) {
  const float sig = fmaf(0.5f, tanh_approx(0.5f * z), 0.5f);
  return fmaf(z * sig, 1.f - sig, sig);
}

__global__ void silu_fwd_kernel(const __nv_bfloat16* __restrict__ z, __nv_bfloat16* __restrict__ h, long long n8) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= n8) return;
  const uint4 A = reinterpret_cast<const uint4*>(z)[i];
  const uint32_t aw[4] = {A.x, A.y, A.z, A.w};
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) o[j] = pack_bf16(silu_of(bf16_lo(aw[j])), silu_of(bf16_hi(aw[j])));
  reinterpret_cast<uint4*>(h)[i] = make_uint4(o[0], o[1], o[2], o[3]);
}

// SiLU of the [T, 4 D] pre-activation of a fused u | q | k | v projection, written as two matrices: u [T, D]
// (contiguous: it gates a LayerNorm that wants whole rows) and q | k | v [T, 3 D].
__global__ void silu_fwd_split_kernel(const __nv_bfloat16* __restrict__ z, __nv_bfloat16* __restrict__ u,
                                      __nv_bfloat16* __restrict__ qkv, long long T, int D) {
  const long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 8;
  const long long width = 4LL * D;
  if (i >= T * width) return;
  const long long r = i / width;
  const int c = static_cast<int>(i - r * width);
  const uint4 A = *reinterpret_cast<const uint4*>(z + i);
  const uint32_t aw[4] = {A.x, A.y, A.z, A.w};
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) o[j] = pack_bf16(silu_of(bf16_lo(aw[j])), silu_of(bf16_hi(aw[j])));
  __nv_bfloat16* dst = c < D ? u + r * D + c : qkv + r * 3LL * D + (c - D);
  *reinterpret_cast<uint4*>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
}

// The fused u | q | k | v projection of an attention block: z is [T, 4 D]; its four column blocks received the
// gradients g0 (bf16, row pitch ld0), g1 (FP32 [T, D]: the attention kernels accumulate dq in fp32), g2 and g3
// (bf16 [T, D]).  dz = (g0 | g1 | g2 | g3) * silu'(z) in one pass instead of a cast, a concatenation and the
// activation's backward.
__global__ void silu_bwd_gather4_kernel(const __nv_bfloat16* __restrict__ z, const __nv_bfloat16* __restrict__ g0,
                                        long long ld0, const float* __restrict__ g1,
                                        const __nv_bfloat16* __restrict__ g2, const __nv_bfloat16* __restrict__ g3,
                                        __nv_bfloat16* __restrict__ dz, long long T, int D) {
  const long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 8;
  const long long width = 4LL * D;
  if (i >= T * width) return;
  const long long r = i / width;
  const int c = static_cast<int>(i - r * width);
  const int part = c / D, cc = c - part * D;
  float g[8];
  if (part == 1) {
    const float4 a = *reinterpret_cast<const float4*>(g1 + r * D + cc);
    const float4 b = *reinterpret_cast<const float4*>(g1 + r * D + cc + 4);
    g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w; g[4] = b.x; g[5] = b.y; g[6] = b.z; g[7] = b.w;
  } else {
    const __nv_bfloat16* src = part == 0 ? g0 + r * ld0 + cc : (part == 2 ? g2 : g3) + r * D + cc;
    const uint4 A = *reinterpret_cast<const uint4*>(src);
    const uint32_t aw[4] = {A.x, A.y, A.z, A.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) { g[2 * j] = bf16_lo(aw[j]); g[2 * j + 1] = bf16_hi(aw[j]); }
  }
  const uint4 Z = *reinterpret_cast<const uint4*>(z + i);
  const uint32_t zw[4] = {Z.x, Z.y, Z.z, Z.w};
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
    o[j] = pack_bf16(g[2 * j] * silu_grad_of(bf16_lo(zw[j])), g[2 * j + 1] * silu_grad_of(bf16_hi(zw[j])));
  *reinterpret_cast<uint4*>(dz + i) = make_uint4(o[0], o[1], o[2], o[3]);
}

// ---- output layer with one unit: y[m] = x[m,:]·w + b ------------------------------------------------
__global__ void gemv_fwd_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int K,
                                const float* __restrict__ w, const float* __restrict__ bias,
                                float* __restrict__ y, long long M) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  float acc = 0.f;
  for (int k = lane * 2; k < K; k += 64) {
    const uint32_t t = *reinterpret_cast<const uint32_t*>(x + row * ld + k);
    acc += bf16_lo(t) * w[k] + bf16_hi(t) * w[k + 1];
  }
  acc = warp_sum(acc);
  if (lane == 0) y[row] = acc + (bias != nullptr ? bias[0] : 0.f);
}

// backward: dx[m,k] = dy[m]*w[k] (masked by relu of x when mask_relu), dw[k] += Σ_m dy[m]*x[m,k], db += Σ dy
__global__ void gemv_bwd_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int K,
                                const float* __restrict__ w, const float* __restrict__ dy, long long M,
                                __nv_bfloat16* __restrict__ dx, long long lddx, int mask_relu,
                                float* __restrict__ dw, float* __restrict__ db, int rows_per_block) {
  // block: 256 threads; thread t owns columns {2t, 2t+1} (+512 strides); loops over its rows
  const long long r0 = static_cast<long long>(blockIdx.x) * rows_per_block;
  const long long r1 = min(M, r0 + rows_per_block);
  for (int k = threadIdx.x * 2; k < K; k += 2 * blockDim.x) {
    const float w0 = w[k], w1 = w[k + 1];
    float a0 = 0.f, a1 = 0.f;
    for (long long r = r0; r < r1; ++r) {
      const float d = dy[r];
      const uint32_t t = *reinterpret_cast<const uint32_t*>(x + r * ld + k);
      const float x0 = bf16_lo(t), x1 = bf16_hi(t);
      a0 += d * x0; a1 += d * x1;
      const float g0 = (mask_relu && !(x0 > 0.f)) ? 0.f : d * w0;
      const float g1 = (mask_relu && !(x1 > 0.f)) ? 0.f : d * w1;
      *reinterpret_cast<uint32_t*>(dx + r * lddx + k) = pack_bf16(g0, g1);
    }
    atomicAdd(dw + k, a0); atomicAdd(dw + k + 1, a1);
  }
  if (db != nullptr && threadIdx.x == 0) {
    float s = 0.f;
    for (long long r = r0; r < r1; ++r) s += dy[r];
    atomicAdd(db, s);
  }
}

}  // namespace ew
}  // namespace recml

using namespace recml::ew;

extern "C" int recml_bce_logits(const void* logits, int logits_bf16, const float* labels, const float* weights,
                                long long n, float grad_scale, float* dlogits_f32, void* dlogits_bf16,
                                float* stats, float* hist_pos, float* hist_neg, int T, cudaStream_t stream) {
  if (n <= 0) return 0;
  int blocks = static_cast<int>((n + 1023) / 1024);
  blocks = blocks > 296 ? 296 : blocks;
  const size_t sh = T > 0 ? 2 * (T + 1) * sizeof(float) : 0;
  if (logits_bf16)
    bce_kernel<__nv_bfloat16><<<blocks, 256, sh, stream>>>(static_cast<const __nv_bfloat16*>(logits), labels, weights, n,
        grad_scale, dlogits_f32, static_cast<__nv_bfloat16*>(dlogits_bf16), stats, hist_pos, hist_neg, T);
  else
    bce_kernel<float><<<blocks, 256, sh, stream>>>(static_cast<const float*>(logits), labels, weights, n, grad_scale,
        dlogits_f32, static_cast<__nv_bfloat16*>(dlogits_bf16), stats, hist_pos, hist_neg, T);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int recml_cast_f32_bf16(const float* in, void* out, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  const long long threads = (n + 3) / 4;
  cast_f32_bf16_kernel<<<static_cast<int>((threads + 255) / 256), 256, 0, stream>>>(in, static_cast<__nv_bfloat16*>(out), n);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int recml_cast_pad_rows(const float* in, int cols_in, void* out, int cols_out, long long ld_out,
                                   long long M, cudaStream_t stream) {
  const long long n = M * cols_out;
  if (n <= 0) return 0;
  cast_pad_rows_kernel<<<static_cast<int>((n + 255) / 256), 256, 0, stream>>>(in, cols_in, static_cast<__nv_bfloat16*>(out),
                                                                             cols_out, ld_out, M);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// out must be zeroed by the caller unless accumulation is wanted.
extern "C" int recml_colsum_bf16(const void* x, long long M, int N, long long ld, float* out, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (N % 8 == 0 && ld % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    const int rows_per_block = 256;
    dim3 grid((N + 255) / 256, static_cast<unsigned>((M + rows_per_block - 1) / rows_per_block));
    colsum8_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), M, N, ld, out, rows_per_block);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
  }
  const int rows_per_block = 512;
  dim3 grid((N + 63) / 64, static_cast<unsigned>((M + rows_per_block - 1) / rows_per_block));
  colsum_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), M, N, ld, out, rows_per_block);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// colsum_dv: optional fp32 [N], pre-zeroed; receives the column sums of dv.
extern "C" int recml_cross_bwd_ew(const void* g, const void* x0, const void* v, void* dv, void* dx0, int accumulate,
                                  long long M, int N, long long ld, float* colsum_dv, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  const int rows_per_block = 128;
  dim3 grid((N + 255) / 256, static_cast<unsigned>((M + rows_per_block - 1) / rows_per_block));
  cross_bwd_ew_kernel<<<grid, 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(g), static_cast<const __nv_bfloat16*>(x0), static_cast<const __nv_bfloat16*>(v),
      static_cast<__nv_bfloat16*>(dv), static_cast<__nv_bfloat16*>(dx0), accumulate, M, N, ld, colsum_dv, rows_per_block);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int recml_add_bf16(const void* a, long long lda, const void* b, long long ldb, void* out, long long ldo,
                              long long M, int N, cudaStream_t stream) {
  const long long n = M * N / 8;
  if (n <= 0) return 0;
  add_bf16_kernel<<<static_cast<int>((n + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(a), lda, static_cast<const __nv_bfloat16*>(b), ldb,
      static_cast<__nv_bfloat16*>(out), ldo, M, N);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int recml_relu_mask_bf16(const void* dy, long long lddy, const void* y, long long ldy, void* out,
                                    long long ldo, long long M, int N, cudaStream_t stream) {
  const long long n = M * N / 8;
  if (n <= 0) return 0;
  relu_mask_kernel<<<static_cast<int>((n + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dy), lddy, static_cast<const __nv_bfloat16*>(y), ldy,
      static_cast<__nv_bfloat16*>(out), ldo, M, N);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int recml_silu_fwd_bf16(const void* z, void* h, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n % 8) return -2;
  const long long n8 = n / 8;
  silu_fwd_kernel<<<static_cast<int>((n8 + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(z), static_cast<__nv_bfloat16*>(h), n8);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int recml_silu_fwd_split(const void* z, void* u, void* qkv, long long T, int D, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D % 8) return -2;
  const long long n8 = T * 4 * D / 8;
  silu_fwd_split_kernel<<<static_cast<int>((n8 + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(z), static_cast<__nv_bfloat16*>(u), static_cast<__nv_bfloat16*>(qkv), T, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int recml_silu_bwd_gather4(const void* z, const void* g0, long long ld0, const float* g1, const void* g2,
                                      const void* g3, void* dz, long long T, int D, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D % 8 || ld0 % 8) return -2;
  const long long n8 = T * 4 * D / 8;
  silu_bwd_gather4_kernel<<<static_cast<int>((n8 + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(z), static_cast<const __nv_bfloat16*>(g0), ld0, g1,
      static_cast<const __nv_bfloat16*>(g2), static_cast<const __nv_bfloat16*>(g3), static_cast<__nv_bfloat16*>(dz), T, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int recml_gemv_fwd(const void* x, long long ld, int K, const float* w, const float* bias, float* y,
                              long long M, cudaStream_t stream) {
  if (M <= 0) return 0;
  gemv_fwd_kernel<<<static_cast<int>((M * 32 + 255) / 256), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), ld, K,
                                                                            w, bias, y, M);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int recml_gemv_bwd(const void* x, long long ld, int K, const float* w, const float* dy, long long M,
                              void* dx, long long lddx, int mask_relu, float* dw, float* db, cudaStream_t stream) {
  if (M <= 0) return 0;
  const int rows_per_block = 64;
  gemv_bwd_kernel<<<static_cast<int>((M + rows_per_block - 1) / rows_per_block), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), ld, K, w, dy, M, static_cast<__nv_bfloat16*>(dx), lddx, mask_relu, dw, db,
      rows_per_block);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
