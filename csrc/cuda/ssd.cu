// Mamba2 selective state-space scan (SSD recurrence) and the depthwise causal conv + SiLU in front
// of it, forward and backward, for sm_100a.
//
//   h_t[p,n] = exp(a_t) * h_{t-1}[p,n] + x_t[p] * b_t[n]        (one state matrix [P, N] per batch x head)
//   y_t[p]   = sum_n h_t[p,n] * c_t[n]
//
// with x = dt * x_raw, a = A * dt <= 0 and b, c shared by all heads of a sample (one group).
// Sequences of a recommender are short (L <= a few hundred) while batch x heads is in the thousands,
// so the scan is parallel over (batch, head) and sequential in time: one CTA per (batch, head) keeps
// the [P, N] state in registers, thread (p, g) owning N/4 interleaved columns of row p.  The forward
// stores the state every kCkpt steps; the backward walks the sequence in reverse in sub-chunks of
// kSub steps: it recomputes the states of a sub-chunk from the nearest checkpoint into shared
// memory, then runs the adjoint recurrence, reading h_{t-1} from there.
#include "common.cuh"

namespace recml {
namespace ssd {

constexpr int kCkpt = 32;   // forward checkpoints the state entering every 32nd step
constexpr int kSub = 8;     // backward keeps the states of 8 steps in shared memory

struct ScanParams {
  const float* x; const float* a; const float* b; const float* c; const float* init;   // init may be null
  long long init_batch_stride;      // 0: one [H,P,N] initial state for all samples
  float* y; float* ckpt;            // ckpt [B, H, n_ckpt, P, N]
  int B, L, H, P, N, n_ckpt;
  // backward only
  const float* dy; float* dx; float* da; float* db; float* dc; float* dinit;   // db / dc are [B, L, H, N] per-head partials
};

__device__ __forceinline__ float quad_sum(float v) {   // over the 4 threads that share a row p
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}

template <int NPT>
__global__ void __launch_bounds__(256) ssd_fwd_kernel(const ScanParams p) {
  constexpr int N = NPT * 4;
  extern __shared__ float smem[];
  const int P = p.P;
  float* sb = smem;                 // [kCkpt][N]
  float* sc = sb + kCkpt * N;       // [kCkpt][N]
  float* sx = sc + kCkpt * N;       // [kCkpt][P]
  float* sy = sx + kCkpt * P;       // [kCkpt][P]
  float* sa = sy + kCkpt * P;       // [kCkpt]
  const int bh = blockIdx.x, bi = bh / p.H, hi = bh % p.H;
  const int tid = threadIdx.x, row = tid >> 2, g = tid & 3;
  float h[NPT];
  if (p.init != nullptr) {
    const float* src = p.init + bi * p.init_batch_stride + (static_cast<long long>(hi) * P + row) * N;
#pragma unroll
    for (int i = 0; i < NPT; ++i) h[i] = src[i * 4 + g];
  } else {
#pragma unroll
    for (int i = 0; i < NPT; ++i) h[i] = 0.f;
  }
  const long long xbase = (static_cast<long long>(bi) * p.L * p.H + hi) * P;   // + t*H*P + row
  for (int t0 = 0; t0 < p.L; t0 += kCkpt) {
    const int steps = min(kCkpt, p.L - t0);
    // checkpoint: the state entering step t0
    float* ck = p.ckpt + ((static_cast<long long>(bh) * p.n_ckpt + t0 / kCkpt) * P + row) * N;
#pragma unroll
    for (int i = 0; i < NPT; ++i) ck[i * 4 + g] = h[i];
    __syncthreads();
    for (int i = tid; i < steps * N; i += blockDim.x) {
      const long long src = (static_cast<long long>(bi) * p.L + t0) * N + i;
      sb[i] = p.b[src];
      sc[i] = p.c[src];
    }
    for (int i = tid; i < steps * P; i += blockDim.x)
      sx[i] = p.x[xbase + static_cast<long long>(t0 + i / P) * p.H * P + (i % P)];
    if (tid < steps) sa[tid] = __expf(p.a[(static_cast<long long>(bi) * p.L + t0 + tid) * p.H + hi]);
    __syncthreads();
    for (int s = 0; s < steps; ++s) {
      const float decay = sa[s], xv = sx[s * P + row];
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < NPT; ++i) {
        h[i] = fmaf(decay, h[i], xv * sb[s * N + i * 4 + g]);
        acc = fmaf(h[i], sc[s * N + i * 4 + g], acc);
      }
      acc = quad_sum(acc);
      if (g == 0) sy[s * P + row] = acc;
    }
    __syncthreads();
    for (int i = tid; i < steps * P; i += blockDim.x)
      p.y[xbase + static_cast<long long>(t0 + i / P) * p.H * P + (i % P)] = sy[i];
  }
}

// Backward.  Shared memory: state history hist[kSub + 1][P][N + 4] (slot s = state after step
// t0 + s - 1, slot 0 = state entering the sub-chunk; the +4 padding keeps the (p, g) accesses on
// distinct banks), then b, c [kSub][N], x, dy [kSub][P], decay [kSub], da partials.
template <int NPT>
__global__ void __launch_bounds__(256) ssd_bwd_kernel(const ScanParams p) {
  constexpr int N = NPT * 4;
  constexpr int LD = N + 4;
  extern __shared__ float smem[];
  const int P = p.P;
  float* hist = smem;                         // [(kSub + 1) * P * LD]
  float* sb = hist + (kSub + 1) * P * LD;     // [kCkpt][N]   (a whole checkpoint interval is staged for the recompute)
  float* sc = sb + kCkpt * N;                 // [kSub][N]
  float* sx = sc + kSub * N;                  // [kCkpt][P]
  float* sdy = sx + kCkpt * P;                // [kSub][P]
  float* sa = sdy + kSub * P;                 // [kCkpt]
  float* sred = sa + kCkpt;                   // [kSub][8] per-warp partials of da
  const int bh = blockIdx.x, bi = bh / p.H, hi = bh % p.H;
  const int tid = threadIdx.x, row = tid >> 2, g = tid & 3, lane = tid & 31, warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;
  const long long xbase = (static_cast<long long>(bi) * p.L * p.H + hi) * P;
  float dh[NPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) dh[i] = 0.f;
  float next_decay = 0.f;                     // exp(a_{t+1}) of the step processed just before (in reverse)
  const int n_sub = (p.L + kSub - 1) / kSub;
  for (int sub = n_sub - 1; sub >= 0; --sub) {
    const int t0 = sub * kSub, steps = min(kSub, p.L - t0);
    const int ck = t0 / kCkpt, tc = ck * kCkpt;          // nearest checkpoint at or before t0
    const int pre = t0 - tc;                              // steps to replay before the sub-chunk
    __syncthreads();
    // stage b, x, decay for [tc, t0 + steps); c and dy only for the sub-chunk
    for (int i = tid; i < (pre + steps) * N; i += blockDim.x) sb[i] = p.b[(static_cast<long long>(bi) * p.L + tc) * N + i];
    for (int i = tid; i < steps * N; i += blockDim.x) sc[i] = p.c[(static_cast<long long>(bi) * p.L + t0) * N + i];
    for (int i = tid; i < (pre + steps) * P; i += blockDim.x)
      sx[i] = p.x[xbase + static_cast<long long>(tc + i / P) * p.H * P + (i % P)];
    for (int i = tid; i < steps * P; i += blockDim.x)
      sdy[i] = p.dy[xbase + static_cast<long long>(t0 + i / P) * p.H * P + (i % P)];
    if (tid < pre + steps) sa[tid] = __expf(p.a[(static_cast<long long>(bi) * p.L + tc + tid) * p.H + hi]);
    // replay the forward from the checkpoint
    float h[NPT];
    const float* ckp = p.ckpt + ((static_cast<long long>(bh) * p.n_ckpt + ck) * P + row) * N;
#pragma unroll
    for (int i = 0; i < NPT; ++i) h[i] = ckp[i * 4 + g];
    __syncthreads();
    for (int s = 0; s < pre; ++s) {
      const float decay = sa[s], xv = sx[s * P + row];
#pragma unroll
      for (int i = 0; i < NPT; ++i) h[i] = fmaf(decay, h[i], xv * sb[s * N + i * 4 + g]);
    }
#pragma unroll
    for (int i = 0; i < NPT; ++i) hist[(0 * P + row) * LD + i * 4 + g] = h[i];
    for (int s = 0; s < steps; ++s) {
      const float decay = sa[pre + s], xv = sx[(pre + s) * P + row];
#pragma unroll
      for (int i = 0; i < NPT; ++i) {
        h[i] = fmaf(decay, h[i], xv * sb[(pre + s) * N + i * 4 + g]);
        hist[((s + 1) * P + row) * LD + i * 4 + g] = h[i];
      }
    }
    __syncthreads();
    // dc_t[n] = sum_p dy_t[p] * h_t[p, n]: one (t, n) pair per thread and round, columns contiguous across lanes
    for (int item = tid; item < steps * N; item += blockDim.x) {
      const int s = item / N, n = item % N;
      float acc = 0.f;
      for (int q = 0; q < P; ++q) acc = fmaf(sdy[s * P + q], hist[((s + 1) * P + q) * LD + n], acc);
      p.dc[((static_cast<long long>(bi) * p.L + t0 + s) * p.H + hi) * N + n] = acc;
    }
    __syncthreads();
    // adjoint recurrence, newest step first; dh_t overwrites the slot of h_t once h_t is no longer needed
    for (int s = steps - 1; s >= 0; --s) {
      const float dyv = sdy[s * P + row];
      float dxv = 0.f, dav = 0.f;
      const float decay = sa[pre + s];
#pragma unroll
      for (int i = 0; i < NPT; ++i) {
        const int n = i * 4 + g;
        dh[i] = fmaf(next_decay, dh[i], dyv * sc[s * N + n]);
        dxv = fmaf(dh[i], sb[(pre + s) * N + n], dxv);
        dav = fmaf(dh[i] * decay, hist[(s * P + row) * LD + n], dav);     // d exp(a)/da = exp(a); uses h_{t-1}
        hist[((s + 1) * P + row) * LD + n] = dh[i];
      }
      next_decay = decay;
      dxv = quad_sum(dxv);
      if (g == 0) p.dx[xbase + static_cast<long long>(t0 + s) * p.H * P + row] = dxv;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) dav += __shfl_xor_sync(0xffffffffu, dav, o);
      if (lane == 0) sred[s * 8 + warp] = dav;
    }
    __syncthreads();
    if (tid < steps) {
      float acc = 0.f;
      for (int w = 0; w < nwarps; ++w) acc += sred[tid * 8 + w];
      p.da[(static_cast<long long>(bi) * p.L + t0 + tid) * p.H + hi] = acc;
    }
    // db_t[n] = sum_p dh_t[p, n] * x_t[p]
    for (int item = tid; item < steps * N; item += blockDim.x) {
      const int s = item / N, n = item % N;
      float acc = 0.f;
      for (int q = 0; q < P; ++q) acc = fmaf(hist[((s + 1) * P + q) * LD + n], sx[(pre + s) * P + q], acc);
      p.db[((static_cast<long long>(bi) * p.L + t0 + s) * p.H + hi) * N + n] = acc;
    }
  }
  // gradient of the initial state: dh carried past step 0
  if (p.dinit != nullptr) {
    float* dst = p.dinit + (static_cast<long long>(bh) * P + row) * N;
#pragma unroll
    for (int i = 0; i < NPT; ++i) dst[i * 4 + g] = next_decay * dh[i];
  }
}

// ---- depthwise causal conv (K taps) + SiLU ------------------------------------------------------------
//   u[t, ch] = bias[ch] + sum_k w[ch, k] * x[t - (K-1) + k, ch];   y = u * sigmoid(u)
template <int K>
__global__ void conv_fwd_kernel(const float* x, const float* w, const float* bias, float* y, int B, int L, int C) {
  const long long total = static_cast<long long>(B) * L * C;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int ch = static_cast<int>(i % C);
    const int t = static_cast<int>((i / C) % L);
    float u = bias != nullptr ? bias[ch] : 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int tt = t - (K - 1) + k;
      if (tt >= 0) u = fmaf(w[ch * K + k], x[i + static_cast<long long>(tt - t) * C], u);
    }
    y[i] = u / (1.f + __expf(-u));
  }
}

// dx[t] = sum_k w[k] * du[t + (K-1) - k];  dw / dbias are reduced per channel by a second kernel.
template <int K>
__global__ void conv_bwd_dx_kernel(const float* x, const float* w, const float* bias, const float* dy, float* dx,
                                   float* du_out, int B, int L, int C) {
  const long long total = static_cast<long long>(B) * L * C;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int ch = static_cast<int>(i % C);
    const int t = static_cast<int>((i / C) % L);
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int to = t + (K - 1) - k;      // output position that read x[t] through tap k
      if (to >= L) continue;
      // recompute u[to] and the SiLU derivative
      float u = bias != nullptr ? bias[ch] : 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j) {
        const int tt = to - (K - 1) + j;
        if (tt >= 0) u = fmaf(w[ch * K + j], x[i + static_cast<long long>(tt - t) * C], u);
      }
      const float sg = 1.f / (1.f + __expf(-u));
      const float du = dy[i + static_cast<long long>(to - t) * C] * sg * (1.f + u * (1.f - sg));
      if (k == K - 1) du_out[i] = du;      // to == t: this thread owns du[t]
      acc = fmaf(w[ch * K + k], du, acc);
    }
    dx[i] = acc;
  }
}

// dw[ch, k] = sum_{b,t} du[b,t,ch] * x[b, t-(K-1)+k, ch];  dbias[ch] = sum du.  One block per 32 channels.
template <int K>
__global__ void __launch_bounds__(256) conv_bwd_dw_kernel(const float* x, const float* du, float* dw, float* dbias,
                                                          int B, int L, int C) {
  __shared__ float part[8][32][K + 1];
  const int lane = threadIdx.x & 31, wy = threadIdx.x >> 5;
  const int ch = blockIdx.x * 32 + lane;
  float acc[K + 1];
#pragma unroll
  for (int k = 0; k <= K; ++k) acc[k] = 0.f;
  if (ch < C) {
    const long long rows = static_cast<long long>(B) * L;
    for (long long r = wy; r < rows; r += 8) {
      const int t = static_cast<int>(r % L);
      const float d = du[r * C + ch];
      acc[K] += d;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const int tt = t - (K - 1) + k;
        if (tt >= 0) acc[k] = fmaf(d, x[(r + tt - t) * C + ch], acc[k]);
      }
    }
  }
#pragma unroll
  for (int k = 0; k <= K; ++k) part[wy][lane][k] = acc[k];
  __syncthreads();
  if (wy == 0 && ch < C) {
#pragma unroll
    for (int k = 0; k <= K; ++k) {
      float s = 0.f;
      for (int j = 0; j < 8; ++j) s += part[j][lane][k];
      if (k < K) dw[ch * K + k] = s; else if (dbias != nullptr) dbias[ch] = s;
    }
  }
}

}  // namespace ssd
}  // namespace recml

using namespace recml::ssd;

extern "C" int recml_ssd_struct_size() { return static_cast<int>(sizeof(ScanParams)); }
extern "C" int recml_ssd_ckpt_interval() { return kCkpt; }

static size_t fwd_smem(int P, int N) { return sizeof(float) * (2 * kCkpt * N + 2 * kCkpt * P + kCkpt); }
static size_t bwd_smem(int P, int N) {
  return sizeof(float) * ((kSub + 1) * P * (N + 4) + kCkpt * N + kSub * N + kCkpt * P + kSub * P + kCkpt + kSub * 8);
}

// P in {8, 16, 32, 64}, N in {16, 32, 64, 128}; anything else returns -10 and the caller falls back.
extern "C" int recml_ssd_scan(const ScanParams* p, int backward, cudaStream_t stream) {
  const int P = p->P, N = p->N;
  if (!(P == 8 || P == 16 || P == 32 || P == 64) || !(N == 16 || N == 32 || N == 64 || N == 128)) return -10;
  const int threads = P * 4;
  const int blocks = p->B * p->H;
  if (blocks <= 0 || p->L <= 0) return 0;
  const size_t smem = backward ? bwd_smem(P, N) : fwd_smem(P, N);
  if (smem > 227 * 1024) return -11;
#define RECML_SSD(NPT)                                                                                     \
  do {                                                                                                     \
    if (backward) {                                                                                        \
      cudaFuncSetAttribute(ssd_bwd_kernel<NPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
      ssd_bwd_kernel<NPT><<<blocks, threads, smem, stream>>>(*p);                                          \
    } else {                                                                                               \
      cudaFuncSetAttribute(ssd_fwd_kernel<NPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
      ssd_fwd_kernel<NPT><<<blocks, threads, smem, stream>>>(*p);                                          \
    }                                                                                                      \
  } while (0)
  switch (N) {
    case 16: RECML_SSD(4); break;
    case 32: RECML_SSD(8); break;
    case 64: RECML_SSD(16); break;
    default: RECML_SSD(32); break;
  }
#undef RECML_SSD
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

static int conv_blocks(long long total) {
  long long b = (total + 255) / 256;
  return static_cast<int>(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

extern "C" int recml_conv1d_silu_fwd(const float* x, const float* w, const float* bias, float* y, int B, int L, int C,
                                     int K, cudaStream_t stream) {
  const long long total = static_cast<long long>(B) * L * C;
  if (total == 0) return 0;
  switch (K) {
    case 2: conv_fwd_kernel<2><<<conv_blocks(total), 256, 0, stream>>>(x, w, bias, y, B, L, C); break;
    case 3: conv_fwd_kernel<3><<<conv_blocks(total), 256, 0, stream>>>(x, w, bias, y, B, L, C); break;
    case 4: conv_fwd_kernel<4><<<conv_blocks(total), 256, 0, stream>>>(x, w, bias, y, B, L, C); break;
    default: return -10;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// du is a [B, L, C] scratch the caller provides; dbias may be null.
extern "C" int recml_conv1d_silu_bwd(const float* x, const float* w, const float* bias, const float* dy, float* dx,
                                     float* du, float* dw, float* dbias, int B, int L, int C, int K,
                                     cudaStream_t stream) {
  const long long total = static_cast<long long>(B) * L * C;
  if (total == 0) return 0;
  const int cb = (C + 31) / 32;
  switch (K) {
#define RECML_CONV(KK)                                                                              \
    case KK:                                                                                        \
      conv_bwd_dx_kernel<KK><<<conv_blocks(total), 256, 0, stream>>>(x, w, bias, dy, dx, du, B, L, C); \
      conv_bwd_dw_kernel<KK><<<cb, 256, 0, stream>>>(x, du, dw, dbias, B, L, C);                    \
      break;
    RECML_CONV(2)
    RECML_CONV(3)
    RECML_CONV(4)
#undef RECML_CONV
    default: return -10;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
