// Jagged HSTU attention for sm_100a:  O = silu(Q·K^T·scale + bias) / n · V   per sequence, where `bias`
// carries the learned relative-position and time-bucket terms AND every mask (causal, sequence end,
// sliding window, segment ids) as a large negative value.
//
// Sequences are packed back to back ([T, H, Dh] bf16, seq_offsets[B+1]).  One CTA owns a 128-query
// tile of one sequence and one head and walks over the key/value tiles it may see (causal: tiles up
// to its own).  Per key tile:
//   TMA (warp 0)        K_j, V_j -> shared memory (2 stages)
//   tcgen05.mma (warp 1) S = Q·K_j^T into tensor memory
//   warps 2..17          (each 32 rows x 32 columns of the score tile) tcgen05.ld S, load the matching
//                        piece of the pair's BIAS TILE, h = s·scale/2 + bias/2, p = h·tanh(h) + h
//                        (= x·sigmoid(x)); bf16 P written to shared memory in the 128-byte-swizzled
//                        K-major layout the tensor core expects
//   tcgen05.mma (warp 1) O += P·V_j    (V consumed as an MN-major operand straight from its [kv, Dh] tile)
// Bias tiles: the bias of a (query tile, key tile) pair depends on the batch (lengths, timestamps) and on
// the two small weight tables, not on the head or the layer, so it is evaluated ONCE per step by
// bias_tile_kernel into bf16 blocks of 128 x 128 (already halved; masked entries hold -15000, for which
// tanh gives exactly -1 and the element and its derivative vanish).  The per-element work of the attention
// kernels is then one fused multiply-add, one tanh and one more fused multiply-add, with no predicates and
// no table lookups.  The backward kernel (one CTA per key tile and head, walking over the query tiles that
// see it) recomputes S and forms dV += P^T·dO, dK += dS^T·Q, dQ += dS·K on the tensor cores; it adds dS
// (fp32 vector reductions) into a gradient block per tile pair, summed over heads and layers, from which
// bias_grad_kernel takes the gradients of the two tables once per step (diagonal sums by a lane-rotating
// accumulator, time buckets by runs of equal buckets).
// CTAs take their tiles from a list sorted by decreasing work (the backward has its own order) with the
// heads varying fastest.  A softmax mode (SASRec / BERT4Rec blocks) shares the pipeline.
// All waits are bounded; a CTA that gives up drains and frees its tensor memory.
#include "tcgen05.cuh"

namespace recml {
namespace hstu {
using namespace recml::tc;

constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int kThreads = 576;        // TMA warp, MMA warp, 16 element-wise warps (four per tensor-memory lane quarter,
constexpr int kCompute = 512;        // each covering 32 rows x 32 columns of a score tile)
constexpr float kBucketSize = 0.301f;

struct Params {
  int T, H, Dh, B, max_seq_len, num_buckets, causal;
  float scale, inv_n;
  const int* seq_offsets;
  const int* tile_seq;        // [n_tiles] sequence of each 128-row tile (-1: unused slot)
  const int* tile_row0;       // [n_tiles] first position (within the sequence) of the tile
  const int* timestamps;      // seconds relative to the earliest timestamp of the batch (int32)
  const float* pos_w;
  const float* ts_w;
  __nv_bfloat16* out;         // fwd: O [T, H*Dh]
  // backward only
  float* dq;                  // [T, H*Dh] fp32, accumulated with atomics (pre-zeroed)
  __nv_bfloat16* dk;          // [T, H*Dh]
  __nv_bfloat16* dv;
  float* dpos_w;              // [2N-1] (pre-zeroed) or null
  float* dts_w;               // [num_buckets+1] (pre-zeroed) or null
  int* status;
  // softmax mode (SASRec / BERT4Rec blocks): P = softmax over the visible keys instead of SiLU / n.
  // The forward needs the whole key row in tensor memory (max_seq_len <= 256: two score tiles) and
  // writes the row log-sum-exp; the backward reads it back together with delta = rowsum(dO * O).
  int mode;                   // Mode below
  float* lse;                 // [T, H]
  const float* delta;         // [T, H] (backward)
  // row pitch in elements of q / k / v / dO when they are column slices of a wider matrix (0: H * Dh)
  int ld_q, ld_k, ld_v, ld_do;
  // Time buckets of every (query tile, key tile) pair, computed once per batch because all heads, layers
  // and both passes use the same ones: pair (qt, kt) of sequence s is the 128 x 128 uint8 block number
  // pair_base[s] + (causal ? qt (qt + 1) / 2 + kt : qt * n_tiles(s) + kt).  Null: buckets are computed inline.
  const unsigned char* bucket_cache;
  const int* pair_base;       // [B + 1]
  int cap_pairs;              // blocks the caches can hold
  // Bias tiles (SiLU mode): pair-indexed like the bucket cache, 16384 bf16 per pair in the element order of
  // the attention kernels' threads (tile_offset below); values are HALF the bias, masked entries -15000.
  const __nv_bfloat16* bias_tiles;
  float* dbias_tiles;         // backward: 16384 fp32 per pair, same order, accumulated with reductions (or null)
  int window;                 // >= 0: query i sees keys i - window .. i + window (intersected with causality)
  const int* segment_ids;     // [T] or null: a query sees only keys of its own segment
  // Decay mode (the quadratic form of the Mamba2 state-space recurrence): P[l, s] = S[l, s] * 2^(cum[l] - cum[s])
  // for s <= l, with q = C and k = B shared by all heads ([T, Dh]), v = X [T, H * Dh].
  const float* cum;           // [H, cum_pitch]: inclusive prefix sums of a * log2(e) along each sequence
  long long cum_pitch;        // >= T + 128 so that a tile may read past the last token
  int qk_shared;              // 1: q / k (and dq / dk) have one head that all heads of v share
  float* dk_acc;              // decay mode: dk accumulated in fp32 [T, Dh] (pre-zeroed) like dq
  // Gradient w.r.t. the (natural-log) prefix sums, [H, cum_pitch], pre-zeroed:
  //   dcum[l] = sum_s dP[l, s] P[l, s] - sum_l' dP[l', l] P[l', l]
  // The row sums are taken where dP and P are formed; the column sums equal x_s . dx_s (dx = P^T dO), taken when dv
  // is read out.  Both use the bf16-rounded P that the tensor cores saw, so the two halves cancel as they should.
  float* dcum;
  const __nv_bfloat16* v_rows;   // v as a plain pointer (row pitch ld_v) for that dot product
  // Attention-weight dropout (SiLU mode): element (head, query token, key token) is kept when a counter-based hash
  // of its indices and the 64-bit key is at or above drop_threshold = p * 2^32; kept weights are scaled by keep_scale
  // = 1 / (1 - p).  The backward pass regenerates the same mask from the same key.
  const unsigned long long* dropout_key;
  unsigned int drop_threshold;
  float keep_scale;
};

enum Mode { kSilu = 0, kSoftmax = 1, kDecay = 2, kSiluDropout = 3, kSoftmaxDropout = 4 };

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}
// per (head, query token) part of the dropout hash, and the per-element decision
__device__ __forceinline__ uint32_t dropout_row_hash(unsigned long long key, int head, int q_token) {
  return mix32(static_cast<uint32_t>(key) ^ (static_cast<uint32_t>(q_token) * 0x9E3779B1u) ^
               (static_cast<uint32_t>(head + 1) * 0x85EBCA6Bu));
}
__device__ __forceinline__ bool dropout_keep(uint32_t row_hash, uint32_t key_hi, int k_token, uint32_t threshold) {
  return mix32(row_hash ^ (static_cast<uint32_t>(k_token) * 0xC2B2AE35u + key_hi)) >= threshold;
}

constexpr float kMaskedHalfBias = -15000.f;

// 16-byte fp32 vector reduction into global memory (no return value)
__device__ __forceinline__ void red_add_v4(float4* dst, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Element (r, c) of a 128 x 128 tile as the attention kernels' threads see it: warp (quarter = r / 32,
// cb = c / 32), lane = r % 32, 32 consecutive columns per thread in vectors of `vec` elements.  A warp's
// vector load or reduction of one vector index touches consecutive memory.
__device__ __forceinline__ int tile_offset(int r, int c, int vec) {
  const int quarter = r >> 5, lane = r & 31, cb = c >> 5, within = c & 31;
  const int per_thread = 32 / vec;
  return (((cb * 4 + quarter) * per_thread + within / vec) * 32 + lane) * vec + within % vec;
}

// Lists the 128-row tiles of every sequence: tile t belongs to sequence tile_seq[t] and starts at
// position tile_row0[t].  Slots beyond the real number of tiles keep -1.  The list is ordered by
// decreasing work so that the CTAs dispatched last are the short ones (under causal masking the
// forward's query tile i visits i + 1 key tiles, the backward's key tile i visits n - i query
// tiles): level w = max_n .. 1 lists, for every sequence with at least w tiles, the tile with w steps.
__global__ void tile_list_kernel(const int* seq_offsets, int B, int* tile_seq, int* tile_row0, int cap, int backward) {
  if (blockIdx.x != 0 || threadIdx.x >= 32) return;
  const int lane = threadIdx.x;
  int max_n = 0;
  for (int b = lane; b < B; b += 32) max_n = max(max_n, (seq_offsets[b + 1] - seq_offsets[b] + BQ - 1) / BQ);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) max_n = max(max_n, __shfl_xor_sync(0xffffffffu, max_n, o));
  int t = 0;
  for (int w = max_n; w >= 1; --w) {
    for (int b0 = 0; b0 < B; b0 += 32) {
      const int b = b0 + lane;
      const int n = b < B ? (seq_offsets[b + 1] - seq_offsets[b] + BQ - 1) / BQ : 0;
      const bool has = n >= w;
      const unsigned mask = __ballot_sync(0xffffffffu, has);
      const int at = t + __popc(mask & ((1u << lane) - 1u));
      if (has && at < cap) { tile_seq[at] = b; tile_row0[at] = (backward ? n - w : w - 1) * BQ; }
      t += __popc(mask);
    }
  }
}

// the single-instruction tanh approximation (one special-function op instead of exp + rcp); exactly -1 / +1
// for arguments of large magnitude
__device__ __forceinline__ float tanh_fast(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
  return t;
}

__device__ __forceinline__ float exp2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 32 consecutive prefix sums, the same for every lane of the warp: 16-byte loads when the address allows
__device__ __forceinline__ void load_cum32(const float* src, float (&dst)[32]) {
  if ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      const float4 t = __ldg(reinterpret_cast<const float4*>(src) + g);
      dst[4 * g] = t.x; dst[4 * g + 1] = t.y; dst[4 * g + 2] = t.z; dst[4 * g + 3] = t.w;
    }
  } else {
#pragma unroll
    for (int e = 0; e < 32; ++e) dst[e] = __ldg(src + e);
  }
}

// bucket = clip(int(ln(clip(|dt|, 1, 1e9)) / 0.301), 0, num_buckets), with ln taken as log2 * ln(2)
__device__ __forceinline__ int time_bucket(int dt, int num_buckets) {
  int a = dt < 0 ? -dt : dt;
  a = a < 1 ? 1 : (a > 1000000000 ? 1000000000 : a);
  const int b = static_cast<int>(__log2f(static_cast<float>(a)) * (0.69314718f / kBucketSize));
  return b > num_buckets ? num_buckets : b;
}

__device__ __forceinline__ int pair_index(const Params& p, int seq, int n_tiles, int qt, int kt) {
  return p.pair_base[seq] + (p.causal ? qt * (qt + 1) / 2 + kt : qt * n_tiles + kt);
}
// byte `col` of the 32 bucket bytes a thread holds for its row (col is a compile-time constant after unrolling)
__device__ __forceinline__ int bucket_byte(const uint32_t (&w)[8], int col) { return (w[col >> 2] >> ((col & 3) * 8)) & 0xff; }

// pair_base[s] = number of cached tile pairs of the sequences before s.
__global__ void pair_base_kernel(const int* seq_offsets, int B, int causal, int* pair_base) {
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  int acc = 0;
  for (int b = 0; b < B; ++b) {
    pair_base[b] = acc;
    const int n = (seq_offsets[b + 1] - seq_offsets[b] + BQ - 1) / BQ;
    acc += causal ? n * (n + 1) / 2 : n * n;
  }
  pair_base[B] = acc;
}

// One block per (query tile of the forward list, key tile): 256 threads, thread = (row, 64-column half).
__global__ void __launch_bounds__(256) bucket_cache_kernel(const int* seq_offsets, const int* tile_seq, const int* tile_row0,
                                                           const int* timestamps, const int* pair_base, int num_buckets,
                                                           int causal, int cap_pairs, unsigned char* cache) {
  const int seq = tile_seq[blockIdx.x];
  if (seq < 0) return;
  const int q0 = tile_row0[blockIdx.x], qt = q0 / BQ, kt = blockIdx.y;
  const int seq_start = seq_offsets[seq];
  const int L = seq_offsets[seq + 1] - seq_start;
  const int nt = (L + BQ - 1) / BQ;
  if (kt >= nt || (causal && kt > qt)) return;
  const int pair = pair_base[seq] + (causal ? qt * (qt + 1) / 2 + kt : qt * nt + kt);
  if (pair >= cap_pairs) return;
  __shared__ int ts_k[BKV];
  const int kv0 = kt * BKV;
  if (threadIdx.x < BKV) ts_k[threadIdx.x] = (kv0 + threadIdx.x < L) ? timestamps[seq_start + kv0 + threadIdx.x] : 0;
  __syncthreads();
  const int r = threadIdx.x >> 1, c0 = (threadIdx.x & 1) * 64;
  const int qi = q0 + r;
  const int tq = qi < L ? timestamps[seq_start + (qi + 1 < L ? qi + 1 : L - 1)] : 0;
  unsigned char* dst = cache + (static_cast<size_t>(pair) << 14) + r * BKV + c0;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t v = 0;
#pragma unroll
      for (int b = 0; b < 4; ++b) v |= static_cast<uint32_t>(time_bucket(tq - ts_k[c0 + g * 16 + j * 4 + b], num_buckets)) << (8 * b);
      w[j] = v;
    }
    *reinterpret_cast<uint4*>(dst + g * 16) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// One lane polls the mbarrier, the result is broadcast: the whole warp takes the same branch, so warp-level
// synchronisation after it can never be left waiting for a lane that gave up.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                          int where, int lane) {
  int ok = 1;
  if (lane == 0) ok = mbar_wait(bar, parity, abort_flag, status, where) ? 1 : 0;
  ok = __shfl_sync(0xffffffffu, ok, 0);
  return ok != 0;
}

// ---- bias tiles: half the bias (position + time-bucket terms) of every visible element, a large negative
// value for every masked one.  One block per (query tile of the forward list, key tile); thread = (row,
// 64-column half).
struct BiasParams {
  const int* seq_offsets; const int* tile_seq; const int* tile_row0; const int* pair_base;
  int causal, cap_pairs, max_seq_len, window, num_buckets;
  const int* segment_ids; const float* pos_w; const float* ts_w;
  const unsigned char* bucket_cache;
  __nv_bfloat16* tiles;
  float* dbias; float* dpos_w; float* dts_w;     // gradient pass
  int* status;
};

__global__ void __launch_bounds__(256) bias_tile_kernel(const BiasParams p) {
  const int seq = p.tile_seq[blockIdx.x];
  if (seq < 0) return;
  const int q0 = p.tile_row0[blockIdx.x], qt = q0 / BQ, kt = blockIdx.y;
  const int seq_start = p.seq_offsets[seq];
  const int L = p.seq_offsets[seq + 1] - seq_start;
  const int nt = (L + BQ - 1) / BQ;
  if (kt >= nt || (p.causal && kt > qt)) return;
  const int pair = p.pair_base[seq] + (p.causal ? qt * (qt + 1) / 2 + kt : qt * nt + kt);
  if (pair >= p.cap_pairs) { report(p.status, kCapacity, 2); return; }
  __shared__ float posw[256];
  __shared__ float tsw[256];
  __shared__ int seg_k[BKV];
  const int kv0 = kt * BKV;
  {
    // element (r, c) needs pos_w[(kv0 + c) - (q0 + r) + N - 1] = window[c - r + 127]
    const int base = kv0 - q0 + p.max_seq_len - 1 - 127;
    const int idx = base + static_cast<int>(threadIdx.x);
    posw[threadIdx.x] = (p.pos_w != nullptr && threadIdx.x < 255 && idx >= 0 && idx < 2 * p.max_seq_len - 1)
                            ? __ldg(p.pos_w + idx) : 0.f;
    tsw[threadIdx.x] = (p.ts_w != nullptr && static_cast<int>(threadIdx.x) <= p.num_buckets) ? __ldg(p.ts_w + threadIdx.x) : 0.f;
    if (threadIdx.x < BKV)
      seg_k[threadIdx.x] = (p.segment_ids != nullptr && kv0 + threadIdx.x < L) ? p.segment_ids[seq_start + kv0 + threadIdx.x] : 0;
  }
  __syncthreads();
  const int r = threadIdx.x >> 1, c0 = (threadIdx.x & 1) * 64;
  const int qi = q0 + r;
  const bool row_ok = qi < L;
  const int seg_q = (p.segment_ids != nullptr && row_ok) ? p.segment_ids[seq_start + qi] : 0;
  const unsigned char* brow = p.bucket_cache != nullptr
      ? p.bucket_cache + (static_cast<size_t>(pair) << 14) + r * BKV + c0 : nullptr;
  __nv_bfloat16* out = p.tiles + (static_cast<size_t>(pair) << 14);
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    uint32_t bytes[2] = {0u, 0u};
    if (brow != nullptr && p.ts_w != nullptr) {
      const uint2 t = *reinterpret_cast<const uint2*>(brow + g * 8);
      bytes[0] = t.x; bytes[1] = t.y;
    }
    float val[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int c = c0 + g * 8 + e;
      const int kj = kv0 + c;
      bool vis = row_ok && kj < L && (!p.causal || kj <= qi);
      if (p.window >= 0) vis = vis && kj >= qi - p.window && kj <= qi + p.window;
      if (p.segment_ids != nullptr) vis = vis && seg_q == seg_k[c];
      float b = posw[c - r + 127];
      if (p.ts_w != nullptr) b += tsw[(bytes[e >> 2] >> ((e & 3) * 8)) & 0xff];
      val[e] = vis ? 0.5f * b : kMaskedHalfBias;
    }
    *reinterpret_cast<uint4*>(out + tile_offset(r, c0 + g * 8, 8)) =
        make_uint4(pack_bf16(val[0], val[1]), pack_bf16(val[2], val[3]), pack_bf16(val[4], val[5]), pack_bf16(val[6], val[7]));
  }
}

// ---- gradients of the two bias tables from the per-pair gradient blocks (which are cleared on the way, so
// the buffer is all zeros again for the next step).  One block of 16 warps per tile pair, the same
// thread-to-element map as the attention kernels.  Masked elements hold exact zeros.
__global__ void __launch_bounds__(512) bias_grad_kernel(const BiasParams p) {
  const int seq = p.tile_seq[blockIdx.x];
  if (seq < 0) return;
  const int q0 = p.tile_row0[blockIdx.x], qt = q0 / BQ, kt = blockIdx.y;
  const int seq_start = p.seq_offsets[seq];
  const int L = p.seq_offsets[seq + 1] - seq_start;
  const int nt = (L + BQ - 1) / BQ;
  if (kt >= nt || (p.causal && kt > qt)) return;
  const int pair = p.pair_base[seq] + (p.causal ? qt * (qt + 1) / 2 + kt : qt * nt + kt);
  if (pair >= p.cap_pairs) return;
  __shared__ float hist[512];           // [0, 255) diagonals, [256, 512) time buckets
  __shared__ float diag[16][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quarter = warp & 3, cb = warp >> 2;
  const int r = quarter * 32 + lane;
  hist[threadIdx.x] = 0.f;
  __syncthreads();
  float ds[32];
  float4* src = reinterpret_cast<float4*>(p.dbias + (static_cast<size_t>(pair) << 14)) + (cb * 4 + quarter) * 8 * 32 + lane;
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    const float4 t = src[g * 32];
    src[g * 32] = make_float4(0.f, 0.f, 0.f, 0.f);
    ds[4 * g] = t.x; ds[4 * g + 1] = t.y; ds[4 * g + 2] = t.z; ds[4 * g + 3] = t.w;
  }
  if (p.dpos_w != nullptr) {
    // This lane's element lies on diagonal (col - lane) of the warp's 32 x 32 block; the partial sum of a
    // diagonal travels one lane up per column, so every lane adds its element to the sum passing through it.
    // The diagonal leaving lane 31 is complete and is parked; after the last column those 31 and the 32
    // diagonals still in flight go to the histogram (bin = c - r + 127).
    float dacc = 0.f;
#pragma unroll
    for (int col = 0; col < 32; ++col) {
      dacc += ds[col];
      if (col < 31) {
        if (lane == 31) diag[warp][col] = dacc;
        const float below = __shfl_sync(0xffffffffu, dacc, (lane + 31) & 31);
        dacc = lane == 0 ? 0.f : below;
      }
    }
    atomicAdd(hist + (cb * 32 + 31 - r + 127), dacc);
    __syncwarp();
    if (lane < 31) atomicAdd(hist + (cb * 32 + lane - (quarter * 32 + 31) + 127), diag[warp][lane]);
  }
  if (p.dts_w != nullptr && p.bucket_cache != nullptr) {
    // along a row the bucket changes rarely (log-spaced buckets, increasing timestamps): runs of equal buckets
    // are summed in a register and flushed with one atomic
    const uint4* bc = reinterpret_cast<const uint4*>(p.bucket_cache + (static_cast<size_t>(pair) << 14) + r * BKV + cb * 32);
    const uint4 b0 = __ldg(bc), b1 = __ldg(bc + 1);
    const uint32_t bk[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
    int run_bucket = -1;
    float run_sum = 0.f;
#pragma unroll
    for (int col = 0; col < 32; ++col) {
      const int bucket = bucket_byte(bk, col);
      if (bucket != run_bucket) {
        if (run_bucket >= 0 && run_sum != 0.f) atomicAdd(hist + 256 + run_bucket, run_sum);
        run_bucket = bucket;
        run_sum = 0.f;
      }
      run_sum += ds[col];
    }
    if (run_bucket >= 0 && run_sum != 0.f) atomicAdd(hist + 256 + run_bucket, run_sum);
  }
  __syncthreads();
  const int kv0 = kt * BKV;
  if (threadIdx.x < 255) {
    const float v = hist[threadIdx.x];
    const int idx = (kv0 - q0) + (static_cast<int>(threadIdx.x) - 127) + p.max_seq_len - 1;
    if (v != 0.f && p.dpos_w != nullptr && idx >= 0 && idx < 2 * p.max_seq_len - 1) atomicAdd(p.dpos_w + idx, v);
  } else if (threadIdx.x >= 256) {
    const int b = threadIdx.x - 256;
    const float v = hist[threadIdx.x];
    if (v != 0.f && p.dts_w != nullptr && b <= p.num_buckets) atomicAdd(p.dts_w + b, v);
  }
}

template <int DH>
struct Smem {
  static constexpr int kSub = DH / 64;                 // 64-column sub-tiles per operand tile
  static constexpr int kTile = BQ * 64 * 2 * kSub;     // bytes of one [128, DH] bf16 tile
  static constexpr int kQ = 0;
  static constexpr int kK = kTile;                     // 2 stages
  static constexpr int kV = kK + 2 * kTile;            // 2 stages
  static constexpr int kP = kV + 2 * kTile;            // [128, 128] bf16 = 32 KB
  static constexpr int kBars = kP + BQ * BKV * 2;
  static constexpr int kTotal = kBars + 128 + 1024;
  static constexpr int kTmemCols = 512;                // S: 2 x 128 columns, O: DH columns
};

template <int DH, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
hstu_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const Params p) {
  constexpr bool SOFTMAX = MODE == kSoftmax || MODE == kSoftmaxDropout, SILU = MODE == kSilu || MODE == kSiluDropout;
  constexpr bool DECAY = MODE == kDecay, DROP = MODE == kSiluDropout || MODE == kSoftmaxDropout;
  using S = Smem<DH>;
  // CTAs are dispatched in linear block order; heads vary fastest so that this order follows the work-sorted list
  const int lin = blockIdx.x + gridDim.x * blockIdx.y;
  const int tile_id = lin / p.H;
  const int seq = p.tile_seq[tile_id];
  if (seq < 0) return;   // whole CTA leaves before touching barriers or tensor memory
  if (SILU && p.pair_base[seq + 1] > p.cap_pairs) {   // the bias tiles of this sequence do not exist
    if (threadIdx.x == 0) report(p.status, kCapacity, 3);
    return;
  }
  const int h = lin % p.H;
  const int q0 = p.tile_row0[tile_id];
  const int seq_start = p.seq_offsets[seq];
  const int L = p.seq_offsets[seq + 1] - seq_start;
  const int tok0 = seq_start + q0;
  const int n_kv = p.causal ? (q0 / BKV + 1) : (L + BKV - 1) / BKV;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + S::kBars;
  // barrier slots: 0 q_full, 1-2 kv_full, 3-4 kv_empty, 5-6 s_full, 7-8 s_empty, 9 p_full, 10 p_empty, 11 o_full
  auto bar = [&](int i) { return bars + 8u * i; };
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ float softmax_xchg[SOFTMAX ? 1024 : 1];     // [parity][column block][row]: row maxima / partial sums
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int i = 0; i <= 6; ++i) mbar_init(bar(i), 1);
    mbar_init(bar(7), kCompute);
    mbar_init(bar(8), kCompute);
    mbar_init(bar(9), kCompute);
    mbar_init(bar(10), 1);
    mbar_init(bar(11), 1);
    for (int i = 12; i <= 15; ++i) mbar_init(bar(i), 128);    // softmax mode: the four warps of a lane quarter
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_slot), S::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // tensor memory: S buffers at columns [0,128) and [128,256), O at [256, 256+DH)
  const uint32_t tmem_o = tmem_slot + 256;
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar(0), S::kTile);
      const int hq = p.qk_shared ? 0 : h * DH;   // column of this head in q / k
      for (int d = 0; d < S::kSub; ++d) tma_load_2d(base + S::kQ + d * 16384, &map_q, hq + 64 * d, tok0, bar(0));
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        if (!mbar_wait(bar(3 + s), ((j >> 1) & 1) ^ 1, abortp, p.status, 40)) break;
        mbar_expect_tx(bar(1 + s), 2 * S::kTile);
        const int row = seq_start + j * BKV;
        for (int d = 0; d < S::kSub; ++d) {
          tma_load_2d(base + S::kK + s * S::kTile + d * 16384, &map_k, hq + 64 * d, row, bar(1 + s));
          tma_load_2d(base + S::kV + s * S::kTile + d * 16384, &map_v, h * DH + 64 * d, row, bar(1 + s));
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = idesc_bf16(BQ, BKV, false, false);
      const uint32_t idesc_o = idesc_bf16(BQ, DH, false, true);
      bool ok = mbar_wait(bar(0), 0, abortp, p.status, 41);
      // S_j = Q·K_j^T goes to S buffer j&1, so the scores of tile j+1 are produced while the element-wise
      // warps still work on tile j
      auto issue_qk = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(bar(1 + s), (j >> 1) & 1, abortp, p.status, 42)) return false;
        if (j >= 2 && !mbar_wait(bar(7 + s), ((j >> 1) - 1) & 1, abortp, p.status, 43)) return false;
        tc_fence_after();
        const uint32_t sk = base + S::kK + s * S::kTile;
#pragma unroll
        for (int d = 0; d < S::kSub; ++d)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_bf16(tmem_slot + s * 128, make_desc(base + S::kQ + d * 16384 + k * 32, 16, 1024),
                        make_desc(sk + d * 16384 + k * 32, 16, 1024), idesc_s, (d | k) ? 1u : 0u);
        tc_commit(bar(5 + s));
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j & 1;
        if (j + 1 < n_kv && !issue_qk(j + 1)) break;
        if (!mbar_wait(bar(9), j & 1, abortp, p.status, 44)) break;   // P_j written
        tc_fence_after();
        const uint32_t sv = base + S::kV + s * S::kTile;
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk)
          tc_mma_bf16(tmem_o, make_desc(base + S::kP + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                      make_desc(sv + kk * 2048, 16384, 1024), idesc_o, (j | kk) ? 1u : 0u);
        tc_commit(bar(3 + s));   // K_j / V_j stage free
        tc_commit(bar(10));      // P buffer free
      }
      tc_commit(bar(11));
    }
  } else {
    const int cw = warp - 2;              // 0..15
    const int quarter = warp & 3;         // tensor-memory lane quarter this warp may read
    const int cb = cw >> 2;               // which 32 key columns of the tile this warp handles
    const int r = quarter * 32 + lane;
    const int qi = q0 + r;
    const bool row_ok = qi < L;
    const int n_tiles_seq = (L + BQ - 1) / BQ;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    bool ok = true;
    float out_scale = SILU ? p.inv_n : 1.f;
    if constexpr (DECAY) {
      // P = S * 2^(cum[l] - cum[s]) below and on the diagonal, 0 above it and for rows past the sequence end
      const float* cum_h = p.cum + static_cast<size_t>(h) * p.cum_pitch + seq_start;
      const float cl = cum_h[qi];
      for (int j = 0; j < n_kv && ok; ++j) {
        const int sb = j & 1;
        float cs[32];
        load_cum32(cum_h + j * BKV + cb * 32, cs);
        if (!warp_wait(bar(5 + sb), (j >> 1) & 1, abortp, p.status, 45, lane)) { ok = false; break; }
        tc_fence_after();
        if (j > 0 && !warp_wait(bar(10), (j - 1) & 1, abortp, p.status, 46, lane)) { ok = false; break; }
        {
          uint32_t v[32];
          tmem_ld32(tmem_slot + sb * 128 + lane_off + cb * 32, v);
          uint8_t* row_ptr = base_ptr + S::kP + (cb >> 1) * 16384 + r * 128;
          const int kj0 = j * BKV + cb * 32;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t packed[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              float pr[2];
#pragma unroll
              for (int u = 0; u < 2; ++u) {
                const int col = g * 8 + 2 * k + u;
                const bool visible = row_ok && kj0 + col <= qi;
                pr[u] = visible ? __uint_as_float(v[col]) * exp2_fast(cl - cs[col]) : 0.f;
              }
              packed[k] = pack_bf16(pr[0], pr[1]);
            }
            const int chunk = ((cb & 1) * 4 + g) ^ (r & 7);
            *reinterpret_cast<uint4*>(row_ptr + chunk * 16) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          }
        }
        tc_fence_before();
        mbar_arrive(bar(7 + sb));
        fence_async_smem();
        mbar_arrive(bar(9));
      }
    } else if constexpr (SOFTMAX) {
      // Streaming softmax.  The four warps that share a row (one per 32-column block of the score tile) agree on
      // the tile's row maximum through shared memory, then each keeps the running sum of its own columns; when
      // the maximum grows the accumulated output is rescaled in tensor memory (it is idle between P_{j-1}·V and
      // P_j·V).  exp is evaluated as 2^(x log2 e - m).
      const float sc2 = p.scale * 1.4426950408889634f;
      uint32_t sm_drop_row = 0, sm_drop_hi = 0;
      if constexpr (DROP) {
        const unsigned long long key = *p.dropout_key;
        sm_drop_row = dropout_row_hash(key, h, tok0 + r);
        sm_drop_hi = static_cast<uint32_t>(key >> 32);
      }
      float m = -INFINITY, l = 0.f;
      float* mx = softmax_xchg + quarter * 32 + lane;      // [parity][cb][row]: + parity * 512 + cb * 128
      const uint32_t xbar = bar(12 + quarter);
      int xphase = 0;
      for (int j = 0; j < n_kv && ok; ++j) {
        const int sb = j & 1;
        if (!warp_wait(bar(5 + sb), (j >> 1) & 1, abortp, p.status, 45, lane)) { ok = false; break; }
        tc_fence_after();
        uint32_t v[32];
        tmem_ld32(tmem_slot + sb * 128 + lane_off + cb * 32, v);
        tc_fence_before();
        mbar_arrive(bar(7 + sb));           // the scores are in registers: this S buffer may be overwritten
        const int kj0 = j * BKV + cb * 32;
        float tmax = -INFINITY;
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const int kj = kj0 + e;
          const bool visible = row_ok && kj < L && (!p.causal || kj <= qi);
          const float x = visible ? __uint_as_float(v[e]) * sc2 : -INFINITY;
          v[e] = __float_as_uint(x);
          tmax = fmaxf(tmax, x);
        }
        mx[sb * 512 + cb * 128] = tmax;
        mbar_arrive(xbar);
        if (!warp_wait(xbar, xphase, abortp, p.status, 48, lane)) { ok = false; break; }
        xphase ^= 1;
        const float* mrow = softmax_xchg + sb * 512 + quarter * 32 + lane;
        const float m_new = fmaxf(fmaxf(m, fmaxf(mrow[0], mrow[128])), fmaxf(mrow[256], mrow[384]));
        const float alpha = m == -INFINITY ? (m_new == -INFINITY ? 1.f : 0.f) : exp2_fast(m - m_new);
        m = m_new;
        float psum = 0.f;
        uint32_t packed[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const float x0 = __uint_as_float(v[e]), x1 = __uint_as_float(v[e + 1]);
          float p0 = x0 == -INFINITY ? 0.f : exp2_fast(x0 - m_new);
          float p1 = x1 == -INFINITY ? 0.f : exp2_fast(x1 - m_new);
          psum += p0 + p1;
          if constexpr (DROP) {      // dropout acts on the normalised weights: the row sum keeps all of them
            const int kt = seq_start + kj0 + e;
            p0 = dropout_keep(sm_drop_row, sm_drop_hi, kt, p.drop_threshold) ? p0 * p.keep_scale : 0.f;
            p1 = dropout_keep(sm_drop_row, sm_drop_hi, kt + 1, p.drop_threshold) ? p1 * p.keep_scale : 0.f;
          }
          packed[e >> 1] = pack_bf16(p0, p1);
        }
        l = fmaf(l, alpha, psum);
        if (j > 0) {
          if (!warp_wait(bar(10), (j - 1) & 1, abortp, p.status, 46, lane)) { ok = false; break; }   // P_{j-1}·V done
          if (__any_sync(0xffffffffu, alpha != 1.f)) {
            tc_fence_after();
#pragma unroll 1
            for (int c = cb; c < DH / 32; c += 4) {
              uint32_t o[32];
              tmem_ld32(tmem_o + lane_off + c * 32, o);
#pragma unroll
              for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
              tmem_st32(tmem_o + lane_off + c * 32, o);
            }
          }
        }
        uint8_t* row_ptr = base_ptr + S::kP + (cb >> 1) * 16384 + r * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int chunk = ((cb & 1) * 4 + g) ^ (r & 7);
          *reinterpret_cast<uint4*>(row_ptr + chunk * 16) =
              make_uint4(packed[4 * g], packed[4 * g + 1], packed[4 * g + 2], packed[4 * g + 3]);
        }
        tc_fence_before();
        fence_async_smem();
        mbar_arrive(bar(9));
      }
      // the row sum is the sum of the four column blocks' partial sums (all scaled to the final maximum)
      if (ok) {
        // (the buffer half that tile n_kv would use: nobody can still be reading it)
        mx[(n_kv & 1) * 512 + cb * 128] = l;
        mbar_arrive(xbar);
        if (!warp_wait(xbar, xphase, abortp, p.status, 49, lane)) ok = false;
        if (ok) {
          const float* lrow = softmax_xchg + (n_kv & 1) * 512 + quarter * 32 + lane;
          l = (lrow[0] + lrow[128]) + (lrow[256] + lrow[384]);
        }
      }
      out_scale = l > 0.f ? 1.f / l : 0.f;
      if (ok && cb == 0 && row_ok && p.lse != nullptr)
        p.lse[static_cast<size_t>(tok0 + r) * p.H + h] = l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : 0.f;
    } else {
      // SiLU mode.  With h = (s * scale + bias) / 2:  silu(2h) = 2h * sigmoid(2h) = h * tanh(h) + h.  The
      // pair's bias tile brings bias / 2 (and the masks); 1 / n is applied once, to the output.
      const float hs = 0.5f * p.scale;
      uint32_t drop_row = 0, drop_hi = 0;
      if constexpr (DROP) {
        const unsigned long long key = *p.dropout_key;
        drop_row = dropout_row_hash(key, h, tok0 + r);
        drop_hi = static_cast<uint32_t>(key >> 32);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int sb = j & 1;
        const uint4* bt = reinterpret_cast<const uint4*>(
            p.bias_tiles + (static_cast<size_t>(pair_index(p, seq, n_tiles_seq, q0 / BQ, j)) << 14)) +
            (cb * 4 + quarter) * 4 * 32 + lane;
        uint4 hb[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) hb[g] = __ldg(bt + g * 32);
        if (!warp_wait(bar(5 + sb), (j >> 1) & 1, abortp, p.status, 45, lane)) { ok = false; break; }
        tc_fence_after();
        if (j > 0 && !warp_wait(bar(10), (j - 1) & 1, abortp, p.status, 46, lane)) { ok = false; break; }
        {
          uint32_t v[32];
          tmem_ld32(tmem_slot + sb * 128 + lane_off + cb * 32, v);
          uint8_t* row_ptr = base_ptr + S::kP + (cb >> 1) * 16384 + r * 128;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const uint32_t w[4] = {hb[g].x, hb[g].y, hb[g].z, hb[g].w};
            uint32_t packed[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float h0 = fmaf(__uint_as_float(v[g * 8 + 2 * k]), hs, bf16_lo(w[k]));
              const float h1 = fmaf(__uint_as_float(v[g * 8 + 2 * k + 1]), hs, bf16_hi(w[k]));
              float p0 = fmaf(h0, tanh_fast(h0), h0), p1 = fmaf(h1, tanh_fast(h1), h1);
              if constexpr (DROP) {
                const int kt = seq_start + j * BKV + cb * 32 + g * 8 + 2 * k;
                p0 = dropout_keep(drop_row, drop_hi, kt, p.drop_threshold) ? p0 * p.keep_scale : 0.f;
                p1 = dropout_keep(drop_row, drop_hi, kt + 1, p.drop_threshold) ? p1 * p.keep_scale : 0.f;
              }
              packed[k] = pack_bf16(p0, p1);
            }
            // 32 columns = 64 bytes = four 16-byte chunks of row r in 64-column sub-tile cb / 2
            const int chunk = ((cb & 1) * 4 + g) ^ (r & 7);
            *reinterpret_cast<uint4*>(row_ptr + chunk * 16) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          }
        }
        tc_fence_before();
        mbar_arrive(bar(7 + sb));   // this S buffer may be overwritten
        fence_async_smem();
        mbar_arrive(bar(9));        // P is in shared memory
      }
    }
    if (ok && warp_wait(bar(11), 0, abortp, p.status, 47, lane)) {
      tc_fence_after();
#pragma unroll 1
      for (int c = cb; c < DH / 32; c += 4) {
        uint32_t v[32];
        tmem_ld32(tmem_o + lane_off + c * 32, v);
        if (row_ok) {
          __nv_bfloat16* dst = p.out + static_cast<size_t>(tok0 + r) * p.H * DH + h * DH + c * 32;
#pragma unroll
          for (int g = 0; g < 4; ++g)
            *reinterpret_cast<uint4*>(dst + g * 8) =
                make_uint4(pack_bf16(__uint_as_float(v[8 * g]) * out_scale, __uint_as_float(v[8 * g + 1]) * out_scale),
                           pack_bf16(__uint_as_float(v[8 * g + 2]) * out_scale, __uint_as_float(v[8 * g + 3]) * out_scale),
                           pack_bf16(__uint_as_float(v[8 * g + 4]) * out_scale, __uint_as_float(v[8 * g + 5]) * out_scale),
                           pack_bf16(__uint_as_float(v[8 * g + 6]) * out_scale, __uint_as_float(v[8 * g + 7]) * out_scale));
        }
      }
    }
  }
  if (*abortp) {
    for (int i = 0; i < 64; ++i) __nanosleep(100000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_slot, S::kTmemCols);
  }
}

// =============================================== backward ===============================================
template <int DH>
struct SmemB {
  static constexpr int kSub = DH / 64;
  static constexpr int kTile = BQ * 64 * 2 * kSub;
  static constexpr int kStages = DH == 64 ? 2 : 1;      // Q_i / dO_i ring
  static constexpr int kK = 0;
  static constexpr int kV = kTile;
  static constexpr int kQ = 2 * kTile;
  static constexpr int kDO = kQ + kStages * kTile;
  static constexpr int kP = kDO + kStages * kTile;      // [128 q, 128 kv] bf16
  static constexpr int kDS = kP + BQ * BKV * 2;
  static constexpr int kBars = kDS + BQ * BKV * 2;
  static constexpr int kTotal = kBars + 128 + 1024;
  // tensor memory columns: [0,128) S then dQ, [128,256) dP, [256,256+DH) dV, [256+DH,256+2DH) dK
  static constexpr int kTmemCols = 512;
};

template <int DH, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
hstu_bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                const Params p) {
  constexpr bool SOFTMAX = MODE == kSoftmax || MODE == kSoftmaxDropout, SILU = MODE == kSilu || MODE == kSiluDropout;
  constexpr bool DECAY = MODE == kDecay, DROP = MODE == kSiluDropout || MODE == kSoftmaxDropout;
  using S = SmemB<DH>;
  const int lin = blockIdx.x + gridDim.x * blockIdx.y;   // heads fastest: dispatch order = work-sorted list order
  const int tile_id = lin / p.H;
  const int seq = p.tile_seq[tile_id];
  if (seq < 0) return;
  if (SILU && p.pair_base[seq + 1] > p.cap_pairs) {
    if (threadIdx.x == 0) report(p.status, kCapacity, 4);
    return;
  }
  const int h = lin % p.H;
  const int kv0 = p.tile_row0[tile_id];
  const int seq_start = p.seq_offsets[seq];
  const int L = p.seq_offsets[seq + 1] - seq_start;
  const int n_q_total = (L + BQ - 1) / BQ;
  const int i_first = p.causal ? kv0 / BQ : 0;
  const int n_it = n_q_total - i_first;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + S::kBars;
  // 0 kv_full, 1-2 qdo_full, 3-4 qdo_empty, 5 sp_full, 6 pds_full, 7 dq_full, 8 dq_empty, 9 final
  auto bar = [&](int i) { return bars + 8u * i; };
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(bar(0), 1);
    mbar_init(bar(1), 1); mbar_init(bar(2), 1);
    mbar_init(bar(3), 1); mbar_init(bar(4), 1);
    mbar_init(bar(5), 1);
    mbar_init(bar(6), kCompute);
    mbar_init(bar(7), 1);
    mbar_init(bar(8), kCompute);
    mbar_init(bar(9), 1);
    mbar_init(bar(10), kCompute);      // S / dP are in registers: their tensor-memory columns may be overwritten
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_slot), S::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // With head dim 64 there is room for dQ in columns of its own (448 of 512 in use) and for two Q / dO stages:
  // the score products of the NEXT query tile are then issued while the element-wise warps still work on this
  // one.  With head dim 128 dQ shares the columns of S and the steps run one after the other.
  constexpr bool kAhead = DH == 64;
  const uint32_t tmem_s = tmem_slot, tmem_dp = tmem_slot + 128, tmem_dv = tmem_slot + 256,
                 tmem_dk = tmem_slot + 256 + DH, tmem_dq = kAhead ? tmem_slot + 256 + 2 * DH : tmem_slot;
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar(0), 2 * S::kTile);
      const int hq = p.qk_shared ? 0 : h * DH;
      for (int d = 0; d < S::kSub; ++d) {
        tma_load_2d(base + S::kK + d * 16384, &map_k, hq + 64 * d, seq_start + kv0, bar(0));
        tma_load_2d(base + S::kV + d * 16384, &map_v, h * DH + 64 * d, seq_start + kv0, bar(0));
      }
      for (int it = 0; it < n_it; ++it) {
        const int st = it % S::kStages;
        if (!mbar_wait(bar(3 + st), ((it / S::kStages) & 1) ^ 1, abortp, p.status, 50)) break;
        mbar_expect_tx(bar(1 + st), 2 * S::kTile);
        const int row = seq_start + (i_first + it) * BQ;
        for (int d = 0; d < S::kSub; ++d) {
          tma_load_2d(base + S::kQ + st * S::kTile + d * 16384, &map_q, hq + 64 * d, row, bar(1 + st));
          tma_load_2d(base + S::kDO + st * S::kTile + d * 16384, &map_do, h * DH + 64 * d, row, bar(1 + st));
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = idesc_bf16(BQ, BKV, false, false);     // S = Q·K^T, dP = dO·V^T
      const uint32_t idesc_t = idesc_bf16(BKV, DH, true, true);       // dV = P^T·dO, dK = dS^T·Q
      const uint32_t idesc_q = idesc_bf16(BQ, DH, false, true);       // dQ = dS·K
      bool ok = mbar_wait(bar(0), 0, abortp, p.status, 51);
      // S = Q_i K^T and dP = dO_i V^T of query tile `it` (its Q / dO stage must have landed)
      auto issue_scores = [&](int it) -> bool {
        const int st = it % S::kStages;
        if (!mbar_wait(bar(1 + st), (it / S::kStages) & 1, abortp, p.status, 52)) return false;
        tc_fence_after();
        const uint32_t sq = base + S::kQ + st * S::kTile, sdo = base + S::kDO + st * S::kTile;
#pragma unroll
        for (int d = 0; d < S::kSub; ++d)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            tc_mma_bf16(tmem_s, make_desc(sq + d * 16384 + k * 32, 16, 1024),
                        make_desc(base + S::kK + d * 16384 + k * 32, 16, 1024), idesc_s, (d | k) ? 1u : 0u);
            tc_mma_bf16(tmem_dp, make_desc(sdo + d * 16384 + k * 32, 16, 1024),
                        make_desc(base + S::kV + d * 16384 + k * 32, 16, 1024), idesc_s, (d | k) ? 1u : 0u);
          }
        tc_commit(bar(5));
        return true;
      };
      if (kAhead && ok && n_it > 0) ok = issue_scores(0);
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it % S::kStages;
        if constexpr (kAhead) {
          // the next tile's scores as soon as this tile's are in the element-wise warps' registers
          if (it + 1 < n_it) {
            if (!mbar_wait(bar(10), it & 1, abortp, p.status, 58)) break;
            if (!issue_scores(it + 1)) break;
          }
        } else {
          if (it > 0 && !mbar_wait(bar(8), (it - 1) & 1, abortp, p.status, 53)) break;   // dQ of tile it-1 read out
          if (!issue_scores(it)) break;
        }
        const uint32_t sq = base + S::kQ + st * S::kTile, sdo = base + S::kDO + st * S::kTile;
        if (!mbar_wait(bar(6), it & 1, abortp, p.status, 54)) break;   // P and dS are in shared memory
        if (kAhead && it > 0 && !mbar_wait(bar(8), (it - 1) & 1, abortp, p.status, 53)) break;   // dQ of tile it-1 read out
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BQ / 16; ++kk) {   // contraction over the 128 query rows
          tc_mma_bf16(tmem_dv, make_desc(base + S::kP + kk * 2048, 16384, 1024), make_desc(sdo + kk * 2048, 16384, 1024),
                      idesc_t, (it | kk) ? 1u : 0u);
          tc_mma_bf16(tmem_dk, make_desc(base + S::kDS + kk * 2048, 16384, 1024), make_desc(sq + kk * 2048, 16384, 1024),
                      idesc_t, (it | kk) ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk)    // contraction over the 128 keys
          tc_mma_bf16(tmem_dq, make_desc(base + S::kDS + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                      make_desc(base + S::kK + kk * 2048, 16384, 1024), idesc_q, kk ? 1u : 0u);
        tc_commit(bar(7));           // dQ ready; P / dS / this Q,dO stage no longer read
        tc_commit(bar(3 + st));
      }
      tc_commit(bar(9));
    }
  } else {
    const int cw = warp - 2;
    const int quarter = warp & 3;
    const int cb = cw >> 2;               // which 32 key columns of the tile this warp handles
    const int r = quarter * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const float hs = 0.5f * p.scale;
    // what multiplies the accumulated dQ: the score scale, and in SiLU mode the 1 / n that P and dS leave out
    const float dq_scale = SILU ? p.scale * p.inv_n : p.scale;
    bool ok = true;
    const float* cum_h = nullptr;
    float cs[32];
    if constexpr (DECAY) {
      cum_h = p.cum + static_cast<size_t>(h) * p.cum_pitch + seq_start;
      load_cum32(cum_h + kv0 + cb * 32, cs);     // this CTA's keys stay the same for all query tiles
    }
    for (int it = 0; it < n_it && ok; ++it) {
      const int q0 = (i_first + it) * BQ;
      const int qi = q0 + r;
      const bool row_ok = qi < L;
      float lse_r = 0.f, delta_r = 0.f;
      uint4 hb[4];
      size_t pair_off = 0;
      float cl = 0.f;
      uint32_t drop_row = 0, drop_hi = 0;
      if constexpr (DROP) {
        const unsigned long long key = *p.dropout_key;
        drop_row = dropout_row_hash(key, h, seq_start + qi);
        drop_hi = static_cast<uint32_t>(key >> 32);
      }
      if constexpr (DECAY) {
        cl = cum_h[qi];
      } else if constexpr (SOFTMAX) {
        if (row_ok) {
          lse_r = p.lse[static_cast<size_t>(seq_start + qi) * p.H + h];
          delta_r = p.delta[static_cast<size_t>(seq_start + qi) * p.H + h];
        }
      } else {
        pair_off = static_cast<size_t>(pair_index(p, seq, n_q_total, i_first + it, kv0 / BKV)) << 14;
        const uint4* bt = reinterpret_cast<const uint4*>(p.bias_tiles + pair_off) + (cb * 4 + quarter) * 4 * 32 + lane;
#pragma unroll
        for (int g = 0; g < 4; ++g) hb[g] = __ldg(bt + g * 32);
      }
      if (!warp_wait(bar(5), it & 1, abortp, p.status, 55, lane)) { ok = false; break; }
      tc_fence_after();
      {
        uint32_t sv[32], dpv[32];
        float row_acc = 0.f;
        tmem_ld32(tmem_s + lane_off + cb * 32, sv);
        tmem_ld32(tmem_dp + lane_off + cb * 32, dpv);
        if constexpr (kAhead) {
          tc_fence_before();
          mbar_arrive(bar(10));
        }
        uint8_t* prow = base_ptr + S::kP + (cb >> 1) * 16384 + r * 128;
        uint8_t* drow = base_ptr + S::kDS + (cb >> 1) * 16384 + r * 128;
        float4* dbias = nullptr;
        if constexpr (SILU) {
          if (p.dbias_tiles != nullptr)
            dbias = reinterpret_cast<float4*>(p.dbias_tiles + pair_off) + (cb * 4 + quarter) * 8 * 32 + lane;
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint32_t pp[4], dd[4];
          float dsv[8];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            float pr[2], dr[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int col = g * 8 + 2 * k + u;       // within the warp's 32 columns
              const float s_raw = __uint_as_float(sv[col]), dp = __uint_as_float(dpv[col]);
              if constexpr (DECAY) {
                // P = S * D, dS = dP * D with D = 2^(cum[l] - cum[s]) on and below the diagonal
                const bool visible = row_ok && kv0 + cb * 32 + col <= qi;
                const float dec = visible ? exp2_fast(cl - cs[col]) : 0.f;
                pr[u] = s_raw * dec;
                dr[u] = dp * dec;
              } else if constexpr (SOFTMAX) {
                const int kj = kv0 + cb * 32 + col;
                const bool visible = row_ok && kj < L && (!p.causal || kj <= qi);
                // P = exp(x - lse);  dS = P * (dP - delta)
                const float pv = visible ? __expf(s_raw * p.scale - lse_r) : 0.f;
                float keep = 1.f;
                if constexpr (DROP)
                  keep = dropout_keep(drop_row, drop_hi, seq_start + kj, p.drop_threshold) ? p.keep_scale : 0.f;
                // O = sum_j P_j M_j V_j with the dropout mask M:  dV uses P M, dS = P (dP M - delta)
                pr[u] = pv * keep;
                dr[u] = visible ? pv * (dp * keep - delta_r) : 0.f;
              } else {
                // h = x / 2;  P = x sigmoid(x) = h tanh(h) + h;  dP/dx = sig + P (1 - sig), sig = (tanh(h) + 1) / 2
                const uint32_t w = k == 0 ? hb[g].x : k == 1 ? hb[g].y : k == 2 ? hb[g].z : hb[g].w;
                const float hv = fmaf(s_raw, hs, u == 0 ? bf16_lo(w) : bf16_hi(w));
                const float t = tanh_fast(hv);
                const float pv = fmaf(hv, t, hv);
                const float sig = fmaf(0.5f, t, 0.5f);
                float keep = 1.f;
                if constexpr (DROP)
                  keep = dropout_keep(drop_row, drop_hi, seq_start + kv0 + cb * 32 + col, p.drop_threshold) ? p.keep_scale : 0.f;
                pr[u] = pv * keep;
                dr[u] = dp * keep * fmaf(pv, 1.f - sig, sig);
              }
              dsv[2 * k + u] = dr[u];
            }
            pp[k] = pack_bf16(pr[0], pr[1]);
            dd[k] = pack_bf16(dr[0], dr[1]);
            if constexpr (DECAY)
              row_acc = fmaf(__uint_as_float(dpv[g * 8 + 2 * k + 1]), bf16_hi(pp[k]),
                             fmaf(__uint_as_float(dpv[g * 8 + 2 * k]), bf16_lo(pp[k]), row_acc));
          }
          const int chunk = ((cb & 1) * 4 + g) ^ (r & 7);
          *reinterpret_cast<uint4*>(prow + chunk * 16) = make_uint4(pp[0], pp[1], pp[2], pp[3]);
          *reinterpret_cast<uint4*>(drow + chunk * 16) = make_uint4(dd[0], dd[1], dd[2], dd[3]);
          if constexpr (SILU) {
            if (dbias != nullptr) {
              // gradient of the bias: dS / n, summed over heads and layers in the pair's gradient block
              red_add_v4(dbias + (2 * g) * 32, dsv[0] * p.inv_n, dsv[1] * p.inv_n, dsv[2] * p.inv_n, dsv[3] * p.inv_n);
              red_add_v4(dbias + (2 * g + 1) * 32, dsv[4] * p.inv_n, dsv[5] * p.inv_n, dsv[6] * p.inv_n, dsv[7] * p.inv_n);
            }
          }
        }
        if constexpr (DECAY) {
          if (row_ok && p.dcum != nullptr) atomicAdd(p.dcum + static_cast<size_t>(h) * p.cum_pitch + seq_start + qi, row_acc);
        }
      }
      tc_fence_before();
      fence_async_smem();
      mbar_arrive(bar(6));
      // dQ tile: wait for the three products of this step, then add it into the fp32 gradient
      if (!warp_wait(bar(7), it & 1, abortp, p.status, 56, lane)) { ok = false; break; }
      tc_fence_after();
#pragma unroll 1
      for (int c = cb; c < DH / 32; c += 4) {
        uint32_t v[32];
        tmem_ld32(tmem_dq + lane_off + c * 32, v);
        if (row_ok) {
          float4* dst = reinterpret_cast<float4*>(
              p.qk_shared ? p.dq + static_cast<size_t>(seq_start + qi) * DH + c * 32
                          : p.dq + static_cast<size_t>(seq_start + qi) * p.H * DH + h * DH + c * 32);
#pragma unroll
          for (int g = 0; g < 8; ++g)
            red_add_v4(dst + g, __uint_as_float(v[4 * g]) * dq_scale, __uint_as_float(v[4 * g + 1]) * dq_scale,
                       __uint_as_float(v[4 * g + 2]) * dq_scale, __uint_as_float(v[4 * g + 3]) * dq_scale);
        }
      }
      tc_fence_before();
      mbar_arrive(bar(8));
    }
    if (ok && warp_wait(bar(9), 0, abortp, p.status, 57, lane)) {
      tc_fence_after();
      const int kj = kv0 + r;
      const bool kv_ok = kj < L;
      const float dv_scale = SILU ? p.inv_n : 1.f, dk_scale = dq_scale;
#pragma unroll 1
      for (int c = cb; c < DH / 32; c += 4) {
        uint32_t v[32], w[32];
        tmem_ld32(tmem_dv + lane_off + c * 32, v);
        tmem_ld32(tmem_dk + lane_off + c * 32, w);
        if (kv_ok) {
          const size_t off = static_cast<size_t>(seq_start + kj) * p.H * DH + h * DH + c * 32;
          if constexpr (DECAY) {
            if (p.dcum != nullptr) {
              const uint4* xr = reinterpret_cast<const uint4*>(
                  p.v_rows + static_cast<size_t>(seq_start + kj) * (p.ld_v > 0 ? p.ld_v : p.H * DH) + h * DH + c * 32);
              float dot = 0.f;
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                const uint4 xv = __ldg(xr + g);
                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (int k = 0; k < 4; ++k)
                  dot = fmaf(__uint_as_float(v[8 * g + 2 * k + 1]), bf16_hi(xw[k]),
                             fmaf(__uint_as_float(v[8 * g + 2 * k]), bf16_lo(xw[k]), dot));
              }
              atomicAdd(p.dcum + static_cast<size_t>(h) * p.cum_pitch + seq_start + kj, -dot);
            }
          }
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            *reinterpret_cast<uint4*>(p.dv + off + g * 8) =
                make_uint4(pack_bf16(__uint_as_float(v[8 * g]) * dv_scale, __uint_as_float(v[8 * g + 1]) * dv_scale),
                           pack_bf16(__uint_as_float(v[8 * g + 2]) * dv_scale, __uint_as_float(v[8 * g + 3]) * dv_scale),
                           pack_bf16(__uint_as_float(v[8 * g + 4]) * dv_scale, __uint_as_float(v[8 * g + 5]) * dv_scale),
                           pack_bf16(__uint_as_float(v[8 * g + 6]) * dv_scale, __uint_as_float(v[8 * g + 7]) * dv_scale));
            if constexpr (!DECAY)
              *reinterpret_cast<uint4*>(p.dk + off + g * 8) =
                  make_uint4(pack_bf16(__uint_as_float(w[8 * g]) * dk_scale, __uint_as_float(w[8 * g + 1]) * dk_scale),
                             pack_bf16(__uint_as_float(w[8 * g + 2]) * dk_scale, __uint_as_float(w[8 * g + 3]) * dk_scale),
                             pack_bf16(__uint_as_float(w[8 * g + 4]) * dk_scale, __uint_as_float(w[8 * g + 5]) * dk_scale),
                             pack_bf16(__uint_as_float(w[8 * g + 6]) * dk_scale, __uint_as_float(w[8 * g + 7]) * dk_scale));
          }
          if constexpr (DECAY) {
            // the key operand is shared by all heads: their gradients meet in one fp32 row
            float4* dst = reinterpret_cast<float4*>(p.dk_acc + static_cast<size_t>(seq_start + kj) * DH + c * 32);
#pragma unroll
            for (int g = 0; g < 8; ++g)
              red_add_v4(dst + g, __uint_as_float(w[4 * g]) * dk_scale, __uint_as_float(w[4 * g + 1]) * dk_scale,
                         __uint_as_float(w[4 * g + 2]) * dk_scale, __uint_as_float(w[4 * g + 3]) * dk_scale);
          }
        }
      }
    }
  }
  if (*abortp) {
    for (int i = 0; i < 64; ++i) __nanosleep(100000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_slot, S::kTmemCols);
  }
}

}  // namespace hstu
}  // namespace recml

using namespace recml::hstu;

extern "C" int recml_hstu_struct_size() { return static_cast<int>(sizeof(Params)); }

extern "C" int recml_hstu_tile_list(const int* seq_offsets, int B, int* tile_seq, int* tile_row0, int cap, int backward,
                                    cudaStream_t stream) {
  cudaMemsetAsync(tile_seq, 0xFF, sizeof(int) * cap, stream);
  tile_list_kernel<<<1, 32, 0, stream>>>(seq_offsets, B, tile_seq, tile_row0, cap, backward);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// Fills pair_base [B + 1] and the bucket blocks of every tile pair the kernels will visit.  `tile_seq` /
// `tile_row0` are the forward tile list (capacity n_tiles); cap_pairs bounds the blocks `cache` can hold.
extern "C" int recml_hstu_bucket_cache(const int* seq_offsets, int B, const int* tile_seq, const int* tile_row0, int n_tiles,
                                       const int* timestamps, int num_buckets, int causal, int max_tiles_per_seq,
                                       int* pair_base, unsigned char* cache, int cap_pairs, cudaStream_t stream) {
  if (B <= 0 || n_tiles <= 0 || max_tiles_per_seq <= 0) return 0;
  if (num_buckets + 1 > 256) return -11;
  pair_base_kernel<<<1, 32, 0, stream>>>(seq_offsets, B, causal, pair_base);
  dim3 grid(n_tiles, max_tiles_per_seq);
  bucket_cache_kernel<<<grid, 256, 0, stream>>>(seq_offsets, tile_seq, tile_row0, timestamps, pair_base, num_buckets, causal,
                                                cap_pairs, cache);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

template <int DH, int MODE>
static int launch_fwd(const void* q, const void* k, const void* v, const Params& p, int n_tiles, cudaStream_t stream) {
  CUtensorMap mq, mk, mv;
  const long long cols = static_cast<long long>(p.H) * DH;
  const long long qk_cols = p.qk_shared ? DH : cols;
  auto pitch = [&](int ld) { return ld > 0 ? static_cast<long long>(ld) : cols; };
  auto qk_pitch = [&](int ld) { return ld > 0 ? static_cast<long long>(ld) : qk_cols; };
  if (recml::tc::make_map_bf16(&mq, q, p.T, qk_cols, qk_pitch(p.ld_q), BQ) || recml::tc::make_map_bf16(&mk, k, p.T, qk_cols, qk_pitch(p.ld_k), BKV) ||
      recml::tc::make_map_bf16(&mv, v, p.T, cols, pitch(p.ld_v), BKV))
    return -2;
  auto kern = hstu_fwd_kernel<DH, MODE>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<DH>::kTotal) != cudaSuccess) return -3;
    configured = true;
  }
  dim3 grid(n_tiles, p.H);
  kern<<<grid, kThreads, Smem<DH>::kTotal, stream>>>(mq, mk, mv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// q, k, v: [T, H, Dh] bf16 contiguous.  n_tiles: capacity of the tile list (>= number of real tiles).
extern "C" int recml_hstu_attn_fwd(const void* q, const void* k, const void* v, const Params* p, int n_tiles,
                                   cudaStream_t stream) {
  if (p->T <= 0 || n_tiles <= 0) return 0;
  if ((p->mode == kSilu || p->mode == kSiluDropout) && (p->bias_tiles == nullptr || p->pair_base == nullptr)) return -12;
  if ((p->mode == kSiluDropout || p->mode == kSoftmaxDropout) && p->dropout_key == nullptr) return -14;
  if (p->mode == kDecay && (p->cum == nullptr || !p->causal || !p->qk_shared || p->cum_pitch < p->T + BKV)) return -13;
  if (p->mode != kDecay && p->qk_shared) return -13;
#define RECML_ATTN_FWD(D)                                                                  \
  switch (p->mode) {                                                                       \
    case kSilu: return launch_fwd<D, kSilu>(q, k, v, *p, n_tiles, stream);                 \
    case kSoftmax: return launch_fwd<D, kSoftmax>(q, k, v, *p, n_tiles, stream);           \
    case kDecay: return launch_fwd<D, kDecay>(q, k, v, *p, n_tiles, stream);               \
    case kSiluDropout: return launch_fwd<D, kSiluDropout>(q, k, v, *p, n_tiles, stream);   \
    case kSoftmaxDropout: return launch_fwd<D, kSoftmaxDropout>(q, k, v, *p, n_tiles, stream); \
    default: return -10;                                                                   \
  }
  if (p->Dh == 64) RECML_ATTN_FWD(64)
  if (p->Dh == 128) RECML_ATTN_FWD(128)
#undef RECML_ATTN_FWD
  return -10;
}

template <int DH, int MODE>
static int launch_bwd(const void* q, const void* k, const void* v, const void* d_o, const Params& p, int n_tiles,
                      cudaStream_t stream) {
  CUtensorMap mq, mk, mv, mdo;
  const long long cols = static_cast<long long>(p.H) * DH;
  const long long qk_cols = p.qk_shared ? DH : cols;
  auto pitch = [&](int ld) { return ld > 0 ? static_cast<long long>(ld) : cols; };
  auto qk_pitch = [&](int ld) { return ld > 0 ? static_cast<long long>(ld) : qk_cols; };
  if (recml::tc::make_map_bf16(&mq, q, p.T, qk_cols, qk_pitch(p.ld_q), BQ) || recml::tc::make_map_bf16(&mk, k, p.T, qk_cols, qk_pitch(p.ld_k), BKV) ||
      recml::tc::make_map_bf16(&mv, v, p.T, cols, pitch(p.ld_v), BKV) || recml::tc::make_map_bf16(&mdo, d_o, p.T, cols, pitch(p.ld_do), BQ))
    return -2;
  auto kern = hstu_bwd_kernel<DH, MODE>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemB<DH>::kTotal) != cudaSuccess) return -3;
    configured = true;
  }
  dim3 grid(n_tiles, p.H);
  kern<<<grid, kThreads, SmemB<DH>::kTotal, stream>>>(mq, mk, mv, mdo, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// dq (fp32), dpos_w, dts_w must be zero on entry; dk / dv are fully written for every token.
// Rows whose key tile contains no query that sees them still get written (with zeros) because every
// key tile of every sequence has a CTA.
extern "C" int recml_hstu_attn_bwd(const void* q, const void* k, const void* v, const void* d_o, const Params* p,
                                   int n_tiles, cudaStream_t stream) {
  if (p->T <= 0 || n_tiles <= 0) return 0;
  if (p->num_buckets + 1 > 256) return -11;
  if ((p->mode == kSilu || p->mode == kSiluDropout) && (p->bias_tiles == nullptr || p->pair_base == nullptr)) return -12;
  if ((p->mode == kSiluDropout || p->mode == kSoftmaxDropout) && p->dropout_key == nullptr) return -14;
  if (p->mode == kDecay && (p->cum == nullptr || !p->causal || !p->qk_shared || p->dk_acc == nullptr || p->cum_pitch < p->T + BKV))
    return -13;
  if (p->mode != kDecay && p->qk_shared) return -13;
#define RECML_ATTN_BWD(D)                                                                  \
  switch (p->mode) {                                                                       \
    case kSilu: return launch_bwd<D, kSilu>(q, k, v, d_o, *p, n_tiles, stream);            \
    case kSoftmax: return launch_bwd<D, kSoftmax>(q, k, v, d_o, *p, n_tiles, stream);      \
    case kDecay: return launch_bwd<D, kDecay>(q, k, v, d_o, *p, n_tiles, stream);          \
    case kSiluDropout: return launch_bwd<D, kSiluDropout>(q, k, v, d_o, *p, n_tiles, stream); \
    case kSoftmaxDropout: return launch_bwd<D, kSoftmaxDropout>(q, k, v, d_o, *p, n_tiles, stream); \
    default: return -10;                                                                   \
  }
  if (p->Dh == 64) RECML_ATTN_BWD(64)
  if (p->Dh == 128) RECML_ATTN_BWD(128)
#undef RECML_ATTN_BWD
  return -10;
}

extern "C" int recml_hstu_bias_struct_size() { return static_cast<int>(sizeof(BiasParams)); }

// pair_base [B + 1] alone (when there is no time-bucket cache to build).
extern "C" int recml_hstu_pair_base(const int* seq_offsets, int B, int causal, int* pair_base, cudaStream_t stream) {
  pair_base_kernel<<<1, 32, 0, stream>>>(seq_offsets, B, causal, pair_base);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// Bias tiles of every tile pair the attention kernels will visit (forward tile list of capacity n_tiles).
extern "C" int recml_hstu_bias_tiles(const BiasParams* p, int n_tiles, int max_tiles_per_seq, cudaStream_t stream) {
  if (n_tiles <= 0 || max_tiles_per_seq <= 0) return 0;
  if (p->num_buckets + 1 > 256) return -11;
  dim3 grid(n_tiles, max_tiles_per_seq);
  bias_tile_kernel<<<grid, 256, 0, stream>>>(*p);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// dpos_w / dts_w (pre-zeroed, either may be null) from the gradient blocks, which are zeroed again.
extern "C" int recml_hstu_bias_grads(const BiasParams* p, int n_tiles, int max_tiles_per_seq, cudaStream_t stream) {
  if (n_tiles <= 0 || max_tiles_per_seq <= 0) return 0;
  dim3 grid(n_tiles, max_tiles_per_seq);
  bias_grad_kernel<<<grid, 512, 0, stream>>>(*p);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
