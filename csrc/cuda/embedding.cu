// Sharded-embedding kernels for sm_100a: the lookup / pooling forward that writes its result
// straight into the destination rank's buffer over NVLink (the all-to-all IS the store), the
// activation-gradient push, and the sort-based dedup + row-optimizer backward.
//
// Data flow per step on rank `me` of W ranks (B = per-rank batch):
//   ids      every rank pushes its jagged ids to all peers (emb_push_ids)             flag chan 0
//   forward  for every (feature it owns a part of, source rank s, sample b) rank `me` gathers the
//            rows it owns, pools them in fp32 and stores the bf16 vector into rank s's pooled
//            buffer with plain peer stores (emb_fwd); in training it also appends
//            (row, gradient-vector index) to an occurrence list                         flag chan 1
//   combine  rank s sums the per-source slots of row-sharded features and writes the dense
//            concat input (emb_combine)
//   backward rank s pushes each feature's activation gradient to the rank(s) owning that
//            feature (emb_push_grads)                                                   flag chan 2
//            owners radix-sort the occurrence list by row (radix_sort.cu; it only needs the forward's
//            output, so it runs beside the dense forward pass), reduce each run of equal rows in
//            fp32 and apply the row optimizer in the same kernel (emb_bwd_update/finalize).
// Peer flags are monotonically increasing sequence numbers; all waits are bounded.
#include <cstdio>
#include <cstdlib>

#include "common.cuh"

namespace recml {
namespace emb {

constexpr int kMaxWorld = 8;
enum Kind : int { kTableWise = 0, kRowWise = 1, kColumnWise = 2 };
enum Combiner : int { kSum = 0, kMean = 1, kSqrtN = 2 };
enum Opt : int { kSGD = 0, kAdagrad = 1, kRowAdagrad = 2, kAdam = 3, kRowAdam = 4, kAdagradMomentum = 5,
                 kFTRL = 6, kLaProp = 7 };

struct FeatDesc {      // one sharded feature as seen by the rank running the kernel
  int feat_index;      // position of the feature in the jagged batch (offset rows f*B .. f*B+B)
  int kind;
  int owner;           // table-wise: owning rank
  int rot;             // row-wise: shard rotation
  int row_base;        // first row of the table inside the stack buffer
  int combiner;
  int dim;             // full embedding dim D of the feature
  int col_lo;          // column-wise: first column held by this rank
  long long slot_off;  // element offset of the feature's block in a destination pooled buffer
  long long grad_off;  // element offset of the feature's block in THIS rank's gradient buffer
  int seq_len;         // >0: sequence feature (no pooling), positions beyond seq_len dropped
  int dst_stride;      // elements between consecutive samples of this feature in the destination
  int vocab;           // rows of the feature's table: ids outside [0, vocab) are reported and ignored
  int tile_shift;      // tiled forward: a warp takes 2^tile_shift consecutive bags of this feature (0..5)
  long long tile_start;  // tiled forward: work units of the features before this one in the launch
};

struct IdPtrs {        // jagged ids of every source rank, in this rank's memory
  const int* values[kMaxWorld];
  const int* offsets[kMaxWorld];
  const float* weights[kMaxWorld];
};
struct PeerBf16 { __nv_bfloat16* p[kMaxWorld]; };
struct PeerFlags { unsigned long long* p[kMaxWorld]; };

// ---- small vector helpers: each lane owns VPL consecutive elements -------------------------------
template <int VPL> struct Vec { float v[VPL]; };

template <int VPL>
__device__ __forceinline__ Vec<VPL> load_f32(const float* p) {
  Vec<VPL> r;
  if constexpr (VPL == 1) { r.v[0] = __ldg(p); }
  else if constexpr (VPL == 2) { float2 t = __ldg(reinterpret_cast<const float2*>(p)); r.v[0] = t.x; r.v[1] = t.y; }
  else {
#pragma unroll
    for (int i = 0; i < VPL / 4; ++i) {
      float4 t = __ldg(reinterpret_cast<const float4*>(p) + i);
      r.v[4 * i] = t.x; r.v[4 * i + 1] = t.y; r.v[4 * i + 2] = t.z; r.v[4 * i + 3] = t.w;
    }
  }
  return r;
}
template <int VPL>
__device__ __forceinline__ Vec<VPL> load_f32_rw(const float* p) {  // no read-only path (data is rewritten)
  Vec<VPL> r;
  if constexpr (VPL == 1) { r.v[0] = *p; }
  else if constexpr (VPL == 2) { float2 t = *reinterpret_cast<const float2*>(p); r.v[0] = t.x; r.v[1] = t.y; }
  else {
#pragma unroll
    for (int i = 0; i < VPL / 4; ++i) {
      float4 t = reinterpret_cast<const float4*>(p)[i];
      r.v[4 * i] = t.x; r.v[4 * i + 1] = t.y; r.v[4 * i + 2] = t.z; r.v[4 * i + 3] = t.w;
    }
  }
  return r;
}
template <int VPL>
__device__ __forceinline__ void store_f32(float* p, const Vec<VPL>& r) {
  if constexpr (VPL == 1) { *p = r.v[0]; }
  else if constexpr (VPL == 2) { *reinterpret_cast<float2*>(p) = make_float2(r.v[0], r.v[1]); }
  else {
#pragma unroll
    for (int i = 0; i < VPL / 4; ++i)
      reinterpret_cast<float4*>(p)[i] = make_float4(r.v[4 * i], r.v[4 * i + 1], r.v[4 * i + 2], r.v[4 * i + 3]);
  }
}
template <int VPL>
__device__ __forceinline__ Vec<VPL> load_bf16(const __nv_bfloat16* p) {
  Vec<VPL> r;
  if constexpr (VPL == 1) { r.v[0] = __bfloat162float(*p); }
  else if constexpr (VPL == 2) { uint32_t t = *reinterpret_cast<const uint32_t*>(p); r.v[0] = bf16_lo(t); r.v[1] = bf16_hi(t); }
  else if constexpr (VPL == 4) {
    uint2 t = *reinterpret_cast<const uint2*>(p);
    r.v[0] = bf16_lo(t.x); r.v[1] = bf16_hi(t.x); r.v[2] = bf16_lo(t.y); r.v[3] = bf16_hi(t.y);
  } else {
    uint4 t = *reinterpret_cast<const uint4*>(p);
    r.v[0] = bf16_lo(t.x); r.v[1] = bf16_hi(t.x); r.v[2] = bf16_lo(t.y); r.v[3] = bf16_hi(t.y);
    r.v[4] = bf16_lo(t.z); r.v[5] = bf16_hi(t.z); r.v[6] = bf16_lo(t.w); r.v[7] = bf16_hi(t.w);
  }
  return r;
}
// Raw (still packed) bf16 elements of one lane: kept packed while several loads are in flight, so a batch of
// loads costs half the registers of converted floats.
template <int VPL> struct RawBf16 { uint32_t w[(VPL + 1) / 2]; };
template <int VPL>
__device__ __forceinline__ RawBf16<VPL> load_raw_bf16(const __nv_bfloat16* p) {
  RawBf16<VPL> r;
  if constexpr (VPL == 1) { r.w[0] = *reinterpret_cast<const unsigned short*>(p); }
  else if constexpr (VPL == 2) { r.w[0] = *reinterpret_cast<const uint32_t*>(p); }
  else if constexpr (VPL == 4) { const uint2 t = *reinterpret_cast<const uint2*>(p); r.w[0] = t.x; r.w[1] = t.y; }
  else { const uint4 t = *reinterpret_cast<const uint4*>(p); r.w[0] = t.x; r.w[1] = t.y; r.w[2] = t.z; r.w[3] = t.w; }
  return r;
}
template <int VPL>
__device__ __forceinline__ void fma_raw_bf16(Vec<VPL>& acc, float gain, const RawBf16<VPL>& r) {
  if constexpr (VPL == 1) { acc.v[0] = fmaf(gain, bf16_lo(r.w[0]), acc.v[0]); }
  else {
#pragma unroll
    for (int i = 0; i < VPL / 2; ++i) {
      acc.v[2 * i] = fmaf(gain, bf16_lo(r.w[i]), acc.v[2 * i]);
      acc.v[2 * i + 1] = fmaf(gain, bf16_hi(r.w[i]), acc.v[2 * i + 1]);
    }
  }
}
template <int VPL>
__device__ __forceinline__ void store_bf16(__nv_bfloat16* p, const Vec<VPL>& r) {
  if constexpr (VPL == 1) { *p = __float2bfloat16(r.v[0]); }
  else if constexpr (VPL == 2) { *reinterpret_cast<uint32_t*>(p) = pack_bf16(r.v[0], r.v[1]); }
  else if constexpr (VPL == 4) {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(r.v[0], r.v[1]), pack_bf16(r.v[2], r.v[3]));
  } else {
    *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16(r.v[0], r.v[1]), pack_bf16(r.v[2], r.v[3]),
                                              pack_bf16(r.v[4], r.v[5]), pack_bf16(r.v[6], r.v[7]));
  }
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// Asks L2 for the 128-byte lines of [ptr, ptr + bytes): issued a window ahead of the loads that need them, so
// those loads pay the L2 latency instead of the DRAM one.
__device__ __forceinline__ void prefetch_l2(const void* ptr, int bytes) {
  const char* c = static_cast<const char*>(ptr);
  for (int o = 0; o < bytes; o += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(c + o));
}

// Raises flag[chan][me] = seq on every rank once ALL blocks of the grid have finished their stores.
__device__ __forceinline__ void grid_done_then_signal(unsigned int* done_counter, const PeerFlags& flags,
                                                      int W, unsigned long long seq) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *done_counter = 0;
      __threadfence_system();
      for (int r = 0; r < W; ++r)
        if (flags.p[r] != nullptr) st_release_sys(flags.p[r], seq);
    }
  }
}

// Every block waits until flags[src] >= seq for all sources (threads 0..W-1 poll one flag each).
// `flags` points at channel c0, source 0; channels are kMaxWorld flags apart; n_chan consecutive channels.
__device__ __forceinline__ bool wait_all_sources(const unsigned long long* flags, int W,
                                                 unsigned long long seq, int* status, int chan,
                                                 int n_chan = 1) {
  __shared__ int ok_shared;
  if (threadIdx.x == 0) ok_shared = 1;
  __syncthreads();
  if (threadIdx.x < W * n_chan) {
    const int c = threadIdx.x / W, src = threadIdx.x % W;
    if (!wait_flag_ge(flags + c * kMaxWorld + src, seq, kDefaultWaitNs, status, (chan + c) * 16 + src)) ok_shared = 0;
  }
  __syncthreads();
  return ok_shared != 0;
}

// =================================== ids: push to all peers =======================================
struct PushIdsParams {
  const int* values; const int* offsets; const float* weights;
  long long nnz; int n_offsets; int W; int me;
  int* dst_values[kMaxWorld]; int* dst_offsets[kMaxWorld]; float* dst_weights[kMaxWorld];
  unsigned int* done_counter; PeerFlags flags; SeqRef seq;
  const unsigned char* need;   // per feature: bit r set when rank r holds part of its table (null: all)
  int n_feats; int B;          // offsets[f*B] is the first id of feature f
};

// The offsets go to every rank; the ids of a feature only to the ranks that own rows of its table
// (one rank for a table-wise feature).  Each id is read once and stored to its destinations.
__global__ void emb_push_ids_kernel(const PushIdsParams p) {
  extern __shared__ int bounds[];   // n_feats + 1 feature boundaries in `values`
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = tid; i < p.n_offsets; i += stride) {
    const int o = p.offsets[i];
    for (int r = 0; r < p.W; ++r) p.dst_offsets[r][i] = o;
  }
  if (p.need != nullptr) {
    for (int f = threadIdx.x; f <= p.n_feats; f += blockDim.x) bounds[f] = p.offsets[static_cast<long long>(f) * p.B];
    __syncthreads();
  }
  for (long long i = tid; i < p.nnz; i += stride) {
    unsigned int mask = 0xffu;
    if (p.need != nullptr) {
      int lo = 0, hi = p.n_feats;     // bounds[lo] <= i < bounds[hi]
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (bounds[mid] <= i) lo = mid; else hi = mid;
      }
      mask = p.need[lo];
    }
    const int v = p.values[i];
    const float w = p.weights != nullptr ? p.weights[i] : 0.f;
    for (int r = 0; r < p.W; ++r) {
      if ((mask >> r) & 1u) {
        p.dst_values[r][i] = v;
        if (p.weights != nullptr) p.dst_weights[r][i] = w;
      }
    }
  }
  grid_done_then_signal(p.done_counter, p.flags, p.W, seq_of(p.seq));
}

// =================================== ids: bucketize by owner, then push =============================
// Every destination rank receives a jagged batch of its own: the offsets of all (feature, sample) bags, and only
// the ids it will look up: all ids of a feature whose table it holds whole (or by columns), the ids of ITS rows
// of a row-sharded table, nothing of the other features (their bags are empty for it).  The owner's lookup
// kernel then gathers every id it is given.  Three launches: count the ids of each row-sharded bag per owner,
// turn the counts into offsets (one block per feature and owner), then write ids and offsets into the peers'
// buffers and raise their flags.
struct BucketFeat { int kind; int owner; int rot; int rw_index; };   // rw_index: position among the row-sharded features
struct BucketizeParams {
  const int* values; const int* offsets; const float* weights;
  int n_feats, B, W, me, n_rw;
  const BucketFeat* feats;   // [n_feats]
  int* cnt;                  // [n_rw, W, B]: ids of bag b owned by rank r, then their exclusive prefix over b
  int* tot;                  // [n_rw, W]
  int* cnt_raw;              // [n_rw, W, B] or null: the counts themselves, kept for the combine and the gradient push
                             // (an owner that got no id of a bag neither writes its slot nor needs its gradient)
  int* dst_values[kMaxWorld]; int* dst_offsets[kMaxWorld]; float* dst_weights[kMaxWorld];
  unsigned int* done_counter; PeerFlags flags; SeqRef seq;
};

__device__ __forceinline__ int row_owner(int id, int W, int rot) {
  int m = id % W;
  if (m < 0) m += W;          // ids outside the vocabulary are reported by the owner's lookup, not here
  return (m + rot) % W;
}

__global__ void __launch_bounds__(256) bucket_count_kernel(const BucketizeParams p) {
  extern __shared__ int rw_feat[];      // [n_rw]: feature index of the j-th row-sharded feature
  for (int f = threadIdx.x; f < p.n_feats; f += blockDim.x)
    if (p.feats[f].kind == kRowWise) rw_feat[p.feats[f].rw_index] = f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long total = static_cast<long long>(p.n_rw) * p.B;
  for (long long jb = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5; jb < total; jb += warps) {
    const int j = static_cast<int>(jb / p.B), b = static_cast<int>(jb % p.B);
    const int fi = rw_feat[j];
    const int rot = p.feats[fi].rot;
    const long long fb = static_cast<long long>(fi) * p.B + b;
    const int o0 = p.offsets[fb], o1 = p.offsets[fb + 1];
    int mine = 0;                   // lane r counts the ids of rank r
    for (int base = o0; base < o1; base += 32) {
      const int i = base + lane;
      const int r = i < o1 ? row_owner(p.values[i], p.W, rot) : -1;
      for (int q = 0; q < p.W; ++q) {
        const int c = __popc(__ballot_sync(0xffffffffu, r == q));
        if (lane == q) mine += c;
      }
    }
    if (lane < p.W) {
      p.cnt[(static_cast<long long>(j) * p.W + lane) * p.B + b] = mine;
      if (p.cnt_raw != nullptr) p.cnt_raw[(static_cast<long long>(j) * p.W + lane) * p.B + b] = mine;
    }
  }
}

// One block per (row-sharded feature, owner): exclusive prefix sum of its B counts in place, total to tot.
__global__ void __launch_bounds__(1024) bucket_scan_kernel(const BucketizeParams p) {
  __shared__ int warp_sums[32];
  __shared__ int carry_s;
  int* c = p.cnt + static_cast<long long>(blockIdx.x) * p.B;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int per = (p.B + 1023) / 1024;
  const int lo = min(static_cast<int>(threadIdx.x) * per, p.B), hi = min(lo + per, p.B);
  int sum = 0;
  for (int i = lo; i < hi; ++i) sum += c[i];
  int incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = warp_sums[lane], wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += t;
    }
    warp_sums[lane] = wi - w;
    if (lane == 31) carry_s = wi;
  }
  __syncthreads();
  int run = warp_sums[warp] + incl - sum;
  for (int i = lo; i < hi; ++i) {
    const int v = c[i];
    c[i] = run;
    run += v;
  }
  if (threadIdx.x == 0) p.tot[blockIdx.x] = carry_s;
}

__global__ void __launch_bounds__(256) bucket_push_kernel(const BucketizeParams p) {
  extern __shared__ int base_s[];      // [W][n_feats + 1]: first id of feature f in rank r's batch
  const int lane = threadIdx.x & 31;
  const int F = p.n_feats;
  int* feat_lo = base_s + p.W * (F + 1);    // [n_feats + 1]: first id of feature f in the local batch
  int* rw_feat = feat_lo + F + 1;           // [n_rw]: feature index of the j-th row-sharded feature
  for (int f = threadIdx.x; f <= F; f += blockDim.x) {
    feat_lo[f] = p.offsets[static_cast<long long>(f) * p.B];
    if (f < F && p.feats[f].kind == kRowWise) rw_feat[p.feats[f].rw_index] = f;
  }
  if (threadIdx.x < p.W) {
    const int r = threadIdx.x;
    int run = 0;
    for (int f = 0; f < F; ++f) {
      base_s[r * (F + 1) + f] = run;
      const BucketFeat bf = p.feats[f];
      const int len = p.offsets[static_cast<long long>(f + 1) * p.B] - p.offsets[static_cast<long long>(f) * p.B];
      if (bf.kind == kRowWise) run += p.tot[bf.rw_index * p.W + r];
      else if (bf.kind == kColumnWise || bf.owner == r) run += len;
    }
    base_s[r * (F + 1) + F] = run;
    if (blockIdx.x == 0) p.dst_offsets[r][static_cast<long long>(F) * p.B] = run;     // end of the last bag
  }
  __syncthreads();
  const long long total = static_cast<long long>(F) * p.B;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  // (a) offsets of the bags of whole features, one thread per bag
  for (long long fb = tid; fb < total; fb += nthreads) {
    const int fi = static_cast<int>(fb / p.B);
    const BucketFeat f = p.feats[fi];
    if (f.kind == kRowWise) continue;
    const int within = p.offsets[fb] - feat_lo[fi];
    for (int r = 0; r < p.W; ++r) {
      const bool needs = f.kind == kColumnWise || f.owner == r;
      p.dst_offsets[r][fb] = base_s[r * (F + 1) + fi] + (needs ? within : 0);
    }
  }
  // (b) ids of whole features, one thread per id: the feature is found by bisection over the feature boundaries
  const long long nnz = feat_lo[F];
  for (long long i = tid; i < nnz; i += nthreads) {
    int lo = 0, hi = F;                 // feat_lo[lo] <= i < feat_lo[hi]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (feat_lo[mid] <= i) lo = mid; else hi = mid;
    }
    const BucketFeat f = p.feats[lo];
    if (f.kind == kRowWise) continue;
    const int v = p.values[i];
    const float w = p.weights != nullptr ? p.weights[i] : 0.f;
    const int within = static_cast<int>(i) - feat_lo[lo];
    const int r0 = f.kind == kColumnWise ? 0 : f.owner, r1 = f.kind == kColumnWise ? p.W : f.owner + 1;
    for (int r = max(r0, 0); r < r1; ++r) {
      const int at = base_s[r * (F + 1) + lo] + within;
      p.dst_values[r][at] = v;
      if (p.weights != nullptr) p.dst_weights[r][at] = w;
    }
  }
  // (c) row-sharded features, one warp per bag: every id goes to the rank that owns its row, behind the ids
  // that rank already got from this bag
  const long long warps = nthreads >> 5;
  const long long rw_total = static_cast<long long>(p.n_rw) * p.B;
  for (long long jb = tid >> 5; jb < rw_total; jb += warps) {
    const int fi = rw_feat[jb / p.B], b = static_cast<int>(jb % p.B);
    const BucketFeat f = p.feats[fi];
    const long long fb = static_cast<long long>(fi) * p.B + b;
    const int o0 = p.offsets[fb], o1 = p.offsets[fb + 1];
    int run = 0;      // lane r: where the next id of rank r goes
    if (lane < p.W) {
      run = base_s[lane * (F + 1) + fi] + p.cnt[(static_cast<long long>(f.rw_index) * p.W + lane) * p.B + b];
      p.dst_offsets[lane][fb] = run;
    }
    for (int base = o0; base < o1; base += 32) {
      const int i = base + lane;
      const bool on = i < o1;
      const int id = on ? p.values[i] : 0;
      const int r = on ? row_owner(id, p.W, f.rot) : p.W;     // idle lanes form a group of their own
      const unsigned int peers = __match_any_sync(0xffffffffu, r);
      const int at = __shfl_sync(0xffffffffu, run, r & 31) + __popc(peers & ((1u << lane) - 1u));
      if (on) {
        p.dst_values[r][at] = id;
        if (p.weights != nullptr) p.dst_weights[r][at] = p.weights[i];
      }
      for (int q = 0; q < p.W; ++q) {
        const int c = __popc(__ballot_sync(0xffffffffu, r == q));
        if (lane == q) run += c;
      }
    }
  }
  grid_done_then_signal(p.done_counter, p.flags, p.W, seq_of(p.seq));
}

// =================================== forward: gather + pool + peer store ===========================
struct FwdParams {
  IdPtrs ids;
  const FeatDesc* feats; int n_feats;
  int W, me, B;
  int dloc;                 // columns of the stack buffer (== dim except for column-wise features)
  const float* table;
  PeerBf16 pooled;          // destination buffers (one per source rank of the ids)
  uint32_t* occ_key; uint32_t* occ_val; float* occ_gain; unsigned int* occ_count; unsigned int occ_cap;
  long long grad_ld;        // >0: gradients will be read in place from a [B, grad_ld] matrix (1 rank):
                            //     occurrence value = (b*grad_ld + grad_off)/8 instead of a buffer row
  const unsigned long long* wait_flags;   // ids channel (null: no wait)
  unsigned int* done_counter; PeerFlags flags; SeqRef seq;  // pooled channel; the ids channel uses the same number
  int* status;
  unsigned int* dropped;    // non-null: ids that do not fit the occurrence list are dropped from the lookup and
                            // counted here (allow_id_dropping); null: an overflow is a kCapacity error
  int prefetch;             // bit 0: ask L2 for a bag's rows as soon as their ids are known; bit 1 (tiled kernel):
                            // let owned ids wait in the warp's queue across chunks
  int tiled;                // 1: no sequence feature in this launch -> the bags-in-tiles kernel
  long long total_tiles;    // tiled: sum over features of W * ceil(B / bags per tile)
  int prefiltered;          // 1: the senders bucketized the ids: every id of a row-sharded pooled feature found here
                            //    is owned (sequence features keep their positions, so they still arrive whole)
};

template <int VPL, bool TRAIN, bool GAINS>
__global__ void __launch_bounds__(256) emb_fwd_kernel(const FwdParams p) {
  const unsigned long long seq = seq_of(p.seq);
  if (p.wait_flags != nullptr && !wait_all_sources(p.wait_flags, p.W, seq, p.status, 0)) return;
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long total = static_cast<long long>(p.n_feats) * p.W * p.B;
  const bool lane_on = lane * VPL < p.dloc;
  for (long long item = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5; item < total;
       item += warps) {
    const int b = static_cast<int>(item % p.B);
    const int s = static_cast<int>((item / p.B) % p.W);
    const FeatDesc f = p.feats[item / (static_cast<long long>(p.B) * p.W)];
    const int* offs = p.ids.offsets[s] + static_cast<long long>(f.feat_index) * p.B + b;
    const int o0 = offs[0], o1 = offs[1];
    const int* vals = p.ids.values[s];
    const float* wts = GAINS ? p.ids.weights[s] : nullptr;
    // combiner denominator over the WHOLE bag (not only the rows this rank owns)
    float scale = 1.f;
    if (GAINS && f.combiner != kSum && f.seq_len == 0) {
      float den = 0.f;
      for (int i = o0 + lane; i < o1; i += 32) {
        const float w = wts != nullptr ? wts[i] : 1.f;
        den += f.combiner == kMean ? w : w * w;
      }
      den = warp_sum(den);
      if (f.combiner == kSqrtN) den = sqrtf(den);
      scale = den != 0.f ? 1.f / den : 0.f;
    }
    const long long gv_base = p.grad_ld > 0
        ? (static_cast<long long>(b) * p.grad_ld + f.grad_off) / 8
        : f.grad_off / p.dloc + (static_cast<long long>(s) * p.B + b) * (f.seq_len > 0 ? f.seq_len : 1);
    const int gv_step = p.grad_ld > 0 ? f.dim / 8 : 1;   // per sequence position
    Vec<VPL> acc;
#pragma unroll
    for (int e = 0; e < VPL; ++e) acc.v[e] = 0.f;
    __nv_bfloat16* dst_base = p.pooled.p[s] + f.slot_off + (f.kind == kColumnWise ? f.col_lo : 0) + lane * VPL;
    const long long slot_row = (f.kind == kRowWise ? static_cast<long long>(p.me) * p.B : 0) + b;
    for (int base = o0; base < o1; base += 32) {
      const int i = base + lane;
      int id = -1;
      float w = 1.f;
      if (i < o1) {
        id = vals[i];
        if (GAINS) w = (wts != nullptr ? wts[i] : 1.f) * scale;
      }
      bool owned = id >= 0;
      if (owned && id >= f.vocab) {      // never form an address from an id the table does not have
        report(p.status, kBadIndex, id);
        owned = false;
      }
      unsigned int lrow = 0;
      if (f.kind == kRowWise) {
        owned = owned && ((p.prefiltered && f.seq_len == 0) || (id % p.W + f.rot) % p.W == p.me);
        lrow = f.row_base + id / p.W;
      } else {
        lrow = f.row_base + id;
      }
      if (f.seq_len > 0 && i - o0 >= f.seq_len) owned = false;
      if (owned && (p.prefetch & 1)) prefetch_l2(p.table + static_cast<size_t>(lrow) * p.dloc, p.dloc * 4);
      unsigned int mask = __ballot_sync(0xffffffffu, owned);
      if (TRAIN && mask != 0) {
        // claim room in the occurrence list; the count may run past the capacity (readers clamp it), and
        // exactly the entries below the capacity get written
        const int n_own = __popc(mask);
        unsigned int pos = 0;
        if (lane == 0) pos = atomicAdd(p.occ_count, static_cast<unsigned int>(n_own));
        pos = __shfl_sync(0xffffffffu, pos, 0);
        const unsigned int at = pos + __popc(mask & ((1u << lane) - 1));
        const bool fits = owned && at < p.occ_cap;
        if (fits) {
          p.occ_key[at] = lrow;
          const unsigned int gv = static_cast<unsigned int>(gv_base + (f.seq_len > 0 ? (i - o0) * gv_step : 0));
          if (GAINS) {
            p.occ_val[at] = at;                       // index into (occ_gv = occ_key slot of vals, gain)
            p.occ_gain[2 * static_cast<size_t>(at)] = __uint_as_float(gv);
            p.occ_gain[2 * static_cast<size_t>(at) + 1] = w;
          } else {
            p.occ_val[at] = gv;
          }
        }
        const unsigned int over = __ballot_sync(0xffffffffu, owned && !fits);
        if (over != 0) {
          if (p.dropped != nullptr) {
            if (lane == 0) atomicAdd(p.dropped, static_cast<unsigned int>(__popc(over)));
            mask &= ~over;      // dropped ids take no part in the lookup either
          } else {
            report(p.status, kCapacity, 1);
          }
        }
      }
      if (f.seq_len > 0) {
        // sequence feature: every position of this 32-wide window is its own output vector; positions
        // this rank does not own (or that lie beyond the bag) are written as zeros so the slot is
        // fully defined
        const int npos = min(32, f.seq_len - (base - o0));
        for (int j = 0; j < npos; ++j) {
          const bool own_j = (mask >> j) & 1u;
          const unsigned int rj = __shfl_sync(0xffffffffu, lrow, j);
          const float wj = __shfl_sync(0xffffffffu, w, j);
          if (lane_on) {
            Vec<VPL> r;
#pragma unroll
            for (int e = 0; e < VPL; ++e) r.v[e] = 0.f;
            if (own_j) {
              r = load_f32<VPL>(p.table + static_cast<size_t>(rj) * p.dloc + lane * VPL);
#pragma unroll
              for (int e = 0; e < VPL; ++e) r.v[e] *= wj;
            }
            store_bf16<VPL>(dst_base + slot_row * f.dst_stride + static_cast<long long>(base - o0 + j) * f.dim, r);
          }
        }
        continue;
      }
      // gather owned rows, several at a time so that many loads are in flight
      constexpr int kDepth = VPL <= 4 ? 8 : 4;
      while (mask) {
        int j[kDepth]; unsigned int rj[kDepth]; float wj[kDepth];
        int n = 0;
#pragma unroll
        for (int u = 0; u < kDepth; ++u) {
          j[u] = mask ? __ffs(mask) - 1 : 0;
          if (mask) { mask &= mask - 1; n = u + 1; }
          rj[u] = __shfl_sync(0xffffffffu, lrow, j[u]);
          wj[u] = __shfl_sync(0xffffffffu, w, j[u]);
        }
        if (lane_on) {
          Vec<VPL> r[kDepth];
#pragma unroll
          for (int u = 0; u < kDepth; ++u)
            if (u < n) r[u] = load_f32<VPL>(p.table + static_cast<size_t>(rj[u]) * p.dloc + lane * VPL);
#pragma unroll
          for (int u = 0; u < kDepth; ++u)
            if (u < n) {
#pragma unroll
              for (int e = 0; e < VPL; ++e) acc.v[e] = fmaf(GAINS ? wj[u] : 1.f, r[u].v[e], acc.v[e]);
            }
        }
      }
    }
    if (f.seq_len > 0) {
      if (lane_on) {
        Vec<VPL> z;
#pragma unroll
        for (int e = 0; e < VPL; ++e) z.v[e] = 0.f;
        // the id loop covered positions [0, 32*ceil(len/32)) ∩ [0, seq_len)
        const int covered = min(f.seq_len, ((o1 - o0 + 31) / 32) * 32);
        for (int pos = covered; pos < f.seq_len; ++pos)
          store_bf16<VPL>(dst_base + slot_row * f.dst_stride + static_cast<long long>(pos) * f.dim, z);
      }
    } else if (lane_on && !(p.prefiltered && f.kind == kRowWise && o1 == o0)) {
      store_bf16<VPL>(dst_base + slot_row * f.dst_stride, acc);      // (a bucketized bag with no id for this rank: no store)
    }
  }
  grid_done_then_signal(p.done_counter, p.flags, p.W, seq);
}

// ---- forward, tiled: 32 consecutive bags of one (feature, source rank) per warp ----------------------
// The kernel above gives every bag its own chain of dependent memory latencies (offsets -> ids -> claim of
// occurrence entries -> rows), which dominates when bags hold one to three ids, as most recommender features
// do.  Here a warp takes up to 32 bags at once: one coalesced load brings their offsets, the ids of all of
// them are contiguous and come in 32-wide chunks, occurrence entries are claimed once per chunk, and the owned
// rows are gathered eight at a time ACROSS bag boundaries, each bag's sum being stored when its last row
// has been added.  The number of bags per warp is a per-feature power of two chosen by the host so that a
// tile holds a few hundred ids (32 bags of a one-id feature, 2 bags of a hundred-id one): a tile is a serial
// chain, and with a small per-GPU batch the longest chains decide the kernel's duration.  Pooled features
// only (a launch with a sequence feature takes the per-bag kernel).
template <int VPL, bool TRAIN, bool GAINS>
__global__ void __launch_bounds__(256, 2) emb_fwd_tiled_kernel(const FwdParams p) {
  const unsigned long long seq = seq_of(p.seq);
  if (p.wait_flags != nullptr && !wait_all_sources(p.wait_flags, p.W, seq, p.status, 0)) return;
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long total = p.total_tiles;
  const bool lane_on = lane * VPL < p.dloc;
  constexpr int kDepth = VPL <= 4 ? 8 : 4;
  for (long long tile = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5; tile < total;
       tile += warps) {
    // the feature whose range of work units holds this one (tile_start is increasing)
    int fi = -1;
    for (int f0 = 0; f0 < p.n_feats; f0 += 32) {
      const int fx = f0 + lane;
      fi += __popc(__ballot_sync(0xffffffffu, fx < p.n_feats && p.feats[fx].tile_start <= tile));
    }
    const FeatDesc f = p.feats[fi];
    const int bpt = 1 << f.tile_shift;
    const int blocks_per = (p.B + bpt - 1) >> f.tile_shift;
    const long long t = tile - f.tile_start;
    const int b0 = static_cast<int>(t % blocks_per) << f.tile_shift;
    const int s = static_cast<int>(t / blocks_per);
    const int nb = min(bpt, p.B - b0);                     // bags of this tile
    const int* offs = p.ids.offsets[s] + static_cast<long long>(f.feat_index) * p.B + b0;
    const int o_mine = offs[min(lane, nb)];               // lane l: first id of bag l (lanes >= nb: the end)
    const int p0 = __shfl_sync(0xffffffffu, o_mine, 0);
    const int p1 = offs[nb];
    const int* vals = p.ids.values[s];
    const float* wts = GAINS ? p.ids.weights[s] : nullptr;
    // combiner denominator of this lane's bag (over the WHOLE bag, not only the rows this rank owns)
    float scale_mine = 1.f;
    if (GAINS && f.combiner != kSum) {
      const int o1 = __shfl_down_sync(0xffffffffu, o_mine, 1);
      const int e = lane == 31 ? p1 : o1;
      float den = 0.f;
      if (lane < nb) {
        for (int i = o_mine; i < e; ++i) {
          const float w = wts != nullptr ? wts[i] : 1.f;
          den += f.combiner == kMean ? w : w * w;
        }
      }
      if (f.combiner == kSqrtN) den = sqrtf(den);
      scale_mine = den != 0.f ? 1.f / den : 0.f;
    }
    __nv_bfloat16* dst_base = p.pooled.p[s] + f.slot_off + (f.kind == kColumnWise ? f.col_lo : 0) + lane * VPL;
    const long long slot_row0 = (f.kind == kRowWise ? static_cast<long long>(p.me) * p.B : 0) + b0;
    Vec<VPL> acc;
#pragma unroll
    for (int e = 0; e < VPL; ++e) acc.v[e] = 0.f;
    int cur = 0;          // bag whose sum is being built; bags below it have been stored
    // Bucketized row-sharded features: the sender knows which owners got ids of a bag and reads only their slots,
    // so a bag of which this rank received nothing is not stored at all.
    unsigned int store_mask = 0xffffffffu;
    if (p.prefiltered && f.kind == kRowWise) {
      const int o_next = __shfl_down_sync(0xffffffffu, o_mine, 1);
      const int o_end = lane == nb - 1 ? p1 : o_next;
      store_mask = __ballot_sync(0xffffffffu, lane < nb && o_end > o_mine);
    }
    auto store_upto = [&](int bag) {      // stores bag `cur` (acc) and zeros for the bags between, then cur = bag
      while (cur < bag) {
        if (lane_on && ((store_mask >> cur) & 1u)) store_bf16<VPL>(dst_base + (slot_row0 + cur) * f.dst_stride, acc);
#pragma unroll
        for (int e = 0; e < VPL; ++e) acc.v[e] = 0.f;
        ++cur;
      }
    };
    unsigned int q_row = 0;
    float q_w = 1.f;
    int q_bag = 0, qn = 0;
    auto drain = [&]() {      // gathers the queued rows kDepth at a time, in order, and adds them to their bags
      for (int t0 = 0; t0 < qn; t0 += kDepth) {
        unsigned int rj[kDepth]; float wj[kDepth]; int bj[kDepth];
        const int n = min(kDepth, qn - t0);
#pragma unroll
        for (int u = 0; u < kDepth; ++u) {
          rj[u] = __shfl_sync(0xffffffffu, q_row, (t0 + u) & 31);
          wj[u] = GAINS ? __shfl_sync(0xffffffffu, q_w, (t0 + u) & 31) : 1.f;
          bj[u] = __shfl_sync(0xffffffffu, q_bag, (t0 + u) & 31);
        }
        Vec<VPL> r[kDepth];
        if (lane_on) {
#pragma unroll
          for (int u = 0; u < kDepth; ++u)
            if (u < n) r[u] = load_f32<VPL>(p.table + static_cast<size_t>(rj[u]) * p.dloc + lane * VPL);
        }
#pragma unroll
        for (int u = 0; u < kDepth; ++u) {
          if (u >= n) break;
          if (bj[u] != cur) store_upto(bj[u]);
          if (lane_on) {
#pragma unroll
            for (int e = 0; e < VPL; ++e) acc.v[e] = fmaf(wj[u], r[u].v[e], acc.v[e]);
          }
        }
      }
      qn = 0;
    };
    for (int base = p0; base < p1; base += 32) {
      const int i = base + lane;
      int id = -1;
      float w = 1.f;
      if (i < p1) id = vals[i];
      // bag of this id: the last lane whose first id is <= i (offsets are non-decreasing; lanes >= nb hold
      // the end of the tile).  Every lane runs the five shuffle steps, whatever it holds.
      int lo = 0, hi = nb;          // o[lo] <= i < o[hi]
#pragma unroll
      for (int step = 0; step < 5; ++step) {
        const int mid = (lo + hi) >> 1;
        const int om = __shfl_sync(0xffffffffu, o_mine, mid);
        if (hi - lo > 1) { if (om <= i) lo = mid; else hi = mid; }
      }
      const int bag = lo;
      if (GAINS) {
        const float sc = __shfl_sync(0xffffffffu, scale_mine, bag);
        if (i < p1) w = (wts != nullptr ? wts[i] : 1.f) * sc;
      }
      bool owned = id >= 0;
      if (owned && id >= f.vocab) {
        report(p.status, kBadIndex, id);
        owned = false;
      }
      unsigned int lrow = 0;
      if (f.kind == kRowWise) {
        owned = owned && ((p.prefiltered && f.seq_len == 0) || (id % p.W + f.rot) % p.W == p.me);
        lrow = f.row_base + id / p.W;
      } else {
        lrow = f.row_base + id;
      }
      if (owned && (p.prefetch & 1)) prefetch_l2(p.table + static_cast<size_t>(lrow) * p.dloc, p.dloc * 4);
      unsigned int mask = __ballot_sync(0xffffffffu, owned);
      if (TRAIN && mask != 0) {
        const int n_own = __popc(mask);
        unsigned int pos = 0;
        if (lane == 0) pos = atomicAdd(p.occ_count, static_cast<unsigned int>(n_own));
        pos = __shfl_sync(0xffffffffu, pos, 0);
        const unsigned int at = pos + __popc(mask & ((1u << lane) - 1));
        const bool fits = owned && at < p.occ_cap;
        if (fits) {
          const int b = b0 + bag;
          const long long gvl = p.grad_ld > 0 ? (static_cast<long long>(b) * p.grad_ld + f.grad_off) / 8
                                              : f.grad_off / p.dloc + (static_cast<long long>(s) * p.B + b);
          const unsigned int gv = static_cast<unsigned int>(gvl);
          p.occ_key[at] = lrow;
          if (GAINS) {
            p.occ_val[at] = at;
            p.occ_gain[2 * static_cast<size_t>(at)] = __uint_as_float(gv);
            p.occ_gain[2 * static_cast<size_t>(at) + 1] = w;
          } else {
            p.occ_val[at] = gv;
          }
        }
        const unsigned int over = __ballot_sync(0xffffffffu, owned && !fits);
        if (over != 0) {
          if (p.dropped != nullptr) {
            if (lane == 0) atomicAdd(p.dropped, static_cast<unsigned int>(__popc(over)));
            mask &= ~over;
          } else {
            report(p.status, kCapacity, 1);
          }
        }
      }
      // Owned ids wait in a queue (entry t in lane t) until a chunk no longer fits behind them: a rank owns only
      // 1/W of a row-sharded feature's ids, and gathering the few rows of each chunk by themselves would leave the
      // loads of a warp one short round trip after the other.
      const int n_own = __popc(mask);
      if (qn + n_own > 32) drain();
      if (n_own > 0) {
        const bool mine = lane >= qn && lane < qn + n_own;
        const int src = mine ? __fns(mask, 0, lane - qn + 1) : 0;
        const unsigned int r_in = __shfl_sync(0xffffffffu, lrow, src);
        const float w_in = GAINS ? __shfl_sync(0xffffffffu, w, src) : 1.f;
        const int b_in = __shfl_sync(0xffffffffu, bag, src);
        if (mine) { q_row = r_in; q_w = w_in; q_bag = b_in; }
        qn += n_own;
        if (!(p.prefetch & 2)) drain();
      }
    }
    drain();
    store_upto(nb);       // the open bag and the (empty or un-owned) bags after it
  }
  grid_done_then_signal(p.done_counter, p.flags, p.W, seq);
}

// =================================== combine: sum source slots, write concat =======================
struct CombineDesc { long long slot_off; int nslots; int dim; int out_col; int seq_len; int rw_index; int pad; };
struct CombineParams {
  const __nv_bfloat16* pooled; const CombineDesc* feats; int n_feats; int B;
  __nv_bfloat16* out; long long ld_out;
  const unsigned long long* wait_flags; int W; int n_chan; SeqRef seq; int* status;
  const int* cnt_raw;       // [n_rw, W, B] or null: ids of bag b this rank sent to owner r (bucketized features: a slot
                            // is read only when its owner received ids of the bag, and only then was it written)
};

__global__ void __launch_bounds__(256) emb_combine_kernel(const CombineParams p) {
  if (p.wait_flags != nullptr && !wait_all_sources(p.wait_flags, p.W, seq_of(p.seq), p.status, 1, p.n_chan)) return;
  // one thread per 16-byte chunk (8 bf16) of one (sample, feature) vector
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (int fi = 0; fi < p.n_feats; ++fi) {
    const CombineDesc f = p.feats[fi];
    const int width = f.dim * (f.seq_len > 0 ? f.seq_len : 1);
    const int chunks = width / 8;
    const long long total = static_cast<long long>(p.B) * chunks;
    const long long slot_stride = static_cast<long long>(p.B) * width;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += stride) {
      const long long b = i / chunks;
      const int e = static_cast<int>(i - b * chunks) * 8;
      const __nv_bfloat16* src = p.pooled + f.slot_off + b * width + e;
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      const int* own = (p.cnt_raw != nullptr && f.rw_index >= 0)
          ? p.cnt_raw + static_cast<long long>(f.rw_index) * p.W * p.B + b : nullptr;
      for (int sl = 0; sl < f.nslots; ++sl) {
        if (own != nullptr && own[static_cast<long long>(sl) * p.B] == 0) continue;
        const uint4 t = *reinterpret_cast<const uint4*>(src + sl * slot_stride);
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { acc[2 * j] += bf16_lo(w[j]); acc[2 * j + 1] += bf16_hi(w[j]); }
      }
      *reinterpret_cast<uint4*>(p.out + b * p.ld_out + f.out_col + e) =
          make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]),
                     pack_bf16(acc[6], acc[7]));
    }
  }
}

// =================================== backward: push activation gradients ===========================
struct PushGradDesc {
  int kind; int owner; int dim; int in_col; int seq_len;
  int rw_index;   // >= 0: position among the bucketized row-sharded features (-1: every owner gets the gradient)
  long long grad_off[kMaxWorld];   // element offset of the feature block in rank r's gradient buffer (-1: none)
};
struct PushGradParams {
  const __nv_bfloat16* grad; long long ld; const PushGradDesc* feats; int n_feats; int B; int W; int me;
  PeerBf16 dst; unsigned int* done_counter; PeerFlags flags; SeqRef seq;
  const int* cnt_raw;   // [n_rw, W, B] or null: owners that received no id of a bag do not need its gradient
};

// Half a warp per (feature, sample): 16 lanes x 16 bytes cover a 128-wide bf16 gradient in one load, which is then
// stored to every rank that holds rows of the feature's table.
__global__ void __launch_bounds__(256) emb_push_grads_kernel(const PushGradParams p) {
  const int lane = threadIdx.x & 31;
  const int sub = lane >> 4, sl = lane & 15;
  const long long halves = (static_cast<long long>(gridDim.x) * blockDim.x) >> 4;
  const long long total = static_cast<long long>(p.n_feats) * p.B;
  for (long long item = (((blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5) << 1) + sub; item < total;
       item += halves) {
    const int fi = static_cast<int>(item % p.n_feats);
    const long long b = item / p.n_feats;
    const PushGradDesc& f = p.feats[fi];
    const int width = f.dim * (f.seq_len > 0 ? f.seq_len : 1);
    const __nv_bfloat16* src = p.grad + b * p.ld + f.in_col;
    const long long row = static_cast<long long>(p.me) * p.B + b;
    if (f.kind == kColumnWise) {
      const int dl = f.dim / p.W;
      for (int e = sl * 2; e < f.dim; e += 32) {
        const int r = e / dl;
        *reinterpret_cast<uint32_t*>(p.dst.p[r] + f.grad_off[r] + row * dl + (e - r * dl)) =
            *reinterpret_cast<const uint32_t*>(src + e);
      }
    } else {
      const int r0 = f.kind == kTableWise ? f.owner : 0;
      const int r1 = f.kind == kTableWise ? f.owner + 1 : p.W;
      unsigned int to = 0;          // the ranks that get this gradient
      for (int r = r0; r < r1; ++r) to |= 1u << r;
      if (p.cnt_raw != nullptr && f.kind == kRowWise && f.rw_index >= 0) {
        const int* own = p.cnt_raw + static_cast<long long>(f.rw_index) * p.W * p.B + b;
        for (int r = 0; r < p.W; ++r)
          if (own[static_cast<long long>(r) * p.B] == 0) to &= ~(1u << r);
      }
      bool vec = (width & 7) == 0 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
      for (int r = r0; r < r1; ++r)
        vec = vec && (reinterpret_cast<uintptr_t>(p.dst.p[r] + f.grad_off[r] + row * width) & 15u) == 0;
      if (vec) {
        for (int e = sl * 8; e < width; e += 128) {
          const uint4 v = *reinterpret_cast<const uint4*>(src + e);
          for (int r = r0; r < r1; ++r)
            if ((to >> r) & 1u) *reinterpret_cast<uint4*>(p.dst.p[r] + f.grad_off[r] + row * width + e) = v;
        }
      } else {
        for (int e = sl * 2; e < width; e += 32) {
          const uint32_t v = *reinterpret_cast<const uint32_t*>(src + e);
          for (int r = r0; r < r1; ++r)
            if ((to >> r) & 1u) *reinterpret_cast<uint32_t*>(p.dst.p[r] + f.grad_off[r] + row * width + e) = v;
        }
      }
    }
  }
  grid_done_then_signal(p.done_counter, p.flags, p.W, seq_of(p.seq));
}

// =================================== backward: segmented reduce + row optimizer ====================
struct BwdParams {
  const uint32_t* keys; const uint32_t* vals; const float* occ_gain; const unsigned int* n_occ;
  const __nv_bfloat16* grads;   // gradient vectors: vector v starts at grads + v * val_scale elements
  long long val_scale;
  float* table; float* slot0; float* slot1; int dloc;
  int opt; float hp[6]; float grad_scale; int slot1_rowwise;
  float* scratch;               // [>= ceil(n / kRange), dloc] partial sums of runs that cross range boundaries (kept zero)
  const unsigned long long* wait_flags; int W; SeqRef seq; int* status;
  const float* hp_dev;          // non-null: the six hyper-parameters are read from device memory (so that a
                                // captured CUDA graph follows a learning-rate schedule) instead of `hp`
  unsigned int n_cap;           // >0: *n_occ is clamped to this (capacity of the occurrence list)
  int reserved;
};

__device__ __forceinline__ float hpv(const BwdParams& p, int i) {
  return p.hp_dev != nullptr ? __ldg(p.hp_dev + i) : p.hp[i];
}
__device__ __forceinline__ unsigned int occ_count_of(const BwdParams& p) {
  const unsigned int n = *p.n_occ;
  return p.n_cap > 0 && n > p.n_cap ? p.n_cap : n;
}

template <int VPL>
__device__ __forceinline__ void apply_row_update(const BwdParams& p, unsigned int row, Vec<VPL> g, int lane,
                                                 bool lane_on) {
  const size_t off = static_cast<size_t>(row) * p.dloc + lane * VPL;
  Vec<VPL> w;
  if (lane_on) w = load_f32_rw<VPL>(p.table + off);
#pragma unroll
  for (int e = 0; e < VPL; ++e) g.v[e] *= p.grad_scale;
  float sq = 0.f;
  if (lane_on) {
#pragma unroll
    for (int e = 0; e < VPL; ++e) sq += g.v[e] * g.v[e];
  }
  const float lr = hpv(p, 0);
  switch (p.opt) {
    case kSGD:
      if (lane_on) {
#pragma unroll
        for (int e = 0; e < VPL; ++e) w.v[e] -= lr * g.v[e];
      }
      break;
    case kRowAdagrad: {
      const float msq = warp_sum(sq) / p.dloc;
      const float s = p.slot0[row] + msq;
      __syncwarp();
      if (lane == 0) p.slot0[row] = s;
      const float inv = lr / (sqrtf(s) + hpv(p, 1));
      if (lane_on) {
#pragma unroll
        for (int e = 0; e < VPL; ++e) w.v[e] -= inv * g.v[e];
      }
      break;
    }
    case kAdagrad:
      if (lane_on) {
        Vec<VPL> a = load_f32_rw<VPL>(p.slot0 + off);
#pragma unroll
        for (int e = 0; e < VPL; ++e) { a.v[e] += g.v[e] * g.v[e]; w.v[e] -= lr * g.v[e] * rsqrtf(a.v[e]); }
        store_f32<VPL>(p.slot0 + off, a);
      }
      break;
    case kAdam:
    case kRowAdam: {
      const float b1 = hpv(p, 1), b2 = hpv(p, 2), eps = hpv(p, 3);
      float vrow = 0.f;
      if (p.opt == kRowAdam) {
        const float msq = warp_sum(sq) / p.dloc;
        vrow = p.slot1[row];
        vrow += (1.f - b2) * (msq - vrow);
        __syncwarp();
        if (lane == 0) p.slot1[row] = vrow;
      }
      if (lane_on) {
        Vec<VPL> m = load_f32_rw<VPL>(p.slot0 + off);
        Vec<VPL> v;
        if (p.opt == kAdam) v = load_f32_rw<VPL>(p.slot1 + off);
#pragma unroll
        for (int e = 0; e < VPL; ++e) {
          m.v[e] += (1.f - b1) * (g.v[e] - m.v[e]);
          float ve = vrow;
          if (p.opt == kAdam) { v.v[e] += (1.f - b2) * (g.v[e] * g.v[e] - v.v[e]); ve = v.v[e]; }
          w.v[e] -= lr * m.v[e] / (sqrtf(ve) + eps);
        }
        store_f32<VPL>(p.slot0 + off, m);
        if (p.opt == kAdam) store_f32<VPL>(p.slot1 + off, v);
      }
      break;
    }
    case kAdagradMomentum:
      if (lane_on) {
        const float k = hpv(p, 1), beta2 = hpv(p, 2), eps = hpv(p, 3), expo = hpv(p, 4);
        const bool nesterov = hpv(p, 5) != 0.f;
        Vec<VPL> a = load_f32_rw<VPL>(p.slot0 + off), mo = load_f32_rw<VPL>(p.slot1 + off);
#pragma unroll
        for (int e = 0; e < VPL; ++e) {
          const float g2 = g.v[e] * g.v[e];
          a.v[e] = beta2 == 1.f ? a.v[e] + g2 : beta2 * a.v[e] + (1.f - beta2) * g2;
          const float s = powf(a.v[e] + eps, -1.f / expo) * g.v[e];
          mo.v[e] = k * mo.v[e] + s;
          w.v[e] -= lr * (nesterov ? k * mo.v[e] + s : mo.v[e]);
        }
        store_f32<VPL>(p.slot0 + off, a);
        store_f32<VPL>(p.slot1 + off, mo);
      }
      break;
    case kFTRL:
      if (lane_on) {
        const float lrp = hpv(p, 1), l1 = hpv(p, 2), l2 = hpv(p, 3), beta = hpv(p, 4);
        const bool mult = hpv(p, 5) != 0.f;
        Vec<VPL> a = load_f32_rw<VPL>(p.slot0 + off), li = load_f32_rw<VPL>(p.slot1 + off);
#pragma unroll
        for (int e = 0; e < VPL; ++e) {
          const float an = a.v[e] + g.v[e] * g.v[e];
          const float po = powf(a.v[e], -lrp), pn = powf(an, -lrp);
          float ln, l1s, den;
          if (mult) { ln = li.v[e] + lr * g.v[e] - (pn - po) * w.v[e]; l1s = l1 * lr; den = pn + 2.f * lr * l2 + beta; }
          else { ln = li.v[e] + g.v[e] - ((pn - po) / lr) * w.v[e]; l1s = l1; den = (pn + beta) / lr + 2.f * l2; }
          const float num = l1 == 0.f ? -ln : fminf(fmaxf(ln, -l1s), l1s) - ln;
          w.v[e] = num / den;
          a.v[e] = an; li.v[e] = ln;
        }
        store_f32<VPL>(p.slot0 + off, a);
        store_f32<VPL>(p.slot1 + off, li);
      }
      break;
    case kLaProp:
      if (lane_on) {
        const float b1 = hpv(p, 1), decay = hpv(p, 2), eps = hpv(p, 3);
        Vec<VPL> mu = load_f32_rw<VPL>(p.slot0 + off), nu = load_f32_rw<VPL>(p.slot1 + off);
#pragma unroll
        for (int e = 0; e < VPL; ++e) {
          nu.v[e] = decay * nu.v[e] + (1.f - decay) * (g.v[e] * g.v[e] + eps);
          mu.v[e] = b1 * mu.v[e] + sqrtf(1.f - b1 * b1) * g.v[e] * rsqrtf(nu.v[e]);
          w.v[e] -= lr * mu.v[e];
        }
        store_f32<VPL>(p.slot0 + off, mu);
        store_f32<VPL>(p.slot1 + off, nu);
      }
      break;
    default: break;
  }
  if (lane_on) store_f32<VPL>(p.table + off, w);
}

// first index i in [0, hi) with keys[i] >= key  (keys sorted ascending)
__device__ __forceinline__ unsigned int lower_bound(const uint32_t* keys, unsigned int hi, uint32_t key) {
  unsigned int lo = 0;
  while (lo < hi) {
    const unsigned int mid = (lo + hi) >> 1;
    if (keys[mid] < key) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// One warp per RANGE of kRange sorted occurrences, walked in 32-wide windows with the running sum
// carried across windows; a persistent grid strides over the ranges.  A run of equal rows that lies
// inside the range is reduced in registers and applied at once; the pieces of a run that crosses
// range boundaries are added (fp32 atomics) into the scratch line of the range where the run STARTS,
// and emb_bwd_finalize applies those afterwards.  Hot rows (Zipf heads with 10^5 occurrences) are
// thereby reduced by thousands of warps in parallel, with one atomic line update per kRange
// occurrences.
//
// The kernel is bound by memory latency (random 256-byte gradient vectors, random table rows), so
// every window first asks L2 for what the NEXT window will read (its gradient vectors) and for the
// table rows and optimizer slots of the runs that end in THIS window; the loads that follow then wait
// for L2, not DRAM.  It uses no shared memory and at most 64 registers so that it can share the SMs with a
// tensor-core GEMM running on another stream: beside this library's GEMM CTA (320 threads x 104 registers,
// ~210 KB of shared memory) an SM was measured to take three 128-thread blocks of 64 registers, but not
// three of 80 (`blocks_per_sm` caps the grid accordingly).
constexpr unsigned int kRange = 128;
constexpr int kBwdThreads = 128;

// At most 64 registers: three blocks then share an SM with a GEMM CTA.  (A 56-register build, one allocation unit of
// 256 registers per warp less, lets four blocks in; it measured the same step time and is not kept.)
template <int VPL, bool GAINS>
__global__ void __launch_bounds__(kBwdThreads, 8) emb_bwd_update_kernel(const BwdParams p) {
  if (p.wait_flags != nullptr && !wait_all_sources(p.wait_flags, p.W, seq_of(p.seq), p.status, 2)) return;
  const int lane = threadIdx.x & 31;
  const unsigned int n = occ_count_of(p);
  const unsigned int warps = (gridDim.x * blockDim.x) >> 5;
  const bool lane_on = lane * VPL < p.dloc;
  const int grad_bytes = p.dloc * 2, row_bytes = p.dloc * 4;
  const bool slot0_row = p.opt == kRowAdagrad, slot1_row = p.opt == kRowAdam;
  constexpr int kBatch = VPL <= 4 ? 8 : 4;
  for (unsigned int range = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; range * kRange < n; range += warps) {
    const unsigned int start = range * kRange;
    const unsigned int end = min(start + kRange, n);
    const bool has_prev = start > 0, has_next = end < n;
    const uint32_t prev_key = has_prev ? p.keys[start - 1] : 0;
    const uint32_t next_key = has_next ? p.keys[end] : 0;
    Vec<VPL> acc;
#pragma unroll
    for (int e = 0; e < VPL; ++e) acc.v[e] = 0.f;
    bool first_run = true;      // no run has been closed yet: the open one may have begun before `start`
    // this window's entries; the next window's are fetched one window ahead
    uint32_t key = 0xffffffffu; unsigned int gv = 0; float gain = 1.f;
    auto fetch = [&](unsigned int w0, uint32_t& k, unsigned int& g, float& gn) {
      k = 0xffffffffu; g = 0; gn = 1.f;
      if (w0 + lane < end) {
        k = p.keys[w0 + lane];
        const uint32_t val = p.vals[w0 + lane];
        g = val;
        if (GAINS) {
          g = __float_as_uint(p.occ_gain[2 * static_cast<size_t>(val)]);
          gn = p.occ_gain[2 * static_cast<size_t>(val) + 1];
        }
        prefetch_l2(p.grads + static_cast<size_t>(g) * p.val_scale, grad_bytes);
      }
    };
    fetch(start, key, gv, gain);
    for (unsigned int w0 = start; w0 < end; w0 += 32u) {
      const int cnt = static_cast<int>(min(32u, end - w0));
      const bool window_is_last = w0 + cnt >= end;
      uint32_t nkey = 0xffffffffu; unsigned int ngv = 0; float ngain = 1.f;
      if (!window_is_last) fetch(w0 + 32u, nkey, ngv, ngain);
      // which entries end a run (inside the range; the range's last entry always closes the open piece)
      const uint32_t after = __shfl_sync(0xffffffffu, nkey, 0);
      uint32_t knext = __shfl_down_sync(0xffffffffu, key, 1);
      if (lane == cnt - 1) knext = after;
      const bool ends_run = lane < cnt && ((window_is_last && lane == cnt - 1) || knext != key);
      const unsigned int last_mask = __ballot_sync(0xffffffffu, ends_run);
      if (ends_run) {
        prefetch_l2(p.table + static_cast<size_t>(key) * p.dloc, row_bytes);
        if (p.slot0 != nullptr) {
          if (slot0_row) prefetch_l2(p.slot0 + key, 4); else prefetch_l2(p.slot0 + static_cast<size_t>(key) * p.dloc, row_bytes);
        }
        if (p.slot1 != nullptr) {
          if (slot1_row) prefetch_l2(p.slot1 + key, 4); else prefetch_l2(p.slot1 + static_cast<size_t>(key) * p.dloc, row_bytes);
        }
      }
      for (int j0 = 0; j0 < cnt; j0 += kBatch) {
        RawBf16<VPL> g[kBatch]; float gj[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          const int j = min(j0 + u, cnt - 1);
          const unsigned int gvj = __shfl_sync(0xffffffffu, gv, j);
          gj[u] = GAINS ? __shfl_sync(0xffffffffu, gain, j) : 1.f;
          if (lane_on && j0 + u < cnt)
            g[u] = load_raw_bf16<VPL>(p.grads + static_cast<size_t>(gvj) * p.val_scale + lane * VPL);
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          const int j = j0 + u;
          if (j >= cnt) break;
          if (lane_on) fma_raw_bf16<VPL>(acc, gj[u], g[u]);
          if (!((last_mask >> j) & 1u)) continue;
          const uint32_t kj = __shfl_sync(0xffffffffu, key, j);
          const bool at_range_end = window_is_last && j == cnt - 1;
          const bool begins = !first_run || !has_prev || (prev_key != kj);
          const bool ends = !at_range_end || !has_next || (next_key != kj);
          if (begins && ends) {
            apply_row_update<VPL>(p, kj, acc, lane, lane_on);
          } else {
            unsigned int slot = range;
            if (!begins) {
              if (lane == 0) slot = lower_bound(p.keys, start, kj) / kRange;
              slot = __shfl_sync(0xffffffffu, slot, 0);
            }
            if (lane_on) {
              float* sp = p.scratch + static_cast<size_t>(slot) * p.dloc + lane * VPL;
#pragma unroll
              for (int e = 0; e < VPL; ++e) atomicAdd(sp + e, acc.v[e]);
            }
          }
#pragma unroll
          for (int e = 0; e < VPL; ++e) acc.v[e] = 0.f;
          first_run = false;
        }
      }
      key = nkey; gv = ngv; gain = ngain;
    }
  }
}

template <int VPL>
__global__ void __launch_bounds__(256) emb_bwd_finalize_kernel(const BwdParams p) {
  const int lane = threadIdx.x & 31;
  const unsigned int n = occ_count_of(p);
  const unsigned int range = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const unsigned int start = range * kRange;
  if (start >= n) return;
  const unsigned int last = min(start + kRange, n) - 1;
  const uint32_t klast = p.keys[last];
  if (!(last + 1 < n && p.keys[last + 1] == klast)) return;            // run does not cross into the next range
  if (p.keys[start] == klast && start > 0 && p.keys[start - 1] == klast) return;  // run started earlier
  const bool lane_on = lane * VPL < p.dloc;
  float* sp = p.scratch + static_cast<size_t>(range) * p.dloc + lane * VPL;
  Vec<VPL> acc;
#pragma unroll
  for (int e = 0; e < VPL; ++e) acc.v[e] = 0.f;
  if (lane_on) {
    acc = load_f32_rw<VPL>(sp);
    Vec<VPL> z;
#pragma unroll
    for (int e = 0; e < VPL; ++e) z.v[e] = 0.f;
    store_f32<VPL>(sp, z);
  }
  apply_row_update<VPL>(p, klast, acc, lane, lane_on);
}

__global__ void tick_kernel(unsigned long long* p) { *p += 1ull; }

static int blocks_for(long long warps_needed, int max_blocks) {
  long long b = (warps_needed + 7) / 8;
  if (b < 1) b = 1;
  return static_cast<int>(b < max_blocks ? b : max_blocks);
}

}  // namespace emb
}  // namespace recml

using namespace recml::emb;

extern "C" int recml_tick(unsigned long long* counter, cudaStream_t stream) {
  tick_kernel<<<1, 1, 0, stream>>>(counter);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int recml_emb_push_ids(const PushIdsParams* p, cudaStream_t stream) {
  long long work = p->nnz > p->n_offsets ? p->nnz : p->n_offsets;
  int blocks = static_cast<int>((work + 1023) / 1024);
  const int cap = 148 * 8;
  blocks = blocks < 1 ? 1 : (blocks > cap ? cap : blocks);
  const size_t smem = p->need != nullptr ? (static_cast<size_t>(p->n_feats) + 1) * sizeof(int) : 0;
  if (smem > 40 * 1024) return -2;
  emb_push_ids_kernel<<<blocks, 256, smem, stream>>>(*p);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

template <int VPL>
static void launch_fwd(const FwdParams& p, bool train, bool gains, int blocks, cudaStream_t stream) {
  if (p.tiled) {
    if (train) {
      if (gains) emb_fwd_tiled_kernel<VPL, true, true><<<blocks, 256, 0, stream>>>(p);
      else emb_fwd_tiled_kernel<VPL, true, false><<<blocks, 256, 0, stream>>>(p);
    } else {
      if (gains) emb_fwd_tiled_kernel<VPL, false, true><<<blocks, 256, 0, stream>>>(p);
      else emb_fwd_tiled_kernel<VPL, false, false><<<blocks, 256, 0, stream>>>(p);
    }
    return;
  }
  if (train) {
    if (gains) emb_fwd_kernel<VPL, true, true><<<blocks, 256, 0, stream>>>(p);
    else emb_fwd_kernel<VPL, true, false><<<blocks, 256, 0, stream>>>(p);
  } else {
    if (gains) emb_fwd_kernel<VPL, false, true><<<blocks, 256, 0, stream>>>(p);
    else emb_fwd_kernel<VPL, false, false><<<blocks, 256, 0, stream>>>(p);
  }
}

static int vpl_for(int dloc) { return dloc <= 32 ? 1 : dloc <= 64 ? 2 : dloc <= 128 ? 4 : dloc <= 256 ? 8 : 0; }

// Resident-block bound: co-operating grids (a kernel whose blocks wait on peers) must fit the GPU.
extern "C" int recml_emb_fwd(const FwdParams* p, int train, int gains, cudaStream_t stream) {
  const int vpl = vpl_for(p->dloc);
  if (vpl == 0 || (p->dloc % vpl) != 0) return -10;
  const long long items = p->tiled ? p->total_tiles : static_cast<long long>(p->n_feats) * p->W * p->B;
  const int blocks = blocks_for(items, 148 * 8);
  switch (vpl) {
    case 1: launch_fwd<1>(*p, train, gains, blocks, stream); break;
    case 2: launch_fwd<2>(*p, train, gains, blocks, stream); break;
    case 4: launch_fwd<4>(*p, train, gains, blocks, stream); break;
    default: launch_fwd<8>(*p, train, gains, blocks, stream); break;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int recml_emb_combine(const CombineParams* p, cudaStream_t stream) {
  const int blocks = blocks_for(static_cast<long long>(p->n_feats) * p->B * 4, 148 * 8);
  emb_combine_kernel<<<blocks, 256, 0, stream>>>(*p);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int recml_emb_push_grads(const PushGradParams* p, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) { recml::prefer_max_shared_carveout(emb_push_grads_kernel); configured = true; }
  // three resident blocks per SM (256 threads x 32 registers each): a GEMM CTA of another stream (the
  // weight-gradient products run at the same time) still finds its threads and registers on every SM
  static const int per_sm = [] { const char* e = getenv("RECML_EMB_PUSH_BLOCKS"); return e ? atoi(e) : 3; }();
  const int blocks = blocks_for(static_cast<long long>(p->n_feats) * p->B, 148 * per_sm);
  emb_push_grads_kernel<<<blocks, 256, 0, stream>>>(*p);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// max_occ: host-side upper bound of *n_occ used to size the grid (the persistent grid strides over the ranges
// that exist).  blocks_per_sm: resident 128-thread blocks per SM: 0 = fill the GPU; -1 = leave room for a GEMM
// CTA of another stream on every SM (three blocks of this 64-register kernel).
extern "C" int recml_emb_bwd_update(const BwdParams* p, long long max_occ, int gains, int blocks_per_sm,
                                    cudaStream_t stream) {
  const int vpl = vpl_for(p->dloc);
  if (vpl == 0 || (p->dloc % vpl) != 0) return -10;
  if (max_occ <= 0) return 0;
  const long long ranges = (max_occ + kRange - 1) / kRange;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  if (blocks_per_sm < 0) blocks_per_sm = 3;      // what fits beside a resident GEMM CTA
  if (blocks_per_sm == 0) blocks_per_sm = 8;
  long long want = (ranges + (kBwdThreads / 32) - 1) / (kBwdThreads / 32);
  const long long cap = static_cast<long long>(sms) * blocks_per_sm;
  const int blocks = static_cast<int>(want < cap ? want : cap);
  const int fin_blocks = static_cast<int>((ranges + 7) / 8);
#define RECML_BWD(V)                                                                      \
  do {                                                                                    \
    static bool configured = false;                                                       \
    if (!configured) {                                                                    \
      recml::prefer_max_shared_carveout(emb_bwd_update_kernel<V, true>);                  \
      recml::prefer_max_shared_carveout(emb_bwd_update_kernel<V, false>);                 \
      recml::prefer_max_shared_carveout(emb_bwd_finalize_kernel<V>);                      \
      configured = true;                                                                  \
    }                                                                                     \
    if (gains) emb_bwd_update_kernel<V, true><<<blocks, kBwdThreads, 0, stream>>>(*p);    \
    else emb_bwd_update_kernel<V, false><<<blocks, kBwdThreads, 0, stream>>>(*p);         \
    emb_bwd_finalize_kernel<V><<<fin_blocks, 256, 0, stream>>>(*p);                       \
  } while (0)
  switch (vpl) {
    case 1: RECML_BWD(1); break;
    case 2: RECML_BWD(2); break;
    case 4: RECML_BWD(4); break;
    default: RECML_BWD(8); break;
  }
#undef RECML_BWD
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int recml_emb_bucketize_push(const BucketizeParams* p, cudaStream_t stream) {
  if (p->W > kMaxWorld || p->n_feats <= 0 || p->B <= 0) return -2;
  const size_t smem = (static_cast<size_t>(p->W + 1) * (p->n_feats + 1) + p->n_rw) * sizeof(int);
  if (smem > 40 * 1024) return -2;
  // (the push kernel's work is one thread per id or per bag of a whole feature, one warp per row-sharded bag)
  const long long bags = static_cast<long long>(p->n_feats) * p->B;
  int blocks = static_cast<int>((bags + 255) / 256);
  const int cap = 148 * 8;
  blocks = blocks < 1 ? 1 : (blocks > cap ? cap : blocks);
  if (p->n_rw > 0) {
    const long long rw_bags = static_cast<long long>(p->n_rw) * p->B;
    int cblocks = static_cast<int>((rw_bags + 7) / 8);
    cblocks = cblocks < 1 ? 1 : (cblocks > cap ? cap : cblocks);
    bucket_count_kernel<<<cblocks, 256, p->n_rw * sizeof(int), stream>>>(*p);
    bucket_scan_kernel<<<p->n_rw * p->W, 1024, 0, stream>>>(*p);
  }
  bucket_push_kernel<<<blocks, 256, smem, stream>>>(*p);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int recml_emb_bucketize_struct_size() { return static_cast<int>(sizeof(BucketizeParams)); }

extern "C" int recml_emb_struct_sizes(int* out) {
  out[0] = sizeof(FeatDesc); out[1] = sizeof(FwdParams); out[2] = sizeof(CombineDesc); out[3] = sizeof(CombineParams);
  out[4] = sizeof(PushGradDesc); out[5] = sizeof(PushGradParams); out[6] = sizeof(BwdParams); out[7] = sizeof(PushIdsParams);
  return 0;
}

// ---------------------------------------------------------------------------------------------------
// Allocation-free variant of the backward update (declared in embedding_static.h).
// ---------------------------------------------------------------------------------------------------
#include <mutex>

#include "embedding_static.h"

namespace recml {
namespace emb {
// Scratch for the partial sums of row runs that cross range boundaries: one line of
// RECML_EMB_STATIC_MAX_DIM floats per range of RECML_EMB_STATIC_RANGE (= kRange) sorted occurrences.  It
// lives in the library image, so every GPU that loads the library holds this 1 MiB until the process exits.
static_assert(RECML_EMB_STATIC_RANGE == kRange, "the static scratch is sized in ranges of kRange occurrences");
static __device__ __align__(256) float
    g_static_scratch[(RECML_EMB_STATIC_MAX_OCC / RECML_EMB_STATIC_RANGE) * RECML_EMB_STATIC_MAX_DIM];
}  // namespace emb
}  // namespace recml

static void static_fail(char* err, int err_len, const char* msg) {
  if (err != nullptr && err_len > 0) snprintf(err, static_cast<size_t>(err_len), "%s", msg);
}

extern "C" int recml_emb_bwd_update_static(const BwdParams* p, long long max_occ, int gains, cudaStream_t stream,
                                           char* err, int err_len) {
  if (p == nullptr) { static_fail(err, err_len, "null parameter block"); return -20; }
  if (max_occ > RECML_EMB_STATIC_MAX_OCC) {
    static_fail(err, err_len, "max_occ exceeds RECML_EMB_STATIC_MAX_OCC (262144 occurrences per call)");
    return -21;
  }
  if (p->dloc > RECML_EMB_STATIC_MAX_DIM) {
    static_fail(err, err_len, "embedding dim exceeds RECML_EMB_STATIC_MAX_DIM (128 columns)");
    return -22;
  }
  if (max_occ <= 0) return 0;
  // In host code `g_static_scratch` is only a handle for the symbol; the device address has to be
  // asked for, once per device, with that device current.
  static std::mutex mu;
  static float* dev_addr[64] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    static_fail(err, err_len, "cudaGetDevice failed or device ordinal out of range");
    return -23;
  }
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev_addr[dev] == nullptr) {
      void* addr = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&addr, recml::emb::g_static_scratch);
      if (e != cudaSuccess || addr == nullptr) {
        static_fail(err, err_len, cudaGetErrorString(e));
        return -24;
      }
      dev_addr[dev] = static_cast<float*>(addr);
    }
    scratch = dev_addr[dev];
  }
  // The array keeps whatever the previous call left behind: clear the lines this call can touch.
  const long long chunks = (max_occ + RECML_EMB_STATIC_RANGE - 1) / RECML_EMB_STATIC_RANGE;
  if (cudaMemsetAsync(scratch, 0, static_cast<size_t>(chunks) * p->dloc * sizeof(float), stream) != cudaSuccess) {
    static_fail(err, err_len, "cudaMemsetAsync on the static scratch failed");
    return -25;
  }
  BwdParams q = *p;
  q.scratch = scratch;
  const int rc = recml_emb_bwd_update(&q, max_occ, gains, 0, stream);
  if (rc != 0) static_fail(err, err_len, "kernel launch failed");
  return rc;
}
