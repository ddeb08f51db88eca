// Stable LSD radix sort of (uint32 key, uint32 value) pairs whose COUNT LIVES ON THE DEVICE.
//
// The embedding backward groups the step's (row, gradient-vector) occurrences by row.  The number of
// occurrences is produced by the forward kernel and never read by the host, so every kernel here takes
// a pointer to the count, is launched over the buffer's capacity and lets the tiles beyond the count
// exit at once.  Only the low `key_bits` bits of the keys take part (rows of a table stack need
// 17..28 bits), in passes of at most 9 bits.
//
// One pass = three kernels:
//   count    every block builds the digit histogram of its tile of 4096 keys         -> hist[bin][tile]
//   scan     exclusive prefix sum over hist in (bin-major, tile-minor) order, i.e. the first output
//            position of every (digit, tile) pair (two kernels: sums of 8192-counter parts, then each
//            part scans itself on top of the sum of the parts before it)
//   scatter  every block ranks its tile's keys stably per digit (warp match + per-warp counters, then a
//            scan over the warps) and writes each pair to its final position of the pass
// No kernel here waits on another block.
#include "common.cuh"

namespace recml {
namespace rsort {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kItems = 16;                      // keys per thread
constexpr int kTile = kThreads * kItems;        // 4096 keys per block
constexpr int kMaxBins = 512;

// The producer's counter may run past the buffer's capacity (it counts what it could not store, too).
__device__ __forceinline__ unsigned int count_of(const unsigned int* n_ptr, unsigned int capacity) {
  const unsigned int n = *n_ptr;
  return n < capacity ? n : capacity;
}

// ---- count ----------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) count_kernel(const uint32_t* __restrict__ keys, const unsigned int* n_ptr,
                                                         unsigned int capacity, unsigned int cap_tiles, int shift,
                                                         int bins, unsigned int* __restrict__ hist) {
  __shared__ unsigned int h[kMaxBins];
  const unsigned int n = count_of(n_ptr, capacity);
  const unsigned int tile = blockIdx.x;
  for (int b = threadIdx.x; b < bins; b += kThreads) h[b] = 0;
  __syncthreads();
  const unsigned int base = tile * kTile;
  if (base < n) {
    const uint32_t mask = static_cast<uint32_t>(bins - 1);
#pragma unroll
    for (int i = 0; i < kItems; ++i) {
      const unsigned int idx = base + i * kThreads + threadIdx.x;
      if (idx < n) atomicAdd(&h[(keys[idx] >> shift) & mask], 1u);
    }
  }
  __syncthreads();
  // tiles beyond the count still publish zeros: the scan covers the whole capacity
  for (int b = threadIdx.x; b < bins; b += kThreads) hist[static_cast<size_t>(b) * cap_tiles + tile] = h[b];
}

// ---- scan: exclusive prefix sum over `total` counters, two kernels, no waiting ---------------------
constexpr int kScanItems = 8;
constexpr int kScanPart = 1024 * kScanItems;

__device__ __forceinline__ unsigned int block_sum_1024(unsigned int x, unsigned int* warp_sums) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  if (lane == 0) warp_sums[warp] = x;
  __syncthreads();
  unsigned int t = warp_sums[lane];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  __syncthreads();
  return t;
}

__global__ void __launch_bounds__(1024) scan_partials_kernel(const unsigned int* __restrict__ data, unsigned int total,
                                                             unsigned int* __restrict__ partial) {
  __shared__ unsigned int warp_sums[32];
  const unsigned int base = blockIdx.x * kScanPart + threadIdx.x * kScanItems;
  unsigned int sum = 0;
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) sum += base + i < total ? data[base + i] : 0u;
  sum = block_sum_1024(sum, warp_sums);
  if (threadIdx.x == 0) partial[blockIdx.x] = sum;
}

__global__ void __launch_bounds__(1024) scan_apply_kernel(unsigned int* __restrict__ data, unsigned int total,
                                                          const unsigned int* __restrict__ partial) {
  __shared__ unsigned int warp_sums[32];
  __shared__ unsigned int warp_incl[32];
  // carry = sum of the parts before this one (a few hundred values at most)
  unsigned int c = 0;
  for (unsigned int i = threadIdx.x; i < blockIdx.x; i += 1024) c += partial[i];
  const unsigned int carry = block_sum_1024(c, warp_sums);
  const unsigned int base = blockIdx.x * kScanPart + threadIdx.x * kScanItems;
  unsigned int v[kScanItems];
  unsigned int sum = 0;
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    v[i] = base + i < total ? data[base + i] : 0u;
    sum += v[i];
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned int incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_incl[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    unsigned int w = warp_incl[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned int t = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += t;
    }
    warp_incl[lane] = w;        // inclusive over warps
  }
  __syncthreads();
  unsigned int excl = carry + incl - sum + (warp > 0 ? warp_incl[warp - 1] : 0u);
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    if (base + i < total) data[base + i] = excl;
    excl += v[i];
  }
}

// ---- scatter ---------------------------------------------------------------------------------------
// Keys are taken warp-striped: warp w, round i, lane l reads index base + (w*kItems + i)*32 + l, so
// "earlier in the tile" means (earlier warp) or (same warp, earlier round) or (same round, lower lane),
// which is the order the ranks below respect.
__global__ void __launch_bounds__(kThreads) scatter_kernel(const uint32_t* __restrict__ keys_in,
                                                           const uint32_t* __restrict__ vals_in,
                                                           uint32_t* __restrict__ keys_out,
                                                           uint32_t* __restrict__ vals_out, const unsigned int* n_ptr,
                                                           unsigned int capacity, unsigned int cap_tiles, int shift,
                                                           int bins, const unsigned int* __restrict__ offsets) {
  // per-warp running digit counters, then warp offsets: at most 4096 keys per tile, so 16 bits do, and the
  // block's 10 KB fit beside a GEMM CTA that owns most of the SM's shared memory
  __shared__ unsigned short cnt[kWarps][kMaxBins];
  __shared__ unsigned int gbase[kMaxBins];           // first output position of (digit, this tile)
  const unsigned int n = count_of(n_ptr, capacity);
  const unsigned int tile = blockIdx.x;
  const unsigned int base = tile * kTile;
  if (base >= n) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int b = threadIdx.x; b < bins * kWarps; b += kThreads) (&cnt[0][0])[(b / bins) * kMaxBins + (b % bins)] = 0;
  for (int b = threadIdx.x; b < bins; b += kThreads) gbase[b] = offsets[static_cast<size_t>(b) * cap_tiles + tile];
  __syncthreads();
  const uint32_t mask = static_cast<uint32_t>(bins - 1);
  uint32_t key[kItems], val[kItems];
  unsigned int rank[kItems];
  const unsigned int lt = (1u << lane) - 1u;
#pragma unroll
  for (int i = 0; i < kItems; ++i) {
    const unsigned int idx = base + (warp * kItems + i) * 32 + lane;
    const bool on = idx < n;
    key[i] = on ? keys_in[idx] : 0xffffffffu;
    val[i] = on ? vals_in[idx] : 0u;
    const uint32_t d = (key[i] >> shift) & mask;
    // lanes holding the same digit (inactive lanes form their own group through bit 31 of the match key)
    const unsigned int peers = __match_any_sync(0xffffffffu, on ? d : 0x80000000u);
    const int leader = __ffs(peers) - 1;
    unsigned int start = 0;
    if (on && lane == leader) {
      start = cnt[warp][d];
      cnt[warp][d] = static_cast<unsigned short>(start + __popc(peers));
    }
    start = __shfl_sync(0xffffffffu, start, leader);
    rank[i] = start + __popc(peers & lt);
    __syncwarp();
  }
  __syncthreads();
  // exclusive scan over the warps for every digit: cnt[w][d] becomes the number of keys with digit d in warps < w
  for (int b = threadIdx.x; b < bins; b += kThreads) {
    unsigned int run = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const unsigned int c = cnt[w][b];
      cnt[w][b] = static_cast<unsigned short>(run);
      run += c;
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < kItems; ++i) {
    const unsigned int idx = base + (warp * kItems + i) * 32 + lane;
    if (idx < n) {
      const uint32_t d = (key[i] >> shift) & mask;
      const unsigned int pos = gbase[d] + cnt[warp][d] + rank[i];
      keys_out[pos] = key[i];
      vals_out[pos] = val[i];
    }
  }
}

}  // namespace rsort
}  // namespace recml

using namespace recml::rsort;

// Scratch words needed for `capacity` pairs: histogram [512 bins][tiles] + one partial sum per scan part.
extern "C" long long recml_radix_sort_scratch_words(long long capacity) {
  const long long tiles = (capacity + kTile - 1) / kTile;
  return tiles * kMaxBins + (tiles * kMaxBins + kScanPart - 1) / kScanPart + 4;
}

// Sorts the first *n_ptr pairs (n <= capacity) by the low `key_bits` bits of the key, stably.  The
// result is left in (keys_a, vals_a) when the return value is 0 and in (keys_b, vals_b) when it is 1;
// negative = bad argument / launch failure.  `scratch` (see above) needs no initialisation.
extern "C" int recml_radix_sort_pairs(uint32_t* keys_a, uint32_t* vals_a, uint32_t* keys_b, uint32_t* vals_b,
                                      const unsigned int* n_ptr, long long capacity, int key_bits,
                                      unsigned int* scratch, int* status, cudaStream_t stream) {
  if (capacity <= 0) return 0;
  if (key_bits < 1 || key_bits > 32 || capacity > 0x7fffffffLL) return -1;
  const unsigned int tiles = static_cast<unsigned int>((capacity + kTile - 1) / kTile);
  const int passes = (key_bits + 8) / 9;
  unsigned int* hist = scratch;
  unsigned int* partial = scratch + static_cast<size_t>(tiles) * kMaxBins;
  uint32_t *ki = keys_a, *vi = vals_a, *ko = keys_b, *vo = vals_b;
  int shift = 0;
  static bool configured = false;
  if (!configured) {
    recml::prefer_max_shared_carveout(count_kernel);
    recml::prefer_max_shared_carveout(scan_partials_kernel);
    recml::prefer_max_shared_carveout(scan_apply_kernel);
    recml::prefer_max_shared_carveout(scatter_kernel);
    configured = true;
  }
  for (int p = 0; p < passes; ++p) {
    // spread the bits evenly over the passes (e.g. 25 bits -> 9, 8, 8)
    const int bits = (key_bits - shift + (passes - p) - 1) / (passes - p);
    const int bins = 1 << bits;
    const unsigned int total = static_cast<unsigned int>(bins) * tiles;
    const unsigned int capu = static_cast<unsigned int>(capacity);
    count_kernel<<<tiles, kThreads, 0, stream>>>(ki, n_ptr, capu, tiles, shift, bins, hist);
    const unsigned int parts = (total + kScanPart - 1) / kScanPart;
    scan_partials_kernel<<<parts, 1024, 0, stream>>>(hist, total, partial);
    scan_apply_kernel<<<parts, 1024, 0, stream>>>(hist, total, partial);
    scatter_kernel<<<tiles, kThreads, 0, stream>>>(ki, vi, ko, vo, n_ptr, capu, tiles, shift, bins, hist);
    uint32_t* t = ki; ki = ko; ko = t;
    t = vi; vi = vo; vo = t;
    shift += bits;
  }
  if (cudaGetLastError() != cudaSuccess) return -2;
  return ki == keys_a ? 0 : 1;
}

extern "C" int recml_radix_sort_passes(int key_bits) { return (key_bits + 8) / 9; }
