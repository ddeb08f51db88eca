// De-duplication of an id list on the device:  ids[n] -> the distinct ids in increasing order, how many there
// are, and for every input position the index of its id among the distinct ones (the "inverse" that expands a
// per-distinct-row result back to the occurrences, or folds per-occurrence gradients onto rows).
//
//   1. (id, position) pairs are sorted by id with the library's radix sort (radix_sort.cu);
//   2. unique_flags_kernel marks the first entry of every run of equal ids and sums the marks per block;
//   3. unique_scan_kernel turns the block sums into exclusive offsets (one block; the list of block sums is short);
//   4. unique_write_kernel numbers the runs (block offset + marks before the entry inside the block), writes
//      every run's id once and every entry's run number at its original position.
//
// The element count is read from device memory, like the sort's, so the caller never synchronises to learn it.
#include <cstdint>

#include "common.cuh"

namespace recml {
namespace idu {

constexpr int kBlock = 1024;
constexpr int kItems = 4;                   // entries per thread
constexpr int kTile = kBlock * kItems;

__device__ __forceinline__ unsigned int count_of(const unsigned int* n_ptr, long long capacity) {
  const unsigned int n = *n_ptr;
  return n > capacity ? static_cast<unsigned int>(capacity) : n;
}

// marks of this thread's entries (bit e: entry e starts a run) and their number
__device__ __forceinline__ unsigned int marks_of(const uint32_t* keys, unsigned int base, unsigned int n, int* cnt) {
  unsigned int m = 0;
  int c = 0;
#pragma unroll
  for (int e = 0; e < kItems; ++e) {
    const unsigned int i = base + e;
    if (i < n && (i == 0 || keys[i] != keys[i - 1])) { m |= 1u << e; ++c; }
  }
  *cnt = c;
  return m;
}

// exclusive prefix of `v` over the block's threads (result for this thread), total in *total for everyone
__device__ __forceinline__ int block_exclusive(int v, int* total) {
  __shared__ int warp_sums[32];
  __shared__ int all;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const int w = warp_sums[lane];
    int wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += t;
    }
    warp_sums[lane] = wi - w;
    if (lane == 31) all = wi;
  }
  __syncthreads();
  *total = all;
  return warp_sums[warp] + incl - v;
}

__global__ void __launch_bounds__(kBlock) unique_flags_kernel(const uint32_t* keys, const unsigned int* n_ptr,
                                                              long long capacity, int* block_sums) {
  const unsigned int n = count_of(n_ptr, capacity);
  const unsigned int base = blockIdx.x * kTile + threadIdx.x * kItems;
  int c = 0, total = 0;
  marks_of(keys, base, n, &c);
  block_exclusive(c, &total);
  if (threadIdx.x == 0) block_sums[blockIdx.x] = total;
}

// block_sums[0 .. blocks) -> exclusive offsets in place; the grand total goes to *n_unique
__global__ void __launch_bounds__(kBlock) unique_scan_kernel(int* block_sums, int blocks, unsigned int* n_unique) {
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int b0 = 0; b0 < blocks; b0 += kBlock) {
    const int i = b0 + threadIdx.x;
    const int v = i < blocks ? block_sums[i] : 0;
    int total = 0;
    const int ex = block_exclusive(v, &total);
    if (i < blocks) block_sums[i] = carry + ex;
    __syncthreads();
    if (threadIdx.x == 0) carry += total;
    __syncthreads();
  }
  if (threadIdx.x == 0) *n_unique = static_cast<unsigned int>(carry);
}

__global__ void __launch_bounds__(kBlock) unique_write_kernel(const uint32_t* keys, const uint32_t* positions,
                                                              const unsigned int* n_ptr, long long capacity,
                                                              const int* block_offsets, uint32_t* unique,
                                                              uint32_t* inverse) {
  const unsigned int n = count_of(n_ptr, capacity);
  const unsigned int base = blockIdx.x * kTile + threadIdx.x * kItems;
  int c = 0, total = 0;
  const unsigned int m = marks_of(keys, base, n, &c);
  int run = block_offsets[blockIdx.x] + block_exclusive(c, &total) - 1;    // run number of the entry before mine
#pragma unroll
  for (int e = 0; e < kItems; ++e) {
    const unsigned int i = base + e;
    if (i >= n) break;
    if ((m >> e) & 1u) {
      ++run;
      unique[run] = keys[i];
    }
    inverse[positions[i]] = static_cast<uint32_t>(run);
  }
}

}  // namespace idu
}  // namespace recml

using namespace recml::idu;

extern "C" long long recml_id_unique_scratch_words(long long capacity) { return (capacity + kTile - 1) / kTile + 4; }

// keys / positions: the SORTED (id, original position) pairs (capacity entries, *n_ptr valid).  unique needs
// room for `capacity` ids, inverse for `capacity` entries; scratch as above; *n_unique receives the count.
extern "C" int recml_id_unique_sorted(const uint32_t* keys, const uint32_t* positions, const unsigned int* n_ptr,
                                      long long capacity, uint32_t* unique, uint32_t* inverse, unsigned int* n_unique,
                                      int* scratch, cudaStream_t stream) {
  if (capacity <= 0) return 0;
  if (capacity > 0x7fffffffLL) return -1;
  const int blocks = static_cast<int>((capacity + kTile - 1) / kTile);
  unique_flags_kernel<<<blocks, kBlock, 0, stream>>>(keys, n_ptr, capacity, scratch);
  unique_scan_kernel<<<1, kBlock, 0, stream>>>(scratch, blocks, n_unique);
  unique_write_kernel<<<blocks, kBlock, 0, stream>>>(keys, positions, n_ptr, capacity, scratch, unique, inverse);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
