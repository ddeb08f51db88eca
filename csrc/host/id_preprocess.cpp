// Host-side id preprocessing: the C++ counterpart of the reference's native input-preprocessing
// module (sample ids -> per-partition CSR with duplicate ids merged, id dropping and per-partition
// statistics), re-targeted at GPU shards.
//
// Two services, both multi-threaded over features / samples:
//   recml_pack_jagged      per-feature id lists -> one KeyedJagged (values / offsets / weights)
//   recml_partition_csr    jagged ids of one table -> ids grouped by owning shard, duplicates of the
//                          same (sample, row) merged by adding their gains, optional dropping beyond a
//                          per-partition cap, and the statistics the embedding planner sizes buffers
//                          with (max ids / max unique ids per partition, drop count).
// Row -> shard follows the MOD layout: shard = (id % shards + rotation) % shards, local row = id / shards.
#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <vector>

#include "host/thread_pool.h"

namespace {

struct Entry {
  int32_t shard, row, sample;
  float gain;
};

// Sorts one shard's entries by (row, sample): LSD radix sort, 11 bits per pass, over only as many bits as
// the largest row and the batch size need (rows and samples are non-negative).
void radix_sort_entries(Entry* lo, Entry* hi, int batch) {
  const size_t n = static_cast<size_t>(hi - lo);
  if (n < 2048) {
    std::sort(lo, hi, [](const Entry& a, const Entry& b) { return a.row != b.row ? a.row < b.row : a.sample < b.sample; });
    return;
  }
  int sample_bits = 1;
  while ((1LL << sample_bits) < batch) ++sample_bits;
  int32_t max_row = 0;
  for (const Entry* p = lo; p < hi; ++p) max_row = std::max(max_row, p->row);
  int row_bits = 1;
  while ((1LL << row_bits) <= max_row) ++row_bits;
  const int total_bits = sample_bits + row_bits;
  auto key = [sample_bits](const Entry& x) {
    return (static_cast<uint64_t>(static_cast<uint32_t>(x.row)) << sample_bits) | static_cast<uint32_t>(x.sample);
  };
  std::vector<Entry> tmp(n);
  Entry* src = lo;
  Entry* dst = tmp.data();
  constexpr int kBits = 11;
  std::vector<size_t> count(1u << kBits);
  for (int shift = 0; shift < total_bits; shift += kBits) {
    std::fill(count.begin(), count.end(), 0);
    for (size_t i = 0; i < n; ++i) ++count[(key(src[i]) >> shift) & ((1u << kBits) - 1)];
    size_t run = 0;
    for (size_t& c : count) { const size_t t = c; c = run; run += t; }
    for (size_t i = 0; i < n; ++i) dst[count[(key(src[i]) >> shift) & ((1u << kBits) - 1)]++] = src[i];
    std::swap(src, dst);
  }
  if (src != lo) std::copy(src, src + n, lo);
}

}  // namespace

extern "C" {

// features[f] points at the ids of feature f (concatenated bags), lengths[f] at its per-sample bag
// sizes (batch entries).  Output buffers are caller-allocated: values[total], offsets[F*batch+1],
// weights_out[total] (may be null, as may weights_in / weights_in[f]).
int recml_pack_jagged(int num_features, int batch, const int64_t* const* features, const int32_t* const* lengths,
                      const float* const* weights_in, int32_t* values, int32_t* offsets, float* weights_out) {
  std::vector<long long> feat_total(num_features + 1, 0);
  for (int f = 0; f < num_features; ++f) {
    long long t = 0;
    for (int b = 0; b < batch; ++b) t += lengths[f][b];
    feat_total[f + 1] = feat_total[f] + t;
  }
  if (feat_total[num_features] > INT32_MAX) return -1;
  recml::ThreadPool::global().parallel_for(num_features, [&](long long f0, long long f1, int) {
    for (long long f = f0; f < f1; ++f) {
      long long pos = feat_total[f];
      for (int b = 0; b < batch; ++b) {
        offsets[f * batch + b] = static_cast<int32_t>(pos);
        pos += lengths[f][b];
      }
      const long long n = feat_total[f + 1] - feat_total[f];
      for (long long i = 0; i < n; ++i) values[feat_total[f] + i] = static_cast<int32_t>(features[f][i]);
      if (weights_out != nullptr) {
        const float* w = (weights_in != nullptr) ? weights_in[f] : nullptr;
        for (long long i = 0; i < n; ++i) weights_out[feat_total[f] + i] = w ? w[i] : 1.0f;
      }
    }
  });
  offsets[static_cast<long long>(num_features) * batch] = static_cast<int32_t>(feat_total[num_features]);
  return 0;
}

// ids[nnz] with offsets[batch+1] (bag b = ids[offsets[b]:offsets[b+1]]), optional gains[nnz].
// Outputs (caller-allocated, capacity nnz): out_rows / out_samples / out_gains sorted by (shard, row, sample);
// shard_ptr[shards+1] delimits each shard's slice; stats[0..2] = max ids per shard, max unique rows
// per shard, dropped ids.  max_ids_per_shard <= 0 disables dropping.  Returns the number of entries kept, -1 for a
// negative id (nothing is written then), -2 for a shard count below 1 or offsets that do not ascend from 0.
long long recml_partition_csr(const int32_t* ids, const int32_t* offsets, const float* gains, int batch, int shards,
                              int rotation, int max_ids_per_shard, int32_t* out_rows, int32_t* out_samples,
                              float* out_gains, int64_t* shard_ptr, int64_t* stats) {
  if (shards < 1 || batch < 0 || offsets[0] != 0) return -2;
  for (int b = 0; b < batch; ++b)
    if (offsets[b + 1] < offsets[b]) return -2;
  const long long nnz = offsets[batch];
  rotation = ((rotation % shards) + shards) % shards;
  std::vector<Entry> e(static_cast<size_t>(nnz));
  std::atomic<int> negative{0};
  recml::ThreadPool::global().parallel_for(batch, [&](long long b0, long long b1, int) {
    for (long long b = b0; b < b1; ++b)
      for (int i = offsets[b]; i < offsets[b + 1]; ++i) {
        const int32_t id = ids[i];
        if (id < 0) { negative.store(1); continue; }
        e[i] = Entry{static_cast<int32_t>((id % shards + rotation) % shards), id / shards, static_cast<int32_t>(b),
                     gains ? gains[i] : 1.0f};
      }
  }, 1024);
  if (negative.load()) return -1;
  // bucket by shard (counting sort), then every shard is sorted by (row, sample), merged and capped on its
  // own thread; the shards' survivors are laid end to end afterwards
  std::vector<long long> start(shards + 1, 0);
  for (long long k = 0; k < nnz; ++k) ++start[e[k].shard + 1];
  for (int s = 0; s < shards; ++s) start[s + 1] += start[s];
  std::vector<Entry> by(static_cast<size_t>(nnz));
  {
    std::vector<long long> at(start.begin(), start.end() - 1);
    for (long long k = 0; k < nnz; ++k) by[at[e[k].shard]++] = e[k];
  }
  std::vector<long long> kept_s(shards, 0), unique_s(shards, 0), dropped_s(shards, 0);
  recml::ThreadPool::global().parallel_for(shards, [&](long long s0, long long s1, int) {
    for (long long s = s0; s < s1; ++s) {
      Entry* lo = by.data() + start[s];
      Entry* hi = by.data() + start[s + 1];
      radix_sort_entries(lo, hi, batch);
      long long in_shard = 0, unique = 0, dropped = 0;
      int32_t last_row = -1;
      Entry* out = lo;
      for (Entry* p = lo; p < hi;) {
        Entry cur = *p++;      // merge duplicates of the same (row, sample)
        while (p < hi && p->row == cur.row && p->sample == cur.sample) cur.gain += (p++)->gain;
        if (max_ids_per_shard > 0 && in_shard >= max_ids_per_shard) { ++dropped; continue; }
        if (cur.row != last_row) { ++unique; last_row = cur.row; }
        *out++ = cur;
        ++in_shard;
      }
      kept_s[s] = in_shard; unique_s[s] = unique; dropped_s[s] = dropped;
    }
  }, 1);
  long long kept = 0, dropped = 0, max_ids = 0, max_unique = 0;
  for (int s = 0; s < shards; ++s) {
    shard_ptr[s] = kept;
    kept += kept_s[s];
    dropped += dropped_s[s];
    max_ids = std::max(max_ids, kept_s[s]);
    max_unique = std::max(max_unique, unique_s[s]);
  }
  recml::ThreadPool::global().parallel_for(shards, [&](long long s0, long long s1, int) {
    for (long long s = s0; s < s1; ++s) {
      const Entry* src = by.data() + start[s];
      const long long base = shard_ptr[s];
      for (long long k = 0; k < kept_s[s]; ++k) {
        out_rows[base + k] = src[k].row;
        out_samples[base + k] = src[k].sample;
        out_gains[base + k] = src[k].gain;
      }
    }
  }, 1);
  shard_ptr[shards] = kept;
  stats[0] = max_ids;
  stats[1] = max_unique;
  stats[2] = dropped;
  return kept;
}

int recml_host_threads() { return recml::ThreadPool::global().size(); }

}  // extern "C"
