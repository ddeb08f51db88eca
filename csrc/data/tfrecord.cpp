// TFRecord files and tf.train.Example / SequenceExample records without TensorFlow: framing with
// masked CRC-32C, a protobuf wire-format walker for the Features message, and a multi-threaded batch
// parser that fills dense int64 / float32 arrays (fixed-length features) or jagged values + row lengths
// (variable-length features).  This is the native input pipeline that replaces the tf.data runtime
// the reference relies on.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <atomic>
#include <cstring>
#include <string>
#include <vector>

#include "host/thread_pool.h"

namespace {

uint32_t g_crc_table[8][256];
bool g_crc_ready = false;

void crc_init() {
  if (g_crc_ready) return;
  for (uint32_t i = 0; i < 256; ++i) {
    uint32_t c = i;
    for (int k = 0; k < 8; ++k) c = (c & 1) ? (c >> 1) ^ 0x82F63B78u : (c >> 1);
    g_crc_table[0][i] = c;
  }
  for (uint32_t i = 0; i < 256; ++i)
    for (int t = 1; t < 8; ++t) g_crc_table[t][i] = (g_crc_table[t - 1][i] >> 8) ^ g_crc_table[0][g_crc_table[t - 1][i] & 0xff];
  g_crc_ready = true;
}

#if defined(__x86_64__)
// The CRC-32C instruction of SSE4.2, eight bytes at a time; used when the CPU has it.
__attribute__((target("sse4.2"))) uint32_t crc32c_hw(const uint8_t* p, size_t n) {
  uint64_t c = 0xffffffffu;
  while (n >= 8) {
    uint64_t v;
    memcpy(&v, p, 8);
    c = __builtin_ia32_crc32di(c, v);
    p += 8;
    n -= 8;
  }
  uint32_t c32 = static_cast<uint32_t>(c);
  while (n--) c32 = __builtin_ia32_crc32qi(c32, *p++);
  return c32 ^ 0xffffffffu;
}
#endif

uint32_t crc32c(const uint8_t* p, size_t n) {
#if defined(__x86_64__)
  static const bool hw = __builtin_cpu_supports("sse4.2");
  if (hw) return crc32c_hw(p, n);
#endif
  crc_init();
  uint32_t c = 0xffffffffu;
  while (n >= 8) {
    uint32_t lo, hi;
    memcpy(&lo, p, 4);
    memcpy(&hi, p + 4, 4);
    lo ^= c;
    c = g_crc_table[7][lo & 0xff] ^ g_crc_table[6][(lo >> 8) & 0xff] ^ g_crc_table[5][(lo >> 16) & 0xff] ^
        g_crc_table[4][lo >> 24] ^ g_crc_table[3][hi & 0xff] ^ g_crc_table[2][(hi >> 8) & 0xff] ^
        g_crc_table[1][(hi >> 16) & 0xff] ^ g_crc_table[0][hi >> 24];
    p += 8;
    n -= 8;
  }
  while (n--) c = g_crc_table[0][(c ^ *p++) & 0xff] ^ (c >> 8);
  return c ^ 0xffffffffu;
}

uint32_t masked(uint32_t crc) { return ((crc >> 15) | (crc << 17)) + 0xa282ead8u; }

struct Slice { const uint8_t* p; size_t n; };

inline bool varint(Slice& s, uint64_t& v) {
  if (s.n > 0 && !(*s.p & 0x80)) {      // keys and most lengths fit one byte
    v = *s.p++;
    --s.n;
    return true;
  }
  v = 0;
  for (int shift = 0; shift < 64 && s.n > 0; shift += 7) {
    const uint8_t b = *s.p++;
    --s.n;
    v |= static_cast<uint64_t>(b & 0x7f) << shift;
    if (!(b & 0x80)) return true;
  }
  return false;
}

inline bool field(Slice& s, uint32_t& num, uint32_t& wire, Slice& payload, uint64_t& scalar) {
  uint64_t key;
  if (!varint(s, key)) return false;
  num = static_cast<uint32_t>(key >> 3);
  wire = static_cast<uint32_t>(key & 7);
  payload = Slice{nullptr, 0};
  scalar = 0;
  if (wire == 0) return varint(s, scalar);
  if (wire == 2) {
    uint64_t len;
    if (!varint(s, len) || len > s.n) return false;
    payload = Slice{s.p, static_cast<size_t>(len)};
    s.p += len;
    s.n -= len;
    return true;
  }
  const size_t w = wire == 1 ? 8 : (wire == 5 ? 4 : 0);
  if (w == 0 || w > s.n) return false;
  payload = Slice{s.p, w};
  s.p += w;
  s.n -= w;
  return true;
}

// Feature { bytes_list = 1; float_list = 2; int64_list = 3 }, each list has `repeated value = 1`.
// Returns false when the bytes do not decode as a Feature to their end (a field that runs past the buffer, an
// unknown wire type, a truncated packed list); what was decoded up to there has been appended.
bool parse_feature(Slice f, std::vector<int64_t>* ints, std::vector<float>* floats, std::vector<std::string>* bytes) {
  uint32_t kind, wire, num;
  Slice pl;
  uint64_t sc;
  bool ok = true;
  while (f.n > 0 && field(f, kind, wire, pl, sc)) {
    if (wire != 2) continue;   // kind: 1 bytes_list, 2 float_list, 3 int64_list
    Slice list = pl;
    while (list.n > 0 && field(list, num, wire, pl, sc)) {
      if (num != 1) continue;
      if (kind == 3 && ints != nullptr) {
        if (wire == 2) {         // packed varints: one terminating byte (high bit clear) per value
          if (pl.n > 0 && (pl.p[pl.n - 1] & 0x80)) ok = false;      // the last value has no end
          size_t n_vals = 0;
          for (size_t i = 0; i < pl.n; ++i) n_vals += !(pl.p[i] & 0x80);
          const size_t at = ints->size();
          ints->resize(at + n_vals);
          int64_t* out = ints->data() + at;
          Slice pk = pl;
          uint64_t v;
          size_t k = 0;
          while (k < n_vals && pk.n > 0 && varint(pk, v)) out[k++] = static_cast<int64_t>(v);
          if (k < n_vals) { ints->resize(at + k); ok = false; }      // truncated payload
        } else if (wire == 0) {
          ints->push_back(static_cast<int64_t>(sc));
        }
      } else if (kind == 2 && floats != nullptr) {
        if (wire == 2) {         // packed floats
          if (pl.n % 4) ok = false;
          const size_t at = floats->size(), n_vals = pl.n / 4;
          floats->resize(at + n_vals);
          if (n_vals) memcpy(floats->data() + at, pl.p, n_vals * 4);
        } else if (wire == 5) {
          float v; memcpy(&v, pl.p, 4); floats->push_back(v);
        }
      } else if (kind == 1 && bytes != nullptr && wire == 2) {
        bytes->emplace_back(reinterpret_cast<const char*>(pl.p), pl.n);
      } else if (wire == 2 && ((kind == 3 && pl.n > 0 && (pl.p[pl.n - 1] & 0x80)) || (kind == 2 && pl.n % 4))) {
        ok = false;              // a list nobody asked for is still checked for a whole number of values
      }
    }
    ok = ok && list.n == 0;
  }
  return ok && f.n == 0;
}

// Structural check of one serialized Example / SequenceExample: every nested message (the feature maps, their
// entries, the features and feature lists) must decode to its last byte.
bool record_ok(Slice example) {
  uint32_t num, wire;
  Slice pl;
  uint64_t sc;
  while (example.n > 0 && field(example, num, wire, pl, sc)) {
    if (wire != 2 || (num != 1 && num != 2)) continue;
    const bool lists = num == 2;
    Slice feats = pl;
    while (feats.n > 0 && field(feats, num, wire, pl, sc)) {
      if (num != 1 || wire != 2) continue;
      Slice entry = pl, val{nullptr, 0};
      while (entry.n > 0 && field(entry, num, wire, pl, sc))
        if (num == 2) val = pl;
      if (entry.n > 0) return false;
      if (!lists) {
        if (!parse_feature(val, nullptr, nullptr, nullptr)) return false;
        continue;
      }
      Slice list = val;
      while (list.n > 0 && field(list, num, wire, pl, sc))
        if (num == 1 && wire == 2 && !parse_feature(pl, nullptr, nullptr, nullptr)) return false;
      if (list.n > 0) return false;
    }
    if (feats.n > 0) return false;
  }
  return example.n == 0;
}

// Example { Features features = 1 }; Features { map<string, Feature> feature = 1 } (map entry: key = 1, value = 2)
bool find_feature(Slice example, const char* name, Slice& out) {
  const size_t name_len = strlen(name);
  uint32_t num, wire;
  Slice pl;
  uint64_t sc;
  while (example.n > 0 && field(example, num, wire, pl, sc)) {
    if (num != 1 || wire != 2) continue;
    Slice feats = pl;
    while (feats.n > 0 && field(feats, num, wire, pl, sc)) {
      if (num != 1 || wire != 2) continue;
      Slice entry = pl, key{nullptr, 0}, val{nullptr, 0};
      while (entry.n > 0 && field(entry, num, wire, pl, sc)) {
        if (num == 1) key = pl;
        if (num == 2) val = pl;
      }
      if (key.n == name_len && memcmp(key.p, name, name_len) == 0) { out = val; return true; }
    }
  }
  return false;
}

// SequenceExample { Features context = 1; FeatureLists feature_lists = 2 };
// FeatureLists { map<string, FeatureList> feature_list = 1 };  FeatureList { repeated Feature feature = 1 }
bool find_feature_list(Slice example, const char* name, Slice& out) {
  const size_t name_len = strlen(name);
  uint32_t num, wire;
  Slice pl;
  uint64_t sc;
  while (example.n > 0 && field(example, num, wire, pl, sc)) {
    if (num != 2 || wire != 2) continue;
    Slice lists = pl;
    while (lists.n > 0 && field(lists, num, wire, pl, sc)) {
      if (num != 1 || wire != 2) continue;
      Slice entry = pl, key{nullptr, 0}, val{nullptr, 0};
      while (entry.n > 0 && field(entry, num, wire, pl, sc)) {
        if (num == 1) key = pl;
        if (num == 2) val = pl;
      }
      if (key.n == name_len && memcmp(key.p, name, name_len) == 0) { out = val; return true; }
    }
  }
  return false;
}

}  // namespace

extern "C" {

uint32_t recml_crc32c(const uint8_t* p, long long n) { return crc32c(p, static_cast<size_t>(n)); }

// Scans a TFRecord file image: fills offsets[i] / lengths[i] of each record payload (up to cap).
// Returns the record count, or -(1+index) of the first record that is corrupt: a frame that runs past the file
// (or a tail too short to hold a frame header) always, a checksum mismatch when verify != 0.
long long recml_tfrecord_index(const uint8_t* data, long long size, long long* offsets, long long* lengths,
                               long long cap, int verify) {
  long long pos = 0, n = 0;
  while (pos + 12 <= size) {
    uint64_t len;
    uint32_t len_crc;
    memcpy(&len, data + pos, 8);
    memcpy(&len_crc, data + pos + 8, 4);
    if (verify && masked(crc32c(data + pos, 8)) != len_crc) return -(1 + n);
    if (len > static_cast<uint64_t>(size) || pos + 12 + static_cast<long long>(len) + 4 > size) return -(1 + n);
    if (verify) {
      uint32_t data_crc;
      memcpy(&data_crc, data + pos + 12 + len, 4);
      if (masked(crc32c(data + pos + 12, len)) != data_crc) return -(1 + n);
    }
    if (n < cap) { offsets[n] = pos + 12; lengths[n] = static_cast<long long>(len); }
    ++n;
    pos += 12 + static_cast<long long>(len) + 4;
  }
  return pos == size ? n : -(1 + n);
}

// Frames one payload as a TFRecord into out (capacity >= len + 16); returns bytes written.
long long recml_tfrecord_frame(const uint8_t* payload, long long len, uint8_t* out) {
  const uint64_t l = static_cast<uint64_t>(len);
  memcpy(out, &l, 8);
  const uint32_t c1 = masked(crc32c(out, 8));
  memcpy(out + 8, &c1, 4);
  memcpy(out + 12, payload, static_cast<size_t>(len));
  const uint32_t c2 = masked(crc32c(payload, static_cast<size_t>(len)));
  memcpy(out + 12 + len, &c2, 4);
  return len + 16;
}

// Index of the first record that does not decode as an Example / SequenceExample (`record_ok`), or -1.
long long recml_validate_examples(const uint8_t* data, const long long* offsets, const long long* lengths,
                                  long long count) {
  std::atomic<long long> first_bad{-1};
  recml::ThreadPool::global().parallel_for(count, [&](long long r0, long long r1, int) {
    for (long long r = r0; r < r1; ++r) {
      if (record_ok(Slice{data + offsets[r], static_cast<size_t>(lengths[r])})) continue;
      long long seen = first_bad.load();
      while ((seen < 0 || r < seen) && !first_bad.compare_exchange_weak(seen, r)) {}
      break;
    }
  }, 64);
  return first_bad.load();
}

// Parses one named feature from `count` serialized Examples in parallel.
//   kind 0: int64, 1: float.   fixed_len > 0: dense output [count, fixed_len] (missing / short values
//   are filled with `default_*`, long ones truncated); fixed_len == 0: only row_lengths are filled on the first
//   pass (values == nullptr) and values are written at the offsets given by `row_starts` on the second.
int recml_parse_examples(const uint8_t* data, const long long* offsets, const long long* lengths, long long count,
                         const char* name, int kind, int fixed_len, long long default_int, float default_float,
                         void* values, long long* row_lengths, const long long* row_starts) {
  int status = 0;
  recml::ThreadPool::global().parallel_for(count, [&](long long r0, long long r1, int) {
    std::vector<int64_t> ints;
    std::vector<float> floats;
    for (long long r = r0; r < r1; ++r) {
      ints.clear();
      floats.clear();
      Slice feat;
      if (find_feature(Slice{data + offsets[r], static_cast<size_t>(lengths[r])}, name, feat))
        parse_feature(feat, kind == 0 ? &ints : nullptr, kind == 1 ? &floats : nullptr, nullptr);
      const long long n = kind == 0 ? static_cast<long long>(ints.size()) : static_cast<long long>(floats.size());
      if (row_lengths != nullptr) row_lengths[r] = n;
      if (values == nullptr) continue;
      if (fixed_len > 0) {
        for (int i = 0; i < fixed_len; ++i) {
          if (kind == 0) static_cast<int64_t*>(values)[r * fixed_len + i] = i < n ? ints[i] : default_int;
          else static_cast<float*>(values)[r * fixed_len + i] = i < n ? floats[i] : default_float;
        }
      } else if (row_starts != nullptr) {
        for (long long i = 0; i < n; ++i) {
          if (kind == 0) static_cast<int64_t*>(values)[row_starts[r] + i] = ints[i];
          else static_cast<float*>(values)[row_starts[r] + i] = floats[i];
        }
      }
    }
  }, 64);
  return status;
}

// Parses one named feature LIST of `count` serialized SequenceExamples: the values of all steps of a
// record are concatenated.  Pass 1 (values == nullptr): row_lengths[r] = number of values, steps[r] =
// number of steps.  Pass 2: values written at row_starts[r].  kind 0: int64, 1: float.
int recml_parse_sequence_examples(const uint8_t* data, const long long* offsets, const long long* lengths,
                                  long long count, const char* name, int kind, void* values, long long* row_lengths,
                                  long long* steps, const long long* row_starts) {
  recml::ThreadPool::global().parallel_for(count, [&](long long r0, long long r1, int) {
    std::vector<int64_t> ints;
    std::vector<float> floats;
    for (long long r = r0; r < r1; ++r) {
      ints.clear();
      floats.clear();
      long long n_steps = 0;
      Slice list;
      if (find_feature_list(Slice{data + offsets[r], static_cast<size_t>(lengths[r])}, name, list)) {
        uint32_t num, wire;
        Slice pl;
        uint64_t sc;
        while (list.n > 0 && field(list, num, wire, pl, sc)) {
          if (num != 1 || wire != 2) continue;
          parse_feature(pl, kind == 0 ? &ints : nullptr, kind == 1 ? &floats : nullptr, nullptr);
          ++n_steps;
        }
      }
      const long long n = kind == 0 ? static_cast<long long>(ints.size()) : static_cast<long long>(floats.size());
      if (row_lengths != nullptr) row_lengths[r] = n;
      if (steps != nullptr) steps[r] = n_steps;
      if (values != nullptr && row_starts != nullptr) {
        for (long long i = 0; i < n; ++i) {
          if (kind == 0) static_cast<int64_t*>(values)[row_starts[r] + i] = ints[i];
          else static_cast<float*>(values)[row_starts[r] + i] = floats[i];
        }
      }
    }
  }, 64);
  return 0;
}

// Decodes a bytes-list feature whose strings are raw little-endian buffers (the `decode_raw` idiom of
// pre-batched Criteo records: one string per sample holding its multi-hot int64 ids).  All strings of
// record r are concatenated into out[r * fixed_bytes ..]; returns the number of records whose total
// length differed from fixed_bytes (those rows are zero-filled past their data).
int recml_parse_raw_bytes(const uint8_t* data, const long long* offsets, const long long* lengths, long long count,
                          const char* name, long long fixed_bytes, uint8_t* out) {
  std::atomic<int> bad{0};
  recml::ThreadPool::global().parallel_for(count, [&](long long r0, long long r1, int) {
    std::vector<std::string> strs;
    for (long long r = r0; r < r1; ++r) {
      strs.clear();
      Slice feat;
      if (find_feature(Slice{data + offsets[r], static_cast<size_t>(lengths[r])}, name, feat))
        parse_feature(feat, nullptr, nullptr, &strs);
      uint8_t* dst = out + r * fixed_bytes;
      long long at = 0;
      for (const std::string& b : strs) {
        const long long n = static_cast<long long>(b.size());
        const long long take = at + n <= fixed_bytes ? n : (fixed_bytes > at ? fixed_bytes - at : 0);
        if (take > 0) memcpy(dst + at, b.data(), static_cast<size_t>(take));
        at += n;
      }
      if (at != fixed_bytes) {
        bad.fetch_add(1);
        if (at < fixed_bytes) memset(dst + at, 0, static_cast<size_t>(fixed_bytes - at));
      }
    }
  }, 8);
  return bad.load();
}

// Pre-batched multi-hot id features (the Criteo records of the reference's loader: feature f of a record is
// a bytes list with one string per sample, each holding multi_hot[f] little-endian int64 ids).  Decodes
// features [0, n_feat) of `count` records into out[r * total + batch * sum(multi_hot[0..f)) + b * multi_hot[f] + j]
// as int32 ids taken modulo vocab[f]: the feature-major value layout the embedding input uses, with no
// intermediate int64 arrays.  One task per (record, feature).  Returns the number of (record, feature)
// pairs whose payload was not exactly batch strings of multi_hot[f] ids (their slots are zero-filled).
int recml_decode_multihot_records(const uint8_t* data, const long long* offsets, const long long* lengths, long long count,
                                  int n_feat, const char* const* names, const int* multi_hot, const long long* vocab,
                                  int batch, int32_t* out) {
  std::vector<long long> start(n_feat + 1, 0);
  for (int f = 0; f < n_feat; ++f) start[f + 1] = start[f] + static_cast<long long>(batch) * multi_hot[f];
  const long long total = start[n_feat];
  std::atomic<int> bad{0};
  recml::ThreadPool::global().parallel_for(count * n_feat, [&](long long t0, long long t1, int) {
    for (long long t = t0; t < t1; ++t) {
      const long long r = t / n_feat;
      const int f = static_cast<int>(t % n_feat);
      const int m = multi_hot[f];
      const long long v = vocab[f] > 0 ? vocab[f] : 1;
      int32_t* dst = out + r * total + start[f];
      long long got = 0;           // samples decoded
      bool ok = true;
      Slice feat;
      if (find_feature(Slice{data + offsets[r], static_cast<size_t>(lengths[r])}, names[f], feat)) {
        uint32_t kind, wire, num;
        Slice pl;
        uint64_t sc;
        while (feat.n > 0 && field(feat, kind, wire, pl, sc)) {
          if (kind != 1 || wire != 2) continue;          // bytes_list
          Slice list = pl;
          while (list.n > 0 && field(list, num, wire, pl, sc)) {
            if (num != 1 || wire != 2) continue;
            if (pl.n != static_cast<size_t>(m) * 8 || got >= batch) { ok = false; continue; }
            for (int j = 0; j < m; ++j) {
              int64_t id;
              memcpy(&id, pl.p + 8 * j, 8);
              long long q = id % v;
              if (q < 0) q += v;                         // numpy's modulo is non-negative
              dst[got * m + j] = static_cast<int32_t>(q);
            }
            ++got;
          }
        }
      }
      if (got != batch || !ok) {
        bad.fetch_add(1);
        if (got < batch) memset(dst + got * m, 0, sizeof(int32_t) * static_cast<size_t>(batch - got) * m);
      }
    }
  }, 1);
  return bad.load();
}

// ---- one pass over every record for many features ---------------------------------------------------
// The per-feature entry point above walks a record's feature map once per requested feature; a batch of
// small Examples with tens of features is parsed an order of magnitude faster by visiting every map entry
// once and routing it to the feature that asked for it.  Records are split into chunks; a chunk writes
// fixed-length features straight into the caller's arrays and collects variable-length values in its own
// buffers, which `recml_parse_multi_fetch` then lays end to end.
struct MultiParse {
  int n_feat = 0;
  long long count = 0, chunk = 0;
  int n_chunks = 0;
  std::vector<int> kind;                               // 0 int64, 1 float
  std::vector<std::vector<std::vector<int64_t>>> ints; // [chunk][feature]
  std::vector<std::vector<std::vector<float>>> floats;
  std::atomic<long long> first_bad{-1};                // lowest index of a record that did not decode to its end
};

void* recml_parse_multi(const uint8_t* data, const long long* offsets, const long long* lengths, long long count,
                        int n_feat, const char* const* names, const int* kinds, const int* fixed_lens,
                        const long long* default_int, const float* default_float, void* const* dense_out,
                        long long* const* row_lengths, const int* sources, long long* const* steps_out) {
  // sources (may be null: all 0): 0 = feature of an Example / context feature of a SequenceExample,
  // 1 = feature list of a SequenceExample (variable length only: the values of all its steps are
  // concatenated and steps_out[f][r] receives the number of steps).
  auto* mp = new MultiParse();
  mp->n_feat = n_feat;
  mp->count = count;
  mp->kind.assign(kinds, kinds + n_feat);
  const int threads = recml::ThreadPool::global().size();
  long long bytes = 0;
  for (long long r = 0; r < count; ++r) bytes += lengths[r];
  // small records are grouped by at least 64 per task; pre-batched records (tens of KB each) go one per task
  const long long min_chunk = count > 0 && bytes / count > 16384 ? 1 : 64;
  mp->chunk = std::max<long long>(min_chunk, (count + threads * 4 - 1) / (threads * 4));
  mp->n_chunks = static_cast<int>((count + mp->chunk - 1) / mp->chunk);
  mp->ints.assign(mp->n_chunks, std::vector<std::vector<int64_t>>(n_feat));
  mp->floats.assign(mp->n_chunks, std::vector<std::vector<float>>(n_feat));
  std::vector<size_t> name_len(n_feat);
  for (int f = 0; f < n_feat; ++f) name_len[f] = strlen(names[f]);
  recml::ThreadPool::global().parallel_for(mp->n_chunks, [&](long long c0, long long c1, int) {
    std::vector<int64_t> iv;
    std::vector<float> fv;
    std::vector<char> seen(n_feat);
    for (long long c = c0; c < c1; ++c) {
      const long long r0 = c * mp->chunk, r1 = std::min(count, r0 + mp->chunk);
      for (int f = 0; f < n_feat; ++f) {     // a first guess of 8 values per record saves most regrowth
        if (fixed_lens[f] > 0) continue;
        if (kinds[f] == 0) mp->ints[c][f].reserve(static_cast<size_t>(r1 - r0) * 8);
        else mp->floats[c][f].reserve(static_cast<size_t>(r1 - r0) * 8);
      }
      for (long long r = r0; r < r1; ++r) {
        std::fill(seen.begin(), seen.end(), 0);
        Slice example{data + offsets[r], static_cast<size_t>(lengths[r])};
        uint32_t num, wire;
        Slice pl;
        uint64_t sc;
        int guess = 0;      // records usually list their features in the same order: try the next one first
        bool ok = true;
        while (example.n > 0 && field(example, num, wire, pl, sc)) {
          if (wire != 2 || (num != 1 && num != 2)) continue;
          const int src = num == 2 ? 1 : 0;
          Slice feats = pl;
          while (feats.n > 0 && field(feats, num, wire, pl, sc)) {
            if (num != 1 || wire != 2) continue;
            Slice entry = pl, key{nullptr, 0}, val{nullptr, 0};
            while (entry.n > 0 && field(entry, num, wire, pl, sc)) {
              if (num == 1) key = pl;
              if (num == 2) val = pl;
            }
            ok = ok && entry.n == 0;
            int f = -1;
            for (int t = 0; t < n_feat; ++t) {
              const int cand = guess + t < n_feat ? guess + t : guess + t - n_feat;
              if (name_len[cand] == key.n && (sources != nullptr ? sources[cand] : 0) == src &&
                  memcmp(key.p, names[cand], key.n) == 0) { f = cand; break; }
            }
            if (f < 0 || seen[f]) continue;
            seen[f] = 1;
            guess = f + 1 < n_feat ? f + 1 : 0;
            if (src == 1) {       // FeatureList { repeated Feature feature = 1 }
              std::vector<int64_t>* di = kinds[f] == 0 ? &mp->ints[c][f] : nullptr;
              std::vector<float>* df = kinds[f] == 0 ? nullptr : &mp->floats[c][f];
              const size_t before = di != nullptr ? di->size() : df->size();
              long long n_steps = 0;
              Slice list = val;
              while (list.n > 0 && field(list, num, wire, pl, sc)) {
                if (num != 1 || wire != 2) continue;
                ok = parse_feature(pl, di, df, nullptr) && ok;
                ++n_steps;
              }
              ok = ok && list.n == 0;
              row_lengths[f][r] = static_cast<long long>((di != nullptr ? di->size() : df->size()) - before);
              if (steps_out != nullptr && steps_out[f] != nullptr) steps_out[f][r] = n_steps;
              continue;
            }
            const int fl = fixed_lens[f];
            if (kinds[f] == 0) {
              std::vector<int64_t>& dst = fl > 0 ? iv : mp->ints[c][f];
              const size_t before = dst.size();
              if (fl > 0) iv.clear();
              ok = parse_feature(val, &dst, nullptr, nullptr) && ok;
              if (fl > 0) {
                int64_t* out = static_cast<int64_t*>(dense_out[f]) + r * fl;
                for (int i = 0; i < fl; ++i) out[i] = i < static_cast<int>(iv.size()) ? iv[i] : default_int[f];
              } else {
                row_lengths[f][r] = static_cast<long long>(dst.size() - before);
              }
            } else {
              std::vector<float>& dst = fl > 0 ? fv : mp->floats[c][f];
              const size_t before = dst.size();
              if (fl > 0) fv.clear();
              ok = parse_feature(val, nullptr, &dst, nullptr) && ok;
              if (fl > 0) {
                float* out = static_cast<float*>(dense_out[f]) + r * fl;
                for (int i = 0; i < fl; ++i) out[i] = i < static_cast<int>(fv.size()) ? fv[i] : default_float[f];
              } else {
                row_lengths[f][r] = static_cast<long long>(dst.size() - before);
              }
            }
          }
          ok = ok && feats.n == 0;
        }
        if (!ok || example.n > 0) {
          long long seen_bad = mp->first_bad.load();
          while ((seen_bad < 0 || r < seen_bad) && !mp->first_bad.compare_exchange_weak(seen_bad, r)) {}
        }
        for (int f = 0; f < n_feat; ++f) {      // features the record does not have
          if (seen[f]) continue;
          const int fl = fixed_lens[f];
          if (fl == 0) {
            row_lengths[f][r] = 0;
            if (steps_out != nullptr && steps_out[f] != nullptr) steps_out[f][r] = 0;
            continue;
          }
          for (int i = 0; i < fl; ++i) {
            if (kinds[f] == 0) static_cast<int64_t*>(dense_out[f])[r * fl + i] = default_int[f];
            else static_cast<float*>(dense_out[f])[r * fl + i] = default_float[f];
          }
        }
      }
    }
  }, 1);
  return mp;
}

// Lowest index of a record that did not decode as an Example / SequenceExample, or -1.
long long recml_parse_multi_first_bad(const void* handle) {
  return static_cast<const MultiParse*>(handle)->first_bad.load();
}

// Total number of values collected for variable-length feature f.
long long recml_parse_multi_size(const void* handle, int f) {
  const auto* mp = static_cast<const MultiParse*>(handle);
  long long n = 0;
  for (int c = 0; c < mp->n_chunks; ++c)
    n += mp->kind[f] == 0 ? static_cast<long long>(mp->ints[c][f].size()) : static_cast<long long>(mp->floats[c][f].size());
  return n;
}

// Copies the values of variable-length feature f, in record order, into out (int64 or float32).
void recml_parse_multi_fetch(const void* handle, int f, void* out) {
  const auto* mp = static_cast<const MultiParse*>(handle);
  std::vector<long long> start(mp->n_chunks + 1, 0);
  for (int c = 0; c < mp->n_chunks; ++c)
    start[c + 1] = start[c] + (mp->kind[f] == 0 ? static_cast<long long>(mp->ints[c][f].size())
                                                : static_cast<long long>(mp->floats[c][f].size()));
  recml::ThreadPool::global().parallel_for(mp->n_chunks, [&](long long c0, long long c1, int) {
    for (long long c = c0; c < c1; ++c) {
      if (mp->kind[f] == 0) {
        const auto& v = mp->ints[c][f];
        if (!v.empty()) memcpy(static_cast<int64_t*>(out) + start[c], v.data(), v.size() * sizeof(int64_t));
      } else {
        const auto& v = mp->floats[c][f];
        if (!v.empty()) memcpy(static_cast<float*>(out) + start[c], v.data(), v.size() * sizeof(float));
      }
    }
  }, 1);
}

void recml_parse_multi_free(void* handle) { delete static_cast<MultiParse*>(handle); }

}  // extern "C"
