// Reader and writer for the OCDBT key-value store layout that the reference's checkpoint manager uses by
// default (a manifest file `manifest.ocdbt`, data files under `d/`, and per-process stores under
// `ocdbt.process_<n>/`): a B+tree of (key -> inline value | reference into a data file) whose nodes and
// manifest share one envelope.  Written from the public description of the format; it has not been checked
// against a file produced by the reference's own stack, which cannot be installed here.
//
// Envelope of every file or node:   magic (uint32, big endian) | length (uint64, little endian, whole
// envelope) | body | CRC-32C (uint32 LE) of everything before it.
//   manifest   magic 0x0cdb3a2a   body = version(varint 0) config version-tree
//   B+tree node magic 0x0cdb20de   body = version(varint 0) compression(varint: 0 none, 1 zstd) payload
// config       = uuid[16] manifest_kind(varint) max_inline_value_bytes(varint) max_decoded_node_bytes(varint)
//                version_tree_arity_log2(u8) compression_method(varint) [zstd level (int32 LE)]
// version tree = data-file-table n_versions(varint) then column-wise: generation_number (delta varints)
//                root_height(u8) root file(varint) offset(varint) length(varint) num_keys(varint)
//                num_tree_bytes(varint) num_indirect_value_bytes(varint) commit_time(uint64 LE);
//                then n_version_nodes(varint) = 0 here
// data-file-table = n(varint) prefix_len[1..n) suffix_len[0..n) base_path_len[0..n) suffix bytes, where the
//                   string compressed is base_path + relative_path
// node payload = height(u8) data-file-table n(varint) key_prefix_len[1..n) key_suffix_len[0..n)
//                [interior: subtree_common_prefix_len[0..n)] key suffix bytes, then
//                leaf:     value_len[0..n) value_kind[0..n) (0 inline, 1 in a data file)
//                          file[k] offset[k] for the out-of-line ones, inline bytes
//                interior: file[0..n) offset[0..n) length[0..n) num_indirect_value_bytes[0..n)
//                          num_tree_bytes[0..n) num_keys[0..n)
#include <dlfcn.h>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "host/thread_pool.h"

extern "C" uint32_t recml_crc32c(const uint8_t* p, long long n);

namespace {

constexpr uint32_t kManifestMagic = 0x0cdb3a2a;
constexpr uint32_t kNodeMagic = 0x0cdb20de;

struct Zstd {
  size_t (*compress)(void*, size_t, const void*, size_t, int) = nullptr;
  size_t (*decompress)(void*, size_t, const void*, size_t) = nullptr;
  size_t (*bound)(size_t) = nullptr;
  unsigned long long (*content_size)(const void*, size_t) = nullptr;
  unsigned (*is_error)(size_t) = nullptr;
  bool ok = false;
};

const Zstd& zstd() {
  static Zstd z;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen("libzstd.so.1", RTLD_NOW);
    if (h == nullptr) h = dlopen("libzstd.so", RTLD_NOW);
    if (h == nullptr) return;
    z.compress = reinterpret_cast<decltype(z.compress)>(dlsym(h, "ZSTD_compress"));
    z.decompress = reinterpret_cast<decltype(z.decompress)>(dlsym(h, "ZSTD_decompress"));
    z.bound = reinterpret_cast<decltype(z.bound)>(dlsym(h, "ZSTD_compressBound"));
    z.content_size = reinterpret_cast<decltype(z.content_size)>(dlsym(h, "ZSTD_getFrameContentSize"));
    z.is_error = reinterpret_cast<decltype(z.is_error)>(dlsym(h, "ZSTD_isError"));
    z.ok = z.compress && z.decompress && z.bound && z.content_size && z.is_error;
  });
  return z;
}

// ---- byte-level helpers ------------------------------------------------------------------------
struct Writer {
  std::string b;
  void u8(uint8_t v) { b.push_back(static_cast<char>(v)); }
  void varint(uint64_t v) {
    while (v >= 0x80) { u8(static_cast<uint8_t>(v) | 0x80); v >>= 7; }
    u8(static_cast<uint8_t>(v));
  }
  void u32be(uint32_t v) { for (int i = 3; i >= 0; --i) u8(static_cast<uint8_t>(v >> (8 * i))); }
  void u32le(uint32_t v) { for (int i = 0; i < 4; ++i) u8(static_cast<uint8_t>(v >> (8 * i))); }
  void u64le(uint64_t v) { for (int i = 0; i < 8; ++i) u8(static_cast<uint8_t>(v >> (8 * i))); }
  void bytes(const std::string& s) { b.append(s); }
};

struct Reader {
  const uint8_t* p;
  size_t n, at = 0;
  bool bad = false;
  uint8_t u8() { if (at >= n) { bad = true; return 0; } return p[at++]; }
  uint64_t varint() {
    uint64_t v = 0;
    for (int shift = 0; shift < 64; shift += 7) {
      const uint8_t c = u8();
      v |= static_cast<uint64_t>(c & 0x7f) << shift;
      if (!(c & 0x80)) return v;
    }
    bad = true;
    return v;
  }
  uint32_t u32be() { uint32_t v = 0; for (int i = 0; i < 4; ++i) v = (v << 8) | u8(); return v; }
  uint32_t u32le() { uint32_t v = 0; for (int i = 0; i < 4; ++i) v |= static_cast<uint32_t>(u8()) << (8 * i); return v; }
  uint64_t u64le() { uint64_t v = 0; for (int i = 0; i < 8; ++i) v |= static_cast<uint64_t>(u8()) << (8 * i); return v; }
  std::string bytes(size_t k) {
    if (at + k > n) { bad = true; return std::string(); }
    std::string s(reinterpret_cast<const char*>(p + at), k);
    at += k;
    return s;
  }
};

std::string envelope(uint32_t magic, const std::string& body) {
  Writer w;
  w.u32be(magic);
  w.u64le(4 + 8 + body.size() + 4);
  w.bytes(body);
  w.u32le(recml_crc32c(reinterpret_cast<const uint8_t*>(w.b.data()), static_cast<long long>(w.b.size())));
  return w.b;
}

// Checks magic / length / checksum and returns the body, or false.
bool open_envelope(const uint8_t* data, size_t n, uint32_t magic, std::string* body) {
  if (n < 16) return false;
  Reader r{data, n};
  if (r.u32be() != magic) return false;
  const uint64_t len = r.u64le();
  if (len != n) return false;
  uint32_t crc = 0;
  for (int i = 0; i < 4; ++i) crc |= static_cast<uint32_t>(data[n - 4 + i]) << (8 * i);
  if (crc != recml_crc32c(data, static_cast<long long>(n - 4))) return false;
  body->assign(reinterpret_cast<const char*>(data + 12), n - 16);
  return true;
}

struct DataFile { std::string base, rel; std::string full() const { return base + rel; } };

void write_file_table(Writer& w, const std::vector<DataFile>& files) {
  w.varint(files.size());
  std::vector<size_t> prefix(files.size(), 0);
  for (size_t i = 1; i < files.size(); ++i) {
    const std::string a = files[i - 1].full(), b = files[i].full();
    size_t k = 0;
    while (k < a.size() && k < b.size() && a[k] == b[k]) ++k;
    prefix[i] = k;
    w.varint(k);
  }
  for (size_t i = 0; i < files.size(); ++i) w.varint(files[i].full().size() - prefix[i]);
  for (const auto& f : files) w.varint(f.base.size());
  for (size_t i = 0; i < files.size(); ++i) w.bytes(files[i].full().substr(prefix[i]));
}

bool read_file_table(Reader& r, std::vector<DataFile>* files) {
  const uint64_t n = r.varint();
  if (r.bad || n > (1u << 20)) return false;
  std::vector<uint64_t> prefix(n, 0), suffix(n), base(n);
  for (uint64_t i = 1; i < n; ++i) prefix[i] = r.varint();
  for (uint64_t i = 0; i < n; ++i) suffix[i] = r.varint();
  for (uint64_t i = 0; i < n; ++i) base[i] = r.varint();
  std::string prev;
  files->clear();
  for (uint64_t i = 0; i < n; ++i) {
    if (prefix[i] > prev.size()) return false;
    std::string full = prev.substr(0, prefix[i]) + r.bytes(suffix[i]);
    if (r.bad || base[i] > full.size()) return false;
    files->push_back({full.substr(0, base[i]), full.substr(base[i])});
    prev = full;
  }
  return !r.bad;
}

struct Ref { uint64_t file = 0, offset = 0, length = 0; };
struct Entry {
  std::string key;
  bool inline_value = true;
  std::string value;     // the bytes, when the writer owns them (always so for inline values)
  const uint8_t* ext = nullptr;   // the bytes, when the caller keeps them alive until the commit
  uint64_t ext_len = 0;
  uint64_t size() const { return ext != nullptr ? ext_len : value.size(); }
  Ref ref;               // out-of-line location (length = value length)
};

constexpr long long kIoSegment = 16 << 20;     // large values are read and written in pieces of this size

// pread / pwrite of [off, off + len) of an open file in segments by all host threads.
bool parallel_io(int fd, uint8_t* rbuf, const uint8_t* wbuf, uint64_t off, uint64_t len) {
  const long long segs = static_cast<long long>((len + kIoSegment - 1) / kIoSegment);
  std::atomic<bool> ok{true};
  recml::ThreadPool::global().parallel_for(segs, [&](long long s0, long long s1, int) {
    for (long long sgm = s0; sgm < s1; ++sgm) {
      uint64_t at = static_cast<uint64_t>(sgm) * kIoSegment;
      const uint64_t end = std::min<uint64_t>(len, at + kIoSegment);
      while (at < end) {
        const ssize_t r = rbuf != nullptr ? ::pread(fd, rbuf + at, end - at, static_cast<off_t>(off + at))
                                          : ::pwrite(fd, wbuf + at, end - at, static_cast<off_t>(off + at));
        if (r <= 0) { ok.store(false); return; }
        at += static_cast<uint64_t>(r);
      }
    }
  }, 1);
  return ok.load();
}

std::string encode_node_payload(const Writer& payload, bool compress) {
  Writer body;
  body.varint(0);
  const Zstd& z = zstd();
  if (compress && z.ok) {
    std::string out(z.bound(payload.b.size()), '\0');
    const size_t k = z.compress(&out[0], out.size(), payload.b.data(), payload.b.size(), 1);
    if (!z.is_error(k)) {
      out.resize(k);
      body.varint(1);
      body.bytes(out);
      return envelope(kNodeMagic, body.b);
    }
  }
  body.varint(0);
  body.bytes(payload.b);
  return envelope(kNodeMagic, body.b);
}

std::string encode_leaf(const std::vector<Entry>& es, const std::vector<DataFile>& files, bool compress) {
  Writer w;
  w.u8(0);
  write_file_table(w, files);
  w.varint(es.size());
  std::vector<size_t> prefix(es.size(), 0);
  for (size_t i = 1; i < es.size(); ++i) {
    const std::string &a = es[i - 1].key, &b = es[i].key;
    size_t k = 0;
    while (k < a.size() && k < b.size() && a[k] == b[k]) ++k;
    prefix[i] = k;
    w.varint(k);
  }
  for (size_t i = 0; i < es.size(); ++i) w.varint(es[i].key.size() - prefix[i]);
  for (size_t i = 0; i < es.size(); ++i) w.bytes(es[i].key.substr(prefix[i]));
  for (const auto& e : es) w.varint(e.inline_value ? e.value.size() : e.ref.length);
  for (const auto& e : es) w.u8(e.inline_value ? 0 : 1);
  for (const auto& e : es) if (!e.inline_value) { w.varint(e.ref.file); w.varint(e.ref.offset); }
  for (const auto& e : es) if (e.inline_value) w.bytes(e.value);
  return encode_node_payload(w, compress);
}

struct Child { std::string first_key; Ref ref; uint64_t num_keys = 0, tree_bytes = 0, indirect_bytes = 0; };

std::string encode_interior(int height, const std::vector<Child>& cs, const std::vector<DataFile>& files, bool compress) {
  Writer w;
  w.u8(static_cast<uint8_t>(height));
  write_file_table(w, files);
  w.varint(cs.size());
  std::vector<size_t> prefix(cs.size(), 0);
  for (size_t i = 1; i < cs.size(); ++i) {
    const std::string &a = cs[i - 1].first_key, &b = cs[i].first_key;
    size_t k = 0;
    while (k < a.size() && k < b.size() && a[k] == b[k]) ++k;
    prefix[i] = k;
    w.varint(k);
  }
  for (size_t i = 0; i < cs.size(); ++i) w.varint(cs[i].first_key.size() - prefix[i]);
  for (size_t i = 0; i < cs.size(); ++i) w.varint(0);      // no common prefix stripped from the subtrees' keys
  for (size_t i = 0; i < cs.size(); ++i) w.bytes(cs[i].first_key.substr(prefix[i]));
  for (const auto& c : cs) w.varint(c.ref.file);
  for (const auto& c : cs) w.varint(c.ref.offset);
  for (const auto& c : cs) w.varint(c.ref.length);
  for (const auto& c : cs) w.varint(c.indirect_bytes);
  for (const auto& c : cs) w.varint(c.tree_bytes);
  for (const auto& c : cs) w.varint(c.num_keys);
  return encode_node_payload(w, compress);
}

bool read_whole(const std::string& path, std::string* out) {
  FILE* f = fopen(path.c_str(), "rb");
  if (f == nullptr) return false;
  fseek(f, 0, SEEK_END);
  const long n = ftell(f);
  fseek(f, 0, SEEK_SET);
  out->resize(static_cast<size_t>(n));
  const size_t got = n > 0 ? fread(&(*out)[0], 1, static_cast<size_t>(n), f) : 0;
  fclose(f);
  return got == static_cast<size_t>(n);
}

bool read_range(const std::string& path, uint64_t off, uint64_t len, std::string* out) {
  FILE* f = fopen(path.c_str(), "rb");
  if (f == nullptr) return false;
  out->resize(len);
  bool ok = fseek(f, static_cast<long>(off), SEEK_SET) == 0;
  ok = ok && (len == 0 || fread(&(*out)[0], 1, len, f) == len);
  fclose(f);
  return ok;
}

// ---- an opened store: every key with where its value lives ---------------------------------------
struct Located { bool inline_value; std::string value; std::string path; uint64_t offset, length; };

struct Store {
  std::string root;
  std::map<std::string, Located> keys;
  std::string error;
  std::vector<std::string> order;

  bool walk(const std::string& dir, const std::string& node_raw, const std::string& key_prefix, int depth) {
    if (depth > 16) { error = "tree too deep"; return false; }
    std::string body;
    if (!open_envelope(reinterpret_cast<const uint8_t*>(node_raw.data()), node_raw.size(), kNodeMagic, &body)) {
      error = "bad B+tree node envelope (magic, length or checksum)";
      return false;
    }
    Reader hb{reinterpret_cast<const uint8_t*>(body.data()), body.size()};
    if (hb.varint() != 0) { error = "unknown node version"; return false; }
    const uint64_t comp = hb.varint();
    std::string payload;
    if (comp == 0) {
      payload = body.substr(hb.at);
    } else if (comp == 1) {
      const Zstd& z = zstd();
      if (!z.ok) { error = "node is zstd-compressed and libzstd is not available"; return false; }
      const unsigned long long raw_size = z.content_size(body.data() + hb.at, body.size() - hb.at);
      if (raw_size > (1ull << 32)) { error = "bad zstd frame"; return false; }
      payload.resize(raw_size);
      const size_t k = z.decompress(&payload[0], payload.size(), body.data() + hb.at, body.size() - hb.at);
      if (z.is_error(k) || k != raw_size) { error = "zstd decompression failed"; return false; }
    } else {
      error = "unknown node compression";
      return false;
    }
    Reader r{reinterpret_cast<const uint8_t*>(payload.data()), payload.size()};
    const int height = r.u8();
    std::vector<DataFile> files;
    if (!read_file_table(r, &files)) { error = "bad data file table"; return false; }
    const uint64_t n = r.varint();
    if (r.bad || n > (1u << 24)) { error = "bad entry count"; return false; }
    std::vector<uint64_t> prefix(n, 0), suffix(n), common(n, 0);
    for (uint64_t i = 1; i < n; ++i) prefix[i] = r.varint();
    for (uint64_t i = 0; i < n; ++i) suffix[i] = r.varint();
    if (height > 0) for (uint64_t i = 0; i < n; ++i) common[i] = r.varint();
    std::vector<std::string> ks(n);
    std::string prev;
    for (uint64_t i = 0; i < n; ++i) {
      if (prefix[i] > prev.size()) { error = "bad key prefix"; return false; }
      ks[i] = prev.substr(0, prefix[i]) + r.bytes(suffix[i]);
      prev = ks[i];
    }
    if (r.bad) { error = "truncated node"; return false; }
    auto file_path = [&](uint64_t id) { return id < files.size() ? dir + "/" + files[id].full() : std::string(); };
    if (height == 0) {
      std::vector<uint64_t> vlen(n);
      std::vector<uint8_t> kind(n);
      for (uint64_t i = 0; i < n; ++i) vlen[i] = r.varint();
      for (uint64_t i = 0; i < n; ++i) kind[i] = r.u8();
      std::vector<Ref> refs(n);
      for (uint64_t i = 0; i < n; ++i) if (kind[i] == 1) { refs[i].file = r.varint(); refs[i].offset = r.varint(); }
      for (uint64_t i = 0; i < n; ++i) {
        Located loc{kind[i] == 0, std::string(), std::string(), 0, vlen[i]};
        if (kind[i] == 0) {
          loc.value = r.bytes(vlen[i]);
        } else {
          loc.path = file_path(refs[i].file);
          loc.offset = refs[i].offset;
          if (loc.path.empty()) { error = "value refers to an unknown data file"; return false; }
        }
        const std::string full = key_prefix + ks[i];
        if (keys.find(full) == keys.end()) order.push_back(full);
        keys[full] = std::move(loc);
      }
      if (r.bad) { error = "truncated leaf"; return false; }
      return true;
    }
    std::vector<Ref> refs(n);
    for (uint64_t i = 0; i < n; ++i) refs[i].file = r.varint();
    for (uint64_t i = 0; i < n; ++i) refs[i].offset = r.varint();
    for (uint64_t i = 0; i < n; ++i) refs[i].length = r.varint();
    for (int col = 0; col < 3; ++col) for (uint64_t i = 0; i < n; ++i) r.varint();   // statistics
    if (r.bad) { error = "truncated interior node"; return false; }
    for (uint64_t i = 0; i < n; ++i) {
      std::string child;
      const std::string path = file_path(refs[i].file);
      if (path.empty() || !read_range(path, refs[i].offset, refs[i].length, &child)) {
        error = "cannot read child node from " + path;
        return false;
      }
      if (common[i] > ks[i].size()) { error = "bad subtree prefix"; return false; }
      if (!walk(dir, child, key_prefix + ks[i].substr(0, common[i]), depth + 1)) return false;
    }
    return true;
  }

  // Reads `dir`/manifest.ocdbt (latest version) and adds its keys, prefixed with key_root.
  bool load(const std::string& dir) {
    std::string raw, body;
    if (!read_whole(dir + "/manifest.ocdbt", &raw)) { error = "cannot read " + dir + "/manifest.ocdbt"; return false; }
    if (!open_envelope(reinterpret_cast<const uint8_t*>(raw.data()), raw.size(), kManifestMagic, &body)) {
      error = "bad manifest envelope (magic, length or checksum)";
      return false;
    }
    Reader r{reinterpret_cast<const uint8_t*>(body.data()), body.size()};
    if (r.varint() != 0) { error = "unknown manifest version"; return false; }
    r.bytes(16);                       // uuid
    r.varint();                        // manifest kind
    r.varint(); r.varint();            // max inline value bytes, max decoded node bytes
    r.u8();                            // version tree arity
    if (r.varint() == 1) r.u32le();    // compression method (+ zstd level)
    std::vector<DataFile> files;
    if (!read_file_table(r, &files)) { error = "bad manifest data file table"; return false; }
    const uint64_t nv = r.varint();
    if (r.bad || nv == 0 || nv > (1u << 20)) { error = "manifest holds no version"; return false; }
    std::vector<uint64_t> gen(nv), file(nv), off(nv), len(nv);
    std::vector<uint8_t> height(nv);
    uint64_t g = 0;
    for (uint64_t i = 0; i < nv; ++i) { g += r.varint(); gen[i] = g; }
    for (uint64_t i = 0; i < nv; ++i) height[i] = r.u8();
    for (uint64_t i = 0; i < nv; ++i) file[i] = r.varint();
    for (uint64_t i = 0; i < nv; ++i) off[i] = r.varint();
    for (uint64_t i = 0; i < nv; ++i) len[i] = r.varint();
    for (int col = 0; col < 3; ++col) for (uint64_t i = 0; i < nv; ++i) r.varint();
    for (uint64_t i = 0; i < nv; ++i) r.u64le();
    if (r.bad) { error = "truncated manifest"; return false; }
    const uint64_t last = nv - 1;     // versions are stored in increasing generation order
    if (len[last] == 0) return true;  // an empty store
    if (file[last] >= files.size()) { error = "root refers to an unknown data file"; return false; }
    std::string node;
    if (!read_range(dir + "/" + files[file[last]].full(), off[last], len[last], &node)) {
      error = "cannot read the root node";
      return false;
    }
    return walk(dir, node, std::string(), 0);
  }
};

struct PendingStore {
  std::string dir;
  std::vector<Entry> entries;     // key + bytes, all kept until commit
  long long inline_limit = 100;
};

void mkdirs(const std::string& path) {
  for (size_t i = 1; i <= path.size(); ++i)
    if (i == path.size() || path[i] == '/') mkdir(path.substr(0, i).c_str(), 0777);
}

}  // namespace

extern "C" {

// ---- reading ----------------------------------------------------------------------------------------
// Opens the store rooted at `dir` (its manifest and, when present, the per-process stores
// `ocdbt.process_<n>` beside it).  Returns a handle, or null with a message in err.
void* recml_ocdbt_open(const char* dir, char* err, int err_len) {
  auto s = std::make_unique<Store>();
  s->root = dir;
  bool any = false, ok = true;
  struct stat st;
  if (stat((s->root + "/manifest.ocdbt").c_str(), &st) == 0) { any = true; ok = s->load(s->root); }
  for (int proc = 0; ok && proc < 4096; ++proc) {
    const std::string sub = s->root + "/ocdbt.process_" + std::to_string(proc);
    if (stat((sub + "/manifest.ocdbt").c_str(), &st) != 0) {
      if (proc > 64) break;      // process directories are numbered densely; allow a few gaps
      continue;
    }
    any = true;
    ok = s->load(sub);
  }
  if (!any) { s->error = std::string("no manifest.ocdbt under ") + dir; ok = false; }
  if (!ok) {
    if (err != nullptr && err_len > 0) snprintf(err, static_cast<size_t>(err_len), "%s", s->error.c_str());
    return nullptr;
  }
  return s.release();
}

void recml_ocdbt_close(void* h) { delete static_cast<Store*>(h); }
long long recml_ocdbt_num_keys(void* h) { return static_cast<long long>(static_cast<Store*>(h)->order.size()); }
const char* recml_ocdbt_key(void* h, long long i) { return static_cast<Store*>(h)->order[static_cast<size_t>(i)].c_str(); }

long long recml_ocdbt_value_size(void* h, const char* key) {
  auto* s = static_cast<Store*>(h);
  auto it = s->keys.find(key);
  return it == s->keys.end() ? -1 : static_cast<long long>(it->second.length);
}

// Copies the value of `key` into out (capacity cap).  Returns its size, -1 unknown key, -2 too small, -3 I/O.
long long recml_ocdbt_read(void* h, const char* key, uint8_t* out, long long cap) {
  auto* s = static_cast<Store*>(h);
  auto it = s->keys.find(key);
  if (it == s->keys.end()) return -1;
  const Located& loc = it->second;
  if (static_cast<long long>(loc.length) > cap) return -2;
  if (loc.inline_value) {
    memcpy(out, loc.value.data(), loc.length);
    return static_cast<long long>(loc.length);
  }
  const int fd = ::open(loc.path.c_str(), O_RDONLY);       // straight into the caller's memory, many threads
  if (fd < 0) return -3;
  const bool ok = parallel_io(fd, out, nullptr, loc.offset, loc.length);
  ::close(fd);
  return ok ? static_cast<long long>(loc.length) : -3;
}

// Copies bytes [value_offset, value_offset + n) of the value of `key` into out: a row range of a large chunk
// without reading the rest of it.  Returns n, -1 unknown key, -2 range outside the value, -3 I/O.
long long recml_ocdbt_read_range(void* h, const char* key, long long value_offset, uint8_t* out, long long n) {
  auto* s = static_cast<Store*>(h);
  auto it = s->keys.find(key);
  if (it == s->keys.end()) return -1;
  const Located& loc = it->second;
  if (value_offset < 0 || n < 0 || static_cast<uint64_t>(value_offset) + static_cast<uint64_t>(n) > loc.length) return -2;
  if (loc.inline_value) {
    memcpy(out, loc.value.data() + value_offset, static_cast<size_t>(n));
    return n;
  }
  const int fd = ::open(loc.path.c_str(), O_RDONLY);
  if (fd < 0) return -3;
  const bool ok = parallel_io(fd, out, nullptr, loc.offset + static_cast<uint64_t>(value_offset), static_cast<uint64_t>(n));
  ::close(fd);
  return ok ? n : -3;
}

// ---- writing ----------------------------------------------------------------------------------------
void* recml_ocdbt_writer_new(const char* dir, long long max_inline_value_bytes) {
  auto* w = new PendingStore();
  w->dir = dir;
  if (max_inline_value_bytes >= 0) w->inline_limit = max_inline_value_bytes;
  return w;
}

int recml_ocdbt_writer_add(void* h, const char* key, const uint8_t* data, long long n) {
  auto* w = static_cast<PendingStore*>(h);
  Entry e;
  e.key = key;
  e.value.assign(reinterpret_cast<const char*>(data), static_cast<size_t>(n));
  w->entries.push_back(std::move(e));
  return 0;
}

// Like recml_ocdbt_writer_add without the copy: the caller keeps [data, data + n) alive and unchanged until the
// commit (or abort) returns.
int recml_ocdbt_writer_add_ref(void* h, const char* key, const uint8_t* data, long long n) {
  auto* w = static_cast<PendingStore*>(h);
  Entry e;
  e.key = key;
  if (n <= w->inline_limit) e.value.assign(reinterpret_cast<const char*>(data), static_cast<size_t>(n));
  else { e.ext = data; e.ext_len = static_cast<uint64_t>(n); }
  w->entries.push_back(std::move(e));
  return 0;
}

// Writes d/<data file> (out-of-line values, then the tree's nodes) and manifest.ocdbt, and frees the writer.
// node_fanout: entries per node (a small value forces a multi-level tree).  Returns 0 or a negative code.
int recml_ocdbt_writer_commit(void* h, int compress_nodes, int node_fanout) {
  std::unique_ptr<PendingStore> w(static_cast<PendingStore*>(h));
  if (node_fanout < 2) node_fanout = 64;
  std::sort(w->entries.begin(), w->entries.end(), [](const Entry& a, const Entry& b) { return a.key < b.key; });
  for (size_t i = 1; i < w->entries.size(); ++i)
    if (w->entries[i].key == w->entries[i - 1].key) return -2;       // duplicate key
  mkdirs(w->dir + "/d");
  // data file name: 32 hex digits derived from the keys (what matters is that the manifest names it)
  uint32_t hsh = 0x811c9dc5u;
  for (const auto& e : w->entries) for (char c : e.key) hsh = (hsh ^ static_cast<uint8_t>(c)) * 16777619u;
  char name[40];
  snprintf(name, sizeof(name), "%08x%08x%08x%08x", hsh, hsh * 2654435761u, static_cast<uint32_t>(w->entries.size()), 0x0cdb0001u);
  const std::vector<DataFile> files = {{"d/", name}};
  const std::string data_path = w->dir + "/d/" + name;
  const int fd = ::open((data_path + ".tmp").c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
  if (fd < 0) return -3;
  uint64_t pos = 0;
  bool ok = true;
  auto append = [&](const std::string& bytes) {        // nodes: small, written where the file ends
    const uint64_t at = pos;
    size_t put = 0;
    while (ok && put < bytes.size()) {
      const ssize_t r = ::pwrite(fd, bytes.data() + put, bytes.size() - put, static_cast<off_t>(at + put));
      if (r <= 0) ok = false; else put += static_cast<size_t>(r);
    }
    pos += bytes.size();
    return at;
  };
  // out-of-line values first: their offsets are fixed up front, then every value is written in 16 MB pieces
  // by all host threads, from the caller's memory when it was added by reference
  uint64_t indirect_total = 0;
  for (auto& e : w->entries) {
    if (static_cast<long long>(e.size()) > w->inline_limit) {
      e.inline_value = false;
      e.ref.file = 0;
      e.ref.length = e.size();
      e.ref.offset = pos;
      pos += e.size();
      indirect_total += e.size();
    }
  }
  if (pos > 0 && ::ftruncate(fd, static_cast<off_t>(pos)) != 0) ok = false;
  for (auto& e : w->entries) {
    if (e.inline_value || !ok) continue;
    const uint8_t* src = e.ext != nullptr ? e.ext : reinterpret_cast<const uint8_t*>(e.value.data());
    ok = parallel_io(fd, nullptr, src, e.ref.offset, e.ref.length);
    e.value.clear();
    e.value.shrink_to_fit();
  }
  // leaves
  std::vector<Child> level;
  for (size_t i = 0; i < w->entries.size(); i += static_cast<size_t>(node_fanout)) {
    const size_t j = std::min(w->entries.size(), i + static_cast<size_t>(node_fanout));
    std::vector<Entry> part(w->entries.begin() + static_cast<long>(i), w->entries.begin() + static_cast<long>(j));
    const std::string node = encode_leaf(part, files, compress_nodes != 0);
    Child c;
    c.first_key = part.front().key;
    c.ref.file = 0; c.ref.length = node.size(); c.ref.offset = append(node);
    c.num_keys = part.size();
    c.tree_bytes = node.size();
    for (const auto& e : part) if (!e.inline_value) c.indirect_bytes += e.ref.length;
    level.push_back(std::move(c));
  }
  int height = 0;
  while (level.size() > 1) {
    ++height;
    std::vector<Child> up;
    for (size_t i = 0; i < level.size(); i += static_cast<size_t>(node_fanout)) {
      const size_t j = std::min(level.size(), i + static_cast<size_t>(node_fanout));
      std::vector<Child> part(level.begin() + static_cast<long>(i), level.begin() + static_cast<long>(j));
      const std::string node = encode_interior(height, part, files, compress_nodes != 0);
      Child c;
      c.first_key = part.front().first_key;
      c.ref.file = 0; c.ref.length = node.size(); c.ref.offset = append(node);
      for (const auto& p : part) { c.num_keys += p.num_keys; c.tree_bytes += p.tree_bytes; c.indirect_bytes += p.indirect_bytes; }
      c.tree_bytes += node.size();
      up.push_back(std::move(c));
    }
    level.swap(up);
  }
  if (::close(fd) != 0) ok = false;
  if (!ok) return -3;
  if (rename((data_path + ".tmp").c_str(), data_path.c_str()) != 0) return -3;
  // manifest
  Writer m;
  m.varint(0);
  for (int i = 0; i < 16; ++i) m.u8(static_cast<uint8_t>((hsh >> ((i % 4) * 8)) ^ (i * 37)));   // uuid
  m.varint(0);                                  // manifest kind: single file
  m.varint(static_cast<uint64_t>(w->inline_limit));
  m.varint(8u << 20);                           // max decoded node bytes
  m.u8(4);                                      // version tree arity log2
  if (compress_nodes && zstd().ok) { m.varint(1); m.u32le(1); } else { m.varint(0); }
  write_file_table(m, files);
  m.varint(1);                                  // one version
  m.varint(1);                                  // generation number
  m.u8(static_cast<uint8_t>(height));
  const Child root = level.empty() ? Child() : level[0];
  m.varint(0); m.varint(root.ref.offset); m.varint(root.ref.length);
  m.varint(root.num_keys); m.varint(root.tree_bytes); m.varint(indirect_total);
  m.u64le(0);                                   // commit time
  m.varint(0);                                  // no version tree nodes
  const std::string manifest = envelope(kManifestMagic, m.b);
  const std::string mpath = w->dir + "/manifest.ocdbt";
  FILE* mf = fopen((mpath + ".tmp").c_str(), "wb");
  if (mf == nullptr) return -4;
  ok = fwrite(manifest.data(), 1, manifest.size(), mf) == manifest.size();
  ok = (fclose(mf) == 0) && ok;
  if (!ok || rename((mpath + ".tmp").c_str(), mpath.c_str()) != 0) return -4;
  return 0;
}

void recml_ocdbt_writer_abort(void* h) { delete static_cast<PendingStore*>(h); }

}  // extern "C"
