// .mim container: read-only memory-mapped reader, section hashing, and a writer
// that produces byte-compatible files.
//
// Layout (reference writer: io/mim/write.go:54-167, Python writer
// tools/golden/gen.py:937-997):
//   preamble 64 B little endian: magic "MIM\0" ("MMF\0" in v0.1 files), u16 major,
//     u16 minor, u32 byte-order mark 0x0A0B0C0D, u32 data alignment, u64 preamble
//     size (64), u64 index length, u64 data offset, u64 data length, u64 file
//     length, 8 zero bytes
//   index: u32 nsections, u32 ntensors, u64 name-pool bytes; section entries of
//     64 B (u32 kind, u32 flags, u64 offset, u64 length, u8 hash kind (1 = SHA-256),
//     7 pad, 32 B hash); tensor rows of 96 B (u32 name offset, u32 name length,
//     u32 dtype, u8 rank, 3 pad, 8 x u64 dims, u64 offset inside the weights
//     section, u64 byte length); name pool
//   then the graph section (kind 3) and the metadata section (kind 2), each on a
//     64-byte boundary, then the weights section (kind 1) on a data-alignment
//     boundary.  Tensor rows are sorted bytewise by name; a tensor starts on a
//     64-byte boundary, or a 4 KiB one when it holds 1 MiB or more.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#define MIM_API extern "C" __attribute__((visibility("default")))

namespace {

// ---------------------------------------------------------------- SHA-256
struct Sha256 {
  uint32_t h[8];
  uint8_t buf[64];
  uint64_t len = 0;
  size_t fill = 0;
  Sha256() {
    static const uint32_t init[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a,
                                     0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
    memcpy(h, init, sizeof(h));
  }
  static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
  void block(const uint8_t* p) {
    static const uint32_t k[64] = {
        0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5,
        0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174,
        0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da,
        0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967,
        0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
        0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070,
        0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3,
        0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
    uint32_t w[64];
    for (int i = 0; i < 16; ++i)
      w[i] = (uint32_t(p[4 * i]) << 24) | (uint32_t(p[4 * i + 1]) << 16) | (uint32_t(p[4 * i + 2]) << 8) | p[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
      uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
      uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
    for (int i = 0; i < 64; ++i) {
      uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25);
      uint32_t ch = (e & f) ^ (~e & g);
      uint32_t t1 = hh + S1 + ch + k[i] + w[i];
      uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22);
      uint32_t mj = (a & b) ^ (a & c) ^ (b & c);
      uint32_t t2 = S0 + mj;
      hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
  }
  void update(const uint8_t* p, size_t n) {
    len += n;
    while (n) {
      size_t take = std::min(n, 64 - fill);
      memcpy(buf + fill, p, take);
      fill += take; p += take; n -= take;
      if (fill == 64) { block(buf); fill = 0; }
    }
  }
  void finish(uint8_t out[32]) {
    uint64_t bits = len * 8;
    uint8_t pad = 0x80;
    update(&pad, 1);
    uint8_t z = 0;
    while (fill != 56) update(&z, 1);
    uint8_t lb[8];
    for (int i = 0; i < 8; ++i) lb[i] = uint8_t(bits >> (56 - 8 * i));
    update(lb, 8);
    for (int i = 0; i < 8; ++i) {
      out[4 * i] = uint8_t(h[i] >> 24); out[4 * i + 1] = uint8_t(h[i] >> 16);
      out[4 * i + 2] = uint8_t(h[i] >> 8); out[4 * i + 3] = uint8_t(h[i]);
    }
  }
};

void sha256(const uint8_t* p, size_t n, uint8_t out[32]) {
  Sha256 s;
  s.update(p, n);
  s.finish(out);
}

template <typename T>
T rd(const uint8_t* p) {
  T v;
  memcpy(&v, p, sizeof(T));
  return v;
}
template <typename T>
void wr(std::vector<uint8_t>& b, size_t off, T v) {
  memcpy(b.data() + off, &v, sizeof(T));
}
uint64_t align_up(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }

thread_local char g_err[256] = "";
int fail(const char* msg) {
  snprintf(g_err, sizeof(g_err), "%s", msg);
  return -1;
}

struct Section {
  uint32_t kind, flags;
  uint64_t off, len;
  uint8_t hash_kind;
  uint8_t hash[32];
};
struct TensorRow {
  std::string name;
  uint32_t dtype;
  uint8_t rank;
  uint64_t dims[8];
  uint64_t off, len;  // offset inside the weights section
};

struct MimFile {
  int fd = -1;
  const uint8_t* base = nullptr;
  size_t size = 0;
  bool owns_map = false;
  char magic[4];
  uint16_t major = 0, minor = 0;
  uint32_t alignment = 0;
  uint64_t data_off = 0, data_len = 0;
  std::vector<Section> sections;
  std::vector<TensorRow> tensors;
};

int parse(MimFile* f) {
  const uint8_t* b = f->base;
  if (f->size < 64) return fail("mim: file shorter than the preamble");
  memcpy(f->magic, b, 4);
  if (memcmp(b, "MIM\0", 4) != 0 && memcmp(b, "MMF\0", 4) != 0) return fail("mim: bad magic");
  f->major = rd<uint16_t>(b + 4);
  f->minor = rd<uint16_t>(b + 6);
  if (rd<uint32_t>(b + 8) != 0x0A0B0C0Du) return fail("mim: byte-order mark mismatch");
  f->alignment = rd<uint32_t>(b + 12);
  const uint64_t psize = rd<uint64_t>(b + 16), ilen = rd<uint64_t>(b + 24);
  f->data_off = rd<uint64_t>(b + 32);
  f->data_len = rd<uint64_t>(b + 40);
  const uint64_t flen = rd<uint64_t>(b + 48);
  if (psize != 64 || flen != f->size || psize + ilen > f->size || f->data_off + f->data_len > f->size)
    return fail("mim: preamble sizes do not fit the file");
  const uint8_t* idx = b + 64;
  if (ilen < 16) return fail("mim: index too short");
  const uint32_t ns = rd<uint32_t>(idx), nt = rd<uint32_t>(idx + 4);
  const uint64_t pool = rd<uint64_t>(idx + 8);
  const uint64_t need = 16 + 64ull * ns + 96ull * nt + pool;
  if (need > ilen) return fail("mim: index tables exceed the index length");
  for (uint32_t i = 0; i < ns; ++i) {
    const uint8_t* e = idx + 16 + 64 * i;
    Section s;
    s.kind = rd<uint32_t>(e); s.flags = rd<uint32_t>(e + 4);
    s.off = rd<uint64_t>(e + 8); s.len = rd<uint64_t>(e + 16);
    s.hash_kind = e[24];
    memcpy(s.hash, e + 32, 32);
    if (s.off + s.len > f->size) return fail("mim: section outside the file");
    f->sections.push_back(s);
  }
  const uint8_t* rows = idx + 16 + 64 * ns;
  const uint8_t* names = rows + 96ull * nt;
  for (uint32_t i = 0; i < nt; ++i) {
    const uint8_t* e = rows + 96 * i;
    TensorRow t;
    const uint32_t no = rd<uint32_t>(e), nl = rd<uint32_t>(e + 4);
    if (uint64_t(no) + nl > pool) return fail("mim: tensor name outside the pool");
    t.name.assign(reinterpret_cast<const char*>(names + no), nl);
    t.dtype = rd<uint32_t>(e + 8);
    t.rank = e[12];
    if (t.rank > 8) return fail("mim: tensor rank above 8");
    for (int d = 0; d < 8; ++d) t.dims[d] = rd<uint64_t>(e + 16 + 8 * d);
    t.off = rd<uint64_t>(e + 80);
    t.len = rd<uint64_t>(e + 88);
    if (t.off + t.len > f->data_len) return fail("mim: tensor outside the weights section");
    f->tensors.push_back(t);
  }
  return 0;
}

}  // namespace

// ---------------------------------------------------------------------------
// Reader C ABI
// ---------------------------------------------------------------------------
MIM_API const char* mimir_mim_last_error() { return g_err; }

MIM_API int mimir_mim_open(const char* path, void** out) {
  int fd = open(path, O_RDONLY);
  if (fd < 0) return fail("mim: cannot open file");
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size <= 0) { close(fd); return fail("mim: cannot stat file"); }
  void* p = mmap(nullptr, st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  if (p == MAP_FAILED) { close(fd); return fail("mim: mmap failed"); }
  MimFile* f = new MimFile();
  f->fd = fd;
  f->base = static_cast<const uint8_t*>(p);
  f->size = st.st_size;
  f->owns_map = true;
  if (parse(f) != 0) {
    munmap(p, st.st_size);
    close(fd);
    delete f;
    return -1;
  }
  *out = f;
  return 0;
}

// Parses a file image that the caller keeps alive (no copy, no mapping).
MIM_API int mimir_mim_parse(const void* data, uint64_t size, void** out) {
  MimFile* f = new MimFile();
  f->base = static_cast<const uint8_t*>(data);
  f->size = size;
  if (parse(f) != 0) { delete f; return -1; }
  *out = f;
  return 0;
}

MIM_API void mimir_mim_close(void* h) {
  MimFile* f = static_cast<MimFile*>(h);
  if (!f) return;
  if (f->owns_map) { munmap(const_cast<uint8_t*>(f->base), f->size); close(f->fd); }
  delete f;
}

MIM_API int mimir_mim_info(void* h, int* major, int* minor, int* alignment, int* ntensors, int* nsections,
                           int* is_mmf) {
  MimFile* f = static_cast<MimFile*>(h);
  *major = f->major; *minor = f->minor; *alignment = static_cast<int>(f->alignment);
  *ntensors = static_cast<int>(f->tensors.size()); *nsections = static_cast<int>(f->sections.size());
  *is_mmf = memcmp(f->magic, "MMF\0", 4) == 0;
  return 0;
}

MIM_API const void* mimir_mim_base(void* h) { return static_cast<MimFile*>(h)->base; }
MIM_API uint64_t mimir_mim_size(void* h) { return static_cast<MimFile*>(h)->size; }

// Tensor i: name (not NUL terminated), dtype code, rank, dims[8], absolute file offset, bytes.
MIM_API int mimir_mim_tensor(void* h, int i, const char** name, int* name_len, int* dtype, int* rank,
                             uint64_t* dims, uint64_t* file_off, uint64_t* nbytes) {
  MimFile* f = static_cast<MimFile*>(h);
  if (i < 0 || i >= static_cast<int>(f->tensors.size())) return fail("mim: tensor index out of range");
  const TensorRow& t = f->tensors[i];
  *name = t.name.data(); *name_len = static_cast<int>(t.name.size());
  *dtype = static_cast<int>(t.dtype); *rank = t.rank;
  for (int d = 0; d < 8; ++d) dims[d] = t.dims[d];
  *file_off = f->data_off + t.off; *nbytes = t.len;
  return 0;
}

// The whole tensor table in one call (a file of 20 000 tensors is indexed in a millisecond instead of
// 20 000 calls): meta[i * 12 + {0: dtype, 1: rank, 2..9: dims, 10: absolute file offset, 11: bytes}],
// name_end[i] = end of name i in the concatenated `names` (name i starts where name i - 1 ends).
// With meta == nullptr returns the number of bytes `names` needs.
MIM_API long long mimir_mim_table(void* h, uint64_t* meta, uint32_t* name_end, char* names, long long names_cap) {
  MimFile* f = static_cast<MimFile*>(h);
  long long total = 0;
  for (const TensorRow& t : f->tensors) total += static_cast<long long>(t.name.size());
  if (!meta) return total;
  if (names_cap < total) return fail("mim: name buffer too small");
  long long pos = 0;
  for (size_t i = 0; i < f->tensors.size(); ++i) {
    const TensorRow& t = f->tensors[i];
    uint64_t* m = meta + i * 12;
    m[0] = t.dtype; m[1] = t.rank;
    for (int d = 0; d < 8; ++d) m[2 + d] = t.dims[d];
    m[10] = f->data_off + t.off; m[11] = t.len;
    memcpy(names + pos, t.name.data(), t.name.size());
    pos += static_cast<long long>(t.name.size());
    name_end[i] = static_cast<uint32_t>(pos);
  }
  return total;
}

MIM_API int mimir_mim_section(void* h, int i, int* kind, int* flags, uint64_t* off, uint64_t* len,
                              uint8_t* hash32) {
  MimFile* f = static_cast<MimFile*>(h);
  if (i < 0 || i >= static_cast<int>(f->sections.size())) return fail("mim: section index out of range");
  const Section& s = f->sections[i];
  *kind = static_cast<int>(s.kind); *flags = static_cast<int>(s.flags); *off = s.off; *len = s.len;
  memcpy(hash32, s.hash, 32);
  return 0;
}

// Re-hashes every SHA-256 section; returns the number of mismatches (0 = intact).
MIM_API int mimir_mim_verify(void* h) {
  MimFile* f = static_cast<MimFile*>(h);
  int bad = 0;
  for (const Section& s : f->sections) {
    if (s.hash_kind != 1) continue;
    uint8_t d[32];
    sha256(f->base + s.off, s.len, d);
    if (memcmp(d, s.hash, 32) != 0) ++bad;
  }
  return bad;
}

MIM_API void mimir_sha256(const void* data, uint64_t n, uint8_t* out32) {
  sha256(static_cast<const uint8_t*>(data), n, out32);
}

// ---------------------------------------------------------------------------
// Writer C ABI
// ---------------------------------------------------------------------------
namespace {
struct PendingTensor {
  std::string name;
  uint32_t dtype;
  uint8_t rank;
  uint64_t dims[8];
  std::vector<uint8_t> data;
};
struct MimWriter {
  uint32_t alignment = 4096;
  uint16_t minor = 2;
  bool mmf = false;
  std::vector<PendingTensor> tensors;
  std::map<uint32_t, std::pair<uint32_t, std::vector<uint8_t>>> extra;  // kind -> (flags, bytes)
};
}  // namespace

MIM_API void* mimir_mim_writer_new(int alignment, int minor, int mmf_magic) {
  MimWriter* w = new MimWriter();
  w->alignment = alignment > 0 ? alignment : 4096;
  w->minor = static_cast<uint16_t>(minor);
  w->mmf = mmf_magic != 0;
  return w;
}
MIM_API void mimir_mim_writer_free(void* h) { delete static_cast<MimWriter*>(h); }

MIM_API int mimir_mim_writer_add_tensor(void* h, const char* name, int name_len, int dtype, int rank,
                                        const uint64_t* dims, const void* data, uint64_t nbytes) {
  MimWriter* w = static_cast<MimWriter*>(h);
  if (rank < 0 || rank > 8) return fail("mim: tensor rank above 8");
  PendingTensor t;
  t.name.assign(name, name_len);
  t.dtype = dtype;
  t.rank = static_cast<uint8_t>(rank);
  for (int d = 0; d < 8; ++d) t.dims[d] = d < rank ? dims[d] : 0;
  t.data.assign(static_cast<const uint8_t*>(data), static_cast<const uint8_t*>(data) + nbytes);
  w->tensors.push_back(std::move(t));
  return 0;
}

// kind 2 = metadata, 3 = graph, others (training, LoRA) are kept opaque.
MIM_API int mimir_mim_writer_set_section(void* h, int kind, int flags, const void* data, uint64_t n) {
  MimWriter* w = static_cast<MimWriter*>(h);
  if (kind == 1) return fail("mim: the weights section is built from the tensors");
  auto& e = w->extra[static_cast<uint32_t>(kind)];
  e.first = flags;
  e.second.assign(static_cast<const uint8_t*>(data), static_cast<const uint8_t*>(data) + n);
  return 0;
}

// Serialises into a malloc'd buffer (caller frees with mimir_mim_free_buffer).
MIM_API int mimir_mim_writer_serialize(void* h, uint8_t** out, uint64_t* out_len) {
  MimWriter* w = static_cast<MimWriter*>(h);
  std::vector<PendingTensor*> order;
  for (auto& t : w->tensors) order.push_back(&t);
  std::sort(order.begin(), order.end(), [](const PendingTensor* a, const PendingTensor* b) { return a->name < b->name; });
  for (size_t i = 1; i < order.size(); ++i)
    if (order[i]->name == order[i - 1]->name) return fail("mim: duplicate tensor name");
  // weights section layout: payloads in the order the tensors were added (the index
  // rows are what is sorted by name)
  std::map<const PendingTensor*, uint64_t> placed;
  uint64_t wlen = 0;
  for (auto& t : w->tensors) {
    const uint64_t al = t.data.size() >= (1u << 20) ? 4096 : 64;
    wlen = align_up(wlen, al);
    placed[&t] = wlen;
    wlen += t.data.size();
  }
  std::vector<uint64_t> offs(order.size());
  for (size_t i = 0; i < order.size(); ++i) offs[i] = placed[order[i]];
  // index: sections listed as weights, graph (3), others ascending except metadata, metadata (2) last
  std::vector<uint32_t> kinds = {1};
  if (w->extra.count(3)) kinds.push_back(3);
  for (auto& kv : w->extra) if (kv.first != 2 && kv.first != 3) kinds.push_back(kv.first);
  if (w->extra.count(2)) kinds.push_back(2);
  uint64_t pool = 0;
  for (auto* t : order) pool += t->name.size();
  const uint64_t ilen = 16 + 64ull * kinds.size() + 96ull * order.size() + pool;
  // file offsets: extra sections in index order after the index, each 64-aligned; weights last
  uint64_t cur = 64 + ilen;
  std::map<uint32_t, uint64_t> sec_off;
  for (uint32_t k : kinds) {
    if (k == 1) continue;
    cur = align_up(cur, 64);
    sec_off[k] = cur;
    cur += w->extra[k].second.size();
  }
  const uint64_t data_off = align_up(cur, w->alignment);
  const uint64_t flen = data_off + wlen;
  std::vector<uint8_t> b(flen, 0);
  memcpy(b.data(), w->mmf ? "MMF\0" : "MIM\0", 4);
  wr<uint16_t>(b, 4, 0); wr<uint16_t>(b, 6, w->minor);
  wr<uint32_t>(b, 8, 0x0A0B0C0Du); wr<uint32_t>(b, 12, w->alignment);
  wr<uint64_t>(b, 16, 64); wr<uint64_t>(b, 24, ilen);
  wr<uint64_t>(b, 32, data_off); wr<uint64_t>(b, 40, wlen); wr<uint64_t>(b, 48, flen);
  // payloads first (hashes need them)
  for (size_t i = 0; i < order.size(); ++i)
    memcpy(b.data() + data_off + offs[i], order[i]->data.data(), order[i]->data.size());
  for (auto& kv : sec_off) memcpy(b.data() + kv.second, w->extra[kv.first].second.data(), w->extra[kv.first].second.size());
  size_t o = 64;
  wr<uint32_t>(b, o, static_cast<uint32_t>(kinds.size()));
  wr<uint32_t>(b, o + 4, static_cast<uint32_t>(order.size()));
  wr<uint64_t>(b, o + 8, pool);
  o += 16;
  for (uint32_t k : kinds) {
    const uint64_t off = k == 1 ? data_off : sec_off[k];
    const uint64_t len = k == 1 ? wlen : w->extra[k].second.size();
    const uint32_t flags = k == 1 ? 1u : w->extra[k].first;
    wr<uint32_t>(b, o, k); wr<uint32_t>(b, o + 4, flags);
    wr<uint64_t>(b, o + 8, off); wr<uint64_t>(b, o + 16, len);
    b[o + 24] = 1;
    sha256(b.data() + off, len, b.data() + o + 32);
    o += 64;
  }
  uint32_t name_off = 0;
  const size_t names = o + 96 * order.size();
  for (size_t i = 0; i < order.size(); ++i) {
    const PendingTensor* t = order[i];
    wr<uint32_t>(b, o, name_off); wr<uint32_t>(b, o + 4, static_cast<uint32_t>(t->name.size()));
    wr<uint32_t>(b, o + 8, t->dtype);
    b[o + 12] = t->rank;
    for (int d = 0; d < 8; ++d) wr<uint64_t>(b, o + 16 + 8 * d, t->dims[d]);
    wr<uint64_t>(b, o + 80, offs[i]); wr<uint64_t>(b, o + 88, t->data.size());
    memcpy(b.data() + names + name_off, t->name.data(), t->name.size());
    name_off += static_cast<uint32_t>(t->name.size());
    o += 96;
  }
  uint8_t* buf = static_cast<uint8_t*>(malloc(flen ? flen : 1));
  if (!buf) return fail("mim: out of memory");
  memcpy(buf, b.data(), flen);
  *out = buf;
  *out_len = flen;
  return 0;
}
MIM_API void mimir_mim_free_buffer(uint8_t* p) { free(p); }

// Writes atomically: temporary file in the same directory, fsync, rename
// (reference: train/checkpoint.go:57-72).
MIM_API int mimir_mim_writer_write(void* h, const char* path) {
  uint8_t* buf = nullptr;
  uint64_t n = 0;
  if (mimir_mim_writer_serialize(h, &buf, &n) != 0) return -1;
  std::string tmp = std::string(path) + ".tmp";
  int fd = open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
  if (fd < 0) { free(buf); return fail("mim: cannot create the temporary file"); }
  uint64_t done = 0;
  while (done < n) {
    ssize_t k = write(fd, buf + done, n - done);
    if (k <= 0) { close(fd); free(buf); unlink(tmp.c_str()); return fail("mim: write failed"); }
    done += static_cast<uint64_t>(k);
  }
  fsync(fd);
  close(fd);
  free(buf);
  if (rename(tmp.c_str(), path) != 0) { unlink(tmp.c_str()); return fail("mim: rename failed"); }
  return 0;
}
