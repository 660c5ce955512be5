// Parquet column-chunk decoder (reference: io/parquet/{parquet,metadata,reader,page,rle,delta,
// thrift}.go: its own decoder of the subset of the format that data-science tools write).
//
// Flat schemas of BOOLEAN / INT32 / INT64 / FLOAT / DOUBLE / BYTE_ARRAY / FIXED_LEN_BYTE_ARRAY;
// data pages V1 and V2; PLAIN, RLE (booleans), dictionary, DELTA_BINARY_PACKED,
// DELTA_LENGTH_BYTE_ARRAY, DELTA_BYTE_ARRAY and BYTE_STREAM_SPLIT; UNCOMPRESSED, SNAPPY (decoder
// below), GZIP (zlib) and ZSTD (libzstd), the last two loaded at run time.  Nested columns, INT96,
// encrypted files and the other codecs are listed but refused.  A file is read through mmap; one
// column chunk of one row group is decoded per call into buffers the handle owns, so a data set of
// any size streams row group by row group.  Nothing trusts a count or size the file declares:
// every read is checked against the bytes that are there, and a failed allocation is an error.
//
// Plain C ABI:
//   mimir_pq_open / close / last_error
//   mimir_pq_counts (rows, row groups, columns), mimir_pq_column (schema), mimir_pq_group_rows
//   mimir_pq_meta (created_by and key/value metadata)
//   mimir_pq_decode (group, column) -> mimir_pq_result (pointers into the handle's buffers)
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <dlfcn.h>

#include <cstdint>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "runtime.h"

namespace mimir {
namespace pq {

enum Status { kOk = 0, kFormat = 1, kUnsupported = 2, kIo = 3, kArgument = 4 };

struct Error {
  int code;
  std::string text;
};
#define PQ_FAIL(c, msg) throw Error{c, std::string(msg)}

// ---------------------------------------------------------------------------
// Byte cursor with bounds checks
// ---------------------------------------------------------------------------
struct Cur {
  const uint8_t* p;
  const uint8_t* end;
  size_t left() const { return static_cast<size_t>(end - p); }
  uint8_t byte() {
    if (p >= end) PQ_FAIL(kFormat, "truncated data");
    return *p++;
  }
  const uint8_t* take(size_t n) {
    if (n > left()) PQ_FAIL(kFormat, "truncated data");
    const uint8_t* q = p;
    p += n;
    return q;
  }
  uint64_t uvarint() {
    uint64_t v = 0;
    for (int shift = 0; shift < 64; shift += 7) {
      const uint8_t b = byte();
      v |= static_cast<uint64_t>(b & 0x7f) << shift;
      if (!(b & 0x80)) return v;
    }
    PQ_FAIL(kFormat, "varint longer than 10 bytes");
  }
  int64_t zigzag() {
    const uint64_t u = uvarint();
    return static_cast<int64_t>(u >> 1) ^ -static_cast<int64_t>(u & 1);
  }
  uint32_t le32() {
    const uint8_t* q = take(4);
    uint32_t v;
    memcpy(&v, q, 4);
    return v;
  }
};

// ---------------------------------------------------------------------------
// Thrift compact protocol: only what the footer and page headers need.  Unknown fields are skipped.
// ---------------------------------------------------------------------------
enum TType { T_STOP = 0, T_TRUE = 1, T_FALSE = 2, T_BYTE = 3, T_I16 = 4, T_I32 = 5, T_I64 = 6, T_DOUBLE = 7,
             T_BINARY = 8, T_LIST = 9, T_SET = 10, T_MAP = 11, T_STRUCT = 12 };

struct Thrift {
  Cur c;
  int depth = 0;

  // returns false at STOP; otherwise the field id and wire type
  bool field(int& last_id, int& id, int& type) {
    const uint8_t h = c.byte();
    if (h == 0) return false;
    type = h & 0x0f;
    const int delta = h >> 4;
    if (delta) id = last_id + delta;
    else id = static_cast<int>(c.zigzag());
    last_id = id;
    return true;
  }
  int64_t i() { return c.zigzag(); }
  std::string str() {
    const uint64_t n = c.uvarint();
    const uint8_t* q = c.take(n);
    return std::string(reinterpret_cast<const char*>(q), n);
  }
  void list(int& elem, uint64_t& n) {
    const uint8_t h = c.byte();
    elem = h & 0x0f;
    n = h >> 4;
    if (n == 15) n = c.uvarint();
    if (n > c.left()) PQ_FAIL(kFormat, "list longer than its bytes");   // every element takes a byte at least
  }
  void skip(int type) {
    if (++depth > 64) PQ_FAIL(kFormat, "structure nested too deeply");
    switch (type) {
      case T_TRUE: case T_FALSE: break;
      case T_BYTE: c.byte(); break;
      case T_I16: case T_I32: case T_I64: c.uvarint(); break;
      case T_DOUBLE: c.take(8); break;
      case T_BINARY: c.take(c.uvarint()); break;
      case T_LIST: case T_SET: {
        int e; uint64_t n;
        list(e, n);
        for (uint64_t k = 0; k < n; ++k) {
          if (e == T_TRUE || e == T_FALSE) c.byte();   // booleans in a list take a byte each
          else skip(e);
        }
        break;
      }
      case T_MAP: {
        const uint64_t n = c.uvarint();
        if (n > c.left()) PQ_FAIL(kFormat, "map longer than its bytes");
        if (n) {
          const uint8_t kv = c.byte();
          for (uint64_t k = 0; k < n; ++k) {
            const int kt = kv >> 4, vt = kv & 0x0f;
            if (kt == T_TRUE || kt == T_FALSE) c.byte(); else skip(kt);
            if (vt == T_TRUE || vt == T_FALSE) c.byte(); else skip(vt);
          }
        }
        break;
      }
      case T_STRUCT: {
        int last = 0, id, t;
        while (field(last, id, t)) skip(t);
        break;
      }
      default: PQ_FAIL(kFormat, "unknown thrift type");
    }
    --depth;
  }
};

// ---------------------------------------------------------------------------
// Metadata model
// ---------------------------------------------------------------------------
enum PType { P_BOOLEAN = 0, P_INT32 = 1, P_INT64 = 2, P_INT96 = 3, P_FLOAT = 4, P_DOUBLE = 5, P_BYTE_ARRAY = 6,
             P_FLBA = 7 };

struct Column {
  std::string name;       // dotted path
  int type = -1;
  int type_length = 0;
  bool nullable = false;
  bool nested = false;    // below a group or repeated: listed, not readable
  int converted = -1;     // ConvertedType, -1 when absent
  int scale = 0, precision = 0;
  std::string logical;    // name of the LogicalType union member, "" when absent
};

struct Chunk {
  int type = -1;
  int codec = 0;
  int64_t num_values = 0;
  int64_t total_compressed = 0;
  int64_t data_page_offset = -1;
  int64_t dict_page_offset = -1;
  bool has_meta = false;
  bool encrypted = false;
  bool external = false;   // file_path set
};

struct Group {
  int64_t rows = 0;
  std::vector<Chunk> chunks;
};

struct File {
  int fd = -1;
  const uint8_t* map = nullptr;
  size_t size = 0;
  int64_t rows = 0;
  std::string created_by;
  std::vector<std::pair<std::string, std::string>> kv;
  std::vector<Column> cols;
  std::vector<Group> groups;
  // result of the last decode
  int r_type = -1;
  int64_t r_count = 0;
  std::vector<uint8_t> values;     // fixed width: count x width; byte arrays: the bytes
  std::vector<int64_t> offsets;    // byte arrays: count + 1
  std::vector<uint8_t> nulls;      // count, 1 = null
  int64_t r_null_count = 0;
  // destinations of a fixed-width decode given by the caller (else the vectors above)
  uint8_t* ext_values = nullptr;
  uint8_t* ext_nulls = nullptr;
  // scratch
  std::vector<uint8_t> page, dict_bytes;
  std::vector<int64_t> dict_offsets;
  std::vector<uint8_t> levels;
  std::vector<uint32_t> idx;
  std::string error;
};

static const char* logical_names[] = {"", "STRING", "MAP", "LIST", "ENUM", "DECIMAL", "DATE", "TIME", "TIMESTAMP", "",
                                      "INTEGER", "UNKNOWN", "JSON", "BSON", "UUID", "FLOAT16"};

static void parse_schema_element(Thrift& t, Column& c, int& repetition, int& children, bool& has_type) {
  int last = 0, id, ty;
  repetition = 0;   // REQUIRED when absent (the root)
  children = 0;
  has_type = false;
  while (t.field(last, id, ty)) {
    switch (id) {
      case 1: c.type = static_cast<int>(t.i()); has_type = true; break;
      case 2: c.type_length = static_cast<int>(t.i()); break;
      case 3: repetition = static_cast<int>(t.i()); break;
      case 4: c.name = t.str(); break;
      case 5: children = static_cast<int>(t.i()); break;
      case 6: c.converted = static_cast<int>(t.i()); break;
      case 7: c.scale = static_cast<int>(t.i()); break;
      case 8: c.precision = static_cast<int>(t.i()); break;
      case 10: {   // LogicalType: a union, the set member names the type
        if (ty != T_STRUCT) { t.skip(ty); break; }
        int l2 = 0, id2, ty2;
        while (t.field(l2, id2, ty2)) {
          if (id2 >= 1 && id2 <= 15) c.logical = logical_names[id2];
          t.skip(ty2);
        }
        break;
      }
      default: t.skip(ty);
    }
  }
}

static void parse_column_meta(Thrift& t, Chunk& c) {
  int last = 0, id, ty;
  c.has_meta = true;
  while (t.field(last, id, ty)) {
    switch (id) {
      case 1: c.type = static_cast<int>(t.i()); break;
      case 4: c.codec = static_cast<int>(t.i()); break;
      case 5: c.num_values = t.i(); break;
      case 7: c.total_compressed = t.i(); break;
      case 9: c.data_page_offset = t.i(); break;
      case 11: c.dict_page_offset = t.i(); break;
      default: t.skip(ty);
    }
  }
}

static void parse_chunk(Thrift& t, Chunk& c) {
  int last = 0, id, ty;
  while (t.field(last, id, ty)) {
    switch (id) {
      case 1: { std::string s = t.str(); c.external = !s.empty(); break; }
      case 3:
        if (ty != T_STRUCT) PQ_FAIL(kFormat, "column metadata is not a structure");
        parse_column_meta(t, c);
        break;
      case 8: c.encrypted = true; t.skip(ty); break;   // crypto_metadata
      case 9: c.encrypted = true; t.skip(ty); break;   // encrypted_column_metadata
      default: t.skip(ty);
    }
  }
}

static void parse_group(Thrift& t, Group& g) {
  int last = 0, id, ty;
  while (t.field(last, id, ty)) {
    switch (id) {
      case 1: {
        int e; uint64_t n;
        if (ty != T_LIST) PQ_FAIL(kFormat, "row group columns are not a list");
        t.list(e, n);
        if (e != T_STRUCT) PQ_FAIL(kFormat, "row group columns are not structures");
        g.chunks.resize(n);
        for (auto& c : g.chunks) parse_chunk(t, c);
        break;
      }
      case 3: g.rows = t.i(); break;
      default: t.skip(ty);
    }
  }
}

static void parse_footer(File& f, const uint8_t* p, size_t n) {
  Thrift t{{p, p + n}};
  int last = 0, id, ty;
  struct Raw { Column c; int repetition; int children; bool has_type; };
  std::vector<Raw> schema;
  while (t.field(last, id, ty)) {
    switch (id) {
      case 2: {
        int e; uint64_t cnt;
        if (ty != T_LIST) PQ_FAIL(kFormat, "schema is not a list");
        t.list(e, cnt);
        if (e != T_STRUCT) PQ_FAIL(kFormat, "schema elements are not structures");
        schema.resize(cnt);
        for (auto& r : schema) parse_schema_element(t, r.c, r.repetition, r.children, r.has_type);
        break;
      }
      case 3: f.rows = t.i(); break;
      case 4: {
        int e; uint64_t cnt;
        if (ty != T_LIST) PQ_FAIL(kFormat, "row groups are not a list");
        t.list(e, cnt);
        if (e != T_STRUCT) PQ_FAIL(kFormat, "row groups are not structures");
        f.groups.resize(cnt);
        for (auto& g : f.groups) parse_group(t, g);
        break;
      }
      case 5: {
        int e; uint64_t cnt;
        if (ty != T_LIST) { t.skip(ty); break; }
        t.list(e, cnt);
        for (uint64_t k = 0; k < cnt; ++k) {
          if (e != T_STRUCT) { t.skip(e); continue; }
          std::string key, val;
          int l2 = 0, id2, ty2;
          while (t.field(l2, id2, ty2)) {
            if (id2 == 1 && ty2 == T_BINARY) key = t.str();
            else if (id2 == 2 && ty2 == T_BINARY) val = t.str();
            else t.skip(ty2);
          }
          f.kv.emplace_back(std::move(key), std::move(val));
        }
        break;
      }
      case 6: f.created_by = t.str(); break;
      case 8: PQ_FAIL(kUnsupported, "encrypted file");
      default: t.skip(ty);
    }
  }
  if (schema.empty()) PQ_FAIL(kFormat, "no schema");
  // Walk the schema tree depth first: leaves become columns; a leaf is readable when it hangs
  // directly below the root and is not repeated.
  struct Frame { int remaining; std::string prefix; bool nested; };
  std::vector<Frame> stack;
  if (schema[0].children < 0 || static_cast<size_t>(schema[0].children) > schema.size())
    PQ_FAIL(kFormat, "schema root declares more children than there are elements");
  stack.push_back({schema[0].children, "", false});
  for (size_t k = 1; k < schema.size(); ++k) {
    while (!stack.empty() && stack.back().remaining == 0) stack.pop_back();
    if (stack.empty()) PQ_FAIL(kFormat, "schema elements outside the tree");
    Frame& fr = stack.back();
    --fr.remaining;
    Raw& r = schema[k];
    const std::string path = fr.prefix.empty() ? r.c.name : fr.prefix + "." + r.c.name;
    const bool nested_here = fr.nested || r.repetition == 2 || stack.size() > 1;
    if (r.children > 0) {
      if (stack.size() >= 64) PQ_FAIL(kFormat, "schema nested deeper than 64 groups");
      if (static_cast<size_t>(r.children) > schema.size()) PQ_FAIL(kFormat, "group declares more children than there are elements");
      stack.push_back({r.children, path, true});
    } else {
      if (!r.has_type) PQ_FAIL(kFormat, "schema leaf without a type");
      Column c = r.c;
      c.name = path;
      c.nullable = r.repetition == 1;
      c.nested = nested_here;
      f.cols.push_back(std::move(c));
    }
  }
  for (auto& g : f.groups)
    if (g.chunks.size() != f.cols.size()) PQ_FAIL(kFormat, "row group with a different number of columns than the schema");
}

// ---------------------------------------------------------------------------
// Decompression
// ---------------------------------------------------------------------------
static void snappy_decode(const uint8_t* src, size_t n, std::vector<uint8_t>& out, size_t want) {
  Cur c{src, src + n};
  const uint64_t len = c.uvarint();
  if (len != want) PQ_FAIL(kFormat, "snappy length differs from the page header");
  out.resize(len);
  size_t o = 0;
  while (c.p < c.end) {
    const uint8_t tag = c.byte();
    const int kind = tag & 3;
    if (kind == 0) {
      size_t l = tag >> 2;
      if (l >= 60) {
        const int nb = static_cast<int>(l) - 59;
        const uint8_t* q = c.take(nb);
        l = 0;
        for (int k = 0; k < nb; ++k) l |= static_cast<size_t>(q[k]) << (8 * k);
      }
      l += 1;
      if (l > len - o) PQ_FAIL(kFormat, "snappy literal past the end");
      memcpy(out.data() + o, c.take(l), l);
      o += l;
    } else {
      size_t l, off;
      if (kind == 1) {
        l = ((tag >> 2) & 7) + 4;
        off = (static_cast<size_t>(tag >> 5) << 8) | c.byte();
      } else if (kind == 2) {
        l = (tag >> 2) + 1;
        const uint8_t* q = c.take(2);
        off = q[0] | (static_cast<size_t>(q[1]) << 8);
      } else {
        l = (tag >> 2) + 1;
        off = c.le32();
      }
      if (off == 0 || off > o || l > len - o) PQ_FAIL(kFormat, "snappy copy out of range");
      uint8_t* d = out.data() + o;
      const uint8_t* s = d - off;
      if (off >= l) memcpy(d, s, l);
      else for (size_t k = 0; k < l; ++k) d[k] = s[k];   // overlapping: byte by byte
      o += l;
    }
  }
  if (o != len) PQ_FAIL(kFormat, "snappy stream shorter than its length");
}

// zlib and zstd are loaded at run time so the library has no link-time dependency on them
struct ZStreamLike {   // layout of z_stream on LP64
  const uint8_t* next_in; unsigned avail_in; unsigned long total_in;
  uint8_t* next_out; unsigned avail_out; unsigned long total_out;
  const char* msg; void* state; void* zalloc; void* zfree; void* opaque;
  int data_type; unsigned long adler; unsigned long reserved;
};
typedef int (*inflateInit2_fn)(ZStreamLike*, int, const char*, int);
typedef int (*inflate_fn)(ZStreamLike*, int);
typedef int (*inflateEnd_fn)(ZStreamLike*);
typedef size_t (*zstd_decompress_fn)(void*, size_t, const void*, size_t);
typedef unsigned (*zstd_iserror_fn)(size_t);

static void* open_any(const char* const* names) {
  for (; *names; ++names)
    if (void* h = dlopen(*names, RTLD_NOW | RTLD_LOCAL)) return h;
  return nullptr;
}

static void gzip_decode(const uint8_t* src, size_t n, std::vector<uint8_t>& out, size_t want) {
  static inflateInit2_fn init = nullptr;
  static inflate_fn run = nullptr;
  static inflateEnd_fn fin = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    static const char* names[] = {"libz.so.1", "libz.so", nullptr};
    if (void* h = open_any(names)) {
      init = reinterpret_cast<inflateInit2_fn>(dlsym(h, "inflateInit2_"));
      run = reinterpret_cast<inflate_fn>(dlsym(h, "inflate"));
      fin = reinterpret_cast<inflateEnd_fn>(dlsym(h, "inflateEnd"));
    }
  });
  if (!init || !run || !fin) PQ_FAIL(kUnsupported, "GZIP pages need libz, which was not found");
  out.resize(want);
  ZStreamLike z;
  memset(&z, 0, sizeof z);
  if (init(&z, 15 + 32, "1.2.11", static_cast<int>(sizeof z)) != 0) PQ_FAIL(kFormat, "cannot start inflate");
  z.next_in = src;
  z.avail_in = static_cast<unsigned>(n);
  z.next_out = out.data();
  z.avail_out = static_cast<unsigned>(want);
  // a page may hold several gzip members one after another
  for (;;) {
    const int rc = run(&z, 4 /* Z_FINISH */);
    if (rc == 1 /* Z_STREAM_END */) {
      if (z.avail_in == 0) break;
      const uint8_t* ni = z.next_in; unsigned ai = z.avail_in;
      uint8_t* no = z.next_out; unsigned ao = z.avail_out;
      fin(&z);
      memset(&z, 0, sizeof z);
      if (init(&z, 15 + 32, "1.2.11", static_cast<int>(sizeof z)) != 0) PQ_FAIL(kFormat, "cannot start inflate");
      z.next_in = ni; z.avail_in = ai; z.next_out = no; z.avail_out = ao;
      continue;
    }
    fin(&z);
    PQ_FAIL(kFormat, "damaged gzip page");
  }
  const bool full = z.avail_out == 0;
  fin(&z);
  if (!full) PQ_FAIL(kFormat, "gzip page shorter than the page header says");
}

static void zstd_decode(const uint8_t* src, size_t n, std::vector<uint8_t>& out, size_t want) {
  static zstd_decompress_fn dec = nullptr;
  static zstd_iserror_fn iserr = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    static const char* names[] = {"libzstd.so.1", "libzstd.so", nullptr};
    if (void* h = open_any(names)) {
      dec = reinterpret_cast<zstd_decompress_fn>(dlsym(h, "ZSTD_decompress"));
      iserr = reinterpret_cast<zstd_iserror_fn>(dlsym(h, "ZSTD_isError"));
    }
  });
  if (!dec || !iserr) PQ_FAIL(kUnsupported, "ZSTD pages need libzstd, which was not found");
  out.resize(want);
  const size_t got = dec(out.data(), want, src, n);
  if (iserr(got)) PQ_FAIL(kFormat, "damaged zstd page");
  if (got != want) PQ_FAIL(kFormat, "zstd page shorter than the page header says");
}

static const char* codec_name(int c) {
  static const char* n[] = {"UNCOMPRESSED", "SNAPPY", "GZIP", "LZO", "BROTLI", "LZ4", "ZSTD", "LZ4_RAW"};
  return c >= 0 && c < 8 ? n[c] : "unknown";
}

// Decompresses [src, src+n) into `out` when the codec asks for it; returns where the bytes are.
static Cur decompress(int codec, const uint8_t* src, size_t n, size_t want, std::vector<uint8_t>& out) {
  if (codec == 0) {
    if (n != want) PQ_FAIL(kFormat, "uncompressed page whose two sizes differ");
    return Cur{src, src + n};
  }
  // What a page may expand to is bounded by its own bytes: deflate and zstd stay under 1032:1 and
  // 2^17:1 of real data; a header that claims more than 2^20:1 is refused before anything is allocated.
  if (want > (n + 1) * (size_t{1} << 20)) PQ_FAIL(kFormat, "page declares more bytes than it could hold");
  try {
    if (codec == 1) snappy_decode(src, n, out, want);
    else if (codec == 2) gzip_decode(src, n, out, want);
    else if (codec == 6) zstd_decode(src, n, out, want);
    else PQ_FAIL(kUnsupported, std::string("codec ") + codec_name(codec));
  } catch (const std::bad_alloc&) {
    PQ_FAIL(kFormat, "page too large to hold in memory");
  }
  return Cur{out.data(), out.data() + out.size()};
}

// ---------------------------------------------------------------------------
// RLE / bit-packed hybrid
// ---------------------------------------------------------------------------
struct Hybrid {
  Cur c;
  int width;
  uint64_t run_left = 0;     // values left in the current run
  bool packed = false;
  uint32_t rle_value = 0;
  uint64_t bit_pos = 0;      // inside the packed run
  const uint8_t* packed_base = nullptr;
  uint64_t packed_values = 0;

  void next_run() {
    const uint64_t h = c.uvarint();
    if (h & 1) {
      const uint64_t groups = h >> 1;
      if (groups == 0) PQ_FAIL(kFormat, "empty bit-packed run");
      if (groups > (uint64_t{1} << 32)) PQ_FAIL(kFormat, "bit-packed run longer than any page");
      const uint64_t bytes = groups * width;
      // the last group of a page may be cut short of its padding
      const uint64_t have = bytes <= c.left() ? bytes : c.left();
      packed_base = c.take(have);
      packed_values = width ? (have * 8) / width : groups * 8;
      run_left = groups * 8 < packed_values ? groups * 8 : packed_values;
      if (width == 0) run_left = groups * 8;
      packed = true;
      bit_pos = 0;
    } else {
      run_left = h >> 1;
      if (run_left == 0) PQ_FAIL(kFormat, "empty run");
      const int nb = (width + 7) / 8;
      const uint8_t* q = c.take(nb);
      rle_value = 0;
      for (int k = 0; k < nb; ++k) rle_value |= static_cast<uint32_t>(q[k]) << (8 * k);
      if (width < 32 && (rle_value >> width)) PQ_FAIL(kFormat, "run value wider than its bit width");
      packed = false;
    }
  }
  // decodes n values into dst
  void read(uint32_t* dst, uint64_t n) {
    while (n) {
      if (run_left == 0) next_run();
      const uint64_t take = n < run_left ? n : run_left;
      if (!packed) {
        for (uint64_t k = 0; k < take; ++k) dst[k] = rle_value;
      } else if (width == 0) {
        for (uint64_t k = 0; k < take; ++k) dst[k] = 0;
      } else {
        const uint32_t mask = width == 32 ? 0xffffffffu : ((1u << width) - 1);
        for (uint64_t k = 0; k < take; ++k) {
          const uint64_t byte = bit_pos >> 3;
          const int sh = static_cast<int>(bit_pos & 7);
          uint64_t w = 0;
          // up to 5 bytes hold one value; never read past the run's bytes
          const uint64_t avail = (packed_values * width + 7) / 8 - byte;
          const int nb = avail < 8 ? static_cast<int>(avail) : 8;
          memcpy(&w, packed_base + byte, nb);
          dst[k] = static_cast<uint32_t>(w >> sh) & mask;
          bit_pos += width;
        }
      }
      dst += take;
      n -= take;
      run_left -= take;
    }
  }
};

// ---------------------------------------------------------------------------
// DELTA_BINARY_PACKED
// ---------------------------------------------------------------------------
// Decodes every value of the stream at c (the header says how many) and leaves c behind it.
static void delta_decode(Cur& c, std::vector<int64_t>& out, uint64_t limit) {
  const uint64_t block = c.uvarint(), minis = c.uvarint(), total = c.uvarint();
  const int64_t first = c.zigzag();
  if (block == 0 || block % 128 || minis == 0 || block % minis || (block / minis) % 32 || block > (1u << 20))
    PQ_FAIL(kFormat, "bad delta block layout");
  if (total > limit) PQ_FAIL(kFormat, "delta stream declares more values than the page");
  const uint64_t per = block / minis;
  out.clear();
  out.reserve(total);
  if (total == 0) return;
  uint64_t prev = static_cast<uint64_t>(first);
  out.push_back(first);
  uint64_t done = 1;
  std::vector<uint8_t> widths(minis);
  while (done < total) {
    const uint64_t min_delta = static_cast<uint64_t>(c.zigzag());
    const uint8_t* w = c.take(minis);
    memcpy(widths.data(), w, minis);
    for (uint64_t m = 0; m < minis && done < total; ++m) {
      const int bw = widths[m];
      if (bw > 64) PQ_FAIL(kFormat, "delta bit width above 64");
      const uint64_t bytes = per * bw / 8;
      const uint8_t* d = c.take(bytes);
      const uint64_t n = total - done < per ? total - done : per;
      uint64_t bit = 0;
      for (uint64_t k = 0; k < n; ++k) {
        uint64_t v = 0;
        if (bw) {
          const uint64_t byte = bit >> 3;
          const int sh = static_cast<int>(bit & 7);
          unsigned __int128 acc = 0;
          const uint64_t avail = bytes - byte;
          const int nb = avail < 9 ? static_cast<int>(avail) : 9;
          memcpy(&acc, d + byte, nb);
          acc >>= sh;
          v = bw == 64 ? static_cast<uint64_t>(acc) : static_cast<uint64_t>(acc) & ((uint64_t{1} << bw) - 1);
          bit += bw;
        }
        prev = prev + min_delta + v;   // wraps like the writer's arithmetic
        out.push_back(static_cast<int64_t>(prev));
      }
      done += n;
    }
  }
}

// ---------------------------------------------------------------------------
// Column chunk decoding
// ---------------------------------------------------------------------------
static int width_of(int type, int type_length) {
  switch (type) {
    case P_BOOLEAN: return 1;
    case P_INT32: case P_FLOAT: return 4;
    case P_INT64: case P_DOUBLE: return 8;
    case P_FLBA: return type_length;
    default: return 0;
  }
}

struct PageHeader {
  int type = -1;
  int64_t uncompressed = -1, compressed = -1;
  // data page v1 / v2, dictionary page
  int64_t num_values = -1, num_nulls = -1, num_rows = -1;
  int encoding = -1, def_encoding = 3;
  int64_t def_bytes = 0, rep_bytes = 0;
  bool v2_compressed = true;
  bool has_sub = false;
};

static void parse_page_header(Thrift& t, PageHeader& h) {
  int last = 0, id, ty;
  while (t.field(last, id, ty)) {
    switch (id) {
      case 1: h.type = static_cast<int>(t.i()); break;
      case 2: h.uncompressed = t.i(); break;
      case 3: h.compressed = t.i(); break;
      case 5: case 7: case 8: {
        if (ty != T_STRUCT) PQ_FAIL(kFormat, "page sub-header is not a structure");
        h.has_sub = true;
        int l2 = 0, id2, ty2;
        while (t.field(l2, id2, ty2)) {
          if (id == 5) {
            if (id2 == 1) h.num_values = t.i();
            else if (id2 == 2) h.encoding = static_cast<int>(t.i());
            else if (id2 == 3) h.def_encoding = static_cast<int>(t.i());
            else t.skip(ty2);
          } else if (id == 7) {
            if (id2 == 1) h.num_values = t.i();
            else if (id2 == 2) h.encoding = static_cast<int>(t.i());
            else t.skip(ty2);
          } else {
            if (id2 == 1) h.num_values = t.i();
            else if (id2 == 2) h.num_nulls = t.i();
            else if (id2 == 3) h.num_rows = t.i();
            else if (id2 == 4) h.encoding = static_cast<int>(t.i());
            else if (id2 == 5) h.def_bytes = t.i();
            else if (id2 == 6) h.rep_bytes = t.i();
            else if (id2 == 7) h.v2_compressed = ty2 == T_TRUE;
            else t.skip(ty2);
          }
        }
        break;
      }
      default: t.skip(ty);
    }
  }
}

static const char* encoding_name(int e) {
  static const char* n[] = {"PLAIN", "GROUP_VAR_INT", "PLAIN_DICTIONARY", "RLE", "BIT_PACKED", "DELTA_BINARY_PACKED",
                            "DELTA_LENGTH_BYTE_ARRAY", "DELTA_BYTE_ARRAY", "RLE_DICTIONARY", "BYTE_STREAM_SPLIT"};
  return e >= 0 && e < 10 ? n[e] : "unknown";
}

struct Decoder {
  File& f;
  const Column& col;
  const Chunk& ch;
  int64_t rows;
  int width;
  bool bytes_like;       // BYTE_ARRAY: variable length
  bool have_dict = false;
  int64_t dict_count = 0;
  int64_t filled = 0;    // rows decoded so far
  std::vector<int64_t> tmp64, tmp64b;
  uint8_t* out = nullptr;      // fixed-width values: rows x width
  uint8_t* nul = nullptr;      // rows, 1 = null

  Decoder(File& f_, const Column& c, const Chunk& k, int64_t r)
      : f(f_), col(c), ch(k), rows(r), width(width_of(c.type, c.type_length)), bytes_like(c.type == P_BYTE_ARRAY) {}

  void prepare() {
    // The output is sized by the declared row count, so the count must be believable for the bytes
    // of the chunk: run-length data can hold thousands of rows per byte, not more.
    if (rows < 0 || rows > (int64_t{1} << 31) || rows > (int64_t{1} << 24) + ch.total_compressed * 4096)
      PQ_FAIL(kFormat, "row group declares more rows than its bytes could hold");
    try {
      if (f.ext_nulls) { nul = f.ext_nulls; memset(nul, 0, static_cast<size_t>(rows)); }
      else { f.nulls.assign(rows, 0); nul = f.nulls.data(); }
      if (bytes_like) {
        f.offsets.assign(rows + 1, 0);
        f.values.clear();
      } else if (f.ext_values) {
        out = f.ext_values;
        memset(out, 0, static_cast<size_t>(rows) * width);
        f.offsets.clear();
      } else {
        f.values.assign(static_cast<size_t>(rows) * width, 0);
        out = f.values.data();
        f.offsets.clear();
      }
    } catch (const std::bad_alloc&) {
      PQ_FAIL(kFormat, "row group too large to hold in memory");
    }
    f.r_null_count = 0;
  }

  // PLAIN values of the column's type from c into the dictionary or the output
  void plain_fixed(Cur& c, uint8_t* dst, int64_t n) {
    if (col.type == P_BOOLEAN) {
      const uint8_t* q = c.take((n + 7) / 8);
      for (int64_t k = 0; k < n; ++k) dst[k] = (q[k >> 3] >> (k & 7)) & 1;
    } else {
      const size_t nb = static_cast<size_t>(n) * width;
      memcpy(dst, c.take(nb), nb);
    }
  }

  void read_dictionary(Cur c, const PageHeader& h) {
    if (h.encoding != 0 && h.encoding != 2) PQ_FAIL(kUnsupported, std::string("dictionary encoded as ") + encoding_name(h.encoding));
    if (h.num_values < 0 || static_cast<uint64_t>(h.num_values) > c.left() * 8 + 1)
      PQ_FAIL(kFormat, "dictionary declares more values than it could hold");
    dict_count = h.num_values;
    if (bytes_like) {
      f.dict_offsets.assign(dict_count + 1, 0);
      f.dict_bytes.clear();
      f.dict_bytes.reserve(c.left());
      for (int64_t k = 0; k < dict_count; ++k) {
        const uint32_t len = c.le32();
        const uint8_t* q = c.take(len);
        f.dict_bytes.insert(f.dict_bytes.end(), q, q + len);
        f.dict_offsets[k + 1] = static_cast<int64_t>(f.dict_bytes.size());
      }
    } else {
      if (col.type == P_BOOLEAN) PQ_FAIL(kFormat, "dictionary of booleans");
      f.dict_bytes.resize(static_cast<size_t>(dict_count) * width);
      plain_fixed(c, f.dict_bytes.data(), dict_count);
    }
    have_dict = true;
  }

  void put_bytes(int64_t row, const uint8_t* q, size_t len) {
    f.values.insert(f.values.end(), q, q + len);
    f.offsets[row + 1] = static_cast<int64_t>(f.values.size());
  }

  // Decodes `present` values from c (encoding enc) into the rows of [filled, filled + n) whose level is set.
  void read_values(Cur c, int enc, int64_t n, int64_t present, const uint8_t* defined) {
    // rows of this page, in order; defined == nullptr means all present
    auto for_rows = [&](auto&& emit) {
      int64_t v = 0;
      for (int64_t k = 0; k < n; ++k) {
        const int64_t row = filled + k;
        if (defined && !defined[k]) {
          nul[row] = 1;
          ++f.r_null_count;
          if (bytes_like) f.offsets[row + 1] = static_cast<int64_t>(f.values.size());
          continue;
        }
        emit(row, v++);
      }
    };
    if (enc == 0) {   // PLAIN
      if (bytes_like) {
        for_rows([&](int64_t row, int64_t) {
          const uint32_t len = c.le32();
          put_bytes(row, c.take(len), len);
        });
      } else if (col.type == P_BOOLEAN) {
        const uint8_t* q = c.take((present + 7) / 8);
        for_rows([&](int64_t row, int64_t v) { out[row] = (q[v >> 3] >> (v & 7)) & 1; });
      } else {
        const uint8_t* q = c.take(static_cast<size_t>(present) * width);
        if (!defined) memcpy(out + static_cast<size_t>(filled) * width, q, static_cast<size_t>(present) * width);
        else for_rows([&](int64_t row, int64_t v) { memcpy(out + row * width, q + v * width, width); });
      }
    } else if (enc == 2 || enc == 8) {   // dictionary indices
      if (!have_dict) PQ_FAIL(kFormat, "dictionary-encoded page without a dictionary");
      const int bw = c.byte();
      if (bw > 32) PQ_FAIL(kFormat, "dictionary index wider than 32 bits");
      f.idx.resize(present);
      Hybrid h{c, bw};
      h.read(f.idx.data(), present);
      for (int64_t k = 0; k < present; ++k)
        if (f.idx[k] >= static_cast<uint64_t>(dict_count)) PQ_FAIL(kFormat, "dictionary index out of range");
      if (bytes_like) {
        for_rows([&](int64_t row, int64_t v) {
          const int64_t a = f.dict_offsets[f.idx[v]], b = f.dict_offsets[f.idx[v] + 1];
          put_bytes(row, f.dict_bytes.data() + a, static_cast<size_t>(b - a));
        });
      } else {
        for_rows([&](int64_t row, int64_t v) {
          memcpy(out + row * width, f.dict_bytes.data() + static_cast<size_t>(f.idx[v]) * width, width);
        });
      }
    } else if (enc == 3) {   // RLE booleans: 4-byte length, then runs of width 1
      if (col.type != P_BOOLEAN) PQ_FAIL(kUnsupported, "RLE values of a column that is not BOOLEAN");
      const uint32_t len = c.le32();
      Cur sub{c.take(len), nullptr};
      sub.end = sub.p + len;
      f.idx.resize(present);
      Hybrid h{sub, 1};
      h.read(f.idx.data(), present);
      for_rows([&](int64_t row, int64_t v) { out[row] = static_cast<uint8_t>(f.idx[v]); });
    } else if (enc == 5) {   // DELTA_BINARY_PACKED
      if (col.type != P_INT32 && col.type != P_INT64) PQ_FAIL(kUnsupported, "DELTA_BINARY_PACKED values of a column that is not an integer");
      delta_decode(c, tmp64, present);
      if (static_cast<int64_t>(tmp64.size()) != present) PQ_FAIL(kFormat, "delta stream with a different count than the page");
      if (col.type == P_INT32)
        for_rows([&](int64_t row, int64_t v) { const int32_t x = static_cast<int32_t>(tmp64[v]); memcpy(out + row * 4, &x, 4); });
      else
        for_rows([&](int64_t row, int64_t v) { memcpy(out + row * 8, &tmp64[v], 8); });
    } else if (enc == 6) {   // DELTA_LENGTH_BYTE_ARRAY
      if (!bytes_like) PQ_FAIL(kUnsupported, "DELTA_LENGTH_BYTE_ARRAY values of a column that is not BYTE_ARRAY");
      delta_decode(c, tmp64, present);
      if (static_cast<int64_t>(tmp64.size()) != present) PQ_FAIL(kFormat, "length stream with a different count than the page");
      for_rows([&](int64_t row, int64_t v) {
        if (tmp64[v] < 0) PQ_FAIL(kFormat, "negative length");
        put_bytes(row, c.take(tmp64[v]), tmp64[v]);
      });
    } else if (enc == 7) {   // DELTA_BYTE_ARRAY: shared prefix lengths, then suffixes
      if (!bytes_like && col.type != P_FLBA) PQ_FAIL(kUnsupported, "DELTA_BYTE_ARRAY values of a column that holds no bytes");
      delta_decode(c, tmp64, present);
      delta_decode(c, tmp64b, present);
      if (static_cast<int64_t>(tmp64.size()) != present || static_cast<int64_t>(tmp64b.size()) != present)
        PQ_FAIL(kFormat, "prefix / suffix streams with a different count than the page");
      std::string prev, cur;
      for_rows([&](int64_t row, int64_t v) {
        const int64_t pl = tmp64[v], sl = tmp64b[v];
        if (pl < 0 || sl < 0 || static_cast<size_t>(pl) > prev.size()) PQ_FAIL(kFormat, "prefix longer than the previous value");
        const uint8_t* q = c.take(sl);
        cur.assign(prev, 0, pl);
        cur.append(reinterpret_cast<const char*>(q), sl);
        if (bytes_like) put_bytes(row, reinterpret_cast<const uint8_t*>(cur.data()), cur.size());
        else {
          if (static_cast<int>(cur.size()) != width) PQ_FAIL(kFormat, "fixed-length value of another length");
          memcpy(out + row * width, cur.data(), width);
        }
        prev.swap(cur);
      });
    } else if (enc == 9) {   // BYTE_STREAM_SPLIT
      if (bytes_like || col.type == P_BOOLEAN) PQ_FAIL(kUnsupported, "BYTE_STREAM_SPLIT values of a column without a fixed width");
      const uint8_t* q = c.take(static_cast<size_t>(present) * width);
      for_rows([&](int64_t row, int64_t v) {
        uint8_t* d = out + row * width;
        for (int b = 0; b < width; ++b) d[b] = q[static_cast<size_t>(b) * present + v];
      });
    } else {
      PQ_FAIL(kUnsupported, std::string("encoding ") + encoding_name(enc));
    }
  }

  // definition levels of n values -> f.levels (1 = present); returns how many are present
  int64_t read_levels(Cur c, int64_t n, int encoding) {
    f.levels.resize(n);
    if (encoding == 3) {
      f.idx.resize(n);
      Hybrid h{c, 1};
      h.read(f.idx.data(), n);
      int64_t present = 0;
      for (int64_t k = 0; k < n; ++k) { f.levels[k] = static_cast<uint8_t>(f.idx[k]); present += f.idx[k]; }
      return present;
    }
    if (encoding == 4) {   // deprecated BIT_PACKED: most significant bit first
      const uint8_t* q = c.take((n + 7) / 8);
      int64_t present = 0;
      for (int64_t k = 0; k < n; ++k) { f.levels[k] = (q[k >> 3] >> (7 - (k & 7))) & 1; present += f.levels[k]; }
      return present;
    }
    PQ_FAIL(kUnsupported, std::string("definition levels encoded as ") + encoding_name(encoding));
  }

  void run() {
    prepare();
    f.r_type = col.type;
    f.r_count = rows;
    if (rows == 0) return;   // nothing to decode; such a chunk may have no page at all
    int64_t start = ch.dict_page_offset > 0 && ch.dict_page_offset < ch.data_page_offset ? ch.dict_page_offset : ch.data_page_offset;
    if (start < 4 || static_cast<uint64_t>(start) >= f.size) PQ_FAIL(kFormat, "column chunk outside the file");
    if (ch.total_compressed < 0 || static_cast<uint64_t>(ch.total_compressed) > f.size - start)
      PQ_FAIL(kFormat, "column chunk longer than the file");
    Cur c{f.map + start, f.map + start + ch.total_compressed};
    int64_t values_seen = 0;
    while (filled < rows) {
      if (c.left() == 0) PQ_FAIL(kFormat, "column chunk ends before its rows");
      Thrift t{c};
      PageHeader h;
      parse_page_header(t, h);
      c = t.c;
      if (h.compressed < 0 || h.uncompressed < 0 || static_cast<uint64_t>(h.compressed) > c.left())
        PQ_FAIL(kFormat, "page longer than its column chunk");
      const uint8_t* body = c.take(h.compressed);
      if (h.type == 2) {   // dictionary page
        if (!h.has_sub) PQ_FAIL(kFormat, "dictionary page without its header");
        if (have_dict) PQ_FAIL(kFormat, "second dictionary page");
        read_dictionary(decompress(ch.codec, body, h.compressed, h.uncompressed, f.page), h);
        continue;
      }
      if (h.type == 1) continue;   // index page
      if (h.type != 0 && h.type != 3) PQ_FAIL(kFormat, "unknown page type");
      if (!h.has_sub) PQ_FAIL(kFormat, "data page without its header");
      const int64_t n = h.num_values;
      if (n < 0 || n > rows - filled) PQ_FAIL(kFormat, "page declares more values than the row group has left");
      const uint8_t* defined = nullptr;
      int64_t present = n;
      if (h.type == 0) {
        Cur d = decompress(ch.codec, body, h.compressed, h.uncompressed, f.page);
        if (col.nullable) {
          Cur lv = d;
          if (h.def_encoding == 3) {
            const uint32_t len = d.le32();
            lv = Cur{d.take(len), nullptr};
            lv.end = lv.p + len;
          } else {
            lv = Cur{d.take((n + 7) / 8), nullptr};
            lv.end = lv.p + (n + 7) / 8;
          }
          present = read_levels(lv, n, h.def_encoding);
          defined = f.levels.data();
        }
        read_values(d, h.encoding, n, present, defined);
      } else {
        if (h.rep_bytes != 0) PQ_FAIL(kUnsupported, "repetition levels (nested column)");
        if (h.def_bytes < 0 || h.def_bytes > h.compressed || h.def_bytes > h.uncompressed) PQ_FAIL(kFormat, "levels longer than their page");
        if (col.nullable) {
          if (h.def_bytes > 0) {
            present = read_levels(Cur{body, body + h.def_bytes}, n, 3);
            defined = f.levels.data();
          }
          if (h.num_nulls >= 0 && n - present != h.num_nulls) PQ_FAIL(kFormat, "null count differs from the levels");
        } else if (h.def_bytes != 0) {
          PQ_FAIL(kFormat, "definition levels of a required column");
        }
        const uint8_t* vb = body + h.def_bytes;
        const size_t vn = static_cast<size_t>(h.compressed - h.def_bytes), vu = static_cast<size_t>(h.uncompressed - h.def_bytes);
        Cur d = h.v2_compressed ? decompress(ch.codec, vb, vn, vu, f.page) : decompress(0, vb, vn, vu, f.page);
        read_values(d, h.encoding, n, present, defined);
      }
      filled += n;
      values_seen += n;
    }
    (void)values_seen;
    f.r_type = col.type;
    f.r_count = rows;
  }
};

static void open_file(File& f, const char* path) {
  f.fd = ::open(path, O_RDONLY);
  if (f.fd < 0) PQ_FAIL(kIo, std::string("cannot open ") + path);
  struct stat st;
  if (fstat(f.fd, &st) != 0) PQ_FAIL(kIo, "cannot stat the file");
  f.size = static_cast<size_t>(st.st_size);
  if (f.size < 12) PQ_FAIL(kFormat, "file shorter than a Parquet header and footer");
  void* m = mmap(nullptr, f.size, PROT_READ, MAP_PRIVATE, f.fd, 0);
  if (m == MAP_FAILED) PQ_FAIL(kIo, "cannot map the file");
  f.map = static_cast<const uint8_t*>(m);
  if (memcmp(f.map + f.size - 4, "PARE", 4) == 0) PQ_FAIL(kUnsupported, "encrypted file");
  if (memcmp(f.map, "PAR1", 4) != 0 || memcmp(f.map + f.size - 4, "PAR1", 4) != 0) PQ_FAIL(kFormat, "not a Parquet file (magic)");
  uint32_t flen;
  memcpy(&flen, f.map + f.size - 8, 4);
  if (flen == 0 || static_cast<size_t>(flen) > f.size - 12) PQ_FAIL(kFormat, "footer longer than the file");
  parse_footer(f, f.map + f.size - 8 - flen, flen);
}

static void close_file(File* f) {
  if (!f) return;
  if (f->map) munmap(const_cast<uint8_t*>(f->map), f->size);
  if (f->fd >= 0) ::close(f->fd);
  delete f;
}

static thread_local std::string g_open_error;

template <typename Fn>
static int guard(File* f, Fn&& fn) {
  try {
    fn();
    return kOk;
  } catch (const Error& e) {
    (f ? f->error : g_open_error) = e.text;
    return e.code;
  } catch (const std::bad_alloc&) {
    (f ? f->error : g_open_error) = "out of memory";
    return kFormat;
  } catch (const std::exception& e) {
    (f ? f->error : g_open_error) = e.what();
    return kFormat;
  }
}

}  // namespace pq
}  // namespace mimir

using namespace mimir::pq;

// Status codes: 0 ok, 1 malformed file, 2 unsupported feature, 3 I/O, 4 bad argument.
MIMIR_API int mimir_pq_open(const char* path, void** out) {
  *out = nullptr;
  File* f = new (std::nothrow) File();
  if (!f) return kIo;
  const int rc = guard(nullptr, [&] { open_file(*f, path); });
  if (rc != kOk) { close_file(f); return rc; }
  *out = f;
  return kOk;
}

MIMIR_API void mimir_pq_close(void* h) { close_file(static_cast<File*>(h)); }

// Message of the last failed call on this handle (or of the last failed open on this thread when h is null).
MIMIR_API const char* mimir_pq_last_error(void* h) {
  return h ? static_cast<File*>(h)->error.c_str() : g_open_error.c_str();
}

MIMIR_API int mimir_pq_counts(void* h, long long* rows, int* groups, int* columns) {
  File* f = static_cast<File*>(h);
  *rows = f->rows;
  *groups = static_cast<int>(f->groups.size());
  *columns = static_cast<int>(f->cols.size());
  return kOk;
}

// info: [type, type_length, nullable, nested, converted type, scale, precision]
MIMIR_API int mimir_pq_column(void* h, int i, char* name, int name_cap, char* logical, int logical_cap, int* info) {
  File* f = static_cast<File*>(h);
  if (i < 0 || i >= static_cast<int>(f->cols.size())) return kArgument;
  const Column& c = f->cols[i];
  snprintf(name, name_cap, "%s", c.name.c_str());
  snprintf(logical, logical_cap, "%s", c.logical.c_str());
  info[0] = c.type; info[1] = c.type_length; info[2] = c.nullable; info[3] = c.nested;
  info[4] = c.converted; info[5] = c.scale; info[6] = c.precision;
  return kOk;
}

MIMIR_API long long mimir_pq_group_rows(void* h, int g) {
  File* f = static_cast<File*>(h);
  return g >= 0 && g < static_cast<int>(f->groups.size()) ? f->groups[g].rows : -1;
}

// i == -1: created_by in `key`; otherwise the i-th key/value pair.  Returns the number of pairs.
MIMIR_API int mimir_pq_meta(void* h, int i, const char** key, long long* key_len, const char** val, long long* val_len) {
  File* f = static_cast<File*>(h);
  if (i == -1) { *key = f->created_by.data(); *key_len = static_cast<long long>(f->created_by.size()); }
  else if (i >= 0 && i < static_cast<int>(f->kv.size())) {
    *key = f->kv[i].first.data(); *key_len = static_cast<long long>(f->kv[i].first.size());
    *val = f->kv[i].second.data(); *val_len = static_cast<long long>(f->kv[i].second.size());
  }
  return static_cast<int>(f->kv.size());
}

// Decodes column `column` of row group `group` into the handle's buffers.
MIMIR_API int mimir_pq_decode(void* h, int group, int column) {
  File* f = static_cast<File*>(h);
  return guard(f, [&] {
    if (group < 0 || group >= static_cast<int>(f->groups.size())) PQ_FAIL(kArgument, "no such row group");
    if (column < 0 || column >= static_cast<int>(f->cols.size())) PQ_FAIL(kArgument, "no such column");
    const Column& c = f->cols[column];
    const Chunk& k = f->groups[group].chunks[column];
    if (c.nested) PQ_FAIL(kUnsupported, "nested column " + c.name);
    if (c.type == P_INT96) PQ_FAIL(kUnsupported, "INT96 column " + c.name);
    if (c.type < 0 || c.type > P_FLBA) PQ_FAIL(kFormat, "unknown physical type");
    if (c.type == P_FLBA && (c.type_length <= 0 || c.type_length > (1 << 20))) PQ_FAIL(kFormat, "fixed-length column without a length");
    if (k.encrypted) PQ_FAIL(kUnsupported, "encrypted column " + c.name);
    if (k.external) PQ_FAIL(kUnsupported, "column chunk in another file");
    if (!k.has_meta) PQ_FAIL(kFormat, "column chunk without metadata");
    if (k.type != c.type) PQ_FAIL(kFormat, "column chunk of another type than the schema");
    Decoder d(*f, c, k, f->groups[group].rows);
    d.run();
  });
}

// Decodes a fixed-width column straight into the caller's memory: `values` holds rows x width bytes
// (booleans one byte each), `nulls` rows bytes (may be null for a required column: then nulls are not
// reported).  Returns the status; *null_count gets the number of nulls.
MIMIR_API int mimir_pq_decode_into(void* h, int group, int column, void* values, long long value_bytes,
                                   unsigned char* nulls, long long* null_count) {
  File* f = static_cast<File*>(h);
  const int rc = guard(f, [&] {
    if (group < 0 || group >= static_cast<int>(f->groups.size())) PQ_FAIL(kArgument, "no such row group");
    if (column < 0 || column >= static_cast<int>(f->cols.size())) PQ_FAIL(kArgument, "no such column");
    const Column& c = f->cols[column];
    const int w = width_of(c.type, c.type_length);
    if (c.type == P_BYTE_ARRAY || w <= 0) PQ_FAIL(kArgument, "column without a fixed width");
    if (value_bytes != f->groups[group].rows * w) PQ_FAIL(kArgument, "destination of another size than the column chunk");
    f->ext_values = static_cast<uint8_t*>(values);
    f->ext_nulls = nulls;
  });
  if (rc != kOk) return rc;
  const int rc2 = mimir_pq_decode(h, group, column);
  f->ext_values = nullptr;
  f->ext_nulls = nullptr;
  *null_count = f->r_null_count;
  return rc2;
}

// Pointers into the handle's buffers, valid until the next decode or close.
// values: fixed width -> count x width bytes (booleans one byte each); BYTE_ARRAY -> the bytes, with offsets[count + 1].
MIMIR_API int mimir_pq_result(void* h, int* type, long long* count, const void** values, long long* value_bytes,
                              const long long** offsets, const unsigned char** nulls, long long* null_count) {
  File* f = static_cast<File*>(h);
  *type = f->r_type;
  *count = f->r_count;
  *values = f->values.data();
  *value_bytes = static_cast<long long>(f->values.size());
  *offsets = reinterpret_cast<const long long*>(f->offsets.data());
  *nulls = f->nulls.data();
  *null_count = f->r_null_count;
  return kOk;
}
