// Reader for .safetensors checkpoint files: the input of Module::update_by_safetensors
// (rai-core/src/nn.rs:39-55), which reads each file whole (std::fs::read), deserialises it and copies
// every view into a Vec (rai-core/src/hlops/from_safetensor.rs:51-91).  Here the file is mapped
// read-only and the views point into the mapping: no host copy happens until a tensor is staged for
// its upload.  Host code only; nothing here touches the GPU.
//
// File layout: 8 bytes little-endian N, N bytes of JSON
//   { "<name>": {"dtype": "BF16", "shape": [r, c], "data_offsets": [begin, end]}, ..., "__metadata__": {...} }
// then the data area; offsets are relative to its start.
#include <fcntl.h>
#include <stdint.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <string>
#include <vector>

#include "ctx.h"

using namespace rb;

struct rb_safetensors {
  struct Entry {
    std::string name;
    int32_t dtype = -1;  // RB_* tag, or -1 for a dtype this library has no tag for
    std::string dtype_name;
    int32_t rank = 0;
    int64_t shape[8] = {};
    uint64_t begin = 0, end = 0;
  };
  int fd = -1;
  void* map = nullptr;
  size_t size = 0;
  size_t data_start = 0;
  std::vector<Entry> entries;
};

namespace {

constexpr uint64_t kMaxHeaderBytes = 100000000ull;  // the format's own cap on the JSON header

struct Json {
  const char* p;
  const char* end;
  std::string err;

  void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\r' || *p == '\t')) ++p; }
  bool fail(const char* what) { if (err.empty()) err = what; return false; }
  bool expect(char c) {
    ws();
    if (p < end && *p == c) { ++p; return true; }
    return fail("unexpected character in the header");
  }
  bool peek(char c) { ws(); return p < end && *p == c; }

  static void utf8(std::string& out, uint32_t cp) {
    if (cp < 0x80) out.push_back((char)cp);
    else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
    else if (cp < 0x10000) {
      out.push_back((char)(0xE0 | (cp >> 12))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
      out.push_back((char)(0x80 | (cp & 0x3F)));
    } else {
      out.push_back((char)(0xF0 | (cp >> 18))); out.push_back((char)(0x80 | ((cp >> 12) & 0x3F)));
      out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F)));
    }
  }
  bool hex4(uint32_t& v) {
    if (end - p < 4) return fail("truncated \\u escape");
    v = 0;
    for (int i = 0; i < 4; ++i, ++p) {
      const char c = *p;
      v <<= 4;
      if (c >= '0' && c <= '9') v |= (uint32_t)(c - '0');
      else if (c >= 'a' && c <= 'f') v |= (uint32_t)(c - 'a' + 10);
      else if (c >= 'A' && c <= 'F') v |= (uint32_t)(c - 'A' + 10);
      else return fail("bad \\u escape");
    }
    return true;
  }
  bool string(std::string& out) {
    out.clear();
    if (!expect('"')) return false;
    while (p < end) {
      const char c = *p++;
      if (c == '"') return true;
      if (c != '\\') { out.push_back(c); continue; }
      if (p >= end) break;
      const char e = *p++;
      switch (e) {
        case '"': out.push_back('"'); break;
        case '\\': out.push_back('\\'); break;
        case '/': out.push_back('/'); break;
        case 'b': out.push_back('\b'); break;
        case 'f': out.push_back('\f'); break;
        case 'n': out.push_back('\n'); break;
        case 'r': out.push_back('\r'); break;
        case 't': out.push_back('\t'); break;
        case 'u': {
          uint32_t cp;
          if (!hex4(cp)) return false;
          if (cp >= 0xD800 && cp < 0xDC00 && end - p >= 6 && p[0] == '\\' && p[1] == 'u') {
            p += 2;
            uint32_t lo;
            if (!hex4(lo)) return false;
            cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
          }
          utf8(out, cp);
          break;
        }
        default: return fail("bad escape in a header string");
      }
    }
    return fail("unterminated string in the header");
  }
  bool uint(uint64_t& v) {
    ws();
    if (p >= end || *p < '0' || *p > '9') return fail("expected a non-negative integer in the header");
    v = 0;
    while (p < end && *p >= '0' && *p <= '9') {
      if (v > (UINT64_MAX - 9) / 10) return fail("integer overflow in the header");
      v = v * 10 + (uint64_t)(*p++ - '0');
    }
    if (p < end && (*p == '.' || *p == 'e' || *p == 'E')) return fail("expected an integer in the header");
    return true;
  }
  // any value, discarded (the "__metadata__" map, unknown keys)
  bool skip(int depth = 0) {
    if (depth > 32) return fail("header nested too deeply");
    ws();
    if (p >= end) return fail("truncated header");
    if (*p == '"') { std::string s; return string(s); }
    if (*p == '{' || *p == '[') {
      const char close = *p == '{' ? '}' : ']';
      const bool obj = *p == '{';
      ++p;
      if (peek(close)) { ++p; return true; }
      while (true) {
        if (obj) { std::string k; if (!string(k) || !expect(':')) return false; }
        if (!skip(depth + 1)) return false;
        if (peek(',')) { ++p; continue; }
        return expect(close);
      }
    }
    const char* q = p;
    while (p < end && *p != ',' && *p != '}' && *p != ']' && *p != ' ' && *p != '\n' && *p != '\r' && *p != '\t') ++p;
    return p > q ? true : fail("bad value in the header");
  }
};

struct DtypeName { const char* name; int32_t tag; int bytes; };
const DtypeName kDtypes[] = {
    {"F64", RB_F64, 8}, {"F32", RB_F32, 4}, {"F16", RB_F16, 2}, {"BF16", RB_BF16, 2}, {"I64", RB_I64, 8}, {"U32", RB_U32, 4},
    {"U8", RB_U8, 1},   {"I32", -1, 4},     {"I16", -1, 2},     {"U16", -1, 2},       {"I8", -1, 1},      {"BOOL", -1, 1},
    {"U64", -1, 8},     {"F8_E4M3", -1, 1}, {"F8_E5M2", -1, 1},
};

bool parse_entry(Json& j, rb_safetensors::Entry& e, int& elem_bytes) {
  bool have_dtype = false, have_shape = false, have_off = false;
  if (!j.expect('{')) return false;
  if (j.peek('}')) return j.fail("a tensor entry is empty");
  while (true) {
    std::string key;
    if (!j.string(key) || !j.expect(':')) return false;
    if (key == "dtype") {
      if (!j.string(e.dtype_name)) return false;
      elem_bytes = 0;
      for (const DtypeName& d : kDtypes)
        if (e.dtype_name == d.name) { e.dtype = d.tag; elem_bytes = d.bytes; }
      if (!elem_bytes) return j.fail("unknown dtype name in the header");
      have_dtype = true;
    } else if (key == "shape") {
      if (!j.expect('[')) return false;
      e.rank = 0;
      if (j.peek(']')) { ++j.p; }
      else {
        while (true) {
          uint64_t v;
          if (!j.uint(v)) return false;
          if (e.rank >= 8) return j.fail("a tensor has more than 8 dimensions");
          if (v > (uint64_t)INT64_MAX) return j.fail("a dimension overflows");
          e.shape[e.rank++] = (int64_t)v;
          if (j.peek(',')) { ++j.p; continue; }
          if (!j.expect(']')) return false;
          break;
        }
      }
      have_shape = true;
    } else if (key == "data_offsets") {
      if (!j.expect('[') || !j.uint(e.begin) || !j.expect(',') || !j.uint(e.end) || !j.expect(']')) return false;
      have_off = true;
    } else if (!j.skip()) {
      return false;
    }
    if (j.peek(',')) { ++j.p; continue; }
    if (!j.expect('}')) return false;
    break;
  }
  if (!(have_dtype && have_shape && have_off)) return j.fail("a tensor entry lacks dtype, shape or data_offsets");
  return true;
}

int close_with(rb_safetensors* st, int code) {
  rb_safetensors_close(st);
  return code;
}

}  // namespace

extern "C" int32_t rb_safetensors_open(const char* path, rb_safetensors** out) {
  RB_REQUIRE(path && out, "rb_safetensors_open: null argument");
  *out = nullptr;
  rb_safetensors* st = new rb_safetensors();
  st->fd = open(path, O_RDONLY);
  if (st->fd < 0) return close_with(st, fail(RB_ERR_INVALID, "safetensors: cannot open '%s'", path));
  struct stat sb;
  if (fstat(st->fd, &sb) != 0 || sb.st_size < 8)
    return close_with(st, fail(RB_ERR_INVALID, "safetensors: '%s' is shorter than its 8-byte header length", path));
  st->size = (size_t)sb.st_size;
  st->map = mmap(nullptr, st->size, PROT_READ, MAP_PRIVATE, st->fd, 0);
  if (st->map == MAP_FAILED) { st->map = nullptr; return close_with(st, fail(RB_ERR_INVALID, "safetensors: cannot map '%s'", path)); }
  const unsigned char* b = (const unsigned char*)st->map;
  uint64_t n = 0;
  for (int i = 7; i >= 0; --i) n = (n << 8) | b[i];
  if (n > kMaxHeaderBytes) return close_with(st, fail(RB_ERR_INVALID, "safetensors: '%s': header of %llu bytes is too large", path, (unsigned long long)n));
  if (n > st->size - 8) return close_with(st, fail(RB_ERR_INVALID, "safetensors: '%s': header length %llu exceeds the file", path, (unsigned long long)n));
  st->data_start = 8 + (size_t)n;
  const uint64_t data_bytes = st->size - st->data_start;

  Json j{(const char*)b + 8, (const char*)b + 8 + n, {}};
  bool ok = j.expect('{');
  if (ok && !j.peek('}')) {
    while (ok) {
      std::string key;
      ok = j.string(key) && j.expect(':');
      if (!ok) break;
      if (key == "__metadata__") ok = j.skip();
      else {
        rb_safetensors::Entry e;
        e.name = key;
        int elem = 0;
        ok = parse_entry(j, e, elem);
        if (ok) {
          // the view must lie inside the data area and hold exactly shape-many elements
          uint64_t numel = 1;
          bool overflow = false;
          for (int d = 0; d < e.rank; ++d) {
            if (e.shape[d] != 0 && numel > UINT64_MAX / (uint64_t)e.shape[d]) overflow = true;
            numel *= (uint64_t)e.shape[d];
          }
          if (overflow || numel > UINT64_MAX / (uint64_t)elem) ok = j.fail("a tensor's size overflows");
          else if (e.begin > e.end || e.end > data_bytes) ok = j.fail("a tensor's data_offsets lie outside the file");
          else if (e.end - e.begin != numel * (uint64_t)elem) ok = j.fail("a tensor's data_offsets do not match its shape and dtype");
          if (ok) st->entries.push_back(std::move(e));
        }
      }
      if (!ok) break;
      if (j.peek(',')) { ++j.p; continue; }
      ok = j.expect('}');
      break;
    }
  } else if (ok) {
    ++j.p;
  }
  if (ok) { j.ws(); if (j.p != j.end) ok = j.fail("trailing bytes after the header object"); }
  if (!ok) return close_with(st, fail(RB_ERR_INVALID, "safetensors: '%s': %s", path, j.err.c_str()));
  // file order of the data, which is the order a sequential reader wants
  std::stable_sort(st->entries.begin(), st->entries.end(),
                   [](const rb_safetensors::Entry& a, const rb_safetensors::Entry& c) { return a.begin < c.begin; });
  *out = st;
  return RB_OK;
}

extern "C" int32_t rb_safetensors_close(rb_safetensors* st) {
  if (!st) return RB_OK;
  if (st->map) munmap(st->map, st->size);
  if (st->fd >= 0) close(st->fd);
  delete st;
  return RB_OK;
}

extern "C" int32_t rb_safetensors_count(const rb_safetensors* st) { return st ? (int32_t)st->entries.size() : 0; }

extern "C" int32_t rb_safetensors_entry(const rb_safetensors* st, int32_t index, const char** name, int32_t* dtype,
                                        int32_t* rank, int64_t* shape8, const void** data, uint64_t* bytes) {
  RB_REQUIRE(st, "rb_safetensors_entry: null file");
  RB_REQUIRE(index >= 0 && index < (int32_t)st->entries.size(), "rb_safetensors_entry: index %d out of range", index);
  const rb_safetensors::Entry& e = st->entries[(size_t)index];
  if (name) *name = e.name.c_str();
  if (dtype) *dtype = e.dtype;
  if (rank) *rank = e.rank;
  if (shape8) for (int d = 0; d < 8; ++d) shape8[d] = d < e.rank ? e.shape[d] : 0;
  if (data) *data = (const char*)st->map + st->data_start + e.begin;
  if (bytes) *bytes = e.end - e.begin;
  return RB_OK;
}
