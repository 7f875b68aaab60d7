// safetensors container: memory-mapped reader with a small JSON parser, and a writer.
//
// File layout: u64 little-endian header length N, N bytes of JSON
//   { "name": {"dtype": "BF16", "shape": [..], "data_offsets": [begin, end]}, ..., "__metadata__": {...} }
// followed by the tensor bytes; offsets are relative to the end of the header.
// Reference counterparts: common/safetensors.h:35-86 (reader + JSON, :329-432) and common/safetensors_writer.h.
#include "common.h"
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace gbh {

struct StTensor { std::string name, dtype; std::vector<int64_t> shape; uint64_t begin = 0, end = 0; };

struct StFile {
  int fd = -1; const uint8_t* map = nullptr; size_t size = 0; size_t data_start = 0;
  std::vector<StTensor> tensors; std::map<std::string, int> index;
  std::map<std::string, std::string> metadata; std::string header;
  ~StFile() { if (map) munmap((void*)map, size); if (fd >= 0) close(fd); }
};

// Minimal recursive-descent JSON reader over the subset safetensors headers use.
struct Json {
  const char* p; const char* end; bool ok = true;
  void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool eat(char c) { ws(); if (p < end && *p == c) { ++p; return true; } return false; }
  bool str(std::string& out) {
    ws();
    if (p >= end || *p != '"') return ok = false;
    ++p; out.clear();
    while (p < end && *p != '"') {
      if (*p == '\\' && p + 1 < end) {
        ++p;
        switch (*p) {
          case 'n': out.push_back('\n'); break; case 't': out.push_back('\t'); break; case 'r': out.push_back('\r'); break;
          case 'b': out.push_back('\b'); break; case 'f': out.push_back('\f'); break;
          case 'u': {
            if (p + 4 >= end) return ok = false;
            unsigned cp = 0;
            for (int i = 1; i <= 4; ++i) { const char c = p[i]; cp = cp * 16 + (c >= '0' && c <= '9' ? c - '0' : (c | 32) - 'a' + 10); }
            p += 4;
            if (cp < 0x80) out.push_back((char)cp);
            else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
            else { out.push_back((char)(0xE0 | (cp >> 12))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F))); }
            break;
          }
          default: out.push_back(*p);
        }
        ++p;
      } else out.push_back(*p++);
    }
    if (p >= end) return ok = false;
    ++p;
    return true;
  }
  bool integer(int64_t& v) {
    ws();
    const char* s = p; bool neg = false;
    if (p < end && *p == '-') { neg = true; ++p; }
    if (p >= end || *p < '0' || *p > '9') { p = s; return ok = false; }
    v = 0;
    while (p < end && *p >= '0' && *p <= '9') v = v * 10 + (*p++ - '0');
    if (neg) v = -v;
    return true;
  }
  // skips any value
  bool skip() {
    ws();
    if (p >= end) return ok = false;
    if (*p == '"') { std::string s; return str(s); }
    if (*p == '{' || *p == '[') {
      const char open = *p, close = open == '{' ? '}' : ']';
      ++p;
      if (eat(close)) return true;
      do {
        if (open == '{') { std::string k; if (!str(k) || !eat(':')) return ok = false; }
        if (!skip()) return false;
      } while (eat(','));
      return eat(close) ? true : (ok = false);
    }
    while (p < end && *p != ',' && *p != '}' && *p != ']') ++p;
    return true;
  }
};

static int parse_header(StFile* f) {
  Json j{f->header.data(), f->header.data() + f->header.size()};
  if (!j.eat('{')) return fail("safetensors: header is not a JSON object");
  if (j.eat('}')) return 0;
  do {
    std::string name;
    if (!j.str(name) || !j.eat(':')) return fail("safetensors: malformed header near byte %ld", (long)(j.p - f->header.data()));
    if (name == "__metadata__") {
      if (!j.eat('{')) return fail("safetensors: __metadata__ is not an object");
      if (!j.eat('}')) {
        do {
          std::string k, v;
          if (!j.str(k) || !j.eat(':')) return fail("safetensors: malformed __metadata__");
          j.ws();
          if (j.p < j.end && *j.p == '"') { if (!j.str(v)) return fail("safetensors: malformed __metadata__ value"); f->metadata[k] = v; }
          else if (!j.skip()) return fail("safetensors: malformed __metadata__ value");
        } while (j.eat(','));
        if (!j.eat('}')) return fail("safetensors: unterminated __metadata__");
      }
      continue;
    }
    StTensor t; t.name = name;
    if (!j.eat('{')) return fail("safetensors: entry %s is not an object", name.c_str());
    do {
      std::string k;
      if (!j.str(k) || !j.eat(':')) return fail("safetensors: malformed entry %s", name.c_str());
      if (k == "dtype") { if (!j.str(t.dtype)) return fail("safetensors: bad dtype of %s", name.c_str()); }
      else if (k == "shape") {
        if (!j.eat('[')) return fail("safetensors: bad shape of %s", name.c_str());
        if (!j.eat(']')) { do { int64_t v; if (!j.integer(v)) return fail("safetensors: bad shape of %s", name.c_str()); t.shape.push_back(v); } while (j.eat(',')); if (!j.eat(']')) return fail("safetensors: bad shape of %s", name.c_str()); }
      } else if (k == "data_offsets") {
        int64_t a, b;
        if (!j.eat('[') || !j.integer(a) || !j.eat(',') || !j.integer(b) || !j.eat(']')) return fail("safetensors: bad data_offsets of %s", name.c_str());
        t.begin = (uint64_t)a; t.end = (uint64_t)b;
      } else if (!j.skip()) return fail("safetensors: malformed entry %s", name.c_str());
    } while (j.eat(','));
    if (!j.eat('}')) return fail("safetensors: unterminated entry %s", name.c_str());
    if (t.end < t.begin || f->data_start + t.end > f->size) return fail("safetensors: tensor %s runs past the end of the file", name.c_str());
    f->index[t.name] = (int)f->tensors.size();
    f->tensors.push_back(std::move(t));
  } while (j.eat(','));
  if (!j.eat('}')) return fail("safetensors: unterminated header");
  return 0;
}

}  // namespace gbh

using namespace gbh;

GBH_API void* gbh_st_open(const char* path) {
  std::unique_ptr<StFile> f(new StFile());
  f->fd = open(path, O_RDONLY);
  if (f->fd < 0) { fail("safetensors: cannot open %s", path); return nullptr; }
  struct stat st;
  if (fstat(f->fd, &st) != 0 || st.st_size < 8) { fail("safetensors: %s is too small", path); return nullptr; }
  f->size = (size_t)st.st_size;
  void* m = mmap(nullptr, f->size, PROT_READ, MAP_PRIVATE, f->fd, 0);
  if (m == MAP_FAILED) { fail("safetensors: mmap of %s failed", path); return nullptr; }
  f->map = (const uint8_t*)m;
  uint64_t n; memcpy(&n, f->map, 8);
  if (n > f->size - 8 || n > (1ull << 30)) { fail("safetensors: implausible header length in %s", path); return nullptr; }
  f->header.assign((const char*)f->map + 8, n);
  f->data_start = 8 + n;
  if (parse_header(f.get()) != 0) return nullptr;
  return f.release();
}
GBH_API void gbh_st_close(void* h) { delete (StFile*)h; }
GBH_API long gbh_st_count(void* h) { return (long)((StFile*)h)->tensors.size(); }
GBH_API int gbh_st_find(void* h, const char* name) { auto* f = (StFile*)h; auto it = f->index.find(name); return it == f->index.end() ? -1 : it->second; }
GBH_API int gbh_st_info(void* h, int i, char* name, int name_cap, char* dtype8, int* n_dims, int64_t* shape8, uint64_t* nbytes) {
  auto* f = (StFile*)h;
  if (i < 0 || i >= (int)f->tensors.size()) return fail("safetensors: index %d out of range", i);
  const StTensor& t = f->tensors[i];
  if (name) snprintf(name, name_cap, "%s", t.name.c_str());
  snprintf(dtype8, 8, "%s", t.dtype.c_str());
  *n_dims = (int)t.shape.size();
  for (size_t d = 0; d < t.shape.size() && d < 8; ++d) shape8[d] = t.shape[d];
  *nbytes = t.end - t.begin;
  return 0;
}
GBH_API const void* gbh_st_data(void* h, int i) {
  auto* f = (StFile*)h;
  if (i < 0 || i >= (int)f->tensors.size()) return nullptr;
  return f->map + f->data_start + f->tensors[i].begin;
}
GBH_API const char* gbh_st_metadata(void* h, const char* key) {
  auto* f = (StFile*)h; auto it = f->metadata.find(key);
  return it == f->metadata.end() ? nullptr : it->second.c_str();
}

// Writer: names / dtypes are NUL-terminated strings, shapes are flattened with ranks[i] entries each.
GBH_API int gbh_st_write(const char* path, int n, const char* const* names, const char* const* dtypes, const int* ranks, const int64_t* shapes,
                         const void* const* data, const uint64_t* nbytes) {
  std::string hdr = "{";
  uint64_t off = 0; const int64_t* sp = shapes;
  for (int i = 0; i < n; ++i) {
    if (i) hdr += ",";
    hdr += "\"" + std::string(names[i]) + "\":{\"dtype\":\"" + dtypes[i] + "\",\"shape\":[";
    for (int d = 0; d < ranks[i]; ++d) { if (d) hdr += ","; hdr += std::to_string(*sp++); }
    hdr += "],\"data_offsets\":[" + std::to_string(off) + "," + std::to_string(off + nbytes[i]) + "]}";
    off += nbytes[i];
  }
  hdr += "}";
  while (hdr.size() % 8) hdr += " ";
  FILE* fp = fopen(path, "wb");
  if (!fp) return fail("safetensors: cannot create %s", path);
  const uint64_t hl = hdr.size();
  bool ok = fwrite(&hl, 8, 1, fp) == 1 && fwrite(hdr.data(), 1, hdr.size(), fp) == hdr.size();
  for (int i = 0; ok && i < n; ++i) ok = fwrite(data[i], 1, nbytes[i], fp) == nbytes[i];
  ok = (fclose(fp) == 0) && ok;
  return ok ? 0 : fail("safetensors: short write to %s", path);
}
