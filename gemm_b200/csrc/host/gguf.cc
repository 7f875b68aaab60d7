// GGUF container: reader (memory-mapped, versions 2 and 3) and writer.
//
// Layout (fixed by the file format; the reference parses it in common/gguf_loader.h:343-485 and has no
// writer): magic "GGUF", u32 version, u64 tensor count, u64 key/value count; key/values = string key,
// u32 value type, value (13 types, arrays may nest strings); tensor infos = name, u32 rank, u64 dims
// (innermost first), u32 ggml type, u64 offset into the data section; the data section starts at the next
// multiple of `general.alignment` (default 32) and every tensor is aligned to it.
#include "common.h"
#include "ggml_types.h"
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

enum KvType : uint32_t { KV_U8 = 0, KV_I8, KV_U16, KV_I16, KV_U32, KV_I32, KV_F32, KV_BOOL, KV_STR, KV_ARR, KV_U64, KV_I64, KV_F64 };

static size_t kv_scalar_size(uint32_t t) {
  switch (t) {
    case KV_U8: case KV_I8: case KV_BOOL: return 1;
    case KV_U16: case KV_I16: return 2;
    case KV_U32: case KV_I32: case KV_F32: return 4;
    case KV_U64: case KV_I64: case KV_F64: return 8;
    default: return 0;
  }
}

struct KvEntry {
  std::string key;
  uint32_t type = 0;
  uint32_t elem_type = 0;           // arrays
  uint64_t count = 0;               // arrays
  const uint8_t* data = nullptr;    // scalar bytes / first array element (numeric arrays) / string bytes
  uint64_t str_len = 0;             // strings
  std::vector<std::pair<const uint8_t*, uint64_t>> strs;   // string arrays
};

struct TensorEntry {
  std::string name;
  uint32_t n_dims = 0;
  uint64_t dims[4] = {1, 1, 1, 1};
  uint32_t type = 0;
  uint64_t offset = 0;
  uint64_t nbytes = 0;
};

struct GgufFile {
  int fd = -1;
  const uint8_t* map = nullptr;
  size_t size = 0;
  uint32_t version = 0;
  uint64_t alignment = 32;
  size_t data_start = 0;
  std::vector<KvEntry> kvs;
  std::vector<TensorEntry> tensors;
  std::map<std::string, int> kv_index, tensor_index;
  ~GgufFile() {
    if (map) munmap((void*)map, size);
    if (fd >= 0) close(fd);
  }
};

struct Cursor {
  const uint8_t* p; const uint8_t* end; bool ok = true;
  template <typename T> T get() {
    T v{};
    if (p + sizeof(T) > end) { ok = false; return v; }
    memcpy(&v, p, sizeof(T)); p += sizeof(T);
    return v;
  }
  bool str(const uint8_t** s, uint64_t* len) {
    *len = get<uint64_t>();
    if (!ok || *len > (uint64_t)(end - p)) { ok = false; return false; }
    *s = p; p += *len;
    return true;
  }
  bool skip(uint64_t n) { if (n > (uint64_t)(end - p)) { ok = false; return false; } p += n; return true; }
};

static int parse(GgufFile* f) {
  Cursor c{f->map, f->map + f->size};
  if (c.get<uint32_t>() != 0x46554747u) return fail("gguf: bad magic");
  f->version = c.get<uint32_t>();
  if (f->version < 2 || f->version > 3) return fail("gguf: unsupported version %u", f->version);
  const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
  if (!c.ok || n_tensors > (1u << 24) || n_kv > (1u << 24)) return fail("gguf: implausible header");
  f->kvs.reserve(n_kv);
  for (uint64_t i = 0; i < n_kv; ++i) {
    KvEntry e;
    const uint8_t* s; uint64_t len;
    if (!c.str(&s, &len)) return fail("gguf: truncated key %lu", (unsigned long)i);
    e.key.assign((const char*)s, len);
    e.type = c.get<uint32_t>();
    if (e.type == KV_STR) {
      if (!c.str(&e.data, &e.str_len)) return fail("gguf: truncated string value of %s", e.key.c_str());
    } else if (e.type == KV_ARR) {
      e.elem_type = c.get<uint32_t>(); e.count = c.get<uint64_t>();
      if (!c.ok) return fail("gguf: truncated array header of %s", e.key.c_str());
      if (e.elem_type == KV_STR) {
        if (e.count > (uint64_t)(c.end - c.p) / 8) return fail("gguf: implausible array length of %s", e.key.c_str());
        e.strs.reserve(e.count);
        for (uint64_t j = 0; j < e.count; ++j) {
          if (!c.str(&s, &len)) return fail("gguf: truncated string array %s", e.key.c_str());
          e.strs.emplace_back(s, len);
        }
      } else {
        const size_t es = kv_scalar_size(e.elem_type);
        if (!es) return fail("gguf: array %s has unsupported element type %u", e.key.c_str(), e.elem_type);
        e.data = c.p;
        if (e.count > (uint64_t)(c.end - c.p) / es || !c.skip(e.count * es)) return fail("gguf: truncated array %s", e.key.c_str());
      }
    } else {
      const size_t es = kv_scalar_size(e.type);
      if (!es) return fail("gguf: key %s has unknown value type %u", e.key.c_str(), e.type);
      e.data = c.p;
      if (!c.skip(es)) return fail("gguf: truncated value of %s", e.key.c_str());
    }
    f->kv_index[e.key] = (int)f->kvs.size();
    f->kvs.push_back(std::move(e));
  }
  auto it = f->kv_index.find("general.alignment");
  if (it != f->kv_index.end() && f->kvs[it->second].type == KV_U32) {
    uint32_t a; memcpy(&a, f->kvs[it->second].data, 4);
    if (a && (a & (a - 1)) == 0) f->alignment = a;
  }
  f->tensors.reserve(n_tensors);
  for (uint64_t i = 0; i < n_tensors; ++i) {
    TensorEntry t;
    const uint8_t* s; uint64_t len;
    if (!c.str(&s, &len)) return fail("gguf: truncated tensor name %lu", (unsigned long)i);
    t.name.assign((const char*)s, len);
    t.n_dims = c.get<uint32_t>();
    if (!c.ok || t.n_dims > 4) return fail("gguf: tensor %s has rank %u", t.name.c_str(), t.n_dims);
    uint64_t n_elem = 1;
    for (uint32_t d = 0; d < t.n_dims; ++d) { t.dims[d] = c.get<uint64_t>(); n_elem *= t.dims[d]; }
    t.type = c.get<uint32_t>(); t.offset = c.get<uint64_t>();
    if (!c.ok) return fail("gguf: truncated tensor info %s", t.name.c_str());
    const TypeInfo* ti = type_info((int)t.type);
    if (!ti) return fail("gguf: tensor %s has unknown type %u", t.name.c_str(), t.type);
    if (t.dims[0] % ti->block) return fail("gguf: tensor %s row length %lu is not a multiple of the %s block", t.name.c_str(), (unsigned long)t.dims[0], ti->name);
    t.nbytes = n_elem / ti->block * ti->bytes;
    f->tensor_index[t.name] = (int)f->tensors.size();
    f->tensors.push_back(std::move(t));
  }
  const size_t pos = (size_t)(c.p - f->map);
  f->data_start = (pos + f->alignment - 1) / f->alignment * f->alignment;
  for (auto& t : f->tensors)
    if (f->data_start + t.offset + t.nbytes > f->size) return fail("gguf: tensor %s runs past the end of the file", t.name.c_str());
  return 0;
}

// ------------------------------------------------------------------------------------------ writer
struct WKv { std::string key; uint32_t type; std::vector<uint8_t> payload; };
struct WTensor { std::string name; uint32_t n_dims; uint64_t dims[4]; uint32_t type; const void* data; uint64_t nbytes; std::vector<uint8_t> owned; };
struct GgufWriter { std::vector<WKv> kvs; std::vector<WTensor> tensors; uint32_t alignment = 32; };

template <typename T> static void put(std::vector<uint8_t>& v, T x) { const uint8_t* p = (const uint8_t*)&x; v.insert(v.end(), p, p + sizeof(T)); }
static void put_str(std::vector<uint8_t>& v, const char* s, uint64_t len) { put<uint64_t>(v, len); v.insert(v.end(), (const uint8_t*)s, (const uint8_t*)s + len); }

}  // namespace gbh

using namespace gbh;

// ------------------------------------------------------------------------------------------ reader C API
GBH_API void* gbh_gguf_open(const char* path) {
  std::unique_ptr<GgufFile> f(new GgufFile());
  f->fd = open(path, O_RDONLY);
  if (f->fd < 0) { fail("gguf: cannot open %s", path); return nullptr; }
  struct stat st;
  if (fstat(f->fd, &st) != 0 || st.st_size < 24) { fail("gguf: %s is too small", path); return nullptr; }
  f->size = (size_t)st.st_size;
  void* m = mmap(nullptr, f->size, PROT_READ, MAP_PRIVATE, f->fd, 0);
  if (m == MAP_FAILED) { fail("gguf: mmap of %s failed", path); return nullptr; }
  f->map = (const uint8_t*)m;
  madvise(m, f->size, MADV_WILLNEED);
  if (parse(f.get()) != 0) return nullptr;
  return f.release();
}
GBH_API void gbh_gguf_close(void* h) { delete (GgufFile*)h; }
GBH_API int gbh_gguf_version(void* h) { return (int)((GgufFile*)h)->version; }
GBH_API long gbh_gguf_n_tensors(void* h) { return (long)((GgufFile*)h)->tensors.size(); }
GBH_API long gbh_gguf_n_kv(void* h) { return (long)((GgufFile*)h)->kvs.size(); }
GBH_API long gbh_gguf_alignment(void* h) { return (long)((GgufFile*)h)->alignment; }
GBH_API int gbh_gguf_find_tensor(void* h, const char* name) {
  auto* f = (GgufFile*)h; auto it = f->tensor_index.find(name);
  return it == f->tensor_index.end() ? -1 : it->second;
}
GBH_API int gbh_gguf_tensor_info(void* h, int i, char* name, int name_cap, int* n_dims, uint64_t* dims4, int* type, uint64_t* nbytes) {
  auto* f = (GgufFile*)h;
  if (i < 0 || i >= (int)f->tensors.size()) return fail("gguf: tensor index %d out of range", i);
  const TensorEntry& t = f->tensors[i];
  if (name) snprintf(name, name_cap, "%s", t.name.c_str());
  *n_dims = (int)t.n_dims; *type = (int)t.type; *nbytes = t.nbytes;
  for (int d = 0; d < 4; ++d) dims4[d] = t.dims[d];
  return 0;
}
GBH_API const void* gbh_gguf_tensor_data(void* h, int i) {
  auto* f = (GgufFile*)h;
  if (i < 0 || i >= (int)f->tensors.size()) return nullptr;
  return f->map + f->data_start + f->tensors[i].offset;
}
GBH_API int gbh_gguf_find_key(void* h, const char* key) {
  auto* f = (GgufFile*)h; auto it = f->kv_index.find(key);
  return it == f->kv_index.end() ? -1 : it->second;
}
GBH_API int gbh_gguf_kv_info(void* h, int i, char* key, int key_cap, int* type, int* elem_type, uint64_t* count) {
  auto* f = (GgufFile*)h;
  if (i < 0 || i >= (int)f->kvs.size()) return fail("gguf: key index %d out of range", i);
  const KvEntry& e = f->kvs[i];
  if (key) snprintf(key, key_cap, "%s", e.key.c_str());
  *type = (int)e.type; *elem_type = (int)e.elem_type; *count = e.type == KV_STR ? e.str_len : e.count;
  return 0;
}
// Scalar value as double (integers, floats, bool).
GBH_API int gbh_gguf_kv_scalar(void* h, int i, double* out) {
  auto* f = (GgufFile*)h;
  if (i < 0 || i >= (int)f->kvs.size()) return fail("gguf: key index %d out of range", i);
  const KvEntry& e = f->kvs[i];
  const uint8_t* p = e.data;
  switch (e.type) {
    case KV_U8: *out = *p; break; case KV_I8: *out = (int8_t)*p; break; case KV_BOOL: *out = *p != 0; break;
    case KV_U16: { uint16_t v; memcpy(&v, p, 2); *out = v; break; } case KV_I16: { int16_t v; memcpy(&v, p, 2); *out = v; break; }
    case KV_U32: { uint32_t v; memcpy(&v, p, 4); *out = v; break; } case KV_I32: { int32_t v; memcpy(&v, p, 4); *out = v; break; }
    case KV_F32: { float v; memcpy(&v, p, 4); *out = v; break; } case KV_U64: { uint64_t v; memcpy(&v, p, 8); *out = (double)v; break; }
    case KV_I64: { int64_t v; memcpy(&v, p, 8); *out = (double)v; break; } case KV_F64: { memcpy(out, p, 8); break; }
    default: return fail("gguf: key %s is not a scalar", e.key.c_str());
  }
  return 0;
}
// String value, or element j of a string array: pointer into the mapping and its length (not NUL terminated).
GBH_API const char* gbh_gguf_kv_string(void* h, int i, long j, uint64_t* len) {
  auto* f = (GgufFile*)h;
  if (i < 0 || i >= (int)f->kvs.size()) return nullptr;
  const KvEntry& e = f->kvs[i];
  if (e.type == KV_STR) { *len = e.str_len; return (const char*)e.data; }
  if (e.type == KV_ARR && e.elem_type == KV_STR && j >= 0 && (uint64_t)j < e.count) { *len = e.strs[j].second; return (const char*)e.strs[j].first; }
  return nullptr;
}
// Numeric array payload (packed little-endian elements of elem_type).
GBH_API const void* gbh_gguf_kv_array_data(void* h, int i) {
  auto* f = (GgufFile*)h;
  if (i < 0 || i >= (int)f->kvs.size()) return nullptr;
  const KvEntry& e = f->kvs[i];
  return (e.type == KV_ARR && e.elem_type != KV_STR) ? e.data : nullptr;
}

// ------------------------------------------------------------------------------------------ writer C API
GBH_API void* gbh_gguf_writer_new(int alignment) { auto* w = new GgufWriter(); if (alignment > 0) w->alignment = (uint32_t)alignment; return w; }
GBH_API void gbh_gguf_writer_free(void* w) { delete (GgufWriter*)w; }
GBH_API int gbh_gguf_writer_kv_scalar(void* wv, const char* key, int type, double value) {
  auto* w = (GgufWriter*)wv; WKv e; e.key = key; e.type = (uint32_t)type;
  switch (type) {
    case KV_U8: put<uint8_t>(e.payload, (uint8_t)value); break; case KV_I8: put<int8_t>(e.payload, (int8_t)value); break;
    case KV_BOOL: put<uint8_t>(e.payload, value != 0); break; case KV_U16: put<uint16_t>(e.payload, (uint16_t)value); break;
    case KV_I16: put<int16_t>(e.payload, (int16_t)value); break; case KV_U32: put<uint32_t>(e.payload, (uint32_t)value); break;
    case KV_I32: put<int32_t>(e.payload, (int32_t)value); break; case KV_F32: put<float>(e.payload, (float)value); break;
    case KV_U64: put<uint64_t>(e.payload, (uint64_t)value); break; case KV_I64: put<int64_t>(e.payload, (int64_t)value); break;
    case KV_F64: put<double>(e.payload, value); break;
    default: return fail("gguf writer: %d is not a scalar type", type);
  }
  w->kvs.push_back(std::move(e));
  return 0;
}
GBH_API int gbh_gguf_writer_kv_string(void* wv, const char* key, const char* s, uint64_t len) {
  auto* w = (GgufWriter*)wv; WKv e; e.key = key; e.type = KV_STR; put_str(e.payload, s, len); w->kvs.push_back(std::move(e)); return 0;
}
// strs: concatenated bytes, lens: length of each
GBH_API int gbh_gguf_writer_kv_string_array(void* wv, const char* key, const char* bytes, const uint64_t* lens, uint64_t n) {
  auto* w = (GgufWriter*)wv; WKv e; e.key = key; e.type = KV_ARR;
  put<uint32_t>(e.payload, KV_STR); put<uint64_t>(e.payload, n);
  for (uint64_t i = 0; i < n; ++i) { put_str(e.payload, bytes, lens[i]); bytes += lens[i]; }
  w->kvs.push_back(std::move(e));
  return 0;
}
GBH_API int gbh_gguf_writer_kv_array(void* wv, const char* key, int elem_type, const void* data, uint64_t n) {
  const size_t es = kv_scalar_size((uint32_t)elem_type);
  if (!es) return fail("gguf writer: bad array element type %d", elem_type);
  auto* w = (GgufWriter*)wv; WKv e; e.key = key; e.type = KV_ARR;
  put<uint32_t>(e.payload, (uint32_t)elem_type); put<uint64_t>(e.payload, n);
  e.payload.insert(e.payload.end(), (const uint8_t*)data, (const uint8_t*)data + n * es);
  w->kvs.push_back(std::move(e));
  return 0;
}
// dims innermost first.  copy != 0 copies the bytes now; otherwise `data` must stay valid until write().
GBH_API int gbh_gguf_writer_tensor(void* wv, const char* name, int n_dims, const uint64_t* dims, int type, const void* data, uint64_t nbytes, int copy) {
  if (n_dims < 1 || n_dims > 4) return fail("gguf writer: tensor %s has rank %d", name, n_dims);
  const TypeInfo* ti = type_info(type);
  if (!ti) return fail("gguf writer: tensor %s has unknown type %d", name, type);
  uint64_t n_elem = 1;
  for (int d = 0; d < n_dims; ++d) n_elem *= dims[d];
  if (dims[0] % ti->block || n_elem / ti->block * ti->bytes != nbytes) return fail("gguf writer: tensor %s: %lu bytes do not match its shape and type", name, (unsigned long)nbytes);
  auto* w = (GgufWriter*)wv; WTensor t; t.name = name; t.n_dims = (uint32_t)n_dims; t.type = (uint32_t)type; t.nbytes = nbytes;
  for (int d = 0; d < 4; ++d) t.dims[d] = d < n_dims ? dims[d] : 1;
  if (copy) { t.owned.assign((const uint8_t*)data, (const uint8_t*)data + nbytes); t.data = nullptr; } else t.data = data;
  w->tensors.push_back(std::move(t));
  return 0;
}
GBH_API int gbh_gguf_writer_write(void* wv, const char* path) {
  auto* w = (GgufWriter*)wv;
  std::vector<uint8_t> head;
  put<uint32_t>(head, 0x46554747u); put<uint32_t>(head, 3);
  put<uint64_t>(head, w->tensors.size());
  bool has_align = false;
  for (auto& e : w->kvs) has_align |= e.key == "general.alignment";
  put<uint64_t>(head, w->kvs.size() + (has_align ? 0 : 1));
  if (!has_align) { put_str(head, "general.alignment", 17); put<uint32_t>(head, KV_U32); put<uint32_t>(head, w->alignment); }
  for (auto& e : w->kvs) { put_str(head, e.key.data(), e.key.size()); put<uint32_t>(head, e.type); head.insert(head.end(), e.payload.begin(), e.payload.end()); }
  uint64_t off = 0;
  std::vector<uint64_t> offs;
  for (auto& t : w->tensors) {
    offs.push_back(off);
    put_str(head, t.name.data(), t.name.size()); put<uint32_t>(head, t.n_dims);
    for (uint32_t d = 0; d < t.n_dims; ++d) put<uint64_t>(head, t.dims[d]);
    put<uint32_t>(head, t.type); put<uint64_t>(head, off);
    off = (off + t.nbytes + w->alignment - 1) / w->alignment * w->alignment;
  }
  FILE* fp = fopen(path, "wb");
  if (!fp) return fail("gguf writer: cannot create %s", path);
  bool ok = fwrite(head.data(), 1, head.size(), fp) == head.size();
  const size_t pad0 = (w->alignment - head.size() % w->alignment) % w->alignment;
  static const uint8_t zeros[4096] = {0};
  ok = ok && fwrite(zeros, 1, pad0, fp) == pad0;
  for (size_t i = 0; ok && i < w->tensors.size(); ++i) {
    auto& t = w->tensors[i];
    const void* src = t.owned.empty() ? t.data : t.owned.data();
    ok = fwrite(src, 1, t.nbytes, fp) == t.nbytes;
    const size_t pad = (w->alignment - t.nbytes % w->alignment) % w->alignment;
    ok = ok && fwrite(zeros, 1, pad, fp) == pad;
  }
  ok = (fclose(fp) == 0) && ok;
  return ok ? 0 : fail("gguf writer: short write to %s", path);
}
