// GGUF v2/v3 reader over mmap, following the parse order and range checks of the
// reference loader (src/core/loader.rs:211-320, tensor_slice :383-390; type table
// src/core/tensor.rs:61-81).  Host code only.
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <map>
#include <new>
#include <string>
#include <vector>

#include "common.cuh"

namespace {

struct meta_value {
  int type = -1;   // GGUF value type
  uint64_t u = 0;  // integers / bool
  double f = 0.0;
  std::string s;
  size_t arr_len = 0;
};

struct tensor_info {
  std::string name;
  std::vector<uint64_t> dims;
  int ggml_type;
  uint64_t offset;
  size_t nbytes;
};

bool type_traits(int t, size_t* block_elems, size_t* block_bytes) {
  static const struct { int t; size_t be, bb; } tab[] = {
      {0, 1, 4}, {1, 1, 2}, {2, 32, 18}, {3, 32, 20}, {6, 32, 22}, {7, 32, 24}, {8, 32, 34}, {9, 32, 36},
      {10, 256, 84}, {11, 256, 110}, {12, 256, 144}, {13, 256, 176}, {14, 256, 210}, {15, 256, 292},
      {16, 1, 1}, {17, 1, 2}, {18, 1, 4}};
  for (auto& e : tab)
    if (e.t == t) {
      *block_elems = e.be;
      *block_bytes = e.bb;
      return true;
    }
  return false;
}

struct reader {
  const uint8_t* p;
  size_t len, pos = 0;
  bool ok = true;
  std::string err;
  bool need(size_t n) {
    if (!ok) return false;
    if (n > len - pos) {
      ok = false;
      err = "unexpected end of GGUF data";
      return false;
    }
    return true;
  }
  template <class T> T rd() {
    T v{};
    if (need(sizeof(T))) {
      memcpy(&v, p + pos, sizeof(T));
      pos += sizeof(T);
    }
    return v;
  }
  std::string str() {
    uint64_t n = rd<uint64_t>();
    if (!ok || !need(n)) return std::string();
    std::string s((const char*)p + pos, (size_t)n);
    pos += n;
    return s;
  }
  meta_value value(int t, int depth = 0) {
    meta_value v;
    v.type = t;
    switch (t) {
      case 0: v.u = rd<uint8_t>(); break;
      case 1: v.u = (uint64_t)(int64_t)rd<int8_t>(); break;
      case 2: v.u = rd<uint16_t>(); break;
      case 3: v.u = (uint64_t)(int64_t)rd<int16_t>(); break;
      case 4: v.u = rd<uint32_t>(); break;
      case 5: v.u = (uint64_t)(int64_t)rd<int32_t>(); break;
      case 6: v.f = rd<float>(); break;
      case 7: v.u = rd<uint8_t>(); break;
      case 8: v.s = str(); break;
      case 10: v.u = rd<uint64_t>(); break;
      case 11: v.u = (uint64_t)rd<int64_t>(); break;
      case 12: v.f = rd<double>(); break;
      case 9: {
        int et = rd<int32_t>();
        uint64_t n = rd<uint64_t>();
        if (depth > 2 || et == 9) {
          ok = false;
          err = "nested GGUF arrays are not supported";
          break;
        }
        v.arr_len = (size_t)n;
        for (uint64_t i = 0; i < n && ok; i++) (void)value(et, depth + 1);
        break;
      }
      default:
        ok = false;
        err = "Unknown meta value type: " + std::to_string(t);
    }
    return v;
  }
};

}  // namespace

struct rmi_gguf {
  uint32_t magic;
  int fd;
  const uint8_t* map;
  size_t len;
  uint32_t version;
  size_t data_offset;
  std::map<std::string, meta_value> meta;
  std::vector<tensor_info> tensors;
};

static constexpr uint32_t RMI_GGUF_MAGIC = 0x524d4947;

static int32_t check_gguf(const rmi_gguf* g) {
  RMI_REQUIRE(g != nullptr && g->magic == RMI_GGUF_MAGIC, RMI_ERR_BAD_HANDLE, "invalid rmi_gguf handle");
  return RMI_OK;
}

extern "C" int32_t rmi_gguf_close(rmi_gguf* g) {
  RMI_TRY(check_gguf(g));
  if (g->map) munmap((void*)g->map, g->len);
  if (g->fd >= 0) close(g->fd);
  g->magic = 0;
  delete g;
  return RMI_OK;
}

extern "C" int32_t rmi_gguf_open(const char* path, rmi_gguf** out) {
  RMI_REQUIRE(path && out, RMI_ERR_BAD_HANDLE, "rmi_gguf_open: null argument");
  *out = nullptr;
  int fd = open(path, O_RDONLY);
  RMI_REQUIRE(fd >= 0, RMI_ERR_IO, "Failed to open GGUF file: %s", path);
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size < 24) {
    close(fd);
    rmi_set_error("GGUF file %s is too short", path);
    return RMI_ERR_FORMAT;
  }
  void* m = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  if (m == MAP_FAILED) {
    close(fd);
    rmi_set_error("Failed to mmap: %s", path);
    return RMI_ERR_IO;
  }
  rmi_gguf* g = new (std::nothrow) rmi_gguf();
  if (!g) {
    munmap(m, (size_t)st.st_size);
    close(fd);
    rmi_set_error("host allocation failed");
    return RMI_ERR_OOM;
  }
  g->magic = RMI_GGUF_MAGIC;
  g->fd = fd;
  g->map = (const uint8_t*)m;
  g->len = (size_t)st.st_size;
  reader r{g->map, g->len};
  auto fail = [&](const std::string& msg) {
    rmi_set_error("%s", msg.c_str());
    rmi_gguf_close(g);
    return (int32_t)RMI_ERR_FORMAT;
  };
  if (memcmp(g->map, "GGUF", 4) != 0) return fail("Invalid GGUF magic");
  r.pos = 4;
  g->version = r.rd<uint32_t>();
  if (g->version < 2 || g->version > 3) return fail("Unsupported GGUF version: " + std::to_string(g->version));
  uint64_t n_tensors = r.rd<uint64_t>(), n_kv = r.rd<uint64_t>();
  // every KV entry needs >= 13 bytes, every tensor entry >= 24 (loader.rs ensure_count)
  if (n_kv > (g->len - r.pos) / 13) return fail("metadata count exceeds GGUF data");
  for (uint64_t i = 0; i < n_kv && r.ok; i++) {
    std::string key = r.str();
    int t = r.rd<int32_t>();
    meta_value v = r.value(t);
    if (r.ok) g->meta[key] = v;
  }
  if (!r.ok) return fail(r.err);
  if (n_tensors > (g->len - r.pos) / 24) return fail("tensor count exceeds GGUF data");
  for (uint64_t i = 0; i < n_tensors && r.ok; i++) {
    tensor_info ti;
    ti.name = r.str();
    uint32_t nd = r.rd<uint32_t>();
    if (!r.ok || nd > (g->len - r.pos) / 8) return fail("tensor dimension count exceeds GGUF data");
    for (uint32_t d = 0; d < nd; d++) ti.dims.push_back(r.rd<uint64_t>());
    ti.ggml_type = r.rd<int32_t>();
    ti.offset = r.rd<uint64_t>();
    size_t be, bb;
    if (r.ok && !type_traits(ti.ggml_type, &be, &bb)) return fail("Unknown GGML type: " + std::to_string(ti.ggml_type));
    unsigned __int128 n_el = 1;
    for (auto d : ti.dims) {
      n_el *= d;
      if (n_el > ((unsigned __int128)1 << 62)) return fail("invalid tensor shape: " + ti.name);
    }
    if (r.ok) {
      ti.nbytes = (size_t)(((uint64_t)n_el + be - 1) / be * bb);
      g->tensors.push_back(ti);
    }
  }
  if (!r.ok) return fail(r.err);
  uint64_t align = 32;
  auto it = g->meta.find("general.alignment");
  if (it != g->meta.end()) align = it->second.u;
  if (align == 0) return fail("GGUF alignment must be nonzero");
  g->data_offset = (r.pos + align - 1) / align * align;
  for (auto& t : g->tensors) {
    if (t.offset > g->len || g->data_offset > g->len - t.offset || t.nbytes > g->len - g->data_offset - t.offset)
      return fail("tensor " + t.name + " exceeds GGUF data");
  }
  *out = g;
  return RMI_OK;
}

extern "C" int32_t rmi_gguf_n_tensors(const rmi_gguf* g, size_t* n) {
  RMI_TRY(check_gguf(g));
  *n = g->tensors.size();
  return RMI_OK;
}

extern "C" int32_t rmi_gguf_tensor(const rmi_gguf* g, const char* name, int32_t* ggml_type, uint64_t dims[4],
                                   int32_t* n_dims, const void** data, size_t* nbytes) {
  RMI_TRY(check_gguf(g));
  for (auto& t : g->tensors)
    if (t.name == name) {
      if (ggml_type) *ggml_type = t.ggml_type;
      if (n_dims) *n_dims = (int32_t)t.dims.size();
      if (dims)
        for (size_t i = 0; i < 4; i++) dims[i] = i < t.dims.size() ? t.dims[i] : 1;
      if (data) *data = g->map + g->data_offset + t.offset;
      if (nbytes) *nbytes = t.nbytes;
      return RMI_OK;
    }
  rmi_set_error("Missing tensor: %s", name);
  return RMI_ERR_FORMAT;
}

static const meta_value* find_meta(const rmi_gguf* g, const char* key) {
  auto it = g->meta.find(key);
  return it == g->meta.end() ? nullptr : &it->second;
}

extern "C" int32_t rmi_gguf_meta_u64(const rmi_gguf* g, const char* key, uint64_t* value) {
  RMI_TRY(check_gguf(g));
  const meta_value* v = find_meta(g, key);
  RMI_REQUIRE(v != nullptr, RMI_ERR_FORMAT, "Missing metadata: %s", key);
  RMI_REQUIRE(v->type != 6 && v->type != 8 && v->type != 9 && v->type != 12, RMI_ERR_FORMAT, "Invalid metadata: %s", key);
  *value = v->u;
  return RMI_OK;
}

extern "C" int32_t rmi_gguf_meta_f64(const rmi_gguf* g, const char* key, double* value) {
  RMI_TRY(check_gguf(g));
  const meta_value* v = find_meta(g, key);
  RMI_REQUIRE(v != nullptr, RMI_ERR_FORMAT, "Missing metadata: %s", key);
  if (v->type == 6 || v->type == 12) *value = v->f;
  else if (v->type == 8 || v->type == 9) {
    rmi_set_error("Invalid metadata: %s", key);
    return RMI_ERR_FORMAT;
  } else *value = (double)v->u;
  return RMI_OK;
}

extern "C" int32_t rmi_gguf_meta_str(const rmi_gguf* g, const char* key, char* buf, size_t buf_len) {
  RMI_TRY(check_gguf(g));
  const meta_value* v = find_meta(g, key);
  RMI_REQUIRE(v != nullptr && v->type == 8, RMI_ERR_FORMAT, "Missing metadata: %s", key);
  RMI_REQUIRE(buf && buf_len > v->s.size(), RMI_ERR_BAD_SHAPE, "buffer too small for %s", key);
  memcpy(buf, v->s.c_str(), v->s.size() + 1);
  return RMI_OK;
}

extern "C" int32_t rmi_weight_upload_gguf(rmi_ctx* ctx, const rmi_gguf* g, const char* name, size_t row_begin,
                                          size_t row_end, rmi_weight** out) {
  RMI_TRY(check_gguf(g));
  int32_t type, nd;
  uint64_t dims[4];
  const void* data;
  size_t nbytes;
  RMI_TRY(rmi_gguf_tensor(g, name, &type, dims, &nd, &data, &nbytes));
  RMI_REQUIRE(nd == 2, RMI_ERR_BAD_SHAPE, "tensor %s has %d dims, a weight matrix needs 2", name, nd);
  if (row_end == (size_t)-1) row_end = (size_t)dims[1];
  // GGUF order: dims[0] is the row length (n_in), dims[1] the row count (n_out)
  return rmi_weight_upload(ctx, type, data, nbytes, (size_t)dims[0], (size_t)dims[1], row_begin, row_end, out);
}
