// safetensors.cu — checkpoint files straight to device tensors
// (catgrad-llm/examples/llama/main.rs:279-354 loads every tensor into a host Vec<f32>, widening
// bf16 element by element, and hands it to the backend; here the file is memory-mapped, the
// header is parsed by a small JSON reader, and each tensor's bytes are copied host -> device
// once, in the element type they are stored in).
#include "safetensors.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>

#include "kernels.h"

cg_safetensors::~cg_safetensors() {
  if (map && map != MAP_FAILED) munmap(map, map_bytes);
}

namespace cg {

namespace {

// Minimal JSON reader for the header: objects, arrays, strings (with escapes), numbers,
// true/false/null.  Only what the tensor entries need is kept.
struct Json {
  const char* p;
  const char* end;
  std::string err;
  void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool fail(const char* m) { if (err.empty()) err = m; return false; }
  bool lit(char c) { ws(); if (p < end && *p == c) { ++p; return true; } return false; }
  bool str(std::string* out) {
    ws();
    if (p >= end || *p != '"') return fail("expected a string");
    ++p;
    out->clear();
    while (p < end && *p != '"') {
      if (*p == '\\') {
        if (++p >= end) return fail("bad escape");
        switch (*p) {
          case 'n': out->push_back('\n'); break;
          case 't': out->push_back('\t'); break;
          case 'r': out->push_back('\r'); break;
          case 'b': out->push_back('\b'); break;
          case 'f': out->push_back('\f'); break;
          case 'u': {
            if (end - p < 5) return fail("bad \\u escape");
            unsigned v = 0;
            for (int i = 1; i <= 4; ++i) {
              const char h = p[i];
              v = v * 16 + (h >= '0' && h <= '9' ? h - '0' : h >= 'a' && h <= 'f' ? h - 'a' + 10 : h >= 'A' && h <= 'F' ? h - 'A' + 10 : 0);
            }
            p += 4;
            // tensor names are ASCII in practice; other code points are kept as UTF-8
            if (v < 0x80) out->push_back((char)v);
            else if (v < 0x800) { out->push_back((char)(0xC0 | (v >> 6))); out->push_back((char)(0x80 | (v & 0x3F))); }
            else { out->push_back((char)(0xE0 | (v >> 12))); out->push_back((char)(0x80 | ((v >> 6) & 0x3F))); out->push_back((char)(0x80 | (v & 0x3F))); }
            break;
          }
          default: out->push_back(*p);
        }
        ++p;
      } else {
        out->push_back(*p++);
      }
    }
    if (p >= end) return fail("unterminated string");
    ++p;
    return true;
  }
  bool integer(int64_t* out) {
    ws();
    const char* s = p;
    if (p < end && *p == '-') ++p;
    while (p < end && *p >= '0' && *p <= '9') ++p;
    if (p == s) return fail("expected a number");
    *out = strtoll(std::string(s, p).c_str(), nullptr, 10);
    // tolerate a fractional part / exponent by skipping it
    while (p < end && (*p == '.' || *p == 'e' || *p == 'E' || *p == '+' || *p == '-' || (*p >= '0' && *p <= '9'))) ++p;
    return true;
  }
  bool skip() {  // any value
    ws();
    if (p >= end) return fail("unexpected end");
    if (*p == '"') { std::string s; return str(&s); }
    if (*p == '{') {
      ++p;
      if (lit('}')) return true;
      do {
        std::string k;
        if (!str(&k) || !lit(':') || !skip()) return fail("bad object");
      } while (lit(','));
      return lit('}') || fail("expected }");
    }
    if (*p == '[') {
      ++p;
      if (lit(']')) return true;
      do { if (!skip()) return false; } while (lit(','));
      return lit(']') || fail("expected ]");
    }
    if (!strncmp(p, "true", 4)) { p += 4; return true; }
    if (!strncmp(p, "false", 5)) { p += 5; return true; }
    if (!strncmp(p, "null", 4)) { p += 4; return true; }
    int64_t v;
    return integer(&v);
  }
};

bool parse_entry(Json& j, StEntry* e, std::string* dtype) {
  if (!j.lit('{')) return j.fail("expected a tensor object");
  bool have_shape = false, have_off = false;
  if (!j.lit('}')) {
    do {
      std::string k;
      if (!j.str(&k) || !j.lit(':')) return j.fail("bad tensor object");
      if (k == "dtype") {
        if (!j.str(dtype)) return false;
      } else if (k == "shape") {
        if (!j.lit('[')) return j.fail("shape must be an array");
        if (!j.lit(']')) {
          do {
            int64_t v;
            if (!j.integer(&v)) return false;
            e->dims.push_back(v);
          } while (j.lit(','));
          if (!j.lit(']')) return j.fail("expected ]");
        }
        have_shape = true;
      } else if (k == "data_offsets") {
        int64_t a, b;
        if (!j.lit('[') || !j.integer(&a) || !j.lit(',') || !j.integer(&b) || !j.lit(']')) return j.fail("bad data_offsets");
        e->begin = (size_t)a;
        e->end = (size_t)b;
        have_off = true;
      } else if (!j.skip()) {
        return false;
      }
    } while (j.lit(','));
    if (!j.lit('}')) return j.fail("expected }");
  }
  return (have_shape && have_off && !dtype->empty()) || j.fail("tensor entry lacks dtype, shape or data_offsets");
}

__global__ void k_widen_bf16(const __nv_bfloat16* in, int64_t n, float* out) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = __bfloat162float(in[i]);
}

}  // namespace

cg_safetensors* st_open(const char* path, std::string* why) {
  auto bad = [&](const std::string& m) -> cg_safetensors* { *why = std::string(path ? path : "(null)") + ": " + m; return nullptr; };
  if (!path) return bad("no path");
  const int fd = open(path, O_RDONLY);
  if (fd < 0) return bad("cannot open");
  struct stat sb;
  if (fstat(fd, &sb) != 0 || sb.st_size < 8) { close(fd); return bad("not a safetensors file (shorter than its length field)"); }
  std::unique_ptr<cg_safetensors> f(new cg_safetensors());
  f->path = path;
  f->map_bytes = (size_t)sb.st_size;
  f->map = mmap(nullptr, f->map_bytes, PROT_READ, MAP_PRIVATE, fd, 0);
  close(fd);
  if (f->map == MAP_FAILED) { f->map = nullptr; return bad("mmap failed"); }
  const uint8_t* b = (const uint8_t*)f->map;
  uint64_t hlen = 0;
  for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | b[i];
  if (hlen > f->map_bytes - 8) return bad("header length exceeds the file");
  f->data = b + 8 + hlen;
  f->data_bytes = f->map_bytes - 8 - (size_t)hlen;
  Json j{(const char*)b + 8, (const char*)b + 8 + hlen, {}};
  if (!j.lit('{')) return bad("header is not a JSON object");
  if (!j.lit('}')) {
    do {
      std::string name;
      if (!j.str(&name) || !j.lit(':')) return bad("bad header: " + j.err);
      if (name == "__metadata__") {
        if (!j.skip()) return bad("bad metadata: " + j.err);
        continue;
      }
      StEntry e;
      std::string dtype;
      e.name = name;
      if (!parse_entry(j, &e, &dtype)) return bad("tensor " + name + ": " + j.err);
      if (dtype == "F32") e.storage = ST_F32;
      else if (dtype == "BF16") e.storage = ST_BF16;
      else return bad("tensor " + name + ": unsupported dtype " + dtype + " (F32 and BF16 are)");  // main.rs:318-320 panics
      if ((int)e.dims.size() > CG_MAX_RANK) return bad("tensor " + name + ": rank above " + std::to_string(CG_MAX_RANK));
      for (int64_t d : e.dims)
        if (d < 0) return bad("tensor " + name + ": negative extent");
      const size_t want = (size_t)e.numel() * storage_bytes(e.storage);
      if (e.end < e.begin || e.end > f->data_bytes || e.end - e.begin != want)
        return bad("tensor " + name + ": data_offsets do not match its shape and dtype");
      f->entries.push_back(std::move(e));
    } while (j.lit(','));
    if (!j.lit('}')) return bad("bad header: expected }");
  }
  return f.release();
}

int st_upload(cg_ctx* c, const cg_safetensors* f, const StEntry& e, cg_tensor** out) {
  const int rank = (int)e.dims.size();
  const bool keep_bf16 = e.storage == ST_BF16 && c->precision == CG_PREC_BF16 && rank >= 2;
  const int64_t n = e.numel();
  Hold r;
  if (e.storage == ST_F32 || keep_bf16) {
    // in a bf16-precision context rank >= 2 f32 tensors are rounded like any upload (cg_ndarray_from_vec_f32)
    if (e.storage == ST_F32) return cg_ndarray_from_vec_f32(c, (const float*)(f->data + e.begin), n, e.dims.data(), rank, out);
    CG_TRY(new_tensor(c, CG_F32, ST_BF16, e.dims.data(), rank, &r.t));
    if (n) CG_CUDA(c, cudaMemcpyAsync(r.t->data(), f->data + e.begin, (size_t)n * 2, cudaMemcpyHostToDevice, c->core->stream));
    *out = r.take();
    return CG_OK;
  }
  // bf16 source, f32 result: the 2-byte elements cross the link, the device widens them
  Hold tmp;
  CG_TRY(new_tensor(c, CG_F32, ST_BF16, e.dims.data(), rank, &tmp.t));
  CG_TRY(new_tensor(c, CG_F32, ST_F32, e.dims.data(), rank, &r.t));
  if (n) {
    CG_CUDA(c, cudaMemcpyAsync(tmp.t->data(), f->data + e.begin, (size_t)n * 2, cudaMemcpyHostToDevice, c->core->stream));
    k_widen_bf16<<<grid_for(n, 256), 256, 0, c->core->stream>>>((const __nv_bfloat16*)tmp.t->data(), n, (float*)r.t->data());
    CG_LAUNCHED(c);
  }
  *out = r.take();
  return CG_OK;
}

int st_upload_into_bf16(cg_ctx* c, const cg_safetensors* f, const StEntry& e, cg_tensor* dst, int64_t at) {
  const int64_t n = e.numel();
  if (dst->storage != ST_BF16 || !dst->contiguous() || at < 0 || at + n > dst->numel())
    return fail(c, CG_ERR_INVALID, "safetensors: bad destination for " + e.name);
  if (!n) return CG_OK;
  __nv_bfloat16* d = (__nv_bfloat16*)dst->data() + at;
  if (e.storage == ST_BF16) {
    CG_CUDA(c, cudaMemcpyAsync(d, f->data + e.begin, (size_t)n * 2, cudaMemcpyHostToDevice, c->core->stream));
    return CG_OK;
  }
  Hold tmp;
  CG_TRY(new_tensor(c, CG_F32, ST_F32, &n, 1, &tmp.t));
  CG_CUDA(c, cudaMemcpyAsync(tmp.t->data(), f->data + e.begin, (size_t)n * 4, cudaMemcpyHostToDevice, c->core->stream));
  return k_launch_to_bf16(c, (const float*)tmp.t->data(), n, d);
}

}  // namespace cg

using namespace cg;

extern "C" {

int32_t cg_safetensors_open(const char* path, cg_safetensors** out, char* err, int64_t err_cap) {
  if (!out) return CG_ERR_INVALID;
  std::string why;
  *out = st_open(path, &why);
  if (*out) return CG_OK;
  if (err && err_cap > 0) {
    strncpy(err, why.c_str(), (size_t)err_cap - 1);
    err[err_cap - 1] = 0;
  }
  return CG_ERR_INVALID;
}

int32_t cg_safetensors_close(cg_safetensors* f) {
  if (!f) return CG_ERR_INVALID;
  delete f;
  return CG_OK;
}

int64_t cg_safetensors_count(const cg_safetensors* f) { return f ? (int64_t)f->entries.size() : -1; }

int32_t cg_safetensors_info(const cg_safetensors* f, int64_t i, const char** name, int32_t* storage, int32_t* rank,
                            int64_t dims[CG_MAX_RANK]) {
  if (!f || i < 0 || i >= (int64_t)f->entries.size()) return CG_ERR_INVALID;
  const StEntry& e = f->entries[(size_t)i];
  if (name) *name = e.name.c_str();
  if (storage) *storage = e.storage;
  if (rank) *rank = (int32_t)e.dims.size();
  if (dims)
    for (size_t k = 0; k < e.dims.size(); ++k) dims[k] = e.dims[k];
  return CG_OK;
}

int32_t cg_safetensors_tensor(cg_ctx* c, const cg_safetensors* f, int64_t i, cg_tensor** out) {
  if (!c || !f || !out || i < 0 || i >= (int64_t)f->entries.size()) return fail(c, CG_ERR_INVALID, "safetensors: bad argument");
  CG_TRY(st_upload(c, f, f->entries[(size_t)i], out));
  // the copy reads pageable (mapped) memory: it has completed when the call returns, but be explicit
  CG_CUDA(c, cudaStreamSynchronize(c->core->stream));
  return CG_OK;
}

}  // extern "C"
