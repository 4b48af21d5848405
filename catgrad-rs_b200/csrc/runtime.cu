// runtime.cu — context, stream-ordered caching allocator, tensor handles and the view
// operations of the trait that need no kernel (broadcast, transpose, slice, reshape of a
// compatible layout).
#include "runtime.h"

#include <algorithm>
#include <cstring>

namespace cg {

// ------------------------------------------------------------------ allocator --------
// One stream per context, so a block freed by the host is safe to hand out again at once:
// whatever still reads it was enqueued earlier on the same stream.

static size_t round_size(size_t bytes) {
  if (bytes < 512) return 512;
  if (bytes < (1u << 20)) return (bytes + 511) & ~size_t(511);
  return (bytes + (1u << 20) - 1) & ~size_t((1u << 20) - 1);
}

void* Core::alloc(size_t bytes, size_t* got) {
  size_t want = round_size(bytes);
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = free_blocks.lower_bound(want);
    if (it != free_blocks.end() && it->first <= want + want / 4 + 4096) {
      void* p = it->second;
      *got = it->first;
      free_blocks.erase(it);
      return p;
    }
  }
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, want);
  if (e != cudaSuccess) {
    cudaGetLastError();
    trim();
    e = cudaMalloc(&p, want);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
  }
  std::lock_guard<std::mutex> g(mu);
  reserved += (int64_t)want;
  *got = want;
  return p;
}

void Core::recycle(void* p, size_t bytes) {
  std::lock_guard<std::mutex> g(mu);
  free_blocks.emplace(bytes, p);
}

void Core::trim() {
  std::multimap<size_t, void*> blocks;
  {
    std::lock_guard<std::mutex> g(mu);
    blocks.swap(free_blocks);
  }
  if (blocks.empty()) return;
  cudaStreamSynchronize(stream);
  for (auto& kv : blocks) {
    cudaFree(kv.second);
    std::lock_guard<std::mutex> g(mu);
    reserved -= (int64_t)kv.first;
  }
}

Core::~Core() {
  cudaSetDevice(device);
  cudaStreamSynchronize(stream);
  for (auto& kv : free_blocks) cudaFree(kv.second);
  if (dev_err) cudaFree(dev_err);
  if (own_stream && stream) cudaStreamDestroy(stream);
}

Buffer::~Buffer() {
  if (owned && ptr && core) core->recycle(ptr, bytes);
}

// ------------------------------------------------------------------ errors -----------

int fail(cg_ctx* c, int code, const std::string& msg) {
  if (c) c->err = msg;
  return code;
}

int cuda_fail(cg_ctx* c, cudaError_t e, const char* what) {
  std::string m = std::string(what) + ": " + cudaGetErrorString(e);
  return fail(c, e == cudaErrorMemoryAllocation ? CG_ERR_OOM : CG_ERR_CUDA, m);
}

// ------------------------------------------------------------------ tensors ----------

int new_tensor(cg_ctx* c, int tag, int storage, const int64_t* dims, int rank, cg_tensor** out) {
  if (rank < 0 || rank > CG_MAX_RANK) return fail(c, CG_ERR_INVALID, "rank out of range");
  auto* t = new cg_tensor();
  t->ctx = c;
  t->tag = tag;
  t->storage = storage;
  t->rank = rank;
  int64_t n = 1;
  for (int i = rank - 1; i >= 0; --i) {
    if (dims[i] < 0) { delete t; return fail(c, CG_ERR_SHAPE, "negative dimension"); }
    t->dims[i] = dims[i];
    t->strides[i] = n;
    n *= dims[i];
  }
  auto buf = std::make_shared<Buffer>();
  buf->core = c->core;
  size_t bytes = (size_t)std::max<int64_t>(n, 1) * storage_bytes(storage);
  buf->ptr = c->core->alloc(bytes, &buf->bytes);
  if (!buf->ptr) {
    delete t;
    return fail(c, CG_ERR_OOM, "out of device memory");
  }
  t->buf = buf;
  *out = t;
  return CG_OK;
}

cg_tensor* new_view(const cg_tensor* x) {
  auto* t = new cg_tensor();
  t->ctx = x->ctx;
  t->tag = x->tag;
  t->storage = x->storage;
  t->rank = x->rank;
  memcpy(t->dims, x->dims, sizeof(t->dims));
  memcpy(t->strides, x->strides, sizeof(t->strides));
  t->offset = x->offset;
  t->buf = x->buf;
  t->has_scalar = x->has_scalar;
  t->scalar_bits = x->scalar_bits;
  return t;
}

void release(cg_tensor* t) {
  if (t && --t->rc == 0) {
    if (t->node) lazy_orphan(t);
    delete t;
  }
}

Iter make_iter(int rank, const int64_t* dims, const int64_t* s0, const int64_t* s1, const int64_t* s2) {
  // collect non-unit dims
  int64_t d[CG_MAX_RANK], a[CG_MAX_RANK], b[CG_MAX_RANK], c[CG_MAX_RANK];
  int r = 0;
  for (int i = 0; i < rank; ++i) {
    if (dims[i] == 1) continue;
    d[r] = dims[i];
    a[r] = s0 ? s0[i] : 0;
    b[r] = s1 ? s1[i] : 0;
    c[r] = s2 ? s2[i] : 0;
    ++r;
  }
  // merge dim i+1 into dim i when every operand steps jointly
  Iter it;
  int o = 0;
  for (int i = 0; i < r; ++i) {
    if (o > 0 && it.s0[o - 1] == a[i] * d[i] && it.s1[o - 1] == b[i] * d[i] && it.s2[o - 1] == c[i] * d[i]) {
      it.dims[o - 1] *= d[i];
      it.s0[o - 1] = a[i];
      it.s1[o - 1] = b[i];
      it.s2[o - 1] = c[i];
    } else {
      it.dims[o] = d[i];
      it.s0[o] = a[i];
      it.s1[o] = b[i];
      it.s2[o] = c[i];
      ++o;
    }
  }
  it.rank = o;
  for (int i = o; i < CG_MAX_RANK; ++i) {
    it.dims[i] = 1;
    it.s0[i] = it.s1[i] = it.s2[i] = 0;
  }
  return it;
}

// Try to express `x` reshaped to `dims` as a view (the rule numpy uses to avoid a copy).
static bool reshape_view(const cg_tensor* x, const int64_t* dims, int rank, int64_t* out_strides) {
  int64_t od[CG_MAX_RANK], os[CG_MAX_RANK];
  int on = 0;
  for (int i = 0; i < x->rank; ++i)
    if (x->dims[i] != 1) { od[on] = x->dims[i]; os[on] = x->strides[i]; ++on; }
  int64_t n = 1;
  for (int i = 0; i < rank; ++i) n *= dims[i];
  if (n == 0) {  // empty: any strides do
    int64_t s = 1;
    for (int i = rank - 1; i >= 0; --i) { out_strides[i] = s; s *= std::max<int64_t>(dims[i], 1); }
    return true;
  }
  int oi = 0, oj = 1, ni = 0, nj = 1;
  while (ni < rank && oi < on) {
    int64_t np = dims[ni], op = od[oi];
    while (np != op) {
      if (np < op) { if (nj >= rank) return false; np *= dims[nj++]; }
      else { if (oj >= on) return false; op *= od[oj++]; }
    }
    for (int ok = oi; ok < oj - 1; ++ok)
      if (os[ok] != od[ok + 1] * os[ok + 1]) return false;
    out_strides[nj - 1] = os[oj - 1];
    for (int nk = nj - 1; nk > ni; --nk) out_strides[nk - 1] = out_strides[nk] * dims[nk];
    ni = nj++;
    oi = oj++;
  }
  // remaining new dims must be 1
  int64_t last = ni > 0 ? out_strides[ni - 1] : 1;
  for (int i = ni; i < rank; ++i) {
    if (dims[i] != 1) return false;
    out_strides[i] = last;
  }
  return oi >= on;
}

}  // namespace cg

using namespace cg;

extern "C" {

int32_t cg_ctx_create(int32_t device, int32_t precision, void* stream, cg_ctx** out) {
  if (!out) return CG_ERR_INVALID;
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || device < 0 || device >= ndev) {
    cudaGetLastError();
    return CG_ERR_CUDA;
  }
  if (cudaSetDevice(device) != cudaSuccess) return CG_ERR_CUDA;
  auto core = std::make_shared<Core>();
  core->device = device;
  if (stream) {
    core->stream = (cudaStream_t)stream;
  } else {
    if (cudaStreamCreateWithFlags(&core->stream, cudaStreamNonBlocking) != cudaSuccess) return CG_ERR_CUDA;
    core->own_stream = true;
  }
  if (cudaMalloc(&core->dev_err, 64) != cudaSuccess) return CG_ERR_OOM;
  cudaMemsetAsync(core->dev_err, 0, 64, core->stream);
  auto* c = new cg_ctx();
  c->core = core;
  c->precision = precision;
  *out = c;
  return CG_OK;
}

int32_t cg_ctx_destroy(cg_ctx* c) {
  if (!c) return CG_ERR_INVALID;
  cudaSetDevice(c->core->device);
  if (c->lazy) lazy_flush(c);
  cudaStreamSynchronize(c->core->stream);
  cg_comm_destroy(c);
  c->core->trim();
  delete c;
  return CG_OK;
}

const char* cg_last_error(cg_ctx* c) { return c ? c->err.c_str() : ""; }

int32_t cg_sync(cg_ctx* c) {
  if (!c) return CG_ERR_INVALID;
  CG_LAZY_FLUSH(c);
  int32_t flag = 0;
  CG_CUDA(c, cudaMemcpyAsync(&flag, c->core->dev_err, 4, cudaMemcpyDeviceToHost, c->core->stream));
  CG_CUDA(c, cudaStreamSynchronize(c->core->stream));
  if (flag != DEV_OK) {
    cudaMemsetAsync(c->core->dev_err, 0, 4, c->core->stream);
    if (flag == DEV_INDEX) return fail(c, CG_ERR_INDEX, "index out of bounds");
    return fail(c, CG_ERR_TIMEOUT, "a bounded device-side wait expired");
  }
  return CG_OK;
}

void* cg_ctx_stream(cg_ctx* c) { return c ? (void*)c->core->stream : nullptr; }
int64_t cg_launch_count(cg_ctx* c) { return c ? c->launches : 0; }
int64_t cg_bytes_reserved(cg_ctx* c) { return c ? c->core->reserved : 0; }

int32_t cg_set_option(cg_ctx* c, const char* name, int64_t value) {
  if (!c || !name) return CG_ERR_INVALID;
  c->opt_generation++;  // decoders re-capture their step graph when a switch may have changed the kernel sequence
  if (!strcmp(name, "gemm")) { c->opt_gemm = (int)value; return CG_OK; }
  if (!strcmp(name, "wait_limit_us")) {
    // limit of every bounded device-side wait (mbarrier, peer flag, grid barrier)
    if (value < 1 || value > 60ll * 1000 * 1000) return fail(c, CG_ERR_INVALID, "wait_limit_us out of range");
    const unsigned long long ns = (unsigned long long)value * 1000ull;
    CG_CUDA(c, cudaMemcpyAsync((char*)c->core->dev_err + 8, &ns, 8, cudaMemcpyHostToDevice, c->core->stream));
    CG_CUDA(c, cudaStreamSynchronize(c->core->stream));  // `ns` is on the stack
    return CG_OK;
  }
  if (!strcmp(name, "resident")) { c->opt_resident = value != 0; return CG_OK; }
  if (!strcmp(name, "lazy")) {
    if (!value) CG_TRY(lazy_flush(c));
    c->lazy = value != 0;
    return CG_OK;
  }
  if (!strcmp(name, "resident_stages")) { c->opt_res_stages = (int)value; return CG_OK; }
  if (!strcmp(name, "resident_attn_group")) {
    if (value != 0 && value != 1 && value != 2 && value != 4) return fail(c, CG_ERR_INVALID, "resident_attn_group must be 0, 1, 2 or 4");
    c->opt_res_group = (int)value;
    return CG_OK;
  }
  if (!strcmp(name, "pdl")) { c->opt_pdl = value != 0; return CG_OK; }
  if (!strcmp(name, "peer")) { c->opt_peer = value != 0; return CG_OK; }
  if (!strcmp(name, "fa")) { c->opt_fa = (int)value; return CG_OK; }
  if (!strcmp(name, "prefill_chunk")) {
    if (value < 64 || value > (1 << 20)) return fail(c, CG_ERR_INVALID, "prefill_chunk out of range");
    c->opt_prefill_chunk = (int)value;
    return CG_OK;
  }
  if (!strcmp(name, "handover")) { c->opt_handover = value != 0; return CG_OK; }
  if (!strcmp(name, "persistent")) { c->opt_persistent = value != 0; return CG_OK; }
  if (!strcmp(name, "pair_cta")) { c->opt_pair_cta = (int)value; return CG_OK; }
  return fail(c, CG_ERR_INVALID, std::string("unknown option ") + name);
}

int32_t cg_tensor_retain(cg_tensor* t) {
  if (!t) return CG_ERR_INVALID;
  t->rc++;
  return CG_OK;
}
int32_t cg_tensor_release(cg_tensor* t) {
  if (!t) return CG_ERR_INVALID;
  release(t);
  return CG_OK;
}
int32_t cg_shape(const cg_tensor* t, int32_t* rank, int64_t dims[CG_MAX_RANK]) {
  if (!t || !rank || !dims) return CG_ERR_INVALID;
  *rank = t->rank;
  for (int i = 0; i < t->rank; ++i) dims[i] = t->dims[i];
  return CG_OK;
}
int32_t cg_dtype_of(const cg_tensor* t, int32_t* dtype) {
  if (!t || !dtype) return CG_ERR_INVALID;
  *dtype = t->tag;
  return CG_OK;
}
int32_t cg_storage_of(const cg_tensor* t, int32_t* storage) {
  if (!t || !storage) return CG_ERR_INVALID;
  *storage = t->storage;
  return CG_OK;
}

// ------------------------------------------------------------------ views ------------

int32_t cg_broadcast(cg_ctx* c, const cg_tensor* x, const int64_t* dims, int32_t rank, cg_tensor** out) {
  if (!c || !x || !out || rank < 0 || rank > CG_MAX_RANK || (rank && !dims)) return fail(c, CG_ERR_INVALID, "bad argument");
  if (x->rank > rank) return fail(c, CG_ERR_SHAPE, "broadcast: target has lower rank");
  int64_t st[CG_MAX_RANK] = {0};
  for (int i = 0; i < x->rank; ++i) {
    int o = rank - x->rank + i;
    if (x->dims[i] == dims[o]) st[o] = x->strides[i];
    else if (x->dims[i] == 1) st[o] = 0;
    else return fail(c, CG_ERR_SHAPE, "broadcast: incompatible shapes");
  }
  cg_tensor* t = new_view(x);
  t->rank = rank;
  for (int i = 0; i < rank; ++i) { t->dims[i] = dims[i]; t->strides[i] = dims[i] == 1 ? 0 : st[i]; }
  if (x->node) lazy_view(c, LV_BROADCAST, t, x, dims, rank);
  *out = t;
  return CG_OK;
}

int32_t cg_transpose(cg_ctx* c, const cg_tensor* x, int32_t d0, int32_t d1, cg_tensor** out) {
  if (!c || !x || !out) return fail(c, CG_ERR_INVALID, "null argument");
  if (d0 < 0 || d1 < 0 || d0 >= x->rank || d1 >= x->rank) return fail(c, CG_ERR_SHAPE, "transpose: axis out of range");
  cg_tensor* t = new_view(x);
  std::swap(t->dims[d0], t->dims[d1]);
  std::swap(t->strides[d0], t->strides[d1]);
  if (x->node) { const int64_t a[2] = {d0, d1}; lazy_view(c, LV_TRANSPOSE, t, x, a, 2); }
  *out = t;
  return CG_OK;
}

int32_t cg_slice(cg_ctx* c, const cg_tensor* x, int32_t dim, int64_t start, int64_t len, cg_tensor** out) {
  if (!c || !x || !out) return fail(c, CG_ERR_INVALID, "null argument");
  if (dim < 0 || dim >= x->rank) return fail(c, CG_ERR_SHAPE, "slice: axis out of range");
  if (start < 0 || len < 0 || start + len > x->dims[dim]) return fail(c, CG_ERR_SHAPE, "slice: range out of bounds");
  cg_tensor* t = new_view(x);
  t->dims[dim] = len;
  t->offset += start * x->strides[dim];
  if (x->node) { const int64_t a[3] = {dim, start, len}; lazy_view(c, LV_SLICE, t, x, a, 3); }
  *out = t;
  return CG_OK;
}

int32_t cg_reshape(cg_ctx* c, const cg_tensor* x, const int64_t* dims, int32_t rank, cg_tensor** out) {
  if (!c || !x || !out || rank < 0 || rank > CG_MAX_RANK || (rank && !dims)) return fail(c, CG_ERR_INVALID, "bad argument");
  int64_t n = 1;
  for (int i = 0; i < rank; ++i) {
    if (dims[i] < 0) return fail(c, CG_ERR_SHAPE, "negative dimension");
    n *= dims[i];
  }
  if (n != x->numel()) return fail(c, CG_ERR_SHAPE, "reshape: element count differs");
  int64_t st[CG_MAX_RANK];
  Hold src;
  const cg_tensor* base = x;
  if (!reshape_view(x, dims, rank, st)) {
    if (x->node) return lazy_reshape_copy(c, x, dims, rank, out);  // the contents do not exist yet
    CG_TRY(as_contiguous(c, x, &src.t));
    base = src.t;
    int64_t s = 1;
    for (int i = rank - 1; i >= 0; --i) { st[i] = s; s *= dims[i]; }
  }
  cg_tensor* t = new_view(base);
  t->rank = rank;
  for (int i = 0; i < rank; ++i) { t->dims[i] = dims[i]; t->strides[i] = st[i]; }
  if (base->node) lazy_view(c, LV_RESHAPE, t, base, dims, rank);
  *out = t;
  return CG_OK;
}

}  // extern "C"
