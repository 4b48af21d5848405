"""Host-side mirror of the catgrad interpreter's `trait Backend`
(catgrad/src/interpreter/backend/mod.rs:22-82) over a C-ABI library.

`TraitBackend` binds, by symbol prefix, any shared library that exports the trait-level
entry points declared in include/catgrad_cuda.h.  Method names, argument order and
meaning follow the trait; failures surface the way the reference backends do:

* `ndarray_from_vec_*` raise `BackendError` (BackendError::ShapeError, mod.rs:88-92);
* every other method raises `BackendPanic`, standing for the `panic!` of the reference
  backends (ndarray.rs:212,255,293,333; candle.rs:413-415).

`CudaBackend` is the product: the prefix `cg_` on libcatgrad_cuda.so, with the extension
entry points (fused kernels, bf16 storage, decoder runner) added.  There is no CPU
fallback: constructing it without the built CUDA library, or without a GPU, raises.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Sequence

import numpy as np

F32 = 0  # Dtype::F32 (catgrad/src/category/core.rs:21-24)
U32 = 1  # Dtype::U32
PREC_F32 = 0
PREC_BF16 = 1

_c_i64p = C.POINTER(C.c_int64)
_c_vp = C.c_void_p


class BackendError(Exception):
    """BackendError::ShapeError (backend/mod.rs:88-92)."""


class BackendPanic(RuntimeError):
    """A condition on which the reference backends panic."""

    def __init__(self, status: int, message: str):
        super().__init__(f"[status {status}] {message}")
        self.status = status
        self.message = message


class TaggedTensor:
    """A backend tensor with its dtype tag (interpreter/types.rs:15-98).  Owns one
    reference to the library handle; copying the Python object shares it."""

    __slots__ = ("_b", "_h", "dtype")

    def __init__(self, backend: "TraitBackend", handle, dtype: int):
        self._b = backend
        self._h = handle
        self.dtype = dtype

    @property
    def shape(self) -> tuple[int, ...]:
        """BackendTensorOps::shape (backend/mod.rs:84-86): host metadata, no sync."""
        rank = C.c_int32()
        dims = (C.c_int64 * 8)()
        self._b._f("shape")(self._h, C.byref(rank), dims)
        return tuple(dims[i] for i in range(rank.value))

    def __del__(self):
        try:
            if self._h is not None:
                self._b._f("tensor_release")(self._h)
                self._h = None
        except Exception:
            pass

    def __repr__(self):
        return f"TaggedTensor({'F32' if self.dtype == F32 else 'U32'}, shape={self.shape})"


def _dims(shape: Sequence[int]):
    arr = (C.c_int64 * max(len(shape), 1))(*[int(d) for d in shape])
    return arr, len(shape)


_BINARY = ("matmul", "add", "sub", "mul", "div", "pow", "lt", "eq")
_UNARY = ("sin", "cos", "neg", "max", "sum", "argmax")


class TraitBackend:
    """The 28 trait methods over `<prefix><method>` symbols of `lib`."""

    def __init__(self, lib: C.CDLL, prefix: str, ctx):
        self._lib = lib
        self._prefix = prefix
        self._ctx = ctx
        self._fn_cache: dict[str, object] = {}
        self._declare()

    # -- plumbing -----------------------------------------------------------------
    def _f(self, name: str):
        fn = self._fn_cache.get(name)
        if fn is None:
            fn = getattr(self._lib, self._prefix + name)
            self._fn_cache[name] = fn
        return fn

    def _declare(self):
        vp, i32, i64 = _c_vp, C.c_int32, C.c_int64
        out = C.POINTER(vp)
        sig = {
            "last_error": ([vp], C.c_char_p),
            "tensor_retain": ([vp], i32),
            "tensor_release": ([vp], i32),
            "shape": ([vp, C.POINTER(i32), _c_i64p], i32),
            "dtype_of": ([vp, C.POINTER(i32)], i32),
            "zeros": ([vp, _c_i64p, i32, i32, out], i32),
            "ndarray_from_vec_f32": ([vp, vp, i64, _c_i64p, i32, out], i32),
            "ndarray_from_vec_u32": ([vp, vp, i64, _c_i64p, i32, out], i32),
            "cast": ([vp, vp, i32, out], i32),
            "broadcast": ([vp, vp, _c_i64p, i32, out], i32),
            "reshape": ([vp, vp, _c_i64p, i32, out], i32),
            "transpose": ([vp, vp, i32, i32, out], i32),
            "topk": ([vp, vp, i64, out, out], i32),
            "compare": ([vp, vp, vp, C.POINTER(i32)], i32),
            "concat": ([vp, vp, vp, i32, out], i32),
            "index": ([vp, vp, i32, vp, out], i32),
            "slice": ([vp, vp, i32, i64, i64, out], i32),
            "arange": ([vp, i64, out], i32),
            "to_vec_f32": ([vp, vp, vp, i64], i32),
            "to_vec_u32": ([vp, vp, vp, i64], i32),
        }
        for name in _BINARY:
            sig[name] = ([vp, vp, vp, out], i32)
        for name in _UNARY:
            sig[name] = ([vp, vp, out], i32)
        for name, (args, res) in sig.items():
            fn = self._f(name)
            fn.argtypes = args
            fn.restype = res

    def _err(self) -> str:
        msg = self._f("last_error")(self._ctx)
        return msg.decode() if msg else ""

    def _check(self, status: int):
        if status != 0:
            raise BackendPanic(status, self._err())

    def _wrap(self, handle, dtype: int | None = None) -> TaggedTensor:
        if dtype is None:
            d = C.c_int32()
            self._f("dtype_of")(handle, C.byref(d))
            dtype = d.value
        return TaggedTensor(self, handle, dtype)

    def _out1(self, name: str, *args) -> TaggedTensor:
        h = _c_vp()
        self._check(self._f(name)(self._ctx, *args, C.byref(h)))
        return self._wrap(h)

    # -- trait methods (backend/mod.rs line in the comment) -----------------------
    def zeros(self, shape, target_dtype) -> TaggedTensor:  # :26
        d, r = _dims(shape)
        return self._out1("zeros", d, r, int(target_dtype))

    def ndarray_from_vec_f32(self, data, shape) -> TaggedTensor:  # :28-32
        a = np.ascontiguousarray(data, dtype=np.float32).reshape(-1)
        d, r = _dims(shape)
        h = _c_vp()
        st = self._f("ndarray_from_vec_f32")(self._ctx, a.ctypes.data, a.size, d, r, C.byref(h))
        if st == 1:
            raise BackendError("ShapeError")
        self._check(st)
        return self._wrap(h, F32)

    def ndarray_from_vec_u32(self, data, shape) -> TaggedTensor:  # :34-38
        a = np.ascontiguousarray(data, dtype=np.uint32).reshape(-1)
        d, r = _dims(shape)
        h = _c_vp()
        st = self._f("ndarray_from_vec_u32")(self._ctx, a.ctypes.data, a.size, d, r, C.byref(h))
        if st == 1:
            raise BackendError("ShapeError")
        self._check(st)
        return self._wrap(h, U32)

    def cast(self, x, target_dtype) -> TaggedTensor:  # :40
        return self._out1("cast", x._h, int(target_dtype))

    def matmul(self, a, b): return self._out1("matmul", a._h, b._h)  # :41
    def add(self, a, b): return self._out1("add", a._h, b._h)  # :42
    def sub(self, a, b): return self._out1("sub", a._h, b._h)  # :43
    def mul(self, a, b): return self._out1("mul", a._h, b._h)  # :44
    def div(self, a, b): return self._out1("div", a._h, b._h)  # :45
    def pow(self, a, b): return self._out1("pow", a._h, b._h)  # :46
    def lt(self, a, b): return self._out1("lt", a._h, b._h)  # :47
    def eq(self, a, b): return self._out1("eq", a._h, b._h)  # :48
    def sin(self, x): return self._out1("sin", x._h)  # :49
    def cos(self, x): return self._out1("cos", x._h)  # :50
    def neg(self, x): return self._out1("neg", x._h)  # :51

    def broadcast(self, x, shape) -> TaggedTensor:  # :52
        d, r = _dims(shape)
        return self._out1("broadcast", x._h, d, r)

    def reshape(self, x, new_shape) -> TaggedTensor:  # :53
        d, r = _dims(new_shape)
        return self._out1("reshape", x._h, d, r)

    def transpose(self, x, dim0, dim1) -> TaggedTensor:  # :54
        return self._out1("transpose", x._h, int(dim0), int(dim1))

    def max(self, x): return self._out1("max", x._h)  # :55
    def sum(self, x): return self._out1("sum", x._h)  # :56
    def argmax(self, x): return self._out1("argmax", x._h)  # :57

    def topk(self, x, k):  # :58
        hv, hi = _c_vp(), _c_vp()
        self._check(self._f("topk")(self._ctx, x._h, int(k), C.byref(hv), C.byref(hi)))
        return self._wrap(hv, F32), self._wrap(hi, U32)

    def compare(self, a, b) -> bool:  # :59
        eq = C.c_int32()
        self._check(self._f("compare")(self._ctx, a._h, b._h, C.byref(eq)))
        return bool(eq.value)

    def concat(self, x, y, dim) -> TaggedTensor:  # :60-65
        return self._out1("concat", x._h, y._h, int(dim))

    def index(self, x, dim, indices) -> TaggedTensor:  # :66-71
        return self._out1("index", x._h, int(dim), indices._h)

    def slice(self, x, dim, start, length) -> TaggedTensor:  # :72-78
        return self._out1("slice", x._h, int(dim), int(start), int(length))

    def arange(self, end) -> TaggedTensor:  # :79
        return self._out1("arange", int(end))

    def to_vec(self, x) -> np.ndarray:  # :81 — flat TaggedVec
        n = int(np.prod(x.shape, dtype=np.int64))
        if x.dtype == F32:
            dst = np.empty(n, dtype=np.float32)
            self._check(self._f("to_vec_f32")(self._ctx, x._h, dst.ctypes.data, n))
        else:
            dst = np.empty(n, dtype=np.uint32)
            self._check(self._f("to_vec_u32")(self._ctx, x._h, dst.ctypes.data, n))
        return dst

    # -- conveniences for tests and drivers (not trait methods) -------------------
    def from_numpy(self, a: np.ndarray) -> TaggedTensor:
        """interpreter::tensor (interpreter/mod.rs:21-31) for a numpy array."""
        if a.dtype == np.uint32:
            return self.ndarray_from_vec_u32(a, a.shape)
        return self.ndarray_from_vec_f32(np.asarray(a, dtype=np.float32), a.shape)

    def to_numpy(self, x: TaggedTensor) -> np.ndarray:
        shape = x.shape
        try:
            flat = self.to_vec(x)
        except BackendPanic:
            # the reference's to_vec panics on a non-standard layout (ndarray.rs:48-49);
            # reshape materialises it first
            flat = self.to_vec(self.reshape(x, shape))
        return flat.reshape(shape)

    def lit_f32(self, v: float) -> TaggedTensor:
        """A rank-0 constant as tensor_constant builds it (interpreter/tensor_op.rs:55-66)."""
        return self.ndarray_from_vec_f32([v], ())

    def lit_u32(self, v: int) -> TaggedTensor:
        """nat_to_u32 (interpreter/tensor_op.rs:68-78)."""
        return self.ndarray_from_vec_u32([v], ())


# ---------------------------------------------------------------------------------------


def library_path() -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "libcatgrad_cuda.so")


_LIB = None


def load_library() -> C.CDLL:
    """Load libcatgrad_cuda.so from the package directory.  Raises if it was not built."""
    global _LIB
    if _LIB is None:
        path = library_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                "(there is no CPU fallback)")
        _LIB = C.CDLL(path)
    return _LIB


class CudaBackend(TraitBackend):
    """`impl Backend for CudaBackend`: device-resident tensors on one B200.

    `precision=PREC_BF16` stores rank>=2 F32 uploads as bf16 and routes their matmuls to the
    tcgen05 kernel; tags stay F32 and `to_vec` returns f32.  `stream` may be a raw
    cudaStream_t (e.g. `torch.cuda.current_stream().cuda_stream`) so the caller can time
    with events on it.
    """

    def __init__(self, device: int = 0, precision: int = PREC_F32, stream: int | None = None):
        lib = load_library()
        lib.cg_ctx_create.argtypes = [C.c_int32, C.c_int32, _c_vp, C.POINTER(_c_vp)]
        lib.cg_ctx_create.restype = C.c_int32
        ctx = _c_vp()
        st = lib.cg_ctx_create(int(device), int(precision), _c_vp(stream) if stream else None, C.byref(ctx))
        if st != 0:
            raise RuntimeError(f"cg_ctx_create failed with status {st} (is a CUDA device present?)")
        super().__init__(lib, "cg_", ctx)
        self.device = device
        self.precision = precision
        self._declare_ext()

    def _declare_ext(self):
        vp, i32, i64, f32 = _c_vp, C.c_int32, C.c_int64, C.c_float
        out = C.POINTER(vp)
        L = self._lib
        for name, args, res in [
            ("cg_ctx_destroy", [vp], i32),
            ("cg_sync", [vp], i32),
            ("cg_ctx_stream", [vp], vp),
            ("cg_launch_count", [vp], i64),
            ("cg_bytes_reserved", [vp], i64),
            ("cg_set_option", [vp, C.c_char_p, i64], i32),
            ("cg_storage_of", [vp, C.POINTER(i32)], i32),
            ("cg_to_bf16", [vp, vp, out], i32),
            ("cg_to_f32", [vp, vp, out], i32),
            ("cg_fused_rmsnorm", [vp, vp, vp, f32, i32, out], i32),
            ("cg_fused_softmax", [vp, vp, f32, out], i32),
            ("cg_fused_act_mul", [vp, vp, vp, i32, out], i32),
            ("cg_fused_rope", [vp, vp, f32, i64, out], i32),
            ("cg_fused_attention", [vp, vp, vp, vp, i64, f32, out], i32),
            ("cg_linear", [vp, vp, vp, out], i32),
            ("cg_linear_glu", [vp, vp, vp, i32, out], i32),
            ("cg_fused_moe", [vp, vp, vp, vp, vp, vp, i32, i32, i32, out, out], i32),
            ("cg_randn", [vp, _c_i64p, i32, C.c_uint64, f32, f32, out], i32),
            ("cg_probe_wait_timeout", [vp], i32),
            ("cg_lazy_stats", [vp, _c_i64p, _c_i64p, _c_i64p], i32),
            ("cg_rope_tables", [vp, f32, i32, f32, f32, f32, f32, f32, i32, i64, i64, out, out], i32),
        ]:
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = res

    def close(self):
        if self._ctx is not None:
            self._lib.cg_ctx_destroy(self._ctx)
            self._ctx = None

    # extensions ------------------------------------------------------------------
    def sync(self):
        self._check(self._lib.cg_sync(self._ctx))

    @property
    def stream(self) -> int:
        return int(self._lib.cg_ctx_stream(self._ctx) or 0)

    def launch_count(self) -> int:
        return int(self._lib.cg_launch_count(self._ctx))

    def bytes_reserved(self) -> int:
        return int(self._lib.cg_bytes_reserved(self._ctx))

    def set_option(self, name: str, value: int):
        self._check(self._lib.cg_set_option(self._ctx, name.encode(), int(value)))

    def rope_tables(self, theta, seq_len, head_dim, scaling: dict | None = None):
        """(cos, sin) [T, d/2] as the decoder builds them; `scaling` is a checkpoint's
        rope_scaling dict ("llama3" or "yarn") or None for the plain formula."""
        rs = scaling or {}
        kind = {None: 0, "llama3": 1, "yarn": 2}[rs.get("rope_type", rs.get("type"))]
        a, b = _c_vp(), _c_vp()
        self._check(self._lib.cg_rope_tables(
            self._ctx, float(theta), kind, float(rs.get("factor", 1.0)), float(rs.get("low_freq_factor", 1.0)),
            float(rs.get("high_freq_factor", 4.0)), float(rs.get("beta_fast", 32.0)), float(rs.get("beta_slow", 1.0)),
            int(rs.get("original_max_position_embeddings", 0)), int(seq_len), int(head_dim), C.byref(a), C.byref(b)))
        return self._wrap(a), self._wrap(b)

    def lazy_stats(self):
        """(trait calls recorded, chains fused, calls pending) of the deferred-evaluation mode."""
        a, b, d = C.c_int64(), C.c_int64(), C.c_int64()
        self._check(self._lib.cg_lazy_stats(self._ctx, C.byref(a), C.byref(b), C.byref(d)))
        return a.value, b.value, d.value

    def probe_wait_timeout(self):
        """Enqueue the failure-path probe: a bounded wait on a flag nothing raises."""
        self._check(self._lib.cg_probe_wait_timeout(self._ctx))

    def storage_of(self, x) -> int:
        s = C.c_int32()
        self._lib.cg_storage_of(x._h, C.byref(s))
        return s.value

    def _ext1(self, name, *args) -> TaggedTensor:
        h = _c_vp()
        self._check(getattr(self._lib, name)(self._ctx, *args, C.byref(h)))
        return self._wrap(h)

    def to_bf16(self, x): return self._ext1("cg_to_bf16", x._h)
    def to_f32(self, x): return self._ext1("cg_to_f32", x._h)

    def fused_rmsnorm(self, x, gamma, eps, plus_one=False):
        return self._ext1("cg_fused_rmsnorm", x._h, gamma._h, C.c_float(eps), int(plus_one))

    def fused_softmax(self, x, softcap=0.0):
        return self._ext1("cg_fused_softmax", x._h, C.c_float(softcap))

    def fused_act_mul(self, gate, up, act=0):
        return self._ext1("cg_fused_act_mul", gate._h, up._h, int(act))

    def fused_rope(self, x, theta, pos0=0):
        return self._ext1("cg_fused_rope", x._h, C.c_float(theta), int(pos0))

    def fused_attention(self, q, k, v, window=0, softcap=0.0):
        return self._ext1("cg_fused_attention", q._h, k._h, v._h, int(window), C.c_float(softcap))

    def linear(self, x, w):
        return self._ext1("cg_linear", x._h, w._h)

    def linear_glu(self, x, w_gate_up, act=0):
        """act(x Wg^T) * (x Wu^T) for the stacked bf16 weight [2F, in] (cg_linear_glu)."""
        return self._ext1("cg_linear_glu", x._h, w_gate_up._h, int(act))

    def peer_exchange(self):
        """(mapped, reason): whether decode-step reductions run over mapped peer memory
        (cg_comm_peer_exchange) after `tp.init_comm`."""
        fn = self._lib.cg_comm_peer_exchange
        fn.argtypes = [_c_vp, C.c_char_p, C.c_int64]
        fn.restype = C.c_int32
        buf = C.create_string_buffer(256)
        ok = fn(self._ctx, buf, 256)
        return bool(ok), buf.value.decode()

    def randn(self, shape, seed, std=1.0, mean=0.0):
        """N(mean, std) samples generated on the device (cg_randn)."""
        dims = (C.c_int64 * max(1, len(shape)))(*shape)
        return self._ext1("cg_randn", dims, len(shape), C.c_uint64(seed), C.c_float(mean), C.c_float(std))

    def fused_moe(self, x, router, gate, up, down, top_k, norm_topk=True, act=0):
        """(out, expert ids) of the mixture-of-experts block (qwen3.rs:64-133) on normalised rows."""
        o, ids = _c_vp(), _c_vp()
        self._check(self._lib.cg_fused_moe(self._ctx, x._h, router._h, gate._h, up._h, down._h, int(top_k),
                                           int(norm_topk), int(act), C.byref(o), C.byref(ids)))
        return self._wrap(o), self._wrap(ids)
