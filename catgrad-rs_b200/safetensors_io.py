"""Reading and writing .safetensors checkpoint files.

Reading goes through the library (`cg_safetensors_*`, `cg_decoder_load_safetensors`): the file is
memory-mapped, the header parsed in C++, and every tensor copied host -> device once in its
stored element type.  `write` produces files in the same format from numpy arrays (F32 or BF16),
for tests and for synthetic checkpoints; it follows the published layout (8-byte little-endian
header length, JSON header, raw little-endian tensor bytes) that the reference reads through
the safetensors crate (catgrad-llm/examples/llama/main.rs:296-330).
"""
from __future__ import annotations

import ctypes as C
import json
import struct

import numpy as np

from .backend import CudaBackend, _c_vp, load_library
from .synth import bf16_round


def write(path: str, named_arrays, dtype: str = "BF16", metadata: dict | None = None) -> None:
    """Write (name, f32 array) pairs.  dtype "BF16" stores rank >= 2 arrays as bf16 (rounded to
    nearest even) and the rest as F32; "F32" stores everything as F32."""
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, a in named_arrays:
        a = np.asarray(a, dtype=np.float32, order="C")   # (ascontiguousarray would turn rank 0 into rank 1)
        if dtype == "BF16" and a.ndim >= 2:
            raw = (bf16_round(a).view(np.uint32) >> np.uint32(16)).astype("<u2").tobytes()
            dt = "BF16"
        else:
            raw = a.astype("<f4").tobytes()
            dt = "F32"
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)   # writers pad the header so the data section is 8-byte aligned
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for b in blobs:
            f.write(b)


def _declare(lib):
    vp, i32, i64 = _c_vp, C.c_int32, C.c_int64
    lib.cg_safetensors_open.argtypes = [C.c_char_p, C.POINTER(vp), C.c_char_p, i64]
    lib.cg_safetensors_open.restype = i32
    lib.cg_safetensors_close.argtypes = [vp]
    lib.cg_safetensors_count.argtypes = [vp]
    lib.cg_safetensors_count.restype = i64
    lib.cg_safetensors_info.argtypes = [vp, i64, C.POINTER(C.c_char_p), C.POINTER(i32), C.POINTER(i32), C.POINTER(i64)]
    lib.cg_safetensors_info.restype = i32
    lib.cg_safetensors_tensor.argtypes = [vp, vp, i64, C.POINTER(vp)]
    lib.cg_safetensors_tensor.restype = i32
    return lib


class File:
    """A memory-mapped checkpoint file; no device is needed to open it or to list its tensors."""

    def __init__(self, path: str):
        self._lib = _declare(load_library())
        h, err = _c_vp(), C.create_string_buffer(512)
        if self._lib.cg_safetensors_open(path.encode(), C.byref(h), err, 512) != 0:
            raise ValueError(err.value.decode())
        self._h = h

    def close(self):
        if self._h is not None:
            self._lib.cg_safetensors_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __len__(self):
        return int(self._lib.cg_safetensors_count(self._h))

    def info(self, i: int):
        """(name, "F32" | "BF16", shape) of tensor i."""
        name, st, rank = C.c_char_p(), C.c_int32(), C.c_int32()
        dims = (C.c_int64 * 8)()
        if self._lib.cg_safetensors_info(self._h, i, C.byref(name), C.byref(st), C.byref(rank), dims) != 0:
            raise IndexError(i)
        return name.value.decode(), {0: "F32", 2: "BF16"}[st.value], tuple(dims[k] for k in range(rank.value))

    def tensor(self, backend: CudaBackend, i: int):
        h = _c_vp()
        backend._check(self._lib.cg_safetensors_tensor(backend._ctx, self._h, i, C.byref(h)))
        return backend._wrap(h)


def load_params(backend: CudaBackend, path: str) -> dict:
    """name -> device tensor for every tensor of the file: the parameter map an interpreter is
    built with (catgrad-llm/examples/llama/main.rs:300-331)."""
    f = File(path)
    try:
        return {f.info(i)[0]: f.tensor(backend, i) for i in range(len(f))}
    finally:
        f.close()
