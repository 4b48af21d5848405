"""The C-ABI library loads and exports every symbol include/catgrad_cuda.h declares; the
checker exports the trait-level subset under its own prefix.  No compute calls."""
import ctypes
import os
import re

from conftest import ROOT, cg, load_oracle_lib


def declared(header, prefix):
    text = open(header).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(" + prefix + r"[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = declared(os.path.join(ROOT, "include", "catgrad_cuda.h"), "cg_")
    assert len(names) > 50
    lib = cg.load_library()
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_oracle_exports_the_trait_subset():
    names = declared(os.path.join(ROOT, "oracle", "oracle.h"), "cgo_")
    lib = load_oracle_lib()
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    # every trait-level entry point of the product has a twin in the checker
    product = set(declared(os.path.join(ROOT, "include", "catgrad_cuda.h"), "cg_"))
    for n in names:
        if n in ("cgo_ctx_create", "cgo_ctx_destroy", "cgo_ctx_threads"):
            continue
        assert "cg_" + n[4:] in product, n


def test_no_cpu_fallback_without_a_device():
    import torch
    if torch.cuda.is_available():
        return
    try:
        cg.CudaBackend(0)
    except RuntimeError as e:
        assert "cg_ctx_create failed" in str(e)
    else:
        raise AssertionError("CudaBackend must not construct without a GPU")


def test_decoder_config_mirror_matches_header():
    text = open(os.path.join(ROOT, "include", "catgrad_cuda.h")).read()
    body = text[text.index("typedef struct cg_decoder_config {"):text.index("} cg_decoder_config;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = re.findall(r"\b(?:int32_t|float)\s+([a-z_0-9]+)\s*;", body)
    assert fields == [f[0] for f in cg.DecoderConfig._fields_]


def test_rust_shim_mirrors_match_header():
    """The Rust binding is source only (no toolchain here), so its ABI mirrors are checked as
    text: the decoder configuration has the header's fields in the header's order and types, and
    every extern function the shim declares exists in the header."""
    text = open(os.path.join(ROOT, "include", "catgrad_cuda.h")).read()
    body = text[text.index("typedef struct cg_decoder_config {"):text.index("} cg_decoder_config;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    want = [(n, "f32" if t == "float" else "i32") for t, n in re.findall(r"\b(int32_t|float)\s+([a-z_0-9]+)\s*;", body)]
    rust_dir = os.path.join(ROOT, "catgrad-rs_b200", "rust", "catgrad-cuda", "src")
    rs = open(os.path.join(rust_dir, "decoder.rs")).read()
    struct = rs[rs.index("pub struct DecoderConfig {"):]
    struct = struct[:struct.index("}")]
    got = re.findall(r"pub\s+([a-z_0-9]+)\s*:\s*(i32|f32)\s*,", struct)
    assert got == want
    product = set(declared(os.path.join(ROOT, "include", "catgrad_cuda.h"), "cg_"))
    for name in ("ffi.rs", "decoder.rs"):
        src = open(os.path.join(rust_dir, name)).read()
        for fn in re.findall(r"\bfn\s+(cg_[a-z0-9_]+)\s*\(", src):
            assert fn in product, (name, fn)
