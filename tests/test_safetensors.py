"""Checkpoint files (.safetensors): header parsing on the host, tensors to the device.

The reference loads checkpoints through the safetensors crate into host Vec<f32>
(catgrad-llm/examples/llama/main.rs:279-354) and stacks mixture-of-experts matrices by repeated
concatenation (:173-264).  The library maps the file, parses the header itself and uploads each
tensor once.  CPU tests cover the parser (no device needed); GPU tests check that a decoder
loaded from files gives exactly the logits of one fed tensor by tensor, including per-expert
tensors landing in the stacked layout.
"""
import json
import struct

import numpy as np
import pytest

from conftest import cg

synth, sio = cg.synth, cg.safetensors_io


def test_header_is_parsed_without_a_device(tmp_path):
    rng = np.random.Generator(np.random.PCG64(3))
    arrays = [("model.embed_tokens.weight", rng.standard_normal((10, 6), dtype=np.float32)),
              ("model.norm.weight", np.ones(6, dtype=np.float32)),
              ("odd \"name\"\\with.escapes", rng.standard_normal((2, 3, 4), dtype=np.float32)),
              ("scalar", np.float32(3.5).reshape(()))]
    path = str(tmp_path / "a.safetensors")
    sio.write(path, arrays, dtype="BF16", metadata={"format": "pt", "note": "{nested: [brackets]}"})
    f = sio.File(path)
    assert len(f) == 4
    assert f.info(0) == ("model.embed_tokens.weight", "BF16", (10, 6))
    assert f.info(1) == ("model.norm.weight", "F32", (6,))
    assert f.info(2) == ("odd \"name\"\\with.escapes", "BF16", (2, 3, 4))
    assert f.info(3) == ("scalar", "F32", ())
    with pytest.raises(IndexError):
        f.info(4)
    f.close()


def _raw(path, header: dict, payload: bytes):
    text = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text + payload)


def test_malformed_files_are_refused_with_a_reason(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    with pytest.raises(ValueError, match="cannot open"):
        sio.File(str(tmp_path / "missing.safetensors"))
    open(p, "wb").write(b"\x01\x02")
    with pytest.raises(ValueError, match="shorter than"):
        sio.File(p)
    open(p, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(ValueError, match="header length"):
        sio.File(p)
    _raw(p, {"w": {"dtype": "F16", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 4)
    with pytest.raises(ValueError, match="unsupported dtype F16"):     # the reference's loader panics on these
        sio.File(p)
    _raw(p, {"w": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8)
    with pytest.raises(ValueError, match="do not match"):
        sio.File(p)
    _raw(p, {"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}, b"\0" * 8)   # data section too short
    with pytest.raises(ValueError, match="do not match"):
        sio.File(p)
    open(p, "wb").write(struct.pack("<Q", 5) + b"[1,2]")
    with pytest.raises(ValueError, match="not a JSON object"):
        sio.File(p)


@pytest.mark.gpu
def test_tensors_reach_the_device_unchanged(tmp_path, cuda, cuda_bf16):
    rng = np.random.Generator(np.random.PCG64(5))
    arrays = [("a", rng.standard_normal((33, 17), dtype=np.float32)), ("g", rng.standard_normal(17).astype(np.float32))]
    for dtype in ("F32", "BF16"):
        path = str(tmp_path / f"t_{dtype}.safetensors")
        sio.write(path, arrays, dtype=dtype)
        for B in (cuda, cuda_bf16):
            params = sio.load_params(B, path)
            want_a = arrays[0][1] if (dtype == "F32" and B is cuda) else synth.bf16_round(arrays[0][1])
            np.testing.assert_array_equal(B.to_numpy(params["a"]), want_a)
            np.testing.assert_array_equal(B.to_numpy(params["g"]), arrays[1][1])
            # bf16 data stays bf16 on a bf16-precision context (storage code 2), f32 elsewhere
            assert B.storage_of(params["a"]) == (2 if B is cuda_bf16 else 0)


SMALL = synth.ModelConfig("small-llama-bf16", 256, 512, 2, 4, 2, 1024, rms_norm_eps=1e-5, rope_theta=500000.0,
                          tie_word_embeddings=True, dtype="bf16")
MOE = synth.ModelConfig("qwen3-moe-small", 128, 256, 2, 4, 2, 512, head_dim=64, arch="qwen3", rope_theta=1e6,
                        num_local_experts=16, num_experts_per_tok=4, moe_intermediate_size=96, norm_topk_prob=True,
                        dtype="bf16")


@pytest.mark.gpu
@pytest.mark.parametrize("cfg,dtype", [(SMALL, "BF16"), (SMALL, "F32"), (MOE, "BF16")], ids=["dense-bf16", "dense-f32", "moe-bf16"])
def test_decoder_loaded_from_files_equals_tensor_by_tensor(tmp_path, cuda_bf16, cfg, dtype):
    C = cuda_bf16
    weights = list(synth.make_weights(cfg, 0))
    # checkpoints store each expert on its own ("...experts.E.gate_proj.weight"); two shard files
    on_disk = []
    for name, w in weights:
        if ".mlp.experts." in name and w.ndim == 3:
            stem, proj = name.rsplit(".", 2)[0], name.rsplit(".", 2)[1]
            on_disk += [(f"{stem}.{e}.{proj}.weight", w[e]) for e in range(w.shape[0])]
        else:
            on_disk.append((name, w))
    half = len(on_disk) // 2
    p1, p2 = str(tmp_path / "m-1.safetensors"), str(tmp_path / "m-2.safetensors")
    sio.write(p1, on_disk[:half], dtype=dtype)
    sio.write(p2, on_disk[half:], dtype=dtype)
    prompt = C.from_numpy(synth.make_tokens(cfg, 2, 20, seed=1))
    a = cg.Decoder(C, cfg, max_seq=32, max_batch=2)
    a.load(weights)
    b = cg.Decoder(C, cfg, max_seq=32, max_batch=2)
    b.load_file(p1, p2)
    la = C.to_numpy(a.prefill(prompt, want_logits=True))
    lb = C.to_numpy(b.prefill(prompt, want_logits=True))
    np.testing.assert_array_equal(la, lb)          # the same bytes reached the same kernels
    la = C.to_numpy(a.decode(3, want_logits=True))
    lb = C.to_numpy(b.decode(3, want_logits=True))
    np.testing.assert_array_equal(la, lb)
    np.testing.assert_array_equal(a.tokens(), b.tokens())
    a.close()
    b.close()
