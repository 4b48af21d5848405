"""catgrad-rs_b200 — a B200-native tensor backend for the catgrad interpreter.

The directory name is not a Python identifier; import it with
`importlib.import_module("catgrad-rs_b200")`.

* `backend`  — `CudaBackend`, the mirror of `trait Backend` over the C ABI
* `graphs`   — the op streams of catgrad's stdlib and catgrad-llm model graphs
* `decoder`  — the fused, KV-cached greedy runner
* `synth`    — seeded synthetic checkpoints and prompts
* `safetensors_io` — .safetensors checkpoint files: library-side reader, numpy writer
* `serve`    — the LM / Tokenizer / Loader interfaces of catgrad-llm's serve.rs; `DecoderLM` with prefix reuse
* `tp`       — tensor-parallel sharding plan and communicator set-up
* `build`    — the nvcc recipe for libcatgrad_cuda.so
"""
from .backend import (  # noqa: F401
    F32, U32, PREC_F32, PREC_BF16, BackendError, BackendPanic, TaggedTensor, TraitBackend,
    CudaBackend, load_library, library_path,
)
from . import graphs, safetensors_io, serve, synth, tp  # noqa: F401
from .decoder import Decoder, DecoderConfig  # noqa: F401
