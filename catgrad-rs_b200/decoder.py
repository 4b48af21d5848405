"""The fused, KV-cached greedy runner over libcatgrad_cuda.so (cg_decoder_* entry points).

It does what the reference's example driver does (catgrad-llm/examples/llama/main.rs:118-169)
with the model graph of catgrad-llm/src/models/llama.rs, but as fused kernels over a device
KV cache instead of one full forward per generated token.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from .backend import CudaBackend, TaggedTensor, U32, _c_vp


class DecoderConfig(C.Structure):
    """Mirror of `cg_decoder_config` (include/catgrad_cuda.h)."""
    _fields_ = [
        ("arch", C.c_int32), ("num_layers", C.c_int32), ("hidden", C.c_int32), ("n_heads", C.c_int32),
        ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("ffn", C.c_int32), ("vocab", C.c_int32),
        ("rms_eps", C.c_float), ("rope_theta", C.c_float), ("tie_embeddings", C.c_int32),
        ("max_seq", C.c_int32), ("max_batch", C.c_int32),
        ("qk_norm", C.c_int32), ("act", C.c_int32), ("norm_plus_one", C.c_int32), ("post_norms", C.c_int32),
        ("embed_scale", C.c_float), ("attn_softcap", C.c_float), ("final_softcap", C.c_float),
        ("sliding_window", C.c_int32), ("window_every", C.c_int32),
        ("rope_scaling", C.c_int32), ("rope_factor", C.c_float), ("rope_low_freq_factor", C.c_float),
        ("rope_high_freq_factor", C.c_float), ("rope_beta_fast", C.c_float), ("rope_beta_slow", C.c_float),
        ("rope_original_max_pos", C.c_int32),
        ("rope_local_theta", C.c_float), ("rope_local_every", C.c_int32),
        ("n_experts", C.c_int32), ("top_k", C.c_int32), ("moe_ffn", C.c_int32), ("norm_topk", C.c_int32),
        ("tp_rank", C.c_int32), ("tp_world", C.c_int32), ("ep_rank", C.c_int32), ("ep_world", C.c_int32),
    ]


class Decoder:
    def __init__(self, backend: CudaBackend, cfg, max_seq: int, max_batch: int, tp_rank: int = 0, tp_world: int = 1,
                 ep_rank: int = 0, ep_world: int = 1, **switches):
        self.B = backend
        L = backend._lib
        vp, i32 = _c_vp, C.c_int32
        out = C.POINTER(vp)
        for name, args in [
            ("cg_decoder_create", [vp, C.POINTER(DecoderConfig), out]),
            ("cg_decoder_destroy", [vp]),
            ("cg_decoder_set_param", [vp, C.c_char_p, vp]),
            ("cg_decoder_finalize", [vp]),
            ("cg_decoder_load_safetensors", [vp, C.c_char_p]),
            ("cg_decoder_reset", [vp]),
            ("cg_decoder_prefill", [vp, vp, out]),
            ("cg_decoder_append", [vp, vp, out]),
            ("cg_decoder_truncate", [vp, C.c_int64]),
            ("cg_decoder_position", [vp, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
            ("cg_decoder_decode", [vp, i32, out]),
            ("cg_decoder_step_with", [vp, vp, out]),
            ("cg_decoder_tokens", [vp, out]),
            ("cg_decoder_generate", [vp, vp, i32, i32, i32, vp]),
            ("cg_decoder_time_gemms", [vp, i32, i32, C.POINTER(C.c_float), C.POINTER(i32)]),
        ]:
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = i32
        c = DecoderConfig()
        c.arch = 0
        c.num_layers = cfg.num_hidden_layers
        c.hidden = cfg.hidden_size
        c.n_heads = cfg.num_attention_heads
        c.n_kv_heads = cfg.num_key_value_heads
        c.head_dim = cfg.get_head_dim()
        c.ffn = cfg.intermediate_size
        c.vocab = cfg.vocab_size
        c.rms_eps = cfg.rms_norm_eps
        c.rope_theta = cfg.rope_theta
        c.tie_embeddings = int(cfg.tie_word_embeddings)
        c.max_seq = max_seq
        c.max_batch = max_batch
        c.tp_rank = tp_rank
        c.tp_world = tp_world
        c.ep_rank = ep_rank
        c.ep_world = ep_world
        rs = getattr(cfg, "rope_scaling", None)
        if rs:
            # {"rope_type": "llama3" | "yarn", "factor": ..., ...} as in a checkpoint's config.json
            kind = {"llama3": 1, "yarn": 2}[rs.get("rope_type", rs.get("type"))]
            c.rope_scaling = kind
            c.rope_factor = rs["factor"]
            c.rope_low_freq_factor = rs.get("low_freq_factor", 1.0)
            c.rope_high_freq_factor = rs.get("high_freq_factor", 4.0)
            c.rope_beta_fast = rs.get("beta_fast", 32.0)
            c.rope_beta_slow = rs.get("beta_slow", 1.0)
            c.rope_original_max_pos = rs["original_max_position_embeddings"]
        arch = getattr(cfg, "arch", "llama")
        if arch == "qwen3":
            c.arch = 1
            c.qk_norm = 1
        elif arch == "gemma":
            c.arch = 2
            c.act = 1
            c.norm_plus_one = 1
            c.post_norms = 1
            c.embed_scale = float(np.sqrt(np.float32(cfg.hidden_size), dtype=np.float32))
            c.tie_embeddings = 1
            c.qk_norm = int(cfg.qk_norm)
            c.attn_softcap = cfg.attn_logit_softcap
            c.final_softcap = cfg.final_logit_softcap
            c.sliding_window = cfg.sliding_window
            c.window_every = 2
            if getattr(cfg, "sliding_window_pattern", 0) > 0 and getattr(cfg, "rope_local_base_freq", 0.0) > 0:
                c.rope_local_theta = cfg.rope_local_base_freq
                c.rope_local_every = cfg.sliding_window_pattern
        if getattr(cfg, "num_local_experts", 0) > 1:
            # mixture-of-experts FFN on the layers whose checkpoint carries a router (qwen3.rs:297-298)
            c.n_experts = cfg.num_local_experts
            c.top_k = cfg.num_experts_per_tok
            c.moe_ffn = cfg.moe_intermediate_size
            c.norm_topk = int(cfg.norm_topk_prob)
        for k, v in switches.items():
            setattr(c, k, v)
        self.cfg = c
        h = vp()
        backend._check(L.cg_decoder_create(backend._ctx, C.byref(c), C.byref(h)))
        self._h = h

    def close(self):
        if self._h is not None:
            self.B._lib.cg_decoder_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_param(self, name: str, t: TaggedTensor):
        self.B._check(self.B._lib.cg_decoder_set_param(self._h, name.encode(), t._h))

    def load(self, named_arrays):
        """Upload (name, f32 array) pairs one at a time and hand them to the decoder."""
        for name, w in named_arrays:
            self.set_param(name, self.B.from_numpy(w))
        self.finalize()

    def load_random(self, cfg, seed: int = 0, std: float = 0.02):
        """A synthetic checkpoint generated on the device: matrices ~ N(0, std), norm gains 1
        (0 where the architecture adds 1).  For models whose weights would take minutes to
        draw and upload from the host; the values differ from `synth.make_weights`."""
        from . import synth
        import zlib
        gain = 0.0 if getattr(cfg, "arch", "llama") == "gemma" else 1.0
        for name, shape in synth.param_shapes(cfg).items():
            if len(shape) == 1:
                t = self.B.randn(shape, 0, std=0.0, mean=gain)
            else:
                t = self.B.randn(shape, (seed << 32) ^ zlib.crc32(name.encode()), std=std)
            self.set_param(name, t)
            del t
        self.finalize()

    def load_file(self, *paths: str):
        """Hand over every tensor of one or more .safetensors files (shards) and finalize."""
        for path in paths:
            self.B._check(self.B._lib.cg_decoder_load_safetensors(self._h, path.encode()))
        self.finalize()

    def finalize(self):
        self.B._check(self.B._lib.cg_decoder_finalize(self._h))

    def reset(self):
        self.B._check(self.B._lib.cg_decoder_reset(self._h))

    def _maybe_logits(self, fn, *args, want_logits=False):
        if want_logits:
            h = _c_vp()
            self.B._check(fn(self._h, *args, C.byref(h)))
            return self.B._wrap(h)
        self.B._check(fn(self._h, *args, None))
        return None

    def prefill(self, tokens: TaggedTensor, want_logits=False):
        return self._maybe_logits(self.B._lib.cg_decoder_prefill, tokens._h, want_logits=want_logits)

    def append(self, tokens: TaggedTensor, want_logits=False):
        """Run [B, S] more tokens on top of the cached positions."""
        return self._maybe_logits(self.B._lib.cg_decoder_append, tokens._h, want_logits=want_logits)

    def truncate(self, positions: int):
        """Forget the cached positions from `positions` on."""
        self.B._check(self.B._lib.cg_decoder_truncate(self._h, int(positions)))

    def position(self):
        """(cached positions, tokens generated since the last prefill / truncate)"""
        a, b = C.c_int64(), C.c_int64()
        self.B._check(self.B._lib.cg_decoder_position(self._h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def decode(self, steps: int, want_logits=False):
        return self._maybe_logits(self.B._lib.cg_decoder_decode, int(steps), want_logits=want_logits)

    def step_with(self, tokens: TaggedTensor, want_logits=False):
        return self._maybe_logits(self.B._lib.cg_decoder_step_with, tokens._h, want_logits=want_logits)

    def tokens(self) -> np.ndarray:
        h = _c_vp()
        self.B._check(self.B._lib.cg_decoder_tokens(self._h, C.byref(h)))
        return self.B.to_numpy(self.B._wrap(h, U32))

    def time_gemms(self, batch: int, iters: int = 20):
        """(ms, launches) of the weight-streaming GEMMs of one decode step, measured on the device."""
        ms, n = C.c_float(), C.c_int32()
        self.B._check(self.B._lib.cg_decoder_time_gemms(self._h, int(batch), int(iters), C.byref(ms), C.byref(n)))
        return ms.value, n.value

    def generate(self, prompt: np.ndarray, n_decode: int) -> np.ndarray:
        """Host buffers in, host buffers out: [B, S] ids -> [B, 1 + n_decode] greedy ids."""
        p = np.ascontiguousarray(prompt, dtype=np.uint32)
        b, s = p.shape
        out = np.empty((b, 1 + n_decode), dtype=np.uint32)
        self.B._check(self.B._lib.cg_decoder_generate(self._h, p.ctypes.data, b, s, int(n_decode), out.ctypes.data))
        return out
