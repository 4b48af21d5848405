"""Seeded synthetic checkpoints and prompts.

The reference downloads Hugging Face checkpoints at run time
(catgrad-llm/src/utils.rs:104-146); none exist offline, so every configuration is run on
random weights of the right shapes: each 2-D parameter ~ N(0, 0.02^2) drawn from
numpy.random.Generator(PCG64(seed)) in sorted Hugging Face name order, norm gains = 1,
token ids uniform in [0, V).  The same host arrays feed the checker and the GPU.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


@dataclass
class ModelConfig:
    """Shape of a Llama-family decoder (field names of catgrad-llm/src/legacy/models/utils.rs:52-112)."""
    name: str
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    vocab_size: int
    head_dim: int = 0
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    dtype: str = "f32"
    arch: str = "llama"               # "llama" | "qwen3" | "gemma"
    # qwen3 (catgrad-llm/src/models/qwen3.rs)
    num_local_experts: int = 0        # > 1: mixture-of-experts FFN on sparse layers
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = False
    decoder_sparse_step: int = 1
    # gemma (catgrad-llm/src/models/gemma3.rs graph; the soft-caps and the window are the
    # Gemma-2 additions of the Gemma-2-2B benchmark shape, composed from reference ops)
    qk_norm: bool = False             # per-head q/k RMSNorm (qwen3 always, gemma3 yes, gemma-2 no)
    attn_logit_softcap: float = 0.0
    final_logit_softcap: float = 0.0
    sliding_window: int = 0           # 0 = none; even layers use it when set
    # gemma3.rs:154-159: layers with (i + 1) % sliding_window_pattern != 0 rotate q/k with
    # rope_local_base_freq, the others with rope_theta (0 = one base everywhere)
    sliding_window_pattern: int = 0
    rope_local_base_freq: float = 0.0
    # frequency rescaling of long-context checkpoints (legacy/models/utils.rs:19-48), e.g.
    # {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
    #  "original_max_position_embeddings": 8192}
    rope_scaling: dict | None = None
    extras: dict = field(default_factory=dict)

    def __post_init__(self):
        if not self.head_dim:
            self.head_dim = self.hidden_size // self.num_attention_heads

    def get_head_dim(self) -> int:
        return self.head_dim


# benchmark configurations (shapes only; weights are synthetic)
TINY_LLAMA = ModelConfig("tiny-llama-f32", 256, 688, 2, 4, 2, 32000, rms_norm_eps=1e-5, rope_theta=10000.0,
                         tie_word_embeddings=False, dtype="f32")
LLAMA_32_1B = ModelConfig("llama-3.2-1b-shape", 2048, 8192, 16, 32, 8, 128256, rms_norm_eps=1e-5,
                          rope_theta=500000.0, tie_word_embeddings=True, dtype="bf16")
LLAMA_3_8B = ModelConfig("llama-3-8b-shape", 4096, 14336, 32, 32, 8, 128256, rms_norm_eps=1e-5,
                         rope_theta=500000.0, tie_word_embeddings=False, dtype="bf16")


GEMMA_2_2B = ModelConfig("gemma-2-2b-shape", 2304, 9216, 26, 8, 4, 256000, head_dim=256, rms_norm_eps=1e-6,
                         rope_theta=10000.0, tie_word_embeddings=True, dtype="bf16", arch="gemma",
                         attn_logit_softcap=50.0, final_logit_softcap=30.0, sliding_window=4096)
QWEN3_30B_A3B = ModelConfig("qwen3-30b-a3b-shape", 2048, 6144, 48, 32, 4, 151936, head_dim=128, rms_norm_eps=1e-6,
                            rope_theta=1e6, tie_word_embeddings=False, dtype="bf16", arch="qwen3",
                            num_local_experts=128, num_experts_per_tok=8, moe_intermediate_size=768,
                            norm_topk_prob=True)


def param_shapes(cfg: ModelConfig) -> dict[str, tuple[int, ...]]:
    """Hugging Face tensor names and shapes of a checkpoint (all weights [out, in]); experts are
    already stacked [E, ...] the way the reference driver stacks them
    (catgrad-llm/examples/llama/main.rs:173-264)."""
    H, F, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    nh, nkv = cfg.num_attention_heads, cfg.num_key_value_heads
    shapes = {"model.embed_tokens.weight": (cfg.vocab_size, H), "model.norm.weight": (H,)}
    if not cfg.tie_word_embeddings:
        shapes["lm_head.weight"] = (cfg.vocab_size, H)
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        shapes[p + "input_layernorm.weight"] = (H,)
        shapes[p + "post_attention_layernorm.weight"] = (H,)
        shapes[p + "self_attn.q_proj.weight"] = (nh * d, H)
        shapes[p + "self_attn.k_proj.weight"] = (nkv * d, H)
        shapes[p + "self_attn.v_proj.weight"] = (nkv * d, H)
        shapes[p + "self_attn.o_proj.weight"] = (H, nh * d)
        if cfg.qk_norm or cfg.arch == "qwen3":
            shapes[p + "self_attn.q_norm.weight"] = (d,)
            shapes[p + "self_attn.k_norm.weight"] = (d,)
        if cfg.arch == "gemma":
            shapes[p + "pre_feedforward_layernorm.weight"] = (H,)
            shapes[p + "post_feedforward_layernorm.weight"] = (H,)
        moe = cfg.num_local_experts > 1 and (i + 1) % cfg.decoder_sparse_step == 0
        if moe:
            E, Fe = cfg.num_local_experts, cfg.moe_intermediate_size
            shapes[p + "mlp.gate.weight"] = (E, H)
            shapes[p + "mlp.experts.gate_proj.weight"] = (E, Fe, H)
            shapes[p + "mlp.experts.up_proj.weight"] = (E, Fe, H)
            shapes[p + "mlp.experts.down_proj.weight"] = (E, H, Fe)
        else:
            shapes[p + "mlp.gate_proj.weight"] = (F, H)
            shapes[p + "mlp.up_proj.weight"] = (F, H)
            shapes[p + "mlp.down_proj.weight"] = (H, F)
    return shapes


def bf16_round(a: np.ndarray) -> np.ndarray:
    """Round f32 to the nearest bf16 (ties to even), returned as f32."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    rounded = (u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))) & np.uint32(0xFFFF0000)
    return rounded.view(np.float32)


def make_weights(cfg: ModelConfig, seed: int = 0, std: float = 0.02):
    """Yield (name, f32 array) in sorted name order.  bf16 configurations get weights already
    rounded to bf16 so the f32 checker and the bf16 device copy hold the same numbers."""
    rng = np.random.Generator(np.random.PCG64(seed))
    shapes = param_shapes(cfg)
    for name in sorted(shapes):
        shp = shapes[name]
        if len(shp) == 1:
            # norm gains: an effective gain of 1 (gemma multiplies by 1 + gamma, so gamma = 0)
            w = np.zeros(shp, dtype=np.float32) if cfg.arch == "gemma" else np.ones(shp, dtype=np.float32)
        else:
            w = rng.standard_normal(shp, dtype=np.float32) * np.float32(std)
            if cfg.dtype == "bf16":
                w = bf16_round(w)
        yield name, w


def make_tokens(cfg: ModelConfig, batch: int, seq: int, seed: int = 1) -> np.ndarray:
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.integers(0, cfg.vocab_size, size=(batch, seq), dtype=np.int64).astype(np.uint32)


def linear_params_per_token(cfg: ModelConfig) -> int:
    """Weights multiplied per token: every linear layer including the LM head, excluding the
    embedding gather."""
    H, F, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    nh, nkv = cfg.num_attention_heads, cfg.num_key_value_heads
    per_layer = H * (nh * d) + 2 * H * (nkv * d) + (nh * d) * H + 3 * H * F
    return cfg.num_hidden_layers * per_layer + cfg.vocab_size * H


def kv_bytes_per_token(cfg: ModelConfig, elem_bytes: int = 2) -> int:
    return 2 * cfg.num_hidden_layers * cfg.num_key_value_heads * cfg.head_dim * elem_bytes
