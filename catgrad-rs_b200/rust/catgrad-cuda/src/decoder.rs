// NOT compiled in this repository's build environment (no Rust toolchain): source only.
//
// The fused, KV-cached greedy runner (cg_decoder_* in include/catgrad_cuda.h): what the
// reference's example driver does in its loop (catgrad-llm/examples/llama/main.rs:118-169),
// as one call.  The checkpoint tensors are handed over under their Hugging Face names, the
// names the reference's loader already uses (main.rs:325); experts stacked [E, ...] the way
// the driver stacks them (main.rs:173-264).
use crate::{ffi, CudaBackend, CudaTensor};
use std::ffi::CString;
use std::os::raw::c_char;

/// Mirror of `cg_decoder_config` (field order and types are part of the ABI).
#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct DecoderConfig {
    pub arch: i32,
    pub num_layers: i32,
    pub hidden: i32,
    pub n_heads: i32,
    pub n_kv_heads: i32,
    pub head_dim: i32,
    pub ffn: i32,
    pub vocab: i32,
    pub rms_eps: f32,
    pub rope_theta: f32,
    pub tie_embeddings: i32,
    pub max_seq: i32,
    pub max_batch: i32,
    pub qk_norm: i32,
    pub act: i32,
    pub norm_plus_one: i32,
    pub post_norms: i32,
    pub embed_scale: f32,
    pub attn_softcap: f32,
    pub final_softcap: f32,
    pub sliding_window: i32,
    pub window_every: i32,
    pub rope_scaling: i32,
    pub rope_factor: f32,
    pub rope_low_freq_factor: f32,
    pub rope_high_freq_factor: f32,
    pub rope_beta_fast: f32,
    pub rope_beta_slow: f32,
    pub rope_original_max_pos: i32,
    pub rope_local_theta: f32,
    pub rope_local_every: i32,
    pub n_experts: i32,
    pub top_k: i32,
    pub moe_ffn: i32,
    pub norm_topk: i32,
    pub tp_rank: i32,
    pub tp_world: i32,
    pub ep_rank: i32,
    pub ep_world: i32,
}

#[repr(C)]
pub struct cg_decoder { _p: [u8; 0] }

extern "C" {
    fn cg_decoder_create(ctx: *mut ffi::cg_ctx, cfg: *const DecoderConfig, out: *mut *mut cg_decoder) -> i32;
    fn cg_decoder_destroy(d: *mut cg_decoder) -> i32;
    fn cg_decoder_set_param(d: *mut cg_decoder, name: *const c_char, t: *const ffi::cg_tensor) -> i32;
    fn cg_decoder_finalize(d: *mut cg_decoder) -> i32;
    fn cg_decoder_generate(d: *mut cg_decoder, prompt: *const u32, batch: i32, seq: i32, n_decode: i32, out: *mut u32) -> i32;
    fn cg_decoder_load_safetensors(d: *mut cg_decoder, path: *const c_char) -> i32;
    fn cg_decoder_append(d: *mut cg_decoder, tokens: *const ffi::cg_tensor, logits_out: *mut *mut ffi::cg_tensor) -> i32;
    fn cg_decoder_truncate(d: *mut cg_decoder, positions: i64) -> i32;
    fn cg_decoder_tokens(d: *mut cg_decoder, out: *mut *mut ffi::cg_tensor) -> i32;
}

pub struct Decoder {
    raw: *mut cg_decoder,
    backend: CudaBackend, // keeps the context alive
}

impl Decoder {
    pub fn new(backend: &CudaBackend, cfg: &DecoderConfig) -> Self {
        let mut raw = std::ptr::null_mut();
        backend.check(unsafe { cg_decoder_create(backend.raw_ctx(), cfg, &mut raw) });
        Decoder { raw, backend: backend.clone() }
    }

    /// Hand over one checkpoint tensor; the decoder keeps its own reference.
    pub fn set_param(&mut self, name: &str, t: &CudaTensor) {
        let c = CString::new(name).expect("parameter name");
        self.backend.check(unsafe { cg_decoder_set_param(self.raw, c.as_ptr(), t.raw()) });
    }

    /// Build the fused weights and the KV cache; the handed-over originals are released.
    pub fn finalize(&mut self) {
        self.backend.check(unsafe { cg_decoder_finalize(self.raw) });
    }

    /// Prefill `prompt` ([batch, seq], row-major) and decode `n_decode` greedy steps; returns
    /// [batch, 1 + n_decode] token ids (the prompt's next token first).
    pub fn generate(&mut self, prompt: &[u32], batch: usize, seq: usize, n_decode: usize) -> Vec<u32> {
        assert_eq!(prompt.len(), batch * seq);
        let mut out = vec![0u32; batch * (1 + n_decode)];
        self.backend.check(unsafe {
            cg_decoder_generate(self.raw, prompt.as_ptr(), batch as i32, seq as i32, n_decode as i32, out.as_mut_ptr())
        });
        out
    }
}

impl Decoder {
    /// Hand over every tensor of a .safetensors file (call once per shard, then `finalize`): replaces
    /// the host-side loading of catgrad-llm/examples/llama/main.rs:279-354.
    pub fn load_safetensors(&mut self, path: &str) {
        let c = CString::new(path).expect("path");
        self.backend.check(unsafe { cg_decoder_load_safetensors(self.raw, c.as_ptr()) });
    }

    /// Run `tokens` (one row) on top of the cached positions and return the greedy next token.
    fn append_row(&mut self, tokens: &[u32]) -> u32 {
        use catgrad::category::core::Shape;
        use catgrad::interpreter::backend::Backend;
        let t = match self.backend.ndarray_from_vec_u32(tokens.to_vec(), Shape(vec![1, tokens.len()])) {
            Ok(catgrad::interpreter::TaggedTensor::U32([t])) => t,
            _ => panic!("token upload failed"),
        };
        self.backend.check(unsafe { cg_decoder_append(self.raw, t.raw(), std::ptr::null_mut()) });
        let mut hist = std::ptr::null_mut();
        self.backend.check(unsafe { cg_decoder_tokens(self.raw, &mut hist) });
        let hist = crate::CudaTensor::from_raw(hist);
        match self.backend.to_vec(catgrad::interpreter::TaggedTensor::U32([hist])) {
            catgrad::interpreter::TaggedVec::U32(v) => *v.last().expect("one generated token"),
            _ => unreachable!(),
        }
    }
}

/// `serve::LM` (catgrad-llm/src/serve.rs:12-20) over the fused decoder, the way the reference's
/// `ModelRunner` implements it (catgrad-llm/src/run.rs:262-305), except that `set_context` keeps the
/// longest common prefix of the old and the new context in the cache instead of all or nothing.
pub struct DecoderLM {
    dec: Decoder,
    eos: Vec<u32>,
    cached: Vec<u32>,
    pending: Vec<u32>,
}

impl DecoderLM {
    pub fn new(dec: Decoder, eos: Vec<u32>) -> Self { DecoderLM { dec, eos, cached: vec![], pending: vec![] } }

    pub fn set_context(&mut self, context: Vec<u32>) {
        let mut n = self.cached.iter().zip(context.iter()).take_while(|(a, b)| a == b).count();
        if n == context.len() && n > 0 { n -= 1; }  // at least one token must run to get a next token
        if n < self.cached.len() {
            self.dec.backend.check(unsafe { cg_decoder_truncate(self.dec.raw, n as i64) });
            self.cached.truncate(n);
        }
        self.pending = context[n..].to_vec();
    }
}

impl Iterator for DecoderLM {
    type Item = u32;
    fn next(&mut self) -> Option<u32> {
        let tokens = std::mem::take(&mut self.pending);
        if tokens.is_empty() { return None; }
        let token = self.dec.append_row(&tokens);
        self.cached.extend(tokens);
        if self.eos.contains(&token) { return None; }  // EOS tokens are not emitted (run.rs:252-255)
        self.pending.push(token);
        Some(token)
    }
}

impl Drop for Decoder {
    fn drop(&mut self) {
        unsafe { cg_decoder_destroy(self.raw); }
    }
}
