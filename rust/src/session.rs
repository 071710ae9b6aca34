//! `B200Session`: the drop-in for `InferenceSession<B>` (akasha-core src/nn/inference.rs:13-327).
//!
//! Same surface (`new`, `replace_cache`, `take_cache`, `prefill`, `decode_step`, `generate`), same
//! `AkashaError` results in the same situations; the graphs, the scratch buffers and the KV cache
//! live inside the library. `Cache<B>` values do not cross the boundary: `replace_cache()`
//! attaches a fresh empty cache, `take_cache()` detaches it (the next `prefill` then fails with
//! `NoCache`, as in the reference).
use crate::ffi::*;
use crate::{check_fatal, last_error, AkashaError, ModelConfig, Real};
use std::os::raw::c_int;
use std::ptr;

/// Owner of a device context and the uploaded weights; shared by sessions and engines
/// (`Arc<ModelWeights<B>>` in the reference, src/nn/inference.rs:15).
pub struct B200Weights {
    pub(crate) ctx: *mut AkCtx,
    pub(crate) w: *mut AkWeights,
    pub cfg: ModelConfig,
    pub bf16: bool,
}

impl B200Weights {
    /// `params`: the tensors in `ModelWeights::params()` order (src/nn/weights.rs:158-171): embedding,
    /// per block norm_1, qkv_proj, out_proj, norm_2, ffn_up, ffn_down, then final_norm, lm_head; matrices
    /// `[in, out]` row-major f32, as the checkpoint stores them. `bf16 = true` keeps bf16 copies on the device
    /// (the fast mode); `false` is the fp32 parity mode.
    pub fn from_params(device: i32, cfg: ModelConfig, params: &[Vec<Real>], bf16: bool) -> Self {
        let mut ctx = ptr::null_mut();
        let mut w = ptr::null_mut();
        unsafe {
            check_fatal(ak_ctx_create(device as c_int, &mut ctx));
            let fcfg = cfg.to_ffi();
            check_fatal(ak_weights_create(ctx, &fcfg, if bf16 { AK_BF16 } else { AK_F32 }, &mut w));
            let count = ak_weights_param_count(w) as usize;
            assert_eq!(count, params.len(), "expected {count} tensors in params() order, got {}", params.len());
            for (i, t) in params.iter().enumerate() {
                assert_eq!(ak_weights_param_len(w, i as u32) as usize, t.len(), "tensor {i}: wrong element count");
                check_fatal(ak_weights_set_param(w, i as u32, t.as_ptr(), t.len() as u64));
            }
        }
        Self { ctx, w, cfg, bf16 }
    }

    /// Load an AKV3 checkpoint (src/nn/checkpoint.rs:98-161); returns the weights and the stored training step.
    pub fn from_checkpoint(device: i32, path: &str, bf16: bool) -> (Self, u64) {
        let cpath = std::ffi::CString::new(path).expect("path contains a NUL byte");
        let mut fcfg = AkModelConfig { vocab_size: 0, dim: 0, num_heads: 0, num_layers: 0, seq_len: 0, ffn_hidden: 0, norm_eps: 0.0, eos_token: 0 };
        let (mut step, mut ctx, mut w) = (0u64, ptr::null_mut(), ptr::null_mut());
        unsafe {
            check_fatal(ak_akv3_read_header(cpath.as_ptr(), &mut fcfg, &mut step));
            check_fatal(ak_ctx_create(device as c_int, &mut ctx));
            check_fatal(ak_weights_create(ctx, &fcfg, if bf16 { AK_BF16 } else { AK_F32 }, &mut w));
            check_fatal(ak_weights_load_akv3(w, cpath.as_ptr(), &mut step));
        }
        let cfg = ModelConfig {
            vocab_size: fcfg.vocab_size,
            dim: fcfg.dim,
            num_heads: fcfg.num_heads,
            num_layers: fcfg.num_layers as usize,
            seq_len: fcfg.seq_len,
            ffn_hidden: fcfg.ffn_hidden,
            norm_eps: fcfg.norm_eps,
            batch_size: 1,
            eos_token: fcfg.eos_token,
        };
        (Self { ctx, w, cfg, bf16 }, step)
    }
}

impl Drop for B200Weights {
    fn drop(&mut self) {
        unsafe {
            ak_weights_destroy(self.w);
            ak_ctx_destroy(self.ctx);
        }
    }
}

/// Decoding settings of `generate` (the positional arguments of src/nn/inference.rs:264-273).
#[derive(Clone, Copy, Debug)]
pub struct Sampling {
    pub temperature: f32,
    pub top_k: usize,
    pub top_p: f32,
    pub repetition_penalty: f32,
    /// The device sampler draws from a counter-based generator keyed by (seed, token index); the reference's
    /// generator is unseeded (src/nn/sampling.rs:73).
    pub seed: u64,
}

impl Sampling {
    /// What `run_chat` passes (src/main.rs:160-162).
    pub fn chat_defaults() -> Self {
        Self { temperature: 0.8, top_k: 40, top_p: 0.95, repetition_penalty: 1.15, seed: 0 }
    }
    pub fn greedy() -> Self {
        Self { temperature: 0.0, top_k: 0, top_p: 1.0, repetition_penalty: 1.0, seed: 0 }
    }
}

pub struct B200Session<'w> {
    weights: &'w B200Weights,
    s: *mut AkSession,
    max_context_len: u32,
}

impl<'w> B200Session<'w> {
    /// `InferenceSession::new` (src/nn/inference.rs:25-40): the cache starts detached.
    pub fn new(weights: &'w B200Weights, max_context_len: u32) -> Self {
        let mut s = ptr::null_mut();
        unsafe { check_fatal(ak_session_create(weights.ctx, weights.w, max_context_len, &mut s)) };
        Self { weights, s, max_context_len }
    }

    fn result(&self, rc: c_int, len: u32) -> Result<(), AkashaError> {
        match rc {
            AK_OK => Ok(()),
            AK_EMPTY_PROMPT => Err(AkashaError::EmptyPrompt),
            AK_PROMPT_TOO_LONG => Err(AkashaError::PromptTooLong { len, max: self.max_context_len }),
            AK_CONTEXT_FULL => Err(AkashaError::ContextFull { max: self.max_context_len }),
            AK_NO_CACHE => Err(AkashaError::NoCache),
            AK_CACHE_NOT_EMPTY => Err(AkashaError::CacheNotEmpty { cur_len: self.cur_len() }),
            other => panic!("akasha-b200: error {other}: {}", last_error()),
        }
    }

    /// `replace_cache(Cache::new(..))` (src/nn/inference.rs:42-54): attach an empty cache.
    pub fn replace_cache(&mut self) {
        unsafe { check_fatal(ak_session_attach_cache(self.s)) };
    }
    /// `take_cache` (src/nn/inference.rs:56-59).
    pub fn take_cache(&mut self) {
        unsafe { check_fatal(ak_session_take_cache(self.s)) };
    }
    /// `Cache::reset` (src/nn/inference_graphs.rs:540-542).
    pub fn reset_cache(&mut self) -> Result<(), AkashaError> {
        let rc = unsafe { ak_session_reset_cache(self.s) };
        self.result(rc, 0)
    }
    pub fn cur_len(&self) -> u32 {
        unsafe { ak_session_cur_len(self.s) }
    }

    /// src/nn/inference.rs:61-176: logits of the last prompt row.
    pub fn prefill(&mut self, prompt_tokens: &[u32]) -> Result<Vec<Real>, AkashaError> {
        let mut logits = vec![0.0 as Real; self.weights.cfg.vocab_size as usize];
        let rc = unsafe {
            ak_session_prefill(self.s, prompt_tokens.as_ptr(), prompt_tokens.len() as u32, logits.as_mut_ptr(), ptr::null_mut())
        };
        self.result(rc, prompt_tokens.len() as u32).map(|_| logits)
    }

    /// src/nn/inference.rs:178-262.
    pub fn decode_step(&mut self, token: u32) -> Result<Vec<Real>, AkashaError> {
        let mut logits = vec![0.0 as Real; self.weights.cfg.vocab_size as usize];
        let rc = unsafe { ak_session_decode_step(self.s, token, logits.as_mut_ptr(), ptr::null_mut()) };
        self.result(rc, 1).map(|_| logits)
    }

    /// src/nn/inference.rs:264-326, returning token ids (the caller decodes them with its tokenizer, as
    /// `generate` does in its last line). Logits never leave the device: `sample_token` runs there.
    pub fn generate(&mut self, prompt_tokens: &[u32], max_new_tokens: usize, how: Sampling) -> Result<Vec<u32>, AkashaError> {
        let mut out = vec![0u32; max_new_tokens.max(1)];
        let mut n_out = 0u32;
        let greedy = how.temperature <= 0.0 && how.repetition_penalty == 1.0;
        let rc = unsafe {
            if greedy {
                ak_session_generate_greedy(self.s, prompt_tokens.as_ptr(), prompt_tokens.len() as u32, max_new_tokens as u32, 1,
                                           out.as_mut_ptr(), &mut n_out)
            } else {
                ak_session_generate(self.s, prompt_tokens.as_ptr(), prompt_tokens.len() as u32, max_new_tokens as u32,
                                    how.temperature, how.top_k as u32, how.top_p, how.repetition_penalty, how.seed, 1,
                                    out.as_mut_ptr(), &mut n_out)
            }
        };
        self.result(rc, prompt_tokens.len() as u32)?;
        out.truncate(n_out as usize);
        Ok(out)
    }

    /// Cached K (post-RoPE) and V rows `0..cur_len` of one layer as `[cur_len, dim]` f32, the layout of the
    /// reference's `Cache` (src/nn/inference_graphs.rs:511-543).
    pub fn read_cache(&mut self, layer: usize) -> (Vec<Real>, Vec<Real>) {
        let n = self.cur_len() as usize * self.weights.cfg.dim as usize;
        let (mut k, mut v) = (vec![0.0; n], vec![0.0; n]);
        unsafe { check_fatal(ak_session_read_cache(self.s, layer as u32, k.as_mut_ptr(), v.as_mut_ptr())) };
        (k, v)
    }
}

impl Drop for B200Session<'_> {
    fn drop(&mut self) {
        unsafe { ak_session_destroy(self.s) };
    }
}
