//! B200 (sm_100a) backend for akasha-core's Prefill/Decode inference path.
//!
//! Three layers over the C ABI of `libakasha_b200.so` (`include/akasha_b200.h`):
//!
//! * [`ffi`]     -- the `extern "C"` block, one declaration per exported symbol;
//! * [`session`] -- `B200Session`, the drop-in for `InferenceSession<B>` (src/nn/inference.rs:13-327):
//!                  same method names, same `AkashaError` mapping, same cache attach/take rules;
//!                  [`engine`] adds continuous batching (no reference counterpart);
//! * [`emit`]    -- the phase-gated emitters (`GraphBuilder<'g, P>` with `Train`/`Prefill`/`Decode`
//!                  marker types and the `FwdPhase`/`FullSeqPhase`/`CachedPhase` bounds of
//!                  src/nn/ops/mod.rs:20-72): one function per forward/cached emitter of
//!                  src/nn/ops/emit.rs with the same name and meta type, recording a launch of
//!                  the matching `ak_*` entry point.
//!
//! Inside akasha-core this crate's modules would live under `src/b200/` behind a `b200` cargo
//! feature and use the crate's own `ModelConfig`, `AkashaError` and meta types; they are
//! restated here (field for field) so that the shim stands alone.
pub mod emit;
pub mod engine;
pub mod ffi;
pub mod meta;
pub mod session;

pub type Real = f32;

/// `ModelConfig` (src/config.rs:2-30).
#[derive(Clone, Copy, Debug, PartialEq)]
pub struct ModelConfig {
    pub vocab_size: u32,
    pub dim: u32,
    pub num_heads: u32,
    pub num_layers: usize,
    pub seq_len: u32,
    pub ffn_hidden: u32,
    pub norm_eps: f32,
    pub batch_size: u32,
    pub eos_token: u32,
}

impl ModelConfig {
    pub fn new(vocab_size: u32, dim: u32, num_heads: u32, num_layers: usize, seq_len: u32) -> Self {
        assert!(num_layers >= 1, "At least one layer is required!");
        assert_eq!(dim % num_heads, 0, "dim must be divisible by num_heads");
        Self {
            vocab_size,
            dim,
            num_heads,
            num_layers,
            seq_len,
            ffn_hidden: dim * 4,
            norm_eps: 1e-5,
            batch_size: 1,
            eos_token: vocab_size - 1,
        }
    }
    pub fn head_dim(&self) -> u32 {
        self.dim / self.num_heads
    }
    pub fn akasha_hall_1() -> Self {
        Self::new(50257, 768, 12, 12, 512)
    }
    pub(crate) fn to_ffi(self) -> ffi::AkModelConfig {
        ffi::AkModelConfig {
            vocab_size: self.vocab_size,
            dim: self.dim,
            num_heads: self.num_heads,
            num_layers: self.num_layers as u32,
            seq_len: self.seq_len,
            ffn_hidden: self.ffn_hidden,
            norm_eps: self.norm_eps,
            eos_token: self.eos_token,
        }
    }
}

/// `AkashaError` (src/lib.rs:10-17); return codes 1..5 of the C ABI map onto it one to one.
#[derive(Debug, Clone, PartialEq, Eq)]
pub enum AkashaError {
    EmptyPrompt,
    PromptTooLong { len: u32, max: u32 },
    ContextFull { max: u32 },
    NoCache,
    CacheNotEmpty { cur_len: u32 },
}

impl std::fmt::Display for AkashaError {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result {
        match self {
            AkashaError::EmptyPrompt => write!(f, "prompt is empty"),
            AkashaError::PromptTooLong { len, max } => write!(f, "prompt is {len} tokens, context window is {max}"),
            AkashaError::ContextFull { max } => write!(f, "context window is full ({max} tokens)"),
            AkashaError::NoCache => write!(f, "no cache attached (call replace_cache or generate first)"),
            AkashaError::CacheNotEmpty { cur_len } => {
                write!(f, "prefill needs an empty cache, this one holds {cur_len} tokens (loop decode_step for a resumed cache)")
            }
        }
    }
}
impl std::error::Error for AkashaError {}

/// Last error text of the library (thread local on the C side).
pub fn last_error() -> String {
    unsafe { std::ffi::CStr::from_ptr(ffi::ak_last_error_string()) }.to_string_lossy().into_owned()
}

/// Codes >= 100 are programming or device errors: the reference panics on those (shape asserts,
/// src/nn/ops/emit.rs:564-572), so does the shim.
pub(crate) fn check_fatal(rc: i32) {
    if rc != 0 {
        panic!("akasha-b200: error {rc}: {}", last_error());
    }
}
