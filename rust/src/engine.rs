//! Continuous batching over the paged KV cache (`ak_engine_*`). The reference serves one session at a
//! time; every sequence an engine runs produces the tokens its own `InferenceSession::generate`
//! (greedy) would, whatever else shares the batch.
use crate::ffi::*;
use crate::session::B200Weights;
use crate::{check_fatal, last_error, AkashaError};
use std::os::raw::c_int;
use std::ptr;

pub struct B200Engine<'w> {
    _weights: &'w B200Weights,
    e: *mut AkEngine,
    max_seq_len: u32,
}

impl<'w> B200Engine<'w> {
    pub fn new(weights: &'w B200Weights, max_seqs: u32, max_seq_len: u32, async_steps: bool) -> Self {
        let cfg = AkEngineConfig { max_seqs, max_seq_len, block_size: 16, use_cuda_graph: 1, async_steps: async_steps as u32, ..Default::default() };
        let mut e = ptr::null_mut();
        unsafe { check_fatal(ak_engine_create(weights.ctx, weights.w, &cfg, &mut e)) };
        Self { _weights: weights, e, max_seq_len }
    }

    /// Queue a sequence; it generates until its total length reaches `max_total_len`.
    pub fn submit(&mut self, prompt: &[u32], max_total_len: u32) -> Result<u64, AkashaError> {
        let mut id = 0u64;
        let rc = unsafe { ak_engine_submit(self.e, prompt.as_ptr(), prompt.len() as u32, max_total_len, &mut id) };
        match rc {
            AK_OK => Ok(id),
            AK_EMPTY_PROMPT => Err(AkashaError::EmptyPrompt),
            AK_PROMPT_TOO_LONG => Err(AkashaError::PromptTooLong { len: prompt.len() as u32, max: self.max_seq_len }),
            AK_CONTEXT_FULL => Err(AkashaError::ContextFull { max: max_total_len.min(self.max_seq_len) }),
            other => panic!("akasha-b200: error {other}: {}", last_error()),
        }
    }

    /// One scheduler step: (running, waiting) afterwards.
    pub fn step(&mut self) -> (u32, u32) {
        let (mut r, mut w) = (0u32, 0u32);
        unsafe { check_fatal(ak_engine_step(self.e, &mut r, &mut w)) };
        (r, w)
    }

    /// Step until nothing runs or waits; returns the number of steps.
    pub fn run_to_completion(&mut self) -> u64 {
        let mut n = 0u64;
        unsafe { check_fatal(ak_engine_run(self.e, 0, &mut n)) };
        n
    }

    /// Tokens generated so far and whether the sequence has finished.
    pub fn poll(&mut self, seq_id: u64) -> (Vec<u32>, bool) {
        let mut out = vec![0u32; self.max_seq_len as usize];
        let (mut n, mut fin) = (0u32, 0 as c_int);
        unsafe { check_fatal(ak_engine_poll(self.e, seq_id, out.as_mut_ptr(), out.len() as u32, &mut n, &mut fin)) };
        out.truncate(n as usize);
        (out, fin != 0)
    }

    pub fn clear_finished(&mut self) {
        unsafe { check_fatal(ak_engine_clear_finished(self.e)) };
    }

    pub fn stats(&mut self) -> AkEngineStats {
        let mut s = AkEngineStats::default();
        unsafe { check_fatal(ak_engine_get_stats(self.e, &mut s)) };
        s
    }
}

impl Drop for B200Engine<'_> {
    fn drop(&mut self) {
        unsafe { ak_engine_destroy(self.e) };
    }
}
