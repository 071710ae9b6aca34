//! Phase-gated emitters for the B200 backend: the counterpart of akasha-core's
//! src/nn/ops/mod.rs:20-72 (phase markers and `GraphBuilder`) and of the forward / cached emitters of
//! src/nn/ops/emit.rs, with the same names, the same meta types and the same trait bounds, so that
//! `build_prefill_layer` / `build_decode_layer` (src/nn/inference_graphs.rs:198-509) compile against
//! them unchanged.
//!
//! The reference's emitters append a node `(shader, bindings, grid)` to wilupgu's `ComputeGraph`;
//! the kernels read their meta buffers at execution time, which is how the decode graph is built
//! once and re-run with four updated metas per token (src/nn/ops/mod.rs:1-10,
//! src/nn/inference_graphs.rs:164-195). The B200 graph keeps that contract: an emitter records a
//! launch closure over device pointers and a `LiveMeta<M>` cell; `B200Graph::execute` replays the
//! closures in append order on the context's stream, each reading the CURRENT value of its meta.
//! Phase gates are compile-time only and cost nothing at run time.
use crate::ffi::*;
use crate::meta::*;
use crate::check_fatal;
use std::cell::Cell;
use std::marker::PhantomData;
use std::rc::Rc;

// ---- phase markers and bounds (src/nn/ops/mod.rs:20-40)
pub struct Train;
pub struct Prefill;
pub struct Decode;

pub trait Phase {}
pub trait FwdPhase: Phase {}
pub trait FullSeqPhase: FwdPhase {} // square causal attention / full-seq RoPE
pub trait CachedPhase: FwdPhase {} // reads/writes the KV cache

impl Phase for Train {}
impl FwdPhase for Train {}
impl FullSeqPhase for Train {}

impl Phase for Prefill {}
impl FwdPhase for Prefill {}
impl FullSeqPhase for Prefill {}
impl CachedPhase for Prefill {}

impl Phase for Decode {}
impl FwdPhase for Decode {}
impl CachedPhase for Decode {}

/// A device buffer of `len` f32 (or u32) elements owned by the graph's user
/// (`Arc<Tensor<B>>` in the reference; here a raw device pointer from `ak_device_malloc`).
#[derive(Clone, Copy)]
pub struct DevBuf {
    pub ptr: *mut std::os::raw::c_void,
    pub len: usize,
}
impl DevBuf {
    fn f32(&self) -> *mut f32 {
        self.ptr as *mut f32
    }
    fn u32(&self) -> *const u32 {
        self.ptr as *const u32
    }
}

/// A meta that may be updated between executions (`foo_with(shape, meta)` in the reference).
pub struct LiveMeta<M: Copy>(Rc<Cell<M>>);
impl<M: Copy> LiveMeta<M> {
    pub fn new(m: M) -> Self {
        Self(Rc::new(Cell::new(m)))
    }
    /// `meta.update(..)`: takes effect at the next `execute` (src/nn/inference_graphs.rs:164-195).
    pub fn set(&self, m: M) {
        self.0.set(m)
    }
    pub fn get(&self) -> M {
        self.0.get()
    }
    fn share(&self) -> Rc<Cell<M>> {
        self.0.clone()
    }
}

/// The recorded launches of one graph (`ComputeGraph<B>`), executed in append order on one stream.
pub struct B200Graph {
    stream: Stream,
    nodes: Vec<Box<dyn Fn(Stream) -> i32>>,
}
impl B200Graph {
    pub fn new(ctx: *mut AkCtx) -> Self {
        Self { stream: unsafe { ak_ctx_stream(ctx) }, nodes: Vec::new() }
    }
    pub fn execute(&self) {
        for n in &self.nodes {
            check_fatal(n(self.stream));
        }
    }
    pub fn synchronize(&self) {
        check_fatal(unsafe { ak_stream_synchronize(self.stream) });
    }
    pub fn len(&self) -> usize {
        self.nodes.len()
    }
    pub fn is_empty(&self) -> bool {
        self.nodes.is_empty()
    }
}

/// `GraphBuilder<'g, B, P>` (src/nn/ops/mod.rs:42-72) with the backend fixed to B200.
pub struct GraphBuilder<'g, P: Phase> {
    pub graph: &'g mut B200Graph,
    _phase: PhantomData<P>,
}
impl<'g> GraphBuilder<'g, Prefill> {
    pub fn prefill(graph: &'g mut B200Graph) -> Self {
        Self { graph, _phase: PhantomData }
    }
}
impl<'g> GraphBuilder<'g, Decode> {
    pub fn decode(graph: &'g mut B200Graph) -> Self {
        Self { graph, _phase: PhantomData }
    }
}

macro_rules! node {
    ($gb:expr, $body:expr) => {
        $gb.graph.nodes.push(Box::new($body))
    };
}

// ---- forward emitters (any FwdPhase): src/nn/ops/emit.rs

/// `C[m,n] = A[m,k] @ B[k,n]`; m == 1 routes to the GEMV inside the library (emit.rs:19-57).
pub fn matmul<P: FwdPhase>(gb: &mut GraphBuilder<'_, P>, a: DevBuf, b: DevBuf, c: DevBuf, shape: MatMulMeta) {
    matmul_with(gb, a, b, c, &LiveMeta::new(shape))
}
pub fn matmul_with<P: FwdPhase>(gb: &mut GraphBuilder<'_, P>, a: DevBuf, b: DevBuf, c: DevBuf, meta: &LiveMeta<MatMulMeta>) {
    let m = meta.share();
    node!(gb, move |s| unsafe { ak_matmul(s, a.f32(), b.f32(), c.f32(), m.get()) });
}

/// `C[m,n] += A[m,k] @ B[k,n]` (emit.rs:91-126).
pub fn matmul_add<P: FwdPhase>(gb: &mut GraphBuilder<'_, P>, a: DevBuf, b: DevBuf, c: DevBuf, shape: MatMulMeta) {
    matmul_add_with(gb, a, b, c, &LiveMeta::new(shape))
}
pub fn matmul_add_with<P: FwdPhase>(gb: &mut GraphBuilder<'_, P>, a: DevBuf, b: DevBuf, c: DevBuf, meta: &LiveMeta<MatMulMeta>) {
    let m = meta.share();
    node!(gb, move |s| unsafe { ak_matmul_add(s, a.f32(), b.f32(), c.f32(), m.get()) });
}

/// emit.rs:151-180.
pub fn rmsnorm<P: FwdPhase>(gb: &mut GraphBuilder<'_, P>, input: DevBuf, weight: DevBuf, output: DevBuf, shape: NormMeta) {
    rmsnorm_with(gb, input, weight, output, &LiveMeta::new(shape))
}
pub fn rmsnorm_with<P: FwdPhase>(gb: &mut GraphBuilder<'_, P>, input: DevBuf, weight: DevBuf, output: DevBuf, meta: &LiveMeta<NormMeta>) {
    let m = meta.share();
    node!(gb, move |s| unsafe { ak_rmsnorm(s, input.f32(), weight.f32(), output.f32(), m.get()) });
}

/// emit.rs:228-257.
pub fn embedding<P: FwdPhase>(gb: &mut GraphBuilder<'_, P>, tokens: DevBuf, table: DevBuf, output: DevBuf, shape: EmbeddingMeta) {
    embedding_with(gb, tokens, table, output, &LiveMeta::new(shape))
}
pub fn embedding_with<P: FwdPhase>(gb: &mut GraphBuilder<'_, P>, tokens: DevBuf, table: DevBuf, output: DevBuf, meta: &LiveMeta<EmbeddingMeta>) {
    let m = meta.share();
    node!(gb, move |s| unsafe { ak_embedding(s, tokens.u32(), table.f32(), output.f32(), m.get()) });
}

/// emit.rs:406-424.
pub fn head_gather<P: FwdPhase>(gb: &mut GraphBuilder<'_, P>, src: DevBuf, dst: DevBuf, shape: HeadMoveMeta) {
    head_gather_with(gb, src, dst, &LiveMeta::new(shape))
}
pub fn head_gather_with<P: FwdPhase>(gb: &mut GraphBuilder<'_, P>, src: DevBuf, dst: DevBuf, meta: &LiveMeta<HeadMoveMeta>) {
    let m = meta.share();
    node!(gb, move |s| unsafe { ak_head_gather(s, src.f32(), dst.f32(), m.get()) });
}

/// emit.rs:686-696.
pub fn silu<P: FwdPhase>(gb: &mut GraphBuilder<'_, P>, buf: DevBuf, len: u32) {
    node!(gb, move |s| unsafe { ak_silu(s, buf.f32(), len) });
}

// ---- full-sequence emitters (Prefill / Train): square causal attention, full-seq RoPE

/// emit.rs:306-313.
pub fn rope<P: FullSeqPhase>(gb: &mut GraphBuilder<'_, P>, buf: DevBuf, shape: RopeMeta) {
    node!(gb, move |s| unsafe { ak_rope(s, buf.f32(), shape) });
}

/// emit.rs:556-597. `l_cache` may be a null `DevBuf` outside training.
pub fn flash_attention<P: FullSeqPhase>(gb: &mut GraphBuilder<'_, P>, q: DevBuf, k: DevBuf, v: DevBuf, out: DevBuf, l_cache: DevBuf,
                                        shape: FlashAttnMeta) {
    assert!(shape.head_dim <= 128, "flash attention supports head_dim <= 128 (emit.rs:564-567)");
    node!(gb, move |s| unsafe { ak_flash_attention(s, q.f32(), k.f32(), v.f32(), out.f32(), l_cache.f32(), shape) });
}

// ---- cached emitters (Prefill / Decode): read or write the KV cache

/// emit.rs:649-675.
pub fn cache_write<P: CachedPhase>(gb: &mut GraphBuilder<'_, P>, src: DevBuf, cache: DevBuf, shape: CacheWriteMeta) {
    cache_write_with(gb, src, cache, &LiveMeta::new(shape))
}
pub fn cache_write_with<P: CachedPhase>(gb: &mut GraphBuilder<'_, P>, src: DevBuf, cache: DevBuf, meta: &LiveMeta<CacheWriteMeta>) {
    let m = meta.share();
    node!(gb, move |s| unsafe { ak_cache_write(s, src.f32(), cache.f32(), m.get()) });
}

// ---- decode-only emitters

/// emit.rs:325-342.
pub fn rope_offset_with(gb: &mut GraphBuilder<'_, Decode>, buf: DevBuf, meta: &LiveMeta<RopeOffsetMeta>) {
    let m = meta.share();
    node!(gb, move |s| unsafe { ak_rope_offset(s, buf.f32(), m.get()) });
}
/// emit.rs:485-504.
pub fn attn_qk_cached_with(gb: &mut GraphBuilder<'_, Decode>, q: DevBuf, k_cache: DevBuf, scores: DevBuf, meta: &LiveMeta<AttnCachedMeta>) {
    let m = meta.share();
    node!(gb, move |s| unsafe { ak_attn_qk_cached(s, q.f32(), k_cache.f32(), scores.f32(), m.get()) });
}
/// emit.rs:528-542.
pub fn softmax_rect_with(gb: &mut GraphBuilder<'_, Decode>, buf: DevBuf, meta: &LiveMeta<SoftmaxRectMeta>) {
    let m = meta.share();
    node!(gb, move |s| unsafe { ak_softmax_rect(s, buf.f32(), m.get()) });
}
/// emit.rs:507-525.
pub fn attn_av_cached_with(gb: &mut GraphBuilder<'_, Decode>, scores: DevBuf, v_cache: DevBuf, out: DevBuf, meta: &LiveMeta<AttnCachedMeta>) {
    let m = meta.share();
    node!(gb, move |s| unsafe { ak_attn_av_cached(s, scores.f32(), v_cache.f32(), out.f32(), m.get()) });
}

#[cfg(test)]
mod phase_gate {
    //! The gates are type-level: `rope` on a Decode builder or `attn_qk_cached_with` on a Prefill builder do
    //! not compile. What can be checked at run time is that recorded nodes read live metas.
    use super::*;

    #[test]
    fn live_meta_is_read_at_execute_time() {
        let m = LiveMeta::new(RopeOffsetMeta { seq_len: 1, dim: 768, head_dim: 64, pos: 0 });
        let shared = m.share();
        m.set(RopeOffsetMeta { seq_len: 1, dim: 768, head_dim: 64, pos: 17 });
        assert_eq!(shared.get().pos, 17);
    }
}
