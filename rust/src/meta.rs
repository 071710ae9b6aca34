//! The typed kernel metas of the inference path, field for field the `#[repr(C)]` structs of
//! akasha-core's src/nn/ops/meta.rs:18-165 (inside akasha-core the shim uses the crate's own types;
//! they are passed to the C ABI BY VALUE).

macro_rules! meta {
    ($(#[$doc:meta])* $name:ident { $($field:ident : $ty:ty),* $(,)? }) => {
        $(#[$doc])*
        #[repr(C)]
        #[derive(Clone, Copy, Debug, PartialEq)]
        pub struct $name { $(pub $field: $ty),* }
    };
}

meta!(/// MatMul family: C is `[m, n]`, contraction length `k`.
      MatMulMeta { m: u32, n: u32, k: u32 });
meta!(/// RMSNorm: `seq_len` rows of `size`.
      NormMeta { seq_len: u32, size: u32, eps: f32 });
meta!(/// HeadGather: `head_dim`-wide slice at `head_offset` of a `full_dim`-wide buffer.
      HeadMoveMeta { seq_len: u32, full_dim: u32, head_dim: u32, head_offset: u32 });
meta!(AttnCachedMeta { attn_len: u32, dim: u32, head_dim: u32 });
meta!(SoftmaxRectMeta { num_rows: u32, width: u32, scale: f32 });
meta!(RopeMeta { seq_len: u32, dim: u32, head_dim: u32, row_offset: u32 });
meta!(RopeOffsetMeta { seq_len: u32, dim: u32, head_dim: u32, pos: u32 });
meta!(CacheWriteMeta { row_count: u32, width: u32, dst_row_offset: u32 });
meta!(EmbeddingMeta { vocab_size: u32, dim: u32, seq_len: u32 });
meta!(FlashAttnMeta { seq_len: u32, dim: u32, head_dim: u32, scale: f32, row_offset: u32 });

impl HeadMoveMeta {
    /// One dim-wide Q/K/V role slice of a fused `[seq_len, 3*dim]` QKV buffer (meta.rs:48-57).
    pub fn qkv_slice(seq_len: u32, dim: u32, role_offset: u32) -> Self {
        Self { seq_len, full_dim: 3 * dim, head_dim: dim, head_offset: role_offset }
    }
}
