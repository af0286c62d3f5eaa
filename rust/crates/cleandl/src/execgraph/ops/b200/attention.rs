//! `Executor`s of `AttentionFwd` / `AttentionBwd` on libcleandl_b200 (SOURCE ONLY, not compiled
//! here).  They take the place of `AttentionExecutor` (crates/cleandl/src/execgraph/ops/attention/
//! exec.rs:358-416), which forwards to flash-attention-rs.  The library implements the dense and
//! the packed layouts, masks None and Causal, bf16, head_dim 128 (GQA included); `AttentionOpts`
//! with paged KV, seqused, softcap, sliding windows, fp8 or other head dimensions keep the
//! existing executor (`supported` below is what `build` asks).
use super::{check, ffi, plain, plain_mut, raw_stream, tensor_ro, tensor_rw};
use crate::{
    context::Context,
    execgraph::{
        op::{Executor, OpIo},
        sym::DimValues,
    },
};
use skycuda::stream::Stream;
use std::{ffi::c_void, ptr};

pub fn supported(head_dim: usize, bf16: bool, paged: bool, seqused: bool, softcap: bool, window: bool) -> bool {
    head_dim == 128 && bf16 && !paged && !seqused && !softcap && !window
}

pub struct B200AttentionFwd {
    pub desc: ffi::CdlAttnDesc,
    pub packed: bool,      // QueryLayout::Packed / KvLayout::Packed (attention/mod.rs:55-79)
    pub max_seqlen_q: i64, // <= 0: the packed total (`None` in the reference)
    pub max_seqlen_k: i64,
    pub save_lse: bool,
}

impl Executor for B200AttentionFwd {
    fn execute(&self, io: &mut OpIo<'_>, stream: &Stream, _cx: &Context) -> anyhow::Result<()> {
        // operands: q, k, v, [cu_seqlens_q, cu_seqlens_k]; outputs: out, [lse]
        let q = tensor_ro(plain(&io.input(0)), stream)?;
        let k = tensor_ro(plain(&io.input(1)), stream)?;
        let v = tensor_ro(plain(&io.input(2)), stream)?;
        let cu = if self.packed {
            Some((tensor_ro(plain(&io.input(3)), stream)?, tensor_ro(plain(&io.input(4)), stream)?))
        } else {
            None
        };
        let o = tensor_rw(plain_mut(io.output(0))?, stream)?;
        let lse = if self.save_lse { Some(tensor_rw(plain_mut(io.output(1))?, stream)?) } else { None };
        let lse_ptr = lse.as_ref().map_or(ptr::null(), |t| t as *const _);
        check(unsafe {
            match &cu {
                Some((cu_q, cu_k)) => ffi::cdl_b200_attn_fwd_packed(
                    &self.desc, &q, &k, &v, cu_q, cu_k, self.max_seqlen_q, self.max_seqlen_k, &o, lse_ptr,
                    raw_stream(stream)),
                None => ffi::cdl_b200_attn_fwd(&self.desc, &q, &k, &v, &o, lse_ptr, raw_stream(stream)),
            }
        })
    }
}

pub struct B200AttentionBwd {
    pub desc: ffi::CdlAttnDesc,
    pub packed: bool,
    pub batch: i64, // packed: number of sequences
    pub heads: i64,
    pub max_seqlen_q: i64,
    pub max_seqlen_k: i64,
    /// Dense layout: scratch for the hint / bound shapes, computed once in `build` with
    /// cdl_b200_attn_bwd_scratch_bytes (two f32 rows per (batch, head, padded query)).
    pub dense_scratch_bytes: usize,
}

impl Executor for B200AttentionBwd {
    fn scratch_bytes(&self, _dims: &DimValues) -> usize {
        if !self.packed {
            return self.dense_scratch_bytes;
        }
        let mut n = 0usize;
        unsafe { ffi::cdl_b200_attn_bwd_packed_scratch_bytes(self.batch, self.max_seqlen_q, self.heads, &mut n) };
        n
    }

    fn execute(&self, io: &mut OpIo<'_>, stream: &Stream, _cx: &Context) -> anyhow::Result<()> {
        // operand order of the reference backward: q, k, v, out, d_out, lse (attention/mod.rs:899-905);
        // outputs dq, dk, dv in the input type (:915-919)
        let t: Vec<_> = (0..6).map(|i| tensor_ro(plain(&io.input(i)), stream)).collect::<Result<_, _>>()?;
        let cu = if self.packed {
            Some((tensor_ro(plain(&io.input(6)), stream)?, tensor_ro(plain(&io.input(7)), stream)?))
        } else {
            None
        };
        let (_, outputs, scratch) = io.split();
        let dq = tensor_rw(plain_mut(&mut outputs[0])?, stream)?;
        let dk = tensor_rw(plain_mut(&mut outputs[1])?, stream)?;
        let dv = tensor_rw(plain_mut(&mut outputs[2])?, stream)?;
        let scratch = scratch.ok_or_else(|| anyhow::anyhow!("attention_bwd needs scratch memory, none was given"))?;
        let (sptr, slen) = (unsafe { scratch.access_mut_on(stream)?.ptr() } as *mut c_void, scratch.len());
        check(unsafe {
            match &cu {
                Some((cu_q, cu_k)) => ffi::cdl_b200_attn_bwd_packed(
                    &self.desc, &t[0], &t[1], &t[2], &t[3], &t[4], &t[5], cu_q, cu_k, self.max_seqlen_q,
                    self.max_seqlen_k, &dq, &dk, &dv, sptr, slen, raw_stream(stream)),
                None => ffi::cdl_b200_attn_bwd(&self.desc, &t[0], &t[1], &t[2], &t[3], &t[4], &t[5], &dq, &dk,
                                               &dv, sptr, slen, raw_stream(stream)),
            }
        })
    }
}
