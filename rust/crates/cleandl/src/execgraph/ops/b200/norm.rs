//! `Executor`s of `NormFwd` (RMSNorm / LayerNorm, plain outputs) and of the RMSNorm backward on
//! libcleandl_b200 (SOURCE ONLY, not compiled here).  The forward takes the place of
//! `SpecializedExecutor` (crates/cleandl/src/execgraph/ops/norm/specialized.rs:116-200); operand
//! order as there: x, then scale, then bias when present; outputs y, then r_inv with save_stats.
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

pub struct B200RmsNormFwd {
    pub has_scale: bool,
    pub has_bias: bool,
    pub save_stats: bool,
    pub eps: f32,
    pub options: ffi::CdlNormOptions,
}

impl Executor for B200RmsNormFwd {
    fn execute(&self, io: &mut OpIo<'_>, stream: &Stream, _cx: &Context) -> anyhow::Result<()> {
        let x = tensor_ro(plain(&io.input(0)), stream)?;
        let scale = if self.has_scale { Some(tensor_ro(plain(&io.input(1)), stream)?) } else { None };
        let bias = if self.has_bias {
            Some(tensor_ro(plain(&io.input(1 + self.has_scale as usize)), stream)?)
        } else {
            None
        };
        let y = tensor_rw(plain_mut(io.output(0))?, stream)?;
        let r_inv = if self.save_stats { Some(tensor_rw(plain_mut(io.output(1))?, stream)?) } else { None };
        let opt = |t: &Option<ffi::CdlTensor>| t.as_ref().map_or(ptr::null(), |t| t as *const _);
        check(unsafe {
            ffi::cdl_b200_rmsnorm_fwd_opt(&x, opt(&scale), opt(&bias), self.eps, &y, opt(&r_inv),
                                          &self.options, raw_stream(stream))
        })
    }
}

/// RMSNorm backward: operands x, dy, [residual_dy], scale, r_inv; outputs dx and dscale
/// (`Access::ReadWrite`: accumulated).  Call sites in the reference:
/// crates/sky-1/src/training/model/decoder.rs:599-607, 684-692.
pub struct B200RmsNormBwd {
    pub cols: usize,
    pub has_residual: bool,
    pub options: ffi::CdlNormOptions,
}

impl Executor for B200RmsNormBwd {
    fn scratch_bytes(&self, dims: &DimValues) -> usize {
        let _ = dims;
        let mut n = 0usize;
        // 1024 partial rows of `cols` f32, whatever the row count
        unsafe { ffi::cdl_b200_rmsnorm_bwd_scratch_bytes(0, self.cols as i64, &mut n) };
        n
    }

    fn execute(&self, io: &mut OpIo<'_>, stream: &Stream, _cx: &Context) -> anyhow::Result<()> {
        let r = self.has_residual as usize;
        let x = tensor_ro(plain(&io.input(0)), stream)?;
        let dy = tensor_ro(plain(&io.input(1)), stream)?;
        let res = if self.has_residual { Some(tensor_ro(plain(&io.input(2)), stream)?) } else { None };
        let scale = tensor_ro(plain(&io.input(2 + r)), stream)?;
        let r_inv = tensor_ro(plain(&io.input(3 + r)), stream)?;
        let dscale = tensor_rw(io.input_mut(4 + r).plain_mut(), stream)?;
        let (_, outputs, scratch) = io.split();
        let dx = tensor_rw(plain_mut(&mut outputs[0])?, stream)?;
        let scratch = scratch.ok_or_else(|| anyhow::anyhow!("norm_bwd needs scratch memory, none was given"))?;
        let (sptr, slen) = (unsafe { scratch.access_mut_on(stream)?.ptr() } as *mut c_void, scratch.len());
        check(unsafe {
            ffi::cdl_b200_rmsnorm_bwd_opt(&x, &dy, res.as_ref().map_or(ptr::null(), |t| t as *const _),
                                          &scale, &r_inv, &dx, &dscale, &self.options, sptr, slen,
                                          raw_stream(stream))
        })
    }
}
