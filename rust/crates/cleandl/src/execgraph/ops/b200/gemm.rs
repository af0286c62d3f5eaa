//! `Executor` of the `Matmul` operator on libcleandl_b200 (SOURCE ONLY, not compiled here).
//!
//! Takes the place of `MatmulExecutor` (crates/cleandl/src/execgraph/ops/matmul.rs:1092-1183),
//! which binds the same operands to a cuBLASLt plan.  The operator's own analysis (transposed
//! views as layouts, `swapped`, C / beta handling, matmul.rs:128-157, 540-660) is unchanged; this
//! executor only needs the bound views: the library reads major-ness from the strides.
use super::{check, ffi, plain, plain_mut, raw_stream, tensor_ro, tensor_rw};
use crate::{
    context::Context,
    execgraph::{
        op::{BuildCx, Executor, OpIo},
        sym::DimValues,
    },
};
use skycuda::stream::Stream;
use std::ptr;

/// One tuner candidate: the library's kernel choice for this node.
pub type Candidate = ffi::CdlMatmulOptions;

pub struct B200MatmulExecutor {
    pub alpha: f32,
    pub beta: f32,
    pub has_c: bool,
    pub options: Candidate,
}

impl B200MatmulExecutor {
    /// What `Matmul::build` calls on an sm_100 device: enumerate the library's candidates for the
    /// hint shapes (heuristic default first, as op.rs:301-318 asks) and let the engine's tuner
    /// time them on hint-shaped buffers, like the cuBLASLt executor does with its algorithm list
    /// (matmul.rs:667-729).
    pub fn build(bcx: &BuildCx<'_>, alpha: f32, beta: f32, has_c: bool) -> anyhow::Result<Self> {
        let candidates = bcx.hint_io(0, |io| {
            let stream = bcx.cx.default_compute_stream();
            let a = tensor_ro(plain(&io.input(0)), stream)?;
            let b = tensor_ro(plain(&io.input(1)), stream)?;
            let d = tensor_rw(plain_mut(io.output(0))?, stream)?;
            let mut list = [Candidate { variant: 0, deterministic: 0 }; 8];
            let mut n = 0i32;
            check(unsafe { ffi::cdl_b200_matmul_candidates(&a, &b, &d, list.as_mut_ptr(), 8, &mut n) })?;
            Ok(list[..n as usize].to_vec())
        })?;
        let key = bcx.tune_key(&("b200_matmul", alpha.to_bits(), beta.to_bits(), has_c))?;
        let (_, executor) = bcx.tune_executor(&key, candidates, |c| {
            Ok(B200MatmulExecutor { alpha, beta, has_c, options: *c })
        })?;
        Ok(executor)
    }
}

impl Executor for B200MatmulExecutor {
    fn scratch_bytes(&self, _dims: &DimValues) -> usize {
        0 // cdl_b200_matmul_scratch_bytes is 0 for every problem: the kernels need none
    }

    fn execute(&self, io: &mut OpIo<'_>, stream: &Stream, _cx: &Context) -> anyhow::Result<()> {
        let a = tensor_ro(plain(&io.input(0)), stream)?;
        let b = tensor_ro(plain(&io.input(1)), stream)?;
        let c = if self.has_c { Some(tensor_ro(plain(&io.input(2)), stream)?) } else { None };
        let d = tensor_rw(plain_mut(io.output(0))?, stream)?;
        check(unsafe {
            ffi::cdl_b200_matmul_opt(
                &a,
                &b,
                c.as_ref().map_or(ptr::null(), |t| t as *const _),
                &d,
                self.alpha,
                self.beta,
                &self.options,
                ptr::null_mut(),
                0,
                raw_stream(stream),
            )
        })
    }
}
