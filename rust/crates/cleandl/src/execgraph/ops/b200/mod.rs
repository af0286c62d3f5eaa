//! Kernel providers for B200 (sm_100a) behind the existing operators: `libcleandl_b200.so` called
//! through its C ABI.  SOURCE ONLY (no Rust toolchain where this was written; not compiled).
//!
//! Graph tracing, validation (`Operator::infer_outputs`), planning, liveness and allocation stay
//! where they are; only what `Operator::build` returns changes.  Each operator's `build` asks
//! [`available`] and, when the device is an sm_100 part and the problem is in the library's
//! domain, returns one of the executors of this module instead of its cuBLASLt / specialized /
//! flash-attention-rs executor.  The executors keep `Executor::execute`'s contract
//! (crates/cleandl/src/execgraph/op.rs:130-142): no allocation, no synchronisation, work on the
//! given stream, an error instead of a panic, empty shapes succeed.
pub mod attention;
pub mod ffi;
pub mod gemm;
pub mod norm;

use crate::{
    execgraph::op::{TensorRef, TensorRefMut},
    tensor::{TensorView, TensorViewMut},
};
use anyhow::{bail, ensure};
use skycuda::stream::Stream;
use skytens_core::data_type::ElementType;
use std::ffi::{c_void, CStr};

/// True when the current device can run the library (compute capability 10.x): the same exact
/// architecture gate as kernel-build-util (crates/kernel-build-util/src/lib.rs:96-107).
pub fn available(device_ordinal: i32) -> bool {
    unsafe { ffi::cdl_b200_device_ok(device_ordinal) == 0 }
}

/// Turns a status of the C ABI into `anyhow::Result`, with the library's thread-local message.
pub(crate) fn check(status: i32) -> anyhow::Result<()> {
    if status == 0 {
        return Ok(());
    }
    let msg = unsafe { CStr::from_ptr(ffi::cdl_b200_last_error()) }
        .to_string_lossy()
        .into_owned();
    bail!("cleandl_b200 ({status}): {msg}")
}

fn dtype_of(ty: ElementType) -> anyhow::Result<i32> {
    Ok(match ty {
        ElementType::Bf16 => ffi::CDL_BF16,
        ElementType::F32 => ffi::CDL_F32,
        ElementType::I32 => ffi::CDL_I32,
        other => bail!("cleandl_b200: element type {other:?} is not supported"),
    })
}

fn descriptor(
    ptr: *mut c_void,
    ty: ElementType,
    shape: &[usize],
    strides: &[usize],
) -> anyhow::Result<ffi::CdlTensor> {
    ensure!(shape.len() <= 4, "cleandl_b200: rank {} exceeds 4", shape.len());
    let mut t = ffi::CdlTensor {
        ptr,
        dtype: dtype_of(ty)?,
        rank: shape.len() as i32,
        shape: [0; 4],
        stride: [0; 4],
    };
    for (i, (&n, &s)) in shape.iter().zip(strides).enumerate() {
        t.shape[i] = n as i64;
        t.stride[i] = s as i64; // element strides, like TensorView's layout (tensor.rs:401-407)
    }
    Ok(t)
}

/// `cdl_tensor` of a read-only operand.  `access_on` records the read on `stream` for the
/// engine's hazard tracking, exactly as the existing executors do before taking a raw pointer
/// (ops/matmul.rs:1166).
pub(crate) fn tensor_ro(t: &TensorView<'_>, stream: &Stream) -> anyhow::Result<ffi::CdlTensor> {
    let ptr = unsafe { t.storage().access_on(stream)?.ptr() } as *mut c_void;
    descriptor(ptr, t.element_type(), t.shape().as_slice(), t.strides().as_slice())
}

/// `cdl_tensor` of an output or read-write operand.
pub(crate) fn tensor_rw(t: &mut TensorViewMut<'_>, stream: &Stream) -> anyhow::Result<ffi::CdlTensor> {
    let (ty, shape, strides) = (t.element_type(), t.shape(), t.strides());
    let ptr = unsafe { t.storage_mut().access_mut_on(stream)?.ptr() } as *mut c_void;
    descriptor(ptr, ty, shape.as_slice(), strides.as_slice())
}

pub(crate) fn plain<'a, 'b>(t: &'b TensorRef<'a>) -> &'b TensorView<'a> {
    t.plain()
}

pub(crate) fn plain_mut<'a, 'b>(t: &'b mut TensorRefMut<'a>) -> anyhow::Result<&'b mut TensorViewMut<'a>> {
    match t {
        TensorRefMut::Plain(v) => Ok(v),
        TensorRefMut::Mx(_) => bail!("cleandl_b200: expected a plain tensor, got a block-scaled one"),
    }
}

/// The raw CUstream handle the C ABI takes as `cdl_stream`.
pub(crate) fn raw_stream(stream: &Stream) -> *mut c_void {
    stream.raw() as *mut c_void
}
