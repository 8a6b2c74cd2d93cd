//! The einsum layer on the device: `Subscripts`, `ContractionTree` and the accumulating executor
//! (`tenferro-einsum/src/lib.rs:239-356, 584-621`).  Parsing, tree optimisation and the tree walk
//! run inside the library; intermediates stay in the context's pool.
use std::ffi::CString;

use tenferro_b200_sys as sys;
use tenferro_device::{Error, Result};

use crate::backend::CudaScalar;
use crate::buffer::CudaBuffer;
use crate::device::Context;
use crate::error::check;

/// `Subscripts` (`tenferro-einsum/src/lib.rs:239-284`).
pub struct Subscripts {
    raw: *mut sys::tfb_subscripts,
}

impl Subscripts {
    /// `Subscripts::new(inputs, output)` with integer labels.
    pub fn new(inputs: &[&[u32]], output: &[u32]) -> Result<Self> {
        let ranks: Vec<usize> = inputs.iter().map(|i| i.len()).collect();
        let ptrs: Vec<*const u32> = inputs.iter().map(|i| i.as_ptr()).collect();
        let mut raw = core::ptr::null_mut();
        // SAFETY: the label arrays outlive the call; the library copies them.
        check(unsafe {
            sys::tfb_subscripts_new(inputs.len(), ranks.as_ptr(), ptrs.as_ptr(), output.len(), output.as_ptr(), &mut raw)
        })?;
        Ok(Self { raw })
    }

    /// `Subscripts::parse("ij,jk->ik")`; parentheses fix the pairwise order.
    pub fn parse(notation: &str) -> Result<Self> {
        let c = CString::new(notation).map_err(|_| Error::InvalidArgument("notation contains NUL".into()))?;
        let mut raw = core::ptr::null_mut();
        // SAFETY: NUL-terminated string, valid out-pointer.
        check(unsafe { sys::tfb_subscripts_parse(c.as_ptr(), &mut raw) })?;
        Ok(Self { raw })
    }
}

impl Drop for Subscripts {
    fn drop(&mut self) {
        // SAFETY: destroyed once.
        unsafe { sys::tfb_subscripts_destroy(self.raw) };
    }
}

/// `ContractionTree` (`tenferro-einsum/src/lib.rs:297-356`).
pub struct ContractionTree {
    raw: *mut sys::tfb_tree,
}

impl ContractionTree {
    /// `ContractionTree::optimize(subscripts, shapes)`.
    pub fn optimize(subscripts: &Subscripts, shapes: &[&[usize]]) -> Result<Self> {
        let ranks: Vec<usize> = shapes.iter().map(|s| s.len()).collect();
        let dims: Vec<*const usize> = shapes.iter().map(|s| s.as_ptr()).collect();
        let mut raw = core::ptr::null_mut();
        // SAFETY: the shape arrays outlive the call.
        check(unsafe { sys::tfb_tree_optimize(subscripts.raw, ranks.as_ptr(), dims.as_ptr(), &mut raw) })?;
        Ok(Self { raw })
    }

    /// `ContractionTree::from_pairs`: intermediates are numbered from `n_inputs` upward.
    pub fn from_pairs(subscripts: &Subscripts, shapes: &[&[usize]], pairs: &[(usize, usize)]) -> Result<Self> {
        let ranks: Vec<usize> = shapes.iter().map(|s| s.len()).collect();
        let dims: Vec<*const usize> = shapes.iter().map(|s| s.as_ptr()).collect();
        let flat: Vec<usize> = pairs.iter().flat_map(|&(a, b)| [a, b]).collect();
        let mut raw = core::ptr::null_mut();
        // SAFETY: as above.
        check(unsafe {
            sys::tfb_tree_from_pairs(subscripts.raw, ranks.as_ptr(), dims.as_ptr(), pairs.len(), flat.as_ptr(), &mut raw)
        })?;
        Ok(Self { raw })
    }

    pub fn output_dims(&self) -> Vec<usize> {
        // SAFETY: a NULL buffer asks for the count only.
        let n = unsafe { sys::tfb_tree_output_dims(self.raw, core::ptr::null_mut(), 0) };
        let mut dims = vec![0usize; n];
        unsafe { sys::tfb_tree_output_dims(self.raw, dims.as_mut_ptr(), n) };
        dims
    }

    /// Multiply-adds of the whole tree.
    pub fn macs(&self) -> f64 {
        // SAFETY: live handle.
        unsafe { sys::tfb_tree_macs(self.raw) }
    }
}

impl Drop for ContractionTree {
    fn drop(&mut self) {
        // SAFETY: destroyed once.
        unsafe { sys::tfb_tree_destroy(self.raw) };
    }
}

/// A strided operand in device memory: buffer plus `Tensor<T>`'s dims / strides / offset
/// (`tenferro-tensor/src/lib.rs:167-181`), with the lazy-conjugate flag of `into_conj`.
pub struct DeviceOperand<'a, T: CudaScalar> {
    pub buffer: &'a CudaBuffer<T>,
    pub dims: &'a [usize],
    pub strides: &'a [isize],
    pub offset: isize,
    pub conj: bool,
}

impl<'a, T: CudaScalar> DeviceOperand<'a, T> {
    fn raw(&self) -> sys::tfb_view {
        sys::tfb_view {
            base: self.buffer.as_device_ptr().cast(),
            rank: self.dims.len(),
            dims: self.dims.as_ptr(),
            strides: self.strides.as_ptr(),
            offset: self.offset,
            flags: if self.conj { sys::TFB_VIEW_CONJ } else { 0 },
        }
    }
}

/// `einsum_with_plan_into` (`tenferro-einsum/src/lib.rs:584-621`):
/// `output = alpha * einsum(operands) + beta * output`.  Enqueues and returns; the other eight
/// entry points reduce to this call on a fresh column-major output.
pub fn einsum_with_plan_into<T: CudaScalar>(
    ctx: &Context,
    tree: &ContractionTree,
    operands: &[DeviceOperand<'_, T>],
    alpha: T,
    beta: T,
    output: &DeviceOperand<'_, T>,
) -> Result<()> {
    let views: Vec<sys::tfb_view> = operands.iter().map(|o| o.raw()).collect();
    let out = output.raw();
    // SAFETY: every view points at slices borrowed for the call; alpha/beta are one scalar each.
    check(unsafe {
        sys::tfb_einsum_with_plan_into(ctx.raw, tree.raw, T::DTYPE, views.len(), views.as_ptr(), (&alpha as *const T).cast(),
                                       (&beta as *const T).cast(), &out)
    })
}
