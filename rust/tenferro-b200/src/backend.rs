//! `impl TensorPrims<Standard> for CudaBackend` (`tenferro-prims/src/lib.rs:278-340`), the CUDA
//! sibling of `CpuBackend` (`:417-439`).
//!
//! The views handed to `execute` must wrap DEVICE memory of the plan's context (a
//! `CudaBuffer<T>` viewed through `strided-view`'s raw constructors).  The trait's view types
//! carry no memory space, so that is the caller's contract, as it is for `tenferro-einsum`,
//! which selects the backend from the tensors' `LogicalMemorySpace` before it calls in
//! (`tenferro-einsum/src/lib.rs:16-20, 179-207`).
use std::marker::PhantomData;
use std::sync::Arc;

use num_complex::{Complex32, Complex64};
use strided_traits::ScalarBase;
use strided_view::{StridedView, StridedViewMut};
use tenferro_algebra::Standard;
use tenferro_b200_sys as sys;
use tenferro_device::{Error, Result};
use tenferro_prims::{Extension, PrimDescriptor, ReduceOp, TensorPrims};

use crate::device::Context;
use crate::error::check;

/// Scalar types of the `Standard` algebra (`tenferro-algebra/src/lib.rs:58-72`) and their dtype code.
pub trait CudaScalar: ScalarBase {
    const DTYPE: sys::tfb_dtype;
}
impl CudaScalar for f32 {
    const DTYPE: sys::tfb_dtype = sys::TFB_F32;
}
impl CudaScalar for f64 {
    const DTYPE: sys::tfb_dtype = sys::TFB_F64;
}
impl CudaScalar for Complex32 {
    const DTYPE: sys::tfb_dtype = sys::TFB_C32;
}
impl CudaScalar for Complex64 {
    const DTYPE: sys::tfb_dtype = sys::TFB_C64;
}

/// dtype of a `ScalarBase` type, or `None` outside the `Standard` algebra.
fn dtype_of<T: ScalarBase>() -> Option<sys::tfb_dtype> {
    use core::any::TypeId;
    let t = TypeId::of::<T>();
    if t == TypeId::of::<f32>() {
        Some(sys::TFB_F32)
    } else if t == TypeId::of::<f64>() {
        Some(sys::TFB_F64)
    } else if t == TypeId::of::<Complex32>() {
        Some(sys::TFB_C32)
    } else if t == TypeId::of::<Complex64>() {
        Some(sys::TFB_C64)
    } else {
        None
    }
}

/// `TensorPrims::Plan<T>` of the CUDA backend: an immutable handle, no type erasure on the Rust
/// side (the element type is part of the type).
pub struct CudaPlan<T: ScalarBase> {
    raw: *mut sys::tfb_plan,
    n_inputs: usize,
    _ctx: Arc<Context>,
    _scalar: PhantomData<T>,
}

// SAFETY: a plan is immutable after creation; `execute` takes `&Plan`.
unsafe impl<T: ScalarBase> Send for CudaPlan<T> {}
unsafe impl<T: ScalarBase> Sync for CudaPlan<T> {}

impl<T: ScalarBase> Drop for CudaPlan<T> {
    fn drop(&mut self) {
        // SAFETY: created by tfb_plan_create, destroyed once.
        unsafe { sys::tfb_plan_destroy(self.raw) };
    }
}

impl<T: ScalarBase> CudaPlan<T> {
    /// Compute over another semiring (`sys::TFB_ALGEBRA_MAX_PLUS`, `sys::TFB_ALGEBRA_MIN_PLUS`; f32
    /// and f64): what an external `impl TensorPrims<MaxPlus> for CudaBackend`
    /// (`tenferro-algebra/src/lib.rs:12-16, 74-106`) calls after `plan` - the descriptor, shapes and
    /// views are those of the Standard plan, only the arithmetic changes.
    pub fn set_algebra(self, algebra: sys::tfb_algebra) -> Result<Self> {
        // SAFETY: live plan handle, plain integer.
        check(unsafe { sys::tfb_plan_set_algebra(self.raw, algebra) })?;
        Ok(self)
    }
}

/// The CUDA backend.  Associated functions only, like `CpuBackend`; the device is the current
/// default (`CudaBackend::set_default_device`), device 0 unless changed.
pub struct CudaBackend;

static DEFAULT_DEVICE: std::sync::atomic::AtomicUsize = std::sync::atomic::AtomicUsize::new(0);

impl CudaBackend {
    pub fn set_default_device(device_id: usize) {
        DEFAULT_DEVICE.store(device_id, std::sync::atomic::Ordering::Relaxed);
    }
    fn context() -> Result<Arc<Context>> {
        Context::get(DEFAULT_DEVICE.load(std::sync::atomic::Ordering::Relaxed))
    }
}

/// Flattened `PrimDescriptor` plus the vectors its pointers refer to.
struct LoweredDesc {
    desc: sys::tfb_desc,
    n_inputs: usize,
    _paired: Vec<u32>,
}

fn lower(desc: &PrimDescriptor) -> LoweredDesc {
    let null32: *const u32 = core::ptr::null();
    let mut d = sys::tfb_desc {
        op: 0, reduce_op: 0, modes_a: null32, n_modes_a: 0, modes_b: null32, n_modes_b: 0, modes_c: null32,
        n_modes_c: 0, paired: null32, n_pairs: 0, batch_dims: core::ptr::null(), n_batch_dims: 0, m: 0, n: 0, k: 0,
    };
    let mut paired_flat = Vec::new();
    let mut n_inputs = 1;
    let mut set_pairs = |pairs: &Vec<(u32, u32)>, flat: &mut Vec<u32>| {
        for &(a, b) in pairs {
            flat.push(a);
            flat.push(b);
        }
    };
    match desc {
        PrimDescriptor::BatchedGemm { batch_dims, m, n, k } => {
            d.op = sys::TFB_OP_BATCHED_GEMM;
            d.batch_dims = batch_dims.as_ptr();
            d.n_batch_dims = batch_dims.len();
            d.m = *m;
            d.n = *n;
            d.k = *k;
            n_inputs = 2;
        }
        PrimDescriptor::Reduce { modes_a, modes_c, op } => {
            d.op = sys::TFB_OP_REDUCE;
            d.reduce_op = match op {
                ReduceOp::Sum => sys::TFB_REDUCE_SUM,
                ReduceOp::Max => sys::TFB_REDUCE_MAX,
                ReduceOp::Min => sys::TFB_REDUCE_MIN,
            };
            d.modes_a = modes_a.as_ptr();
            d.n_modes_a = modes_a.len();
            d.modes_c = modes_c.as_ptr();
            d.n_modes_c = modes_c.len();
        }
        PrimDescriptor::Trace { modes_a, modes_c, paired }
        | PrimDescriptor::AntiTrace { modes_a, modes_c, paired }
        | PrimDescriptor::AntiDiag { modes_a, modes_c, paired } => {
            d.op = match desc {
                PrimDescriptor::Trace { .. } => sys::TFB_OP_TRACE,
                PrimDescriptor::AntiTrace { .. } => sys::TFB_OP_ANTI_TRACE,
                _ => sys::TFB_OP_ANTI_DIAG,
            };
            d.modes_a = modes_a.as_ptr();
            d.n_modes_a = modes_a.len();
            d.modes_c = modes_c.as_ptr();
            d.n_modes_c = modes_c.len();
            set_pairs(paired, &mut paired_flat);
            d.n_pairs = paired.len();
        }
        PrimDescriptor::Permute { modes_a, modes_b } => {
            d.op = sys::TFB_OP_PERMUTE;
            d.modes_a = modes_a.as_ptr();
            d.n_modes_a = modes_a.len();
            d.modes_b = modes_b.as_ptr();
            d.n_modes_b = modes_b.len();
        }
        PrimDescriptor::Contract { modes_a, modes_b, modes_c } => {
            d.op = sys::TFB_OP_CONTRACT;
            d.modes_a = modes_a.as_ptr();
            d.n_modes_a = modes_a.len();
            d.modes_b = modes_b.as_ptr();
            d.n_modes_b = modes_b.len();
            d.modes_c = modes_c.as_ptr();
            d.n_modes_c = modes_c.len();
            n_inputs = 2;
        }
        PrimDescriptor::ElementwiseMul => {
            d.op = sys::TFB_OP_ELEMENTWISE_MUL;
            n_inputs = 2;
        }
    }
    d.paired = paired_flat.as_ptr();
    LoweredDesc { desc: d, n_inputs, _paired: paired_flat }
}

/// A `tfb_view` over a strided view of device memory.  The dims/strides vectors are returned
/// beside it because the struct only points at them.
fn raw_view<T>(ptr: *const T, dims: &[usize], strides: &[isize]) -> (sys::tfb_view, Vec<usize>, Vec<isize>) {
    let d = dims.to_vec();
    let s = strides.to_vec();
    let v = sys::tfb_view {
        base: ptr as *mut core::ffi::c_void, // element 0 of the view: offset already applied
        rank: d.len(),
        dims: d.as_ptr(),
        strides: s.as_ptr(),
        offset: 0,
        flags: 0,
    };
    (v, d, s)
}

impl TensorPrims<Standard> for CudaBackend {
    type Plan<T: ScalarBase> = CudaPlan<T>;

    fn plan<T: ScalarBase>(desc: &PrimDescriptor, shapes: &[&[usize]]) -> Result<CudaPlan<T>> {
        let dtype = dtype_of::<T>()
            .ok_or_else(|| Error::InvalidArgument("CudaBackend supports f32, f64, Complex32, Complex64".into()))?;
        let ctx = Self::context()?;
        let lowered = lower(desc);
        let ranks: Vec<usize> = shapes.iter().map(|s| s.len()).collect();
        let dims: Vec<*const usize> = shapes.iter().map(|s| s.as_ptr()).collect();
        let mut raw = core::ptr::null_mut();
        // SAFETY: every pointer inside `lowered.desc`, `ranks` and `dims` refers to memory that
        // lives until the call returns; the library copies what it keeps.
        check(unsafe {
            sys::tfb_plan_create(ctx.raw, &lowered.desc, dtype, shapes.len(), ranks.as_ptr(), dims.as_ptr(), &mut raw)
        })?;
        Ok(CudaPlan { raw, n_inputs: lowered.n_inputs, _ctx: ctx, _scalar: PhantomData })
    }

    fn execute<T: ScalarBase>(
        plan: &CudaPlan<T>,
        alpha: T,
        inputs: &[&StridedView<T>],
        beta: T,
        output: &mut StridedViewMut<T>,
    ) -> Result<()> {
        if inputs.len() != plan.n_inputs {
            return Err(Error::InvalidArgument(format!("plan takes {} inputs, got {}", plan.n_inputs, inputs.len())));
        }
        let mut keep = Vec::with_capacity(inputs.len() + 1);
        let mut views = Vec::with_capacity(inputs.len());
        for v in inputs {
            let (raw, d, s) = raw_view(v.ptr(), v.dims(), v.strides());
            views.push(raw);
            keep.push((d, s));
        }
        let (out, od, os) = raw_view(output.ptr() as *const T, output.dims(), output.strides());
        keep.push((od, os));
        // SAFETY: alpha/beta point to one scalar of the plan's dtype; the views point to vectors
        // held in `keep` until the call returns.  The call only enqueues (the output's
        // completion is the context's next event).
        check(unsafe {
            sys::tfb_execute(plan.raw, (&alpha as *const T).cast(), views.len(), views.as_ptr(), (&beta as *const T).cast(), &out)
        })
    }

    fn has_extension_for<T: ScalarBase>(ext: Extension) -> bool {
        let code = match ext {
            Extension::Contract => sys::TFB_EXT_CONTRACT,
            Extension::ElementwiseMul => sys::TFB_EXT_ELEMENTWISE_MUL,
        };
        match dtype_of::<T>() {
            // SAFETY: plain integers in, integer out.
            Some(dtype) => unsafe { sys::tfb_has_extension(dtype, code) != 0 },
            None => false,
        }
    }
}
