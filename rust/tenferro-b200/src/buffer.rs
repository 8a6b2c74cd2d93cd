//! `CudaBuffer<T>`: owned device storage, the payload of the `DataBuffer::Cuda` variant that
//! `tenferro-tensor/src/lib.rs:133-137` reserves.
use std::marker::PhantomData;
use std::sync::Arc;

use strided_traits::ScalarBase;
use tenferro_b200_sys as sys;
use tenferro_device::Result;

use crate::device::{CompletionEvent, Context};
use crate::error::check;

/// `len` elements of `T` in the memory pool of one context.  Dropping the buffer returns the
/// block to the pool in stream order: kernels already enqueued that read or write it finish
/// first, so a tensor may be dropped right after the call that consumed it
/// (the `_owned` einsum variants, `tenferro-einsum/src/lib.rs:432-498`, rely on this).
pub struct CudaBuffer<T: ScalarBase> {
    ctx: Arc<Context>,
    ptr: *mut T,
    len: usize,
    /// Completion of the latest write, shared by every view of the buffer.
    pub event: Option<CompletionEvent>,
    _owns: PhantomData<T>,
}

// SAFETY: the buffer is a device allocation; host threads only pass its address around.
unsafe impl<T: ScalarBase + Send> Send for CudaBuffer<T> {}
unsafe impl<T: ScalarBase + Sync> Sync for CudaBuffer<T> {}

impl<T: ScalarBase> CudaBuffer<T> {
    /// Uninitialised storage for `len` elements.
    pub fn uninit(ctx: Arc<Context>, len: usize) -> Result<Self> {
        let mut raw = core::ptr::null_mut();
        // SAFETY: live context, valid out-pointer.
        check(unsafe { sys::tfb_alloc(ctx.raw, len.max(1) * core::mem::size_of::<T>(), &mut raw) })?;
        Ok(Self { ctx, ptr: raw.cast(), len, event: None, _owns: PhantomData })
    }

    /// Zero-filled storage (`Tensor::zeros`, `tenferro-tensor/src/lib.rs:336`).
    pub fn zeros(ctx: Arc<Context>, len: usize) -> Result<Self> {
        let mut buf = Self::uninit(ctx, len)?;
        // SAFETY: the block holds `len * size_of::<T>()` bytes.
        check(unsafe { sys::tfb_memset_async(buf.ctx.raw, buf.ptr.cast(), 0, len * core::mem::size_of::<T>()) })?;
        buf.event = Some(buf.ctx.record_event()?);
        Ok(buf)
    }

    /// Copy of a host slice (`Tensor::from_slice`, `tenferro-tensor/src/lib.rs:360`).  Waits for
    /// the copy: `data` is borrowed only for the call.
    pub fn from_slice(ctx: Arc<Context>, data: &[T]) -> Result<Self> {
        let buf = Self::uninit(ctx, data.len())?;
        let bytes = core::mem::size_of_val(data);
        // SAFETY: the block holds `bytes` bytes and `data` outlives the synchronise below.
        check(unsafe { sys::tfb_memcpy_h2d_async(buf.ctx.raw, buf.ptr.cast(), data.as_ptr().cast(), bytes) })?;
        buf.ctx.synchronize()?;
        Ok(buf)
    }

    /// Host copy of the contents (waits for pending work).
    pub fn to_vec(&self) -> Result<Vec<T>>
    where
        T: Clone + Default,
    {
        let mut out = vec![T::default(); self.len];
        self.ctx.synchronize()?;
        // SAFETY: both sides hold `len` elements.
        check(unsafe {
            sys::tfb_memcpy_d2h_async(self.ctx.raw, out.as_mut_ptr().cast(), self.ptr.cast(), self.len * core::mem::size_of::<T>())
        })?;
        self.ctx.synchronize()?;
        Ok(out)
    }

    pub fn as_device_ptr(&self) -> *mut T {
        self.ptr
    }
    pub fn len(&self) -> usize {
        self.len
    }
    pub fn is_empty(&self) -> bool {
        self.len == 0
    }
    pub fn context(&self) -> &Arc<Context> {
        &self.ctx
    }

    /// `to_memory_space_async` between GPUs (`tenferro-tensor/src/lib.rs:660-671`): a peer copy on
    /// the destination's stream, ordered behind this buffer's latest write.
    pub fn copy_to_device(&self, dst_ctx: Arc<Context>) -> Result<CudaBuffer<T>> {
        let mut dst = CudaBuffer::<T>::uninit(dst_ctx, self.len)?;
        let pending;
        let ev = match &self.event {
            Some(ev) => ev,
            None => {
                pending = self.ctx.record_event()?;
                &pending
            }
        };
        dst.ctx.wait_event(ev)?;
        // SAFETY: both blocks hold `len` elements on the named devices.
        check(unsafe {
            sys::tfb_memcpy_p2p_async(dst.ctx.raw, dst.ptr.cast(), dst.ctx.device_id() as i32, self.ptr.cast(),
                                      self.ctx.device_id() as i32, self.len * core::mem::size_of::<T>())
        })?;
        dst.event = Some(dst.ctx.record_event()?);
        Ok(dst)
    }
}

impl<T: ScalarBase> Drop for CudaBuffer<T> {
    fn drop(&mut self) {
        // SAFETY: the block came from tfb_alloc of the same context and is freed once.
        let st = unsafe { sys::tfb_free(self.ctx.raw, self.ptr.cast()) };
        debug_assert_eq!(st, sys::TFB_OK, "tfb_free failed");  // errors cannot leave a destructor
    }
}
