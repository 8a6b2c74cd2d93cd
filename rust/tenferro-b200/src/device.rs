//! Context, events and transfers: the CUDA half of `tenferro-device`
//! (`tenferro-device/src/lib.rs:30-105`) and of `CompletionEvent`
//! (`tenferro-tensor/src/lib.rs:301-309, 677-713`).
use std::collections::HashMap;
use std::sync::{Arc, Mutex, OnceLock};

use tenferro_b200_sys as sys;
use tenferro_device::{ComputeDevice, Error, LogicalMemorySpace, OpKind, Result};

use crate::error::check;

/// One per CUDA device in use: a stream (one in-order queue) and a stream-ordered pool.
/// `TensorPrims` has no receiver (`tenferro-prims/src/lib.rs:259-262`), so contexts live in a
/// process-wide registry keyed by device id.
pub struct Context {
    pub(crate) raw: *mut sys::tfb_ctx,
    device_id: i32,
}

// SAFETY: the C library serialises access to a context's mutable state internally (stream
// order on the device, a mutex around its caches); handles are plain pointers.
unsafe impl Send for Context {}
unsafe impl Sync for Context {}

impl Context {
    /// A new context of its own (own stream, own pool): for work that should overlap the
    /// registry's context of the same device, chained through events.
    pub fn new(device_id: usize) -> Result<Self> {
        let mut raw = core::ptr::null_mut();
        // SAFETY: `raw` is a valid out-pointer; on failure it stays NULL and nothing is owned.
        check(unsafe { sys::tfb_ctx_create(device_id as i32, &mut raw) })?;
        Ok(Self { raw, device_id: device_id as i32 })
    }

    /// The shared context of `ComputeDevice::Cuda { device_id }`.
    pub fn get(device_id: usize) -> Result<Arc<Context>> {
        static REGISTRY: OnceLock<Mutex<HashMap<usize, Arc<Context>>>> = OnceLock::new();
        let mut map = REGISTRY
            .get_or_init(|| Mutex::new(HashMap::new()))
            .lock()
            .map_err(|_| Error::DeviceError("context registry poisoned".into()))?;
        if let Some(ctx) = map.get(&device_id) {
            return Ok(ctx.clone());
        }
        let ctx = Arc::new(Context::new(device_id)?);
        map.insert(device_id, ctx.clone());
        Ok(ctx)
    }

    pub fn device_id(&self) -> usize {
        self.device_id as usize
    }

    /// `LogicalMemorySpace::GpuMemory { space_id }` this context computes on.
    pub fn memory_space(&self) -> LogicalMemorySpace {
        LogicalMemorySpace::GpuMemory { space_id: self.device_id as usize }
    }

    /// Blocks until everything enqueued so far has run.  A kernel that gave up a bounded wait
    /// surfaces here as `Error::DeviceError`.
    pub fn synchronize(&self) -> Result<()> {
        // SAFETY: `raw` is a live context for the lifetime of `self`.
        check(unsafe { sys::tfb_ctx_synchronize(self.raw) })
    }

    /// Records what `f` enqueues on this context into a graph instead of running it
    /// (`tfb_ctx_capture_begin` / `_end`).  The sequence must have run once before: first uses
    /// build plans and offset tables with calls that capture does not allow.
    pub fn capture<F: FnOnce() -> Result<()>>(&self, f: F) -> Result<CapturedGraph> {
        // SAFETY: `raw` is a live context for the lifetime of `self`.
        check(unsafe { sys::tfb_ctx_capture_begin(self.raw) })?;
        let body = f();
        let mut graph = core::ptr::null_mut();
        // SAFETY: valid context and out-pointer; ends the capture whatever `f` returned.
        let ended = check(unsafe { sys::tfb_ctx_capture_end(self.raw, &mut graph) });
        body?;
        ended?;
        Ok(CapturedGraph { raw: graph })
    }

    /// Marks all work enqueued so far.
    pub fn record_event(&self) -> Result<CompletionEvent> {
        let mut ev = core::ptr::null_mut();
        // SAFETY: valid context and out-pointer.
        check(unsafe { sys::tfb_event_record(self.raw, &mut ev) })?;
        Ok(CompletionEvent { raw: ev })
    }

    /// Later work of this context waits for `ev`; the host does not block.
    pub fn wait_event(&self, ev: &CompletionEvent) -> Result<()> {
        // SAFETY: both handles are live.
        check(unsafe { sys::tfb_event_wait(self.raw, ev.raw) })
    }

    /// Asynchronous host -> device copy.  `src` must stay alive and unchanged until the copy has
    /// run (page-locked memory for a truly asynchronous transfer).
    ///
    /// # Safety
    /// `dst` must be a device allocation of at least `bytes` bytes owned by this device.
    pub unsafe fn h2d(&self, dst: *mut u8, src: &[u8], bytes: usize) -> Result<()> {
        debug_assert!(bytes <= src.len());
        check(sys::tfb_memcpy_h2d_async(self.raw, dst.cast(), src.as_ptr().cast(), bytes))
    }

    /// Asynchronous device -> host copy.
    ///
    /// # Safety
    /// `src` must be a device allocation of at least `bytes` bytes; `dst` must not be read
    /// before the copy has completed.
    pub unsafe fn d2h(&self, dst: &mut [u8], src: *const u8, bytes: usize) -> Result<()> {
        debug_assert!(bytes <= dst.len());
        check(sys::tfb_memcpy_d2h_async(self.raw, dst.as_mut_ptr().cast(), src.cast(), bytes))
    }
}

impl Drop for Context {
    fn drop(&mut self) {
        // SAFETY: the handle came from tfb_ctx_create and is dropped once.
        unsafe { sys::tfb_ctx_destroy(self.raw) };
    }
}

/// A captured sequence of calls (`tfb_graph_*`); `launch` replays it on the context's stream with
/// the pointers and scalars the captured calls were given.
pub struct CapturedGraph {
    pub(crate) raw: *mut sys::tfb_graph,
}

// SAFETY: the handle is only read by `launch`; CUDA graph launches may come from any thread.
unsafe impl Send for CapturedGraph {}

impl CapturedGraph {
    pub fn launch(&self) -> Result<()> {
        // SAFETY: live handle.
        check(unsafe { sys::tfb_graph_launch(self.raw) })
    }
}

impl Drop for CapturedGraph {
    fn drop(&mut self) {
        // SAFETY: the handle came from tfb_ctx_capture_end and is destroyed once.
        unsafe { sys::tfb_graph_destroy(self.raw) }
    }
}

/// `CompletionEvent` (`tenferro-tensor/src/lib.rs:301-309`): completion of enqueued device work.
pub struct CompletionEvent {
    pub(crate) raw: *mut sys::tfb_event,
}

// SAFETY: a CUDA event handle may be waited on and queried from any thread.
unsafe impl Send for CompletionEvent {}
unsafe impl Sync for CompletionEvent {}

impl CompletionEvent {
    /// `Tensor::wait` (`tenferro-tensor/src/lib.rs:677-704`).
    pub fn wait(&self) -> Result<()> {
        // SAFETY: live handle.
        check(unsafe { sys::tfb_event_synchronize(self.raw) })
    }

    /// `Tensor::is_ready` (`tenferro-tensor/src/lib.rs:706-713`).
    pub fn is_ready(&self) -> Result<bool> {
        let mut ready = 0;
        // SAFETY: live handle, valid out-pointer.
        check(unsafe { sys::tfb_event_query(self.raw, &mut ready) })?;
        Ok(ready != 0)
    }
}

impl Drop for CompletionEvent {
    fn drop(&mut self) {
        // SAFETY: dropped once.
        unsafe { sys::tfb_event_destroy(self.raw) };
    }
}

fn op_kind_code(op: OpKind) -> i32 {
    match op {
        OpKind::Contract => sys::TFB_KIND_CONTRACT,
        OpKind::BatchedGemm => sys::TFB_KIND_BATCHED_GEMM,
        OpKind::Reduce => sys::TFB_KIND_REDUCE,
        OpKind::Trace => sys::TFB_KIND_TRACE,
        OpKind::Permute => sys::TFB_KIND_PERMUTE,
        OpKind::ElementwiseMul => sys::TFB_KIND_ELEMENTWISE_MUL,
    }
}

/// The CUDA arm of `preferred_compute_devices` (`tenferro-device/src/lib.rs:92-105`): the owning
/// GPU first, then peers that can map its memory.  `MainMemory` has no CUDA device.
pub fn preferred_compute_devices(space: LogicalMemorySpace, op: OpKind) -> Result<Vec<ComputeDevice>> {
    let (kind, id) = match space {
        LogicalMemorySpace::MainMemory => (sys::TFB_SPACE_MAIN_MEMORY, 0),
        LogicalMemorySpace::GpuMemory { space_id } => (sys::TFB_SPACE_GPU_MEMORY, space_id),
    };
    let mut out = [sys::tfb_compute_device { kind: 0, device_id: 0 }; 16];
    let mut n = 0usize;
    // SAFETY: `out` holds 16 entries and `cap` says so.
    let st = unsafe { sys::tfb_preferred_compute_devices(kind, id, op_kind_code(op), out.as_mut_ptr(), out.len(), &mut n) };
    if st == sys::TFB_ERR_NO_COMPATIBLE_DEVICE {
        return Err(Error::NoCompatibleComputeDevice { space, op });
    }
    check(st)?;
    Ok(out[..n.min(out.len())]
        .iter()
        .map(|d| match d.kind {
            sys::TFB_DEVICE_CUDA => ComputeDevice::Cuda { device_id: d.device_id as usize },
            sys::TFB_DEVICE_HIP => ComputeDevice::Hip { device_id: d.device_id as usize },
            _ => ComputeDevice::Cpu { device_id: d.device_id as usize },
        })
        .collect())
}
