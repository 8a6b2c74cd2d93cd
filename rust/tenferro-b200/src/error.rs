//! `tfb_status` -> `tenferro_device::Error` (`tenferro-device/src/lib.rs:109-159`).
//!
//! The C side reports one integer per `Error` variant plus a thread-local message.  The
//! structured variants (`ShapeMismatch { expected, got }` ...) are rebuilt from the message,
//! which the library formats as the variant's own `Display` text; where that fails the text
//! travels as `InvalidArgument`.
use tenferro_b200_sys as sys;
use tenferro_device::{Error, LogicalMemorySpace, OpKind, Result};

/// The calling thread's last error message.
pub(crate) fn last_error() -> String {
    // SAFETY: a NULL buffer with capacity 0 only asks for the length; the second call writes at
    // most `cap` bytes including the terminator into a buffer of that size.
    unsafe {
        let n = sys::tfb_last_error(core::ptr::null_mut(), 0);
        let mut buf = vec![0u8; n + 1];
        sys::tfb_last_error(buf.as_mut_ptr().cast(), buf.len());
        buf.truncate(n);
        String::from_utf8_lossy(&buf).into_owned()
    }
}

fn numbers_after(text: &str, key: &str) -> Option<Vec<usize>> {
    let rest = &text[text.find(key)? + key.len()..];
    let rest = rest.trim_start();
    let body = if let Some(inner) = rest.strip_prefix('[') { &inner[..inner.find(']')?] } else { rest };
    let nums: Vec<usize> = body
        .split(|c: char| !c.is_ascii_digit())
        .filter(|s| !s.is_empty())
        .take(if rest.starts_with('[') { usize::MAX } else { 1 })
        .filter_map(|s| s.parse().ok())
        .collect();
    if nums.is_empty() { None } else { Some(nums) }
}

/// `GpuMemory { space_id: N }` if the text names one, else `MainMemory`.
fn space_in(text: &str) -> LogicalMemorySpace {
    match numbers_after(text, "space_id:") {
        Some(n) => LogicalMemorySpace::GpuMemory { space_id: n[0] },
        None => LogicalMemorySpace::MainMemory,
    }
}

/// Turn a status code into `Result`, consuming the thread's message on failure.
pub fn check(status: sys::tfb_status) -> Result<()> {
    if status == sys::TFB_OK {
        return Ok(());
    }
    let msg = last_error();
    Err(match status {
        sys::TFB_ERR_SHAPE_MISMATCH => match (numbers_after(&msg, "expected"), numbers_after(&msg, "got")) {
            (Some(expected), Some(got)) => Error::ShapeMismatch { expected, got },
            _ => Error::InvalidArgument(msg),
        },
        sys::TFB_ERR_RANK_MISMATCH => match (numbers_after(&msg, "expected"), numbers_after(&msg, "got")) {
            (Some(e), Some(g)) => Error::RankMismatch { expected: e[0], got: g[0] },
            _ => Error::InvalidArgument(msg),
        },
        sys::TFB_ERR_DEVICE => Error::DeviceError(msg),
        // The library names the space and the op in the message; the typed fields are filled by
        // the callers that know them (see `device::preferred_compute_devices`).
        sys::TFB_ERR_NO_COMPATIBLE_DEVICE => Error::NoCompatibleComputeDevice {
            space: LogicalMemorySpace::MainMemory,
            op: OpKind::Contract,
        },
        sys::TFB_ERR_CROSS_MEMORY_SPACE => match msg.split_once(" and ") {
            Some((left, right)) => Error::CrossMemorySpaceOperation { left: space_in(left), right: space_in(right) },
            None => Error::InvalidArgument(msg),
        },
        sys::TFB_ERR_INVALID_ARGUMENT | sys::TFB_ERR_STRIDED => Error::InvalidArgument(msg),
        _ => Error::DeviceError(format!("unknown status {status}: {msg}")),
    })
}
