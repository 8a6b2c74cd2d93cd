//! `CudaBackend`: tenferro's `TensorPrims<Standard>` on NVIDIA B200 (sm_100a).
//!
//! Uncompiled here (no Rust toolchain on the build machines); see `rust/README.md`.
//!
//! Layering follows the reference workspace:
//! * [`device`]  - what `tenferro-device` gains: context, stream-ordered pool, events, copies;
//! * [`buffer`]  - `CudaBuffer<T>`, the payload of `DataBuffer::Cuda`
//!                 (`tenferro-tensor/src/lib.rs:133-137`);
//! * [`backend`] - `impl TensorPrims<Standard> for CudaBackend`
//!                 (`tenferro-prims/src/lib.rs:278-340`, beside `CpuBackend` at `:417-439`);
//! * [`einsum`]  - `Subscripts`, `ContractionTree` and `einsum_with_plan_into` executed on the
//!                 device (`tenferro-einsum/src/lib.rs:239-356, 584-621`).
pub mod backend;
pub mod buffer;
pub mod device;
pub mod einsum;
mod error;

pub use backend::{CudaBackend, CudaPlan};
pub use buffer::CudaBuffer;
pub use device::{CapturedGraph, CompletionEvent, Context};
pub use error::check;
