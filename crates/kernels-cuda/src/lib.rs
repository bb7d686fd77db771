//! CUDA backend of RunIT's kernel layer for the quantized decode path (fused-dequant GEMV family and the
//! MoE block).  `dispatch` keeps the function names and argument order of `bare_metal_kernels::dispatch`
//! (crates/kernels/src/dispatch.rs) so that `WeightBuf` and `Executor` in crates/engine compile against
//! either backend.
pub mod context;
pub mod dispatch;
pub mod error;
pub mod ffi;

pub use context::{CudaContext, DeviceBuffer};
pub use error::{KernelError, Result};
