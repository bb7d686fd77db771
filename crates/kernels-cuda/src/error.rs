//! Same variants as crates/kernels/src/error.rs:4-22 so callers match on them unchanged.
use thiserror::Error;

#[derive(Debug, Error)]
pub enum KernelError {
    #[error("no CUDA device (B200) available")]
    NoDevice,
    #[error("failed to load library: {0}")]
    LibraryLoad(String),
    #[error("kernel not found: {0}")]
    PipelineNotFound(String),
    #[error("kernel creation failed: {0}")]
    PipelineCreate(String),
    #[error("dispatch error: {0}")]
    Dispatch(String),
    #[error("buffer size mismatch: expected {expected}, got {actual}")]
    BufferSize { expected: usize, actual: usize },
}

pub type Result<T> = std::result::Result<T, KernelError>;
