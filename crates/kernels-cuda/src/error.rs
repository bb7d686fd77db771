//! `KernelError` with the variants, field names and shapes of crates/kernels/src/error.rs:4-22, so that callers that
//! construct or match on them compile unchanged.  The CUDA library has no shader library to load and no pipeline
//! objects: `LibraryLoad` reports a failure to create the context (`path` = the shared library, `reason` = the
//! status), `PipelineNotFound` / `PipelineCreate` are kept for source compatibility and never produced.
use thiserror::Error;

#[derive(Error, Debug)]
pub enum KernelError {
    #[error("no CUDA device (B200, sm_100a) found")]
    NoDevice,

    #[error("failed to load the kernel library from '{path}': {reason}")]
    LibraryLoad { path: String, reason: String },

    #[error("pipeline function '{0}' not found")]
    PipelineNotFound(String),

    #[error("failed to create compute pipeline for '{name}': {reason}")]
    PipelineCreate { name: String, reason: String },

    #[error("kernel dispatch error: {0}")]
    Dispatch(String),

    #[error("buffer size mismatch: expected {expected} bytes, got {actual}")]
    BufferSize { expected: usize, actual: usize },
}

pub type Result<T> = std::result::Result<T, KernelError>;
