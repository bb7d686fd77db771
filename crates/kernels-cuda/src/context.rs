//! `CudaContext` / `DeviceBuffer`: the roles of `MetalContext` and `metal::Buffer`
//! (crates/kernels/src/context.rs:137-304).
use std::ffi::{c_void, CStr};

use crate::error::{KernelError, Result};
use crate::ffi;

/// One CUDA stream on one GPU.  Not `Sync`, like `MetalContext` (context.rs:158).
pub struct CudaContext {
    pub(crate) raw: *mut ffi::runit_ctx_t,
}

/// Device memory owned by the caller; ops never allocate or retain it.
pub struct DeviceBuffer {
    pub(crate) ptr: *mut c_void,
    len: usize,
    ctx: *mut ffi::runit_ctx_t,
}

impl CudaContext {
    /// `MetalContext::new()` (context.rs:163-205).
    pub fn new(device: i32) -> Result<Self> {
        let mut raw = std::ptr::null_mut();
        match unsafe { ffi::runit_ctx_create(device, &mut raw) } {
            ffi::RUNIT_OK => Ok(Self { raw }),
            ffi::RUNIT_ERR_NO_DEVICE => Err(KernelError::NoDevice),
            s => Err(KernelError::LibraryLoad { path: "librunit_cuda.so".to_string(), reason: format!("runit_ctx_create returned status {s}") }),
        }
    }

    /// `MetalContext::new_buffer` (context.rs:215-220).  `host_visible` gives the CPU-readable kind the
    /// engine uses for scratch it touches from the host (forward.rs:1494-1505, 1973).
    pub fn new_buffer(&self, len: usize, host_visible: bool) -> Result<DeviceBuffer> {
        let mut ptr = std::ptr::null_mut();
        let flags = if host_visible { ffi::RUNIT_BUF_HOST_VISIBLE } else { ffi::RUNIT_BUF_DEVICE };
        self.check(unsafe { ffi::runit_buf_alloc(self.raw, len, flags, &mut ptr) })?;
        Ok(DeviceBuffer { ptr, len, ctx: self.raw })
    }

    pub fn upload(&self, buf: &DeviceBuffer, data: &[u8]) -> Result<()> {
        if data.len() > buf.len {
            return Err(KernelError::BufferSize { expected: buf.len, actual: data.len() });
        }
        self.check(unsafe { ffi::runit_memcpy_h2d(self.raw, buf.ptr, data.as_ptr() as *const c_void, data.len()) })?;
        self.flush()
    }

    pub fn download(&self, buf: &DeviceBuffer, out: &mut [u8]) -> Result<()> {
        if out.len() > buf.len {
            return Err(KernelError::BufferSize { expected: buf.len, actual: out.len() });
        }
        self.check(unsafe { ffi::runit_memcpy_d2h(self.raw, out.as_mut_ptr() as *mut c_void, buf.ptr, out.len()) })?;
        self.flush()
    }

    /// `MetalContext::flush` (context.rs:289-296): waits for the stream; also surfaces deferred errors.
    pub fn flush(&self) -> Result<()> {
        self.check(unsafe { ffi::runit_flush(self.raw) })
    }

    pub(crate) fn last_error(&self) -> String {
        unsafe { CStr::from_ptr(ffi::runit_last_error_string(self.raw)) }.to_string_lossy().into_owned()
    }

    pub(crate) fn check(&self, status: i32) -> Result<()> {
        match status {
            ffi::RUNIT_OK => Ok(()),
            ffi::RUNIT_ERR_NO_DEVICE => Err(KernelError::NoDevice),
            ffi::RUNIT_ERR_BUFFER_SIZE => Err(KernelError::BufferSize { expected: 0, actual: 0 }),
            _ => Err(KernelError::Dispatch(self.last_error())),
        }
    }
}

impl Drop for CudaContext {
    fn drop(&mut self) {
        unsafe { ffi::runit_ctx_destroy(self.raw) };
    }
}

impl DeviceBuffer {
    pub fn len(&self) -> usize {
        self.len
    }
    pub fn is_empty(&self) -> bool {
        self.len == 0
    }
    pub fn as_ptr(&self) -> *const c_void {
        self.ptr
    }
}

impl Drop for DeviceBuffer {
    fn drop(&mut self) {
        unsafe { ffi::runit_buf_free(self.ctx, self.ptr) };
    }
}
