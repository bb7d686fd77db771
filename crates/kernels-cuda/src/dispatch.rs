//! Same free functions as crates/kernels/src/dispatch.rs for the quantized decode path, forwarding to
//! librunit_cuda.so.  `ctx: &MetalContext` becomes `&CudaContext`, `&metal::Buffer` becomes `&DeviceBuffer`.
use crate::context::{CudaContext, DeviceBuffer};
use crate::error::Result;
use crate::ffi;

type B = DeviceBuffer;

pub fn gemv_q8_0_f32in_f32out(ctx: &CudaContext, weight: &B, input: &B, output: &B, m: u32, k: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_gemv_q8_0_f32in_f32out(ctx.raw, weight.ptr, input.ptr, output.ptr, m, k) })
}
pub fn gemv_q8_0_f32in(ctx: &CudaContext, weight: &B, input: &B, output: &B, m: u32, k: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_gemv_q8_0_f32in(ctx.raw, weight.ptr, input.ptr, output.ptr, m, k) })
}
pub fn gemv_q8_0_f16(ctx: &CudaContext, weight: &B, input: &B, output: &B, m: u32, k: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_gemv_q8_0_f16(ctx.raw, weight.ptr, input.ptr, output.ptr, m, k) })
}
pub fn gemv_q4_0_f32in_f32out(ctx: &CudaContext, weight: &B, input: &B, output: &B, m: u32, k: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_gemv_q4_0_f32in_f32out(ctx.raw, weight.ptr, input.ptr, output.ptr, m, k) })
}
pub fn gemv_q4_0_f32in(ctx: &CudaContext, weight: &B, input: &B, output: &B, m: u32, k: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_gemv_q4_0_f32in(ctx.raw, weight.ptr, input.ptr, output.ptr, m, k) })
}
pub fn gemv_q4_0_f16(ctx: &CudaContext, weight: &B, input: &B, output: &B, m: u32, k: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_gemv_q4_0_f16(ctx.raw, weight.ptr, input.ptr, output.ptr, m, k) })
}
pub fn gemv_q4k_f32in_f32out(ctx: &CudaContext, weight: &B, input: &B, output: &B, m: u32, k: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_gemv_q4k_f32in_f32out(ctx.raw, weight.ptr, input.ptr, output.ptr, m, k) })
}
pub fn gemv_q4k_f16(ctx: &CudaContext, weight: &B, input: &B, output: &B, m: u32, k: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_gemv_q4k_f16(ctx.raw, weight.ptr, input.ptr, output.ptr, m, k) })
}
pub fn gemv_f16w_f32in(ctx: &CudaContext, weight: &B, input: &B, output: &B, m: u32, k: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_gemv_f16w_f32in(ctx.raw, weight.ptr, input.ptr, output.ptr, m, k) })
}
pub fn gemv_q8_0_add_f32_f32in(ctx: &CudaContext, weight: &B, input: &B, output: &B, residual: &B, m: u32, k: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_gemv_q8_0_add_f32_f32in(ctx.raw, weight.ptr, input.ptr, output.ptr, residual.ptr, m, k) })
}
pub fn gemv_q8_0_add_f16(ctx: &CudaContext, weight: &B, input: &B, output: &B, residual: &B, m: u32, k: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_gemv_q8_0_add_f16(ctx.raw, weight.ptr, input.ptr, output.ptr, residual.ptr, m, k) })
}
pub fn gemv_q8_0_add_f32res_f16(ctx: &CudaContext, weight: &B, input: &B, output: &B, residual: &B, m: u32, k: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_gemv_q8_0_add_f32res_f16(ctx.raw, weight.ptr, input.ptr, output.ptr, residual.ptr, m, k) })
}
pub fn gemv_q4_0_add_f32_f32in(ctx: &CudaContext, weight: &B, input: &B, output: &B, residual: &B, m: u32, k: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_gemv_q4_0_add_f32_f32in(ctx.raw, weight.ptr, input.ptr, output.ptr, residual.ptr, m, k) })
}
pub fn gemv_q4_0_add_f16(ctx: &CudaContext, weight: &B, input: &B, output: &B, residual: &B, m: u32, k: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_gemv_q4_0_add_f16(ctx.raw, weight.ptr, input.ptr, output.ptr, residual.ptr, m, k) })
}
pub fn gemv_q4k_add_f32_f32in(ctx: &CudaContext, weight: &B, input: &B, output: &B, residual: &B, m: u32, k: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_gemv_q4k_add_f32_f32in(ctx.raw, weight.ptr, input.ptr, output.ptr, residual.ptr, m, k) })
}
pub fn gemv_q4k_add_f16(ctx: &CudaContext, weight: &B, input: &B, output: &B, residual: &B, m: u32, k: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_gemv_q4k_add_f16(ctx.raw, weight.ptr, input.ptr, output.ptr, residual.ptr, m, k) })
}
pub fn gemv_q4k_add_f32res_f16(ctx: &CudaContext, weight: &B, input: &B, output: &B, residual: &B, m: u32, k: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_gemv_q4k_add_f32res_f16(ctx.raw, weight.ptr, input.ptr, output.ptr, residual.ptr, m, k) })
}
/// `use_mr` / `_wide` launch-shape variants of the reference (dispatch.rs:1083-1117, 1397-1447) are the same kernel here.
pub use gemv_q8_0_add_f32_f32in as gemv_q8_0_add_f32_f32in_mr;
pub use gemv_q8_0_f32in_f32out as gemv_q8_0_f32in_f32out_mr;

#[allow(clippy::too_many_arguments)]
pub fn fused_qkv_q8_0_f32(ctx: &CudaContext, w_q: &B, w_k: &B, w_v: &B, x_vec: &B, out_q: &B, out_k: &B, out_v: &B,
                          q_dim: u32, kv_dim: u32, k: u32) -> Result<()> {
    ctx.check(unsafe {
        ffi::runit_fused_qkv_q8_0_f32(ctx.raw, w_q.ptr, w_k.ptr, w_v.ptr, x_vec.ptr, out_q.ptr, out_k.ptr, out_v.ptr, q_dim, kv_dim, k)
    })
}

#[allow(clippy::too_many_arguments)]
pub fn fused_qkv_bias_q8_0_f32(ctx: &CudaContext, w_q: &B, w_k: &B, w_v: &B, x_vec: &B, out_q: &B, out_k: &B, out_v: &B,
                               bias_q: &B, bias_k: &B, bias_v: &B, q_dim: u32, kv_dim: u32, k: u32) -> Result<()> {
    ctx.check(unsafe {
        ffi::runit_fused_qkv_bias_q8_0_f32(ctx.raw, w_q.ptr, w_k.ptr, w_v.ptr, x_vec.ptr, out_q.ptr, out_k.ptr, out_v.ptr,
                                           bias_q.ptr, bias_k.ptr, bias_v.ptr, q_dim, kv_dim, k)
    })
}

pub fn fused_ffn_q8_0_f32(ctx: &CudaContext, w_gate: &B, w_up: &B, x_vec: &B, act_out: &B, ff_dim: u32, k: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_fused_ffn_q8_0_f32(ctx.raw, w_gate.ptr, w_up.ptr, x_vec.ptr, act_out.ptr, ff_dim, k) })
}

pub fn fused_ffn_q4_0_f32(ctx: &CudaContext, w_gate: &B, w_up: &B, x_vec: &B, act_out: &B, ff_dim: u32, k: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_fused_ffn_q4_0_f32(ctx.raw, w_gate.ptr, w_up.ptr, x_vec.ptr, act_out.ptr, ff_dim, k) })
}

pub fn dequant_q4k_f16(ctx: &CudaContext, input: &B, output: &B, n_blocks: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_dequant_q4k_f16(ctx.raw, input.ptr, output.ptr, n_blocks) })
}

pub fn silu_mul_f16(ctx: &CudaContext, gate: &B, up: &B, out: &B, n: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_silu_mul_f16(ctx.raw, gate.ptr, up.ptr, out.ptr, n) })
}

pub fn silu_mul_f32(ctx: &CudaContext, gate: &B, up: &B, out: &B, n: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_silu_mul_f32(ctx.raw, gate.ptr, up.ptr, out.ptr, n) })
}

pub fn scale_accumulate_f16(ctx: &CudaContext, src: &B, acc: &B, weight: f32, n: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_scale_accumulate_f16(ctx.raw, src.ptr, acc.ptr, weight, n) })
}

pub fn add_f16_into_f32(ctx: &CudaContext, src: &B, acc: &B, n: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_add_f16_into_f32(ctx.raw, src.ptr, acc.ptr, n) })
}

/// Device-side replacement of `ctx.flush()` + `topk_softmax` (crates/engine/src/forward.rs:1654-1657):
/// indices (i32) and weights (f32) stay on the device.
#[allow(clippy::too_many_arguments)]
pub fn moe_route_topk(ctx: &CudaContext, logits: &B, logits_f16: bool, num_experts: u32, top_k: u32, renorm: bool,
                      tokens: u32, out_idx: &B, out_w: &B) -> Result<()> {
    ctx.check(unsafe {
        ffi::runit_moe_route_topk(ctx.raw, logits.ptr, logits_f16 as i32, num_experts, top_k, renorm as i32, tokens, out_idx.ptr, out_w.ptr)
    })
}

pub fn rms_norm_f32_f32(ctx: &CudaContext, x: &B, y: &B, gamma: &B, eps: f32, hidden: u32, num_rows: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_rms_norm_f32_f32(ctx.raw, x.ptr, y.ptr, gamma.ptr, eps, hidden, num_rows) })
}

pub fn rms_norm_f32_f32_f32g(ctx: &CudaContext, x: &B, y: &B, gamma: &B, eps: f32, hidden: u32, num_rows: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_rms_norm_f32_f32_f32g(ctx.raw, x.ptr, y.ptr, gamma.ptr, eps, hidden, num_rows) })
}

#[allow(clippy::too_many_arguments)]
pub fn fused_rope_qk_f32(ctx: &CudaContext, q: &B, k: &B, head_dim: u32, q_heads: u32, kv_heads: u32, pos: u32, theta: f32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_fused_rope_qk_f32(ctx.raw, q.ptr, k.ptr, head_dim, q_heads, kv_heads, pos, theta) })
}

pub fn kv_copy_to_cache_f16(ctx: &CudaContext, src: &B, dst: &B, pos: u32, max_seq: u32, head_dim: u32, num_kv_heads: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_kv_copy_to_cache_f16(ctx.raw, src.ptr, dst.ptr, pos, max_seq, head_dim, num_kv_heads) })
}

pub fn kv_copy_to_cache_f32(ctx: &CudaContext, src: &B, dst: &B, pos: u32, max_seq: u32, head_dim: u32, num_kv_heads: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_kv_copy_to_cache_f32(ctx.raw, src.ptr, dst.ptr, pos, max_seq, head_dim, num_kv_heads) })
}

#[allow(clippy::too_many_arguments)]
pub fn decode_attention_f32(ctx: &CudaContext, q: &B, k: &B, v: &B, out: &B, batch: u32, kv_len: u32, num_heads: u32,
                            num_kv_heads: u32, head_dim: u32, kv_head_stride: u32) -> Result<()> {
    ctx.check(unsafe {
        ffi::runit_decode_attention_f32(ctx.raw, q.ptr, k.ptr, v.ptr, out.ptr, batch, kv_len, num_heads, num_kv_heads, head_dim, kv_head_stride)
    })
}

#[allow(clippy::too_many_arguments)]
pub fn decode_attention_f16(ctx: &CudaContext, q: &B, k: &B, v: &B, out: &B, batch: u32, kv_len: u32, num_heads: u32,
                            num_kv_heads: u32, head_dim: u32, kv_head_stride: u32) -> Result<()> {
    ctx.check(unsafe {
        ffi::runit_decode_attention_f16(ctx.raw, q.ptr, k.ptr, v.ptr, out.ptr, batch, kv_len, num_heads, num_kv_heads, head_dim, kv_head_stride)
    })
}

pub fn argmax_f16(ctx: &CudaContext, input: &B, result: &B, n: u32) -> Result<()> {
    ctx.check(unsafe { ffi::runit_argmax_f16(ctx.raw, input.ptr, result.ptr, n) })
}
