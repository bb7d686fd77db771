//! `extern "C"` declarations of include/runit_cuda.h (one per exported function used by the engine).
#![allow(non_camel_case_types)]
use std::ffi::c_void;
use std::os::raw::c_char;

#[repr(C)]
pub struct runit_ctx_t {
    _private: [u8; 0],
}
#[repr(C)]
pub struct runit_graph_t {
    _private: [u8; 0],
}

pub const RUNIT_OK: i32 = 0;
pub const RUNIT_ERR_NO_DEVICE: i32 = 1;
pub const RUNIT_ERR_BUFFER_SIZE: i32 = 3;
pub const RUNIT_BUF_DEVICE: i32 = 0;
pub const RUNIT_BUF_HOST_VISIBLE: i32 = 1;

type P = *const c_void;
type M = *mut c_void;
type Ctx = *mut runit_ctx_t;

extern "C" {
    pub fn runit_ctx_create(device: i32, out: *mut Ctx) -> i32;
    pub fn runit_ctx_destroy(ctx: Ctx) -> i32;
    pub fn runit_flush(ctx: Ctx) -> i32;
    pub fn runit_last_error_string(ctx: Ctx) -> *const c_char;
    pub fn runit_buf_alloc(ctx: Ctx, bytes: usize, flags: i32, dptr: *mut M) -> i32;
    pub fn runit_buf_free(ctx: Ctx, dptr: M) -> i32;
    pub fn runit_memcpy_h2d(ctx: Ctx, dst: M, src: P, bytes: usize) -> i32;
    pub fn runit_memcpy_d2h(ctx: Ctx, dst: M, src: P, bytes: usize) -> i32;
    pub fn runit_graph_begin(ctx: Ctx) -> i32;
    pub fn runit_graph_end(ctx: Ctx, out: *mut *mut runit_graph_t) -> i32;
    pub fn runit_graph_launch(ctx: Ctx, g: *mut runit_graph_t) -> i32;

    // Q8_0 (dispatch.rs:1280-1388, 813-871, 903-921)
    pub fn runit_gemv_q8_0_f32in_f32out(ctx: Ctx, w: P, x: P, y: M, m: u32, k: u32) -> i32;
    pub fn runit_gemv_q8_0_add_f32_f32in(ctx: Ctx, w: P, x: P, y: M, r: P, m: u32, k: u32) -> i32;
    pub fn runit_gemv_q8_0_f32in(ctx: Ctx, w: P, x: P, y: M, m: u32, k: u32) -> i32;
    pub fn runit_gemv_q8_0_f16(ctx: Ctx, w: P, x: P, y: M, m: u32, k: u32) -> i32;
    pub fn runit_gemv_q8_0_add_f16(ctx: Ctx, w: P, x: P, y: M, r: P, m: u32, k: u32) -> i32;
    pub fn runit_gemv_q8_0_add_f32res_f16(ctx: Ctx, w: P, x: P, y: M, r: P, m: u32, k: u32) -> i32;
    pub fn runit_fused_qkv_q8_0_f32(ctx: Ctx, wq: P, wk: P, wv: P, x: P, oq: M, ok: M, ov: M, q_dim: u32, kv_dim: u32, k: u32) -> i32;
    pub fn runit_fused_qkv_bias_q8_0_f32(ctx: Ctx, wq: P, wk: P, wv: P, x: P, oq: M, ok: M, ov: M, bq: P, bk: P, bv: P,
                                         q_dim: u32, kv_dim: u32, k: u32) -> i32;
    pub fn runit_fused_ffn_q8_0_f32(ctx: Ctx, wg: P, wu: P, x: P, act: M, ff: u32, k: u32) -> i32;
    // Q4_0 (dispatch.rs:1456-1544)
    pub fn runit_gemv_q4_0_f32in_f32out(ctx: Ctx, w: P, x: P, y: M, m: u32, k: u32) -> i32;
    pub fn runit_gemv_q4_0_add_f32_f32in(ctx: Ctx, w: P, x: P, y: M, r: P, m: u32, k: u32) -> i32;
    pub fn runit_gemv_q4_0_f32in(ctx: Ctx, w: P, x: P, y: M, m: u32, k: u32) -> i32;
    pub fn runit_gemv_q4_0_f16(ctx: Ctx, w: P, x: P, y: M, m: u32, k: u32) -> i32;
    pub fn runit_gemv_q4_0_add_f16(ctx: Ctx, w: P, x: P, y: M, r: P, m: u32, k: u32) -> i32;
    pub fn runit_fused_ffn_q4_0_f32(ctx: Ctx, wg: P, wu: P, x: P, act: M, ff: u32, k: u32) -> i32;
    // Q4_K (dispatch.rs:358, 585, 621, 756, 1229, 1251)
    pub fn runit_gemv_q4k_f32in_f32out(ctx: Ctx, w: P, x: P, y: M, m: u32, k: u32) -> i32;
    pub fn runit_gemv_q4k_add_f32_f32in(ctx: Ctx, w: P, x: P, y: M, r: P, m: u32, k: u32) -> i32;
    pub fn runit_gemv_q4k_f16(ctx: Ctx, w: P, x: P, y: M, m: u32, k: u32) -> i32;
    pub fn runit_gemv_q4k_add_f16(ctx: Ctx, w: P, x: P, y: M, r: P, m: u32, k: u32) -> i32;
    pub fn runit_gemv_q4k_add_f32res_f16(ctx: Ctx, w: P, x: P, y: M, r: P, m: u32, k: u32) -> i32;
    pub fn runit_dequant_q4k_f16(ctx: Ctx, input: P, output: M, n_blocks: u32) -> i32;
    // MoE glue and router (dispatch.rs:15, 35, 270, 316, 1639)
    pub fn runit_gemv_f16w_f32in(ctx: Ctx, w: P, x: P, y: M, m: u32, k: u32) -> i32;
    pub fn runit_silu_mul_f16(ctx: Ctx, gate: P, up: P, out: M, n: u32) -> i32;
    pub fn runit_silu_mul_f32(ctx: Ctx, gate: P, up: P, out: M, n: u32) -> i32;
    pub fn runit_scale_accumulate_f16(ctx: Ctx, src: P, acc: M, weight: f32, n: u32) -> i32;
    pub fn runit_add_f16_into_f32(ctx: Ctx, src: P, acc: M, n: u32) -> i32;
    // device-side routing and the whole block (no twin)
    pub fn runit_moe_route_topk(ctx: Ctx, logits: P, logits_f16: i32, e: u32, k: u32, renorm: i32, t: u32, idx: M, w: M) -> i32;
    pub fn runit_moe_scratch_bytes(t: u32, h: u32, ff: u32, e: u32, k: u32) -> usize;
    pub fn runit_moe_layer_q4k(ctx: Ctx, router: P, gate: P, up: P, down: P, x: P, residual: P, out: M, idx: M, w: M,
                               scratch: M, scratch_bytes: usize, t: u32, h: u32, ff: u32, e: u32, k: u32, renorm: i32) -> i32;
    // other decode ops (dispatch.rs:152, 177, 945, 1159, 1183, 697, 1575, 1615)
    pub fn runit_rms_norm_f32_f32(ctx: Ctx, x: P, y: M, gamma: P, eps: f32, hidden: u32, rows: u32) -> i32;
    pub fn runit_rms_norm_f32_f32_f32g(ctx: Ctx, x: P, y: M, gamma: P, eps: f32, hidden: u32, rows: u32) -> i32;
    pub fn runit_fused_rope_qk_f32(ctx: Ctx, q: M, k: M, head_dim: u32, q_heads: u32, kv_heads: u32, pos: u32, theta: f32) -> i32;
    pub fn runit_kv_copy_to_cache_f16(ctx: Ctx, src: P, dst: M, pos: u32, max_seq: u32, head_dim: u32, kv_heads: u32) -> i32;
    pub fn runit_kv_copy_to_cache_f32(ctx: Ctx, src: P, dst: M, pos: u32, max_seq: u32, head_dim: u32, kv_heads: u32) -> i32;
    pub fn runit_decode_attention_f16(ctx: Ctx, q: P, k: P, v: P, out: M, batch: u32, kv_len: u32, heads: u32, kv_heads: u32,
                                      head_dim: u32, kv_head_stride: u32) -> i32;
    pub fn runit_decode_attention_f32(ctx: Ctx, q: P, k: P, v: P, out: M, batch: u32, kv_len: u32, heads: u32, kv_heads: u32,
                                      head_dim: u32, kv_head_stride: u32) -> i32;
    pub fn runit_argmax_f16(ctx: Ctx, input: P, result: M, n: u32) -> i32;
}
