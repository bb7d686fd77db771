// Device helpers shared by the fused-dequant GEMV kernels and the MoE expert kernels.
//
// Dequantisation without integer->float conversion instructions: a 4-bit field at bit p of a
// word is turned into the float 2^23 + q*2^p by one LOP3 ((v & (15<<p)) | 0x4B000000), and
// one packed FADD removes the 2^23 (and, for Q4_0, the -8 offset).  The factor 2^p is
// cancelled by pre-scaling the activation vector once per stage (exact: powers of two), so
// the per-weight cost is one LOP3, half a packed FADD and half a packed FFMA (sm_100
// add.f32x2 / fma.f32x2).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace runit {

constexpr uint32_t kMagic = 0x4B000000u;   // 2^23 as float bits
constexpr float kTwo23 = 8388608.0f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// 16/8/4-byte asynchronous global->shared copies (LDGSTS); .cg bypasses L1 for the 16-byte
// weight stream (read once), .ca is required for the smaller sizes.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) { return __fadd2_rn(a, b); }

__device__ __forceinline__ float2 bits2(uint32_t a, uint32_t b) {
    return make_float2(__uint_as_float(a), __uint_as_float(b));
}

__device__ __forceinline__ float half_bits_to_float(uint32_t h16) {
    return __half2float(__ushort_as_half((unsigned short)(h16 & 0xFFFFu)));
}

__device__ __forceinline__ float silu(float v) { return v / (1.0f + __expf(-v)); }

// ─────────────── Q4_K scale/min table of one superblock header ───────────────
// header words: h.x = d | dmin<<16, h.y = scales[0..3], h.z = scales[4..7], h.w = scales[8..11].
// Byte j of sl/ml = scale/min of sub-block j (j<4); byte j of sh/mh = those of sub-block j+4
// (get_scale_min_k4, crates/engine/src/forward.rs:359-369).
struct Q4KScales {
    uint32_t sl, ml, sh, mh;
};
__device__ __forceinline__ Q4KScales q4k_unpack_scales(uint4 h) {
    Q4KScales s;
    s.sl = h.y & 0x3F3F3F3Fu;
    s.ml = h.z & 0x3F3F3F3Fu;
    s.sh = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
    s.mh = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
    return s;
}
__device__ __forceinline__ float byte_to_float(uint32_t w, int j) {
    return (float)((w >> (8 * j)) & 0xFFu);
}

// Pre-scale factors applied to the activation vector so that the 2^p of each nibble position
// cancels.  Q4_K: element l of a 32-element sub-block sits in byte l%4 of its qs word; low
// nibbles (first half of a 64-element pair) at bit 8b or, for b==3, bit 12 of (v>>12); high
// nibbles at bit 8b+4, or bit 8/16 of (v>>12) for b==2/3.
__device__ __forceinline__ float q4k_xscale(int elem_in_unit) {
    const int b = elem_in_unit & 3;
    const bool hi = (elem_in_unit >> 5) & 1;
    // lo: 2^0, 2^-8, 2^-16, 2^-12      hi: 2^-4, 2^-12, 2^-8, 2^-16
    const int sh = hi ? (b == 0 ? 4 : (b == 1 ? 12 : (b == 2 ? 8 : 16)))
                      : (b == 0 ? 0 : (b == 1 ? 8 : (b == 2 ? 16 : 12)));
    return __uint_as_float((uint32_t)(127 - sh) << 23);
}

// Q4_0: element e of a 256-element unit (8 blocks of 18 bytes): block b=e/32, byte i=(e%32)/2,
// h=e%2 (low/high nibble).  The byte sits at unit offset 18b+2+i, i.e. byte position
// bp=(2b+2+i)%4 of its word.  Fields: bp0 (bit 0, bit 4); bp1 (8, 12); bp2 (16, bit 8 of v>>12);
// bp3 (bit 12 and bit 16 of v>>12).
__device__ __forceinline__ int q4_0_shift(int bp, int h) {
    return bp == 0 ? (h ? 4 : 0) : bp == 1 ? (h ? 12 : 8) : bp == 2 ? (h ? 8 : 16) : (h ? 16 : 12);
}
__device__ __forceinline__ float q4_0_xscale(int elem_in_unit) {
    const int b = elem_in_unit >> 5, i = (elem_in_unit & 31) >> 1, h = elem_in_unit & 1;
    const int bp = (2 * b + 2 + i) & 3;
    return __uint_as_float((uint32_t)(127 - q4_0_shift(bp, h)) << 23);
}

}  // namespace runit
