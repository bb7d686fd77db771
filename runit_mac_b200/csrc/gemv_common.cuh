// Device helpers shared by the fused-dequant GEMV kernels and the MoE expert kernels.
//
// Dequantisation without integer->float conversion instructions.  Weights are handled as
// 64-bit register pairs P = (word 2n, word 2n+1) exactly as they arrive from a 128-bit
// shared-memory load.  A 4-bit (or 8-bit) field at bit p of BOTH words becomes the packed
// float pair (2^23 + q*2^p, 2^23 + q'*2^p) with one 64-bit logic op (two LOP3), one packed
// add.f32x2 removes the 2^23 (and the -8 / -128 offsets), and one packed fma.f32x2 multiplies
// by the activation pair.  The factor 2^p is cancelled by pre-scaling the activations once per
// stage (exact: powers of two), and the activations are stored permuted so that a 128-bit load
// yields exactly the pairs the fields need.  Per weight: one LOP3, half an add.f32x2, half an
// fma.f32x2 — and no register-pair shuffling.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace runit {

constexpr uint64_t kMagic2 = 0x4B0000004B000000ull;   // (2^23, 2^23) as packed float bits
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
template <int CPB>
__device__ __forceinline__ void cp_async(uint32_t dst, const void* src) {
    if (CPB == 16) cp_async16(dst, src);
    else if (CPB == 8) cp_async8(dst, src);
    else cp_async4(dst, src);
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// Packed f32x2 arithmetic on 64-bit registers (sm_100: add.f32x2 / fma.f32x2).
__device__ __forceinline__ uint64_t fadd2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
// One LOP3 per 32-bit half: ((word & MASK) | 2^23-bits) and ((word & MASK) ^ C).  Written as explicit
// lop3.b32 because 64-bit and/or pairs are not fused into one LOP3 per half by the compiler.
template <uint32_t MASK>
__device__ __forceinline__ uint64_t field_or_magic(uint64_t P) {
    uint64_t out;
    asm("{\n .reg .b32 lo, hi, a, b;\n mov.b64 {lo, hi}, %1;\n"
        " lop3.b32 a, lo, %2, 0x4B000000, 0xEA;\n lop3.b32 b, hi, %2, 0x4B000000, 0xEA;\n"
        " mov.b64 %0, {a, b};\n}"
        : "=l"(out)
        : "l"(P), "n"(MASK));
    return out;
}
template <uint32_t MASK, uint32_t C>
__device__ __forceinline__ uint64_t field_xor(uint64_t P) {
    uint64_t out;
    asm("{\n .reg .b32 lo, hi, a, b;\n mov.b64 {lo, hi}, %1;\n"
        " lop3.b32 a, lo, %2, %3, 0x6A;\n lop3.b32 b, hi, %2, %3, 0x6A;\n"
        " mov.b64 %0, {a, b};\n}"
        : "=l"(out)
        : "l"(P), "n"(MASK), "n"(C));
    return out;
}
__host__ __device__ constexpr uint64_t pack2(uint32_t lo, uint32_t hi) { return ((uint64_t)hi << 32) | lo; }
__device__ __forceinline__ uint64_t packf(float v) {
    const uint32_t b = __float_as_uint(v);
    return pack2(b, b);
}
__device__ __forceinline__ float sum2(uint64_t v) {
    return __uint_as_float((uint32_t)v) + __uint_as_float((uint32_t)(v >> 32));
}
// 4-bit field at bit p of both words
__host__ __device__ constexpr uint64_t nib_mask(int p) { return (0xFull << p) | (0xFull << (p + 32)); }
__host__ __device__ constexpr uint64_t byte_mask(int p) { return (0xFFull << p) | (0xFFull << (p + 32)); }

__device__ __forceinline__ float half_bits_to_float(uint32_t h16) {
    return __half2float(__ushort_as_half((unsigned short)(h16 & 0xFFFFu)));
}
__device__ __forceinline__ float exp2_neg(int sh) { return __uint_as_float((uint32_t)(127 - sh) << 23); }

__device__ __forceinline__ float silu(float v) { return v / (1.0f + __expf(-v)); }

// ─────────────── Q4_K scale/min table of one superblock header ───────────────
// header words: h.x = d | dmin<<16, h.y = scales[0..3], h.z = scales[4..7], h.w = scales[8..11].
// Byte j of sl/ml = scale/min of sub-block j (j<4); byte j of sh/mh = those of sub-block j+4
// (get_scale_min_k4, crates/engine/src/forward.rs:359-369).
struct Q4KScales {
    uint32_t sl, ml, sh, mh;
};
__device__ __forceinline__ Q4KScales q4k_unpack_scales(uint32_t hy, uint32_t hz, uint32_t hw) {
    Q4KScales s;
    s.sl = hy & 0x3F3F3F3Fu;
    s.ml = hz & 0x3F3F3F3Fu;
    s.sh = (hw & 0x0F0F0F0Fu) | ((hy >> 2) & 0x30303030u);
    s.mh = ((hw >> 4) & 0x0F0F0F0Fu) | ((hz >> 2) & 0x30303030u);
    return s;
}
__device__ __forceinline__ float byte_to_float(uint32_t w, int j) {
    return (float)((w >> (8 * j)) & 0xFFu);
}

// ─────────────── activation layout: permutation and pre-scale per format ───────────────
// pos8: within a group of 8 elements the stored order is e0,e4,e1,e5,e2,e6,e3,e7 (pairs that sit
// at the same byte position of two consecutive weight words).
__device__ __forceinline__ int pos8(int t) { return t < 4 ? 2 * t : 2 * (t - 4) + 1; }

// Q4_K, element l (0..31) of a sub-block, hi = second half of the 64-element pair: byte l%4 of
// its word.  Low nibbles sit at bit 8b (b==3: bit 12 of P>>12); high nibbles at bit 8b+4
// (b==2,3: bits 8,16 of P>>12).
__device__ __forceinline__ int q4k_shift(int b, bool hi) {
    return hi ? (b == 0 ? 4 : (b == 1 ? 12 : (b == 2 ? 8 : 16))) : (b == 0 ? 0 : (b == 1 ? 8 : (b == 2 ? 16 : 12)));
}
// Q4_0, element e (0..31) of a block: byte i=e/2, nibble h=e%2, byte position b=i%4 of its
// (realigned) word: field at bit 8b+4h, fields above bit 16 taken from P>>12.
__device__ __forceinline__ int q4_0_shift(int b, int h) {
    const int p = 8 * b + 4 * h;
    return p <= 16 ? p : p - 12;
}
// Q8_0, byte position b of the word: bits 0 / 8 of P (b = 0, 1) or of P>>16 (b = 2, 3).
__device__ __forceinline__ int q8_0_shift(int b) { return (b & 1) ? 8 : 0; }

}  // namespace runit
