// Integer dot-product path of the fused-dequant GEMV (batch 1).
//
// Measured on B200: lop3 / shf / cvt issue on one pipe at 64 lanes/clk/SM, while fma.f32x2, add.f32x2 and
// dp4a issue on the other at 64 instructions/clk/SM.  The float path (gemv_kernels.cuh) spends one lop3 plus
// half an add.f32x2 and half an fma.f32x2 per weight and is bound by issue slots below the HBM rate.  Here the
// activations of a 32-element block are turned, once per stage, into a 24-bit block-fixed-point number
// x ~ v * 2^s (|v| < 2^22, s from the block maximum rounded up to a power of two, so x*2^-s is exact before the
// one rounding to integer) and split into three signed 8-bit limbs v = a0 + 256 a1 + 65536 a2.  The weight
// nibbles of a word are separated with three logic ops per 8 weights and multiplied with dp4a: 0.75 dp4a per
// weight, integer accumulation (exact), one int->float conversion per 32 weights, scales applied in f32.
// The only deviation from the f32 product is the rounding of x to 2^-22 of its block maximum — the size of
// the rounding error of an f32 accumulation — so results stay within a few 1e-7 of an f64 evaluation of the same sums.
#pragma once

#include "gemv_common.cuh"

namespace runit {

__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {   // signed x signed
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {   // unsigned bytes of a x signed bytes of b
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Layout of the prepared activations of one unit (in place of the raw f32 slice):
//   block b (32 elements), limb l: 32 bytes at b*96 + l*32;  then scale[NB] (f32) and vsum[NB] (i32).
template <int NB>
struct IntX {
    static constexpr int LIMBS = 0, SCALE = NB * 96, VSUM = NB * 96 + NB * 4, BYTES = NB * 96 + NB * 8;
};

// Quantise this lane's EPL consecutive elements v[] (block of 32 = 32/EPL lanes) and store limbs, scale, sum.
//   ORDER 0: natural element order inside the block; ORDER 1 (Q4_0): even elements first, then odd ones.
template <int EPL, int NB, int ORDER>
__device__ __forceinline__ void prep_int_block(uint8_t* xq, const float (&v)[EPL], int lane) {
    constexpr int LPB = 32 / EPL;                 // lanes per block
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; i++) m = fmaxf(m, fabsf(v[i]));
#pragma unroll
    for (int o = 1; o < LPB; o <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const uint32_t e = __float_as_uint(m) >> 23;  // biased exponent of the block maximum
    const bool live = e >= 22u && e < 255u;       // zero / denormal-tiny (or non-finite) blocks contribute nothing
    const float inv = live ? __uint_as_float((275u - e) << 23) : 0.f;     // 2^22 / 2^(e-126)
    const float scale = live ? __uint_as_float((e - 21u) << 23) : 0.f;    // 2^(e-126) / 2^22
    int a0[EPL], a1[EPL], a2[EPL], vs = 0;
#pragma unroll
    for (int i = 0; i < EPL; i++) {
        const int q = __float2int_rn(v[i] * inv);   // exact product, one rounding; |q| < 2^22
        vs += q;
        a0[i] = (int)(int8_t)q;
        const int q1 = (q - a0[i]) >> 8;
        a1[i] = (int)(int8_t)q1;
        a2[i] = (q1 - a1[i]) >> 8;
    }
#pragma unroll
    for (int o = 1; o < LPB; o <<= 1) vs += __shfl_xor_sync(0xffffffffu, vs, o);
    const int blk = lane / LPB, t = lane % LPB;
    uint8_t* base = xq + blk * 96;
    auto pack4 = [](int x0, int x1, int x2, int x3) -> uint32_t {
        return __byte_perm(__byte_perm((uint32_t)x0, (uint32_t)x1, 0x0040), __byte_perm((uint32_t)x2, (uint32_t)x3, 0x0040), 0x5410);
    };
    if (EPL == 8) {
        if (ORDER == 0) {
#pragma unroll
            for (int l = 0; l < 3; l++) {
                const int* a = l == 0 ? a0 : (l == 1 ? a1 : a2);
                uint2 w;
                w.x = pack4(a[0], a[1], a[2], a[3]);
                w.y = pack4(a[4], a[5], a[6], a[7]);
                *reinterpret_cast<uint2*>(base + l * 32 + t * 8) = w;
            }
        } else {
#pragma unroll
            for (int l = 0; l < 3; l++) {
                const int* a = l == 0 ? a0 : (l == 1 ? a1 : a2);
                *reinterpret_cast<uint32_t*>(base + l * 32 + t * 4) = pack4(a[0], a[2], a[4], a[6]);        // even elements
                *reinterpret_cast<uint32_t*>(base + l * 32 + 16 + t * 4) = pack4(a[1], a[3], a[5], a[7]);   // odd elements
            }
        }
    } else {   // EPL == 4 (Q8_0)
#pragma unroll
        for (int l = 0; l < 3; l++) {
            const int* a = l == 0 ? a0 : (l == 1 ? a1 : a2);
            *reinterpret_cast<uint32_t*>(base + l * 32 + t * 4) = pack4(a[0], a[1], a[2], a[3]);
        }
    }
    if (t == 0) {
        reinterpret_cast<float*>(xq + IntX<NB>::SCALE)[blk] = scale;
        reinterpret_cast<int*>(xq + IntX<NB>::VSUM)[blk] = vs;
    }
}

// 32 weights (8 words of unsigned 4-bit values in bytes) x one activation block: sum q*v as an int.
__device__ __forceinline__ int dot32_u4(const uint32_t (&q)[8], const uint8_t* xblk) {
    const uint4* xl = reinterpret_cast<const uint4*>(xblk);
    int s0[2] = {0, 0}, s1[2] = {0, 0}, s2[2] = {0, 0};   // one accumulator set per 16-byte half: short chains
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const uint4 l0 = xl[h], l1 = xl[2 + h], l2 = xl[4 + h];
        const uint32_t x0[4] = {l0.x, l0.y, l0.z, l0.w}, x1[4] = {l1.x, l1.y, l1.z, l1.w}, x2[4] = {l2.x, l2.y, l2.z, l2.w};
#pragma unroll
        for (int c = 0; c < 4; c++) {
            s0[h] = dp4a_us(q[4 * h + c], x0[c], s0[h]);
            s1[h] = dp4a_us(q[4 * h + c], x1[c], s1[h]);
            s2[h] = dp4a_us(q[4 * h + c], x2[c], s2[h]);
        }
    }
    return (s0[0] + s0[1]) + ((s1[0] + s1[1]) << 8) + ((s2[0] + s2[1]) << 16);   // |sum| <= 15 * 32 * 2^22 < 2^31
}

// One Q4_K superblock: formula of crates/kernels/shaders/gemv_q4k.metal:85-122.
__device__ __forceinline__ float unit_q4k_i8(const uint8_t* up, const uint8_t* xq) {
    const uint4* u = reinterpret_cast<const uint4*>(up);
    const uint4 h = u[0];
    const float d = half_bits_to_float(h.x), dmin = half_bits_to_float(h.x >> 16);
    const Q4KScales s = q4k_unpack_scales(h.y, h.z, h.w);
    const float* sx = reinterpret_cast<const float*>(xq + IntX<8>::SCALE);
    const int* sv = reinterpret_cast<const int*>(xq + IntX<8>::VSUM);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const uint4 qa = u[1 + 2 * j], qb = u[2 + 2 * j];
        const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
        uint32_t lo[8], hi[8];
#pragma unroll
        for (int c = 0; c < 8; c++) {
            lo[c] = w[c] & 0x0F0F0F0Fu;
            hi[c] = (w[c] >> 4) & 0x0F0F0F0Fu;
        }
        const int sl = dot32_u4(lo, xq + (2 * j) * 96), sh = dot32_u4(hi, xq + (2 * j + 1) * 96);
        const float xl = sx[2 * j], xh = sx[2 * j + 1];
        const float dl = d * (float)((s.sl >> (8 * j)) & 0xFFu), ml = dmin * (float)((s.ml >> (8 * j)) & 0xFFu);
        const float dh = d * (float)((s.sh >> (8 * j)) & 0xFFu), mh = dmin * (float)((s.mh >> (8 * j)) & 0xFFu);
        acc += xl * (dl * (float)sl - ml * (float)sv[2 * j]) + xh * (dh * (float)sh - mh * (float)sv[2 * j + 1]);
    }
    return acc;
}

// Eight Q4_0 blocks: formula of crates/kernels/shaders/gemv_q4_0.metal:26-49 (low nibble = even element).
__device__ __forceinline__ float unit_q4_0_i8(const uint8_t* up, const uint8_t* xq, int nblk) {
    const uint4* u4 = reinterpret_cast<const uint4*>(up);
    uint32_t w[36];
#pragma unroll
    for (int i = 0; i < 9; i++) {
        const uint4 q = u4[i];
        w[4 * i] = q.x; w[4 * i + 1] = q.y; w[4 * i + 2] = q.z; w[4 * i + 3] = q.w;
    }
    const float* sx = reinterpret_cast<const float*>(xq + IntX<8>::SCALE);
    const int* sv = reinterpret_cast<const int*>(xq + IntX<8>::VSUM);
    float acc = 0.f;
#pragma unroll
    for (int blk = 0; blk < 8; blk++) {
        if (blk < nblk) {
            const int o0 = 18 * blk, s = (o0 + 2) >> 2;
            const uint32_t dw = w[o0 >> 2];
            const float d = half_bits_to_float((o0 & 2) ? (dw >> 16) : dw);
            uint32_t q[8];   // q[0..3]: even elements (low nibbles) of the 4 quant words, q[4..7]: odd elements
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t Q = ((o0 + 2) & 2) ? __funnelshift_r(w[s + i], w[s + i + 1], 16) : w[s + i];
                q[i] = Q & 0x0F0F0F0Fu;
                q[4 + i] = (Q >> 4) & 0x0F0F0F0Fu;
            }
            const int sq = dot32_u4(q, xq + blk * 96);
            acc += (d * sx[blk]) * (float)(sq - 8 * sv[blk]);   // sum (q-8) v
        }
    }
    return acc;
}

// Four Q8_0 blocks: formula of crates/kernels/shaders/gemv_q8_0.metal:24-36.
__device__ __forceinline__ float unit_q8_0_i8(const uint8_t* up, const uint8_t* xq, int nblk) {
    const uint2* u2 = reinterpret_cast<const uint2*>(up);
    uint32_t w[34];
#pragma unroll
    for (int i = 0; i < 17; i++) {
        const uint2 q = u2[i];
        w[2 * i] = q.x; w[2 * i + 1] = q.y;
    }
    const float* sx = reinterpret_cast<const float*>(xq + IntX<4>::SCALE);
    float acc = 0.f;
#pragma unroll
    for (int blk = 0; blk < 4; blk++) {
        if (blk < nblk) {
            const int o0 = 34 * blk, s = (o0 + 2) >> 2;
            const uint32_t dw = w[o0 >> 2];
            const float d = half_bits_to_float((o0 & 2) ? (dw >> 16) : dw);
            const uint4* xl = reinterpret_cast<const uint4*>(xq + blk * 96);
            int s0 = 0, s1 = 0, s2 = 0;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const uint4 l0 = xl[h], l1 = xl[2 + h], l2 = xl[4 + h];
                const uint32_t x0[4] = {l0.x, l0.y, l0.z, l0.w}, x1[4] = {l1.x, l1.y, l1.z, l1.w}, x2[4] = {l2.x, l2.y, l2.z, l2.w};
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const int wi = s + 4 * h + c;
                    const uint32_t Q = ((o0 + 2) & 2) ? __funnelshift_r(w[wi], w[wi + 1], 16) : w[wi];
                    s0 = dp4a_ss(Q, x0[c], s0);
                    s1 = dp4a_ss(Q, x1[c], s1);
                    s2 = dp4a_ss(Q, x2[c], s2);
                }
            }
            // |q| up to 127: the limb sums are combined in f32 (each is exact, < 2^20)
            acc += (d * sx[blk]) * fmaf(65536.f, (float)s2, fmaf(256.f, (float)s1, (float)s0));
        }
    }
    return acc;
}

}  // namespace runit
