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

// Bit pattern of max |v| over a block of 32 activations held by LPB lanes with EPL values each; a NaN or an Inf anywhere
// in the block gives a pattern with exponent 255 (fmaxf alone would drop a NaN).  The 0 * v products are exact zeros for
// finite v and NaN otherwise; the cross-lane maximum is taken on the bit patterns, which order like the magnitudes.
template <int EPL, int LPB>
__device__ __forceinline__ uint32_t block_max_bits(const float (&v)[EPL]) {
    float m = 0.f, z = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; i++) {
        m = fmaxf(m, fabsf(v[i]));
        z = fmaf(v[i], 0.f, z);
    }
    uint32_t mb = __float_as_uint(fabsf(m + z));
#pragma unroll
    for (int o = 1; o < LPB; o <<= 1) mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, o));
    return mb;
}

// Layout of the prepared activations of one unit (in place of the raw f32 slice):
//   block b (32 elements), limb l: 32 bytes at b*96 + l*32;  then scale[NB] (f32) and vsum[NB] (i32).
template <int NB>
struct IntX {
    static constexpr int LIMBS = 0, SCALE = NB * 96, VSUM = NB * 96 + NB * 4, BYTES = NB * 96 + NB * 8;
};

// Quantise this lane's EPL consecutive elements v[] (block of 32 = 32/EPL lanes) and store limbs, scale, sum.
//   ORDER 0: natural element order inside the block; ORDER 1 (Q4_0): even elements first, then odd ones.
//   LIMBS 3: 23-bit integers (the text above).  LIMBS 2: 16-bit integers in two signed bytes, |q| <= 127 * 256 + 127 (the
//   top sliver of a binade takes half the scale): activations rounded to 2^-16 .. 2^-15 of their block maximum, a third
//   fewer dp4a and shared-memory reads; the third limb's 32 bytes stay unused.
template <int EPL, int NB, int ORDER, int LIMBS = 3>
__device__ __forceinline__ void prep_int_block(uint8_t* xq, const float (&v)[EPL], int lane) {
    constexpr int LPB = 32 / EPL;                 // lanes per block
    const uint32_t mb = block_max_bits<EPL, LPB>(v);
    const float m = __uint_as_float(mb);
    (void)m;
    const uint32_t e = mb >> 23;                  // biased exponent of the block maximum (255: a non-finite activation)
    const bool live = e >= 22u && e < 255u;       // zero / denormal-tiny blocks contribute nothing
    const uint32_t sh = (LIMBS == 2 && live && m * __uint_as_float((268u - e) << 23) > 32639.0f) ? 1u : 0u;
    const float inv = live ? __uint_as_float(((LIMBS == 2 ? 268u - sh : 275u) - e) << 23) : 0.f;     // 2^22 (2^14) / 2^(e-126)
    // a block that holds an Inf or a NaN gets a NaN scale: every row's sum becomes NaN, as a non-finite activation
    // does (to +-Inf or NaN) in the reference's f32 multiply-add chain
    const float scale = live ? __uint_as_float((e - (LIMBS == 2 ? 14u - sh : 21u)) << 23)
                             : (e == 255u ? __uint_as_float(0x7FC00000u) : 0.f);    // 1 / inv
    int a0[EPL], a1[EPL], a2[EPL], vs = 0;
#pragma unroll
    for (int i = 0; i < EPL; i++) {
        const int q = live ? __float2int_rn(v[i] * inv) : 0;   // exact product, one rounding; |q| < 2^22 (2^15)
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
            for (int l = 0; l < LIMBS; l++) {
                const int* a = l == 0 ? a0 : (l == 1 ? a1 : a2);
                uint2 w;
                w.x = pack4(a[0], a[1], a[2], a[3]);
                w.y = pack4(a[4], a[5], a[6], a[7]);
                *reinterpret_cast<uint2*>(base + l * 32 + t * 8) = w;
            }
        } else {
#pragma unroll
            for (int l = 0; l < LIMBS; l++) {
                const int* a = l == 0 ? a0 : (l == 1 ? a1 : a2);
                *reinterpret_cast<uint32_t*>(base + l * 32 + t * 4) = pack4(a[0], a[2], a[4], a[6]);        // even elements
                *reinterpret_cast<uint32_t*>(base + l * 32 + 16 + t * 4) = pack4(a[1], a[3], a[5], a[7]);   // odd elements
            }
        }
    } else {   // EPL == 4 (Q8_0)
#pragma unroll
        for (int l = 0; l < LIMBS; l++) {
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
            int s0 = 0, s1 = 0;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const uint4 l0 = xl[h], l1 = xl[2 + h];
                const uint32_t x0[4] = {l0.x, l0.y, l0.z, l0.w}, x1[4] = {l1.x, l1.y, l1.z, l1.w};
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const int wi = s + 4 * h + c;
                    const uint32_t Q = ((o0 + 2) & 2) ? __funnelshift_r(w[wi], w[wi + 1], 16) : w[wi];
                    s0 = dp4a_ss(Q, x0[c], s0);
                    s1 = dp4a_ss(Q, x1[c], s1);
                }
            }
            // two limbs (16-bit activations): |s1 * 256 + s0| <= 32 * 127 * 32639 < 2^28, exact in int32
            acc += (d * sx[blk]) * (float)(s1 * 256 + s0);
        }
    }
    return acc;
}

// ───────────────────────── integer tensor-core path (batch 1, 4-bit formats) ─────────────────────────
// The dp4a path above still issues ~2.9 instructions per weight and lane, which holds the largest matrices at ~0.75 of
// the HBM rate.  Here a warp's 32 rows x 256 K unit goes through mma.sync.m16n8k32 (u8 x s8 -> s32): one MMA = 16 rows x
// one 32-element block, the nibbles are its A operand after one mask, and the MMA's eight columns carry FOUR blocks at
// once: the activations are 16-bit block-fixed-point numbers q = 256 hi + lo (two signed bytes), the lane group that
// feeds column c supplies limb c&1 of block c>>1 of the current group of four blocks and zeros in the other three MMAs
// of the group, so the four MMAs accumulate into one register tile whose column pair (2t, 2t+1) holds the (hi, lo) dot
// products of the group's t-th block.  Lane (g, t) then owns the scales of two blocks of rows g and g+8: one conversion
// and two FMAs per row and block, about one instruction per weight and lane in total.
// Deviation from the exact product: the activations are rounded to 2^-16 .. 2^-15 of their block maximum (power-of-two
// block scale); the integer sums are exact.

template <int NB>
struct MmaX {   // prepared activations of one unit: per block 32 high bytes + 32 low bytes, then scale[NB], scale*sum(q)[NB]
    static constexpr int SCALE = NB * 64, SUM = NB * 64 + NB * 4, BYTES = NB * 64 + NB * 8;
};

// Quantise this lane's 8 consecutive elements (4 lanes per 32-block).  Blocks >= nblk (past the end of K) become zeros.
//   ORDER 0 (Q4_K): a lane's 8 bytes are its elements in order (K slots 4t..4t+3 and 16+4t..16+4t+3 of the MMA are
//   the elements 8t..8t+7).  ORDER 1 (Q4_0): even elements first (low nibbles of the lane's weight word), then odd.
template <int NB, int ORDER>
__device__ __forceinline__ void prep_mma_block(uint8_t* xq, float (&v)[8], int lane, int nblk) {
    const int blk = lane >> 2, t = lane & 3;
    const uint32_t mb = block_max_bits<8, 4>(v);
    const float m = __uint_as_float(mb);
    // Power-of-two scale (scaling is exact, small-integer activations stay exact): m in [2^e, 2^(e+1)) maps to
    // |q| < 2^15; the two signed bytes reach 127 * 256 + 127 = 32639, so the top sliver of a binade takes half the scale.
    const uint32_t eb = mb >> 23;                                 // biased exponent of the block maximum (255: non-finite)
    const bool live = blk < nblk && eb >= 20u && eb < 255u;       // zero or denormal-tiny blocks contribute nothing
    const uint32_t sh = live && m * __uint_as_float((268u - eb) << 23) > 32639.0f ? 1u : 0u;
    const float inv = live ? __uint_as_float((268u - eb - sh) << 23) : 0.f;     // 2^(14 - e - sh)
    // a block that holds an Inf or a NaN gets a NaN scale (and a NaN scale * sum): every row's result becomes NaN, as a
    // non-finite activation does (to +-Inf or NaN) in the reference's f32 multiply-add chain
    const float scale = live ? __uint_as_float((eb - 14u + sh) << 23)           // 1 / inv
                             : ((blk < nblk && eb == 255u) ? __uint_as_float(0x7FC00000u) : 0.f);
    uint32_t q[8], qa[8];
    int vs = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int qi = live ? __float2int_rn(v[i] * inv) : 0;
        vs += qi;
        q[i] = (uint32_t)qi;            // low limb = byte 0 as a signed byte
        qa[i] = (uint32_t)(qi + 128);   // high limb = (q - low) >> 8 = byte 1 of q + 128
    }
    vs += __shfl_xor_sync(0xffffffffu, vs, 1);
    vs += __shfl_xor_sync(0xffffffffu, vs, 2);
    auto pack_b0 = [](uint32_t x0, uint32_t x1, uint32_t x2, uint32_t x3) -> uint32_t {
        return __byte_perm(__byte_perm(x0, x1, 0x0040), __byte_perm(x2, x3, 0x0040), 0x5410);
    };
    auto pack_b1 = [](uint32_t x0, uint32_t x1, uint32_t x2, uint32_t x3) -> uint32_t {
        return __byte_perm(__byte_perm(x0, x1, 0x0051), __byte_perm(x2, x3, 0x0051), 0x5410);
    };
    uint2 hi, lo;
    if (ORDER == 0) {
        hi = make_uint2(pack_b1(qa[0], qa[1], qa[2], qa[3]), pack_b1(qa[4], qa[5], qa[6], qa[7]));
        lo = make_uint2(pack_b0(q[0], q[1], q[2], q[3]), pack_b0(q[4], q[5], q[6], q[7]));
    } else {
        hi = make_uint2(pack_b1(qa[0], qa[2], qa[4], qa[6]), pack_b1(qa[1], qa[3], qa[5], qa[7]));
        lo = make_uint2(pack_b0(q[0], q[2], q[4], q[6]), pack_b0(q[1], q[3], q[5], q[7]));
    }
    *reinterpret_cast<uint2*>(xq + blk * 64 + t * 8) = hi;
    *reinterpret_cast<uint2*>(xq + blk * 64 + 32 + t * 8) = lo;
    if (t == 0) {
        reinterpret_cast<float*>(xq + MmaX<NB>::SCALE)[blk] = scale;
        reinterpret_cast<float*>(xq + MmaX<NB>::SUM)[blk] = scale * (float)vs;
    }
}

// c += A (16 rows x 32 K, unsigned bytes) x B (32 K x 8 columns, signed bytes)
__device__ __forceinline__ void mma_u8s8_acc(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// B fragments of one unit for this lane: limb g&1 of the (g>>1)-th block of each of the two groups of four blocks, kept
// only in the MMA whose index equals g>>1.  INTERLEAVED = false: group r holds blocks 4r..4r+3 (Q4_0);
// true: group 0 holds the even blocks, group 1 the odd ones (Q4_K: low-nibble and high-nibble halves of the four chunks).
struct MmaB {
    uint32_t b[2][4][2];
};
template <bool INTERLEAVED>
__device__ __forceinline__ MmaB load_mma_b(const uint8_t* xq, int g, int t) {
    MmaB r;
    const uint32_t sel = (uint32_t)g >> 1;
#pragma unroll
    for (int grp = 0; grp < 2; grp++) {
        const uint32_t blk = INTERLEAVED ? 2 * sel + grp : 4 * grp + sel;
        const uint2 w = *reinterpret_cast<const uint2*>(xq + blk * 64 + (g & 1) * 32 + 8 * t);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t mask = sel == (uint32_t)i ? 0xFFFFFFFFu : 0u;
            r.b[grp][i][0] = w.x & mask;
            r.b[grp][i][1] = w.y & mask;
        }
    }
    return r;
}

// One Q4_K superblock of 32 rows (wb = the warp's box, row pitch 144): formula of
// crates/kernels/shaders/gemv_q4k.metal:85-122.  Chunk ch (32 bytes) holds elements 64ch..64ch+31 in its low nibbles
// (scale/min index ch) and 64ch+32..64ch+63 in its high nibbles (scale/min index ch+4): the low-nibble MMAs of the four
// chunks form one group, the high-nibble ones the other, so lane (g, t) ends up with scale indices t and t+4.
// acc[2*mt + h] += partial dot product of row 16*mt + g + 8*h (the four lanes of a row group are added after the K loop).
__device__ __forceinline__ void unit_q4k_mma(const uint8_t* wb, const uint8_t* xq, int lane, float (&acc)[4]) {
    const int g = lane >> 2, t = lane & 3;
    const float2 xs = reinterpret_cast<const float2*>(xq + MmaX<8>::SCALE)[t];   // activation blocks 2t (low) and 2t+1 (high)
    const float2 sx = reinterpret_cast<const float2*>(xq + MmaX<8>::SUM)[t];
    const MmaB B = load_mma_b<true>(xq, g, t);
    const uint32_t sel = 0x4440u | (uint32_t)t;            // byte t of a word, zero-extended
#pragma unroll
    for (int mt = 0; mt < 2; mt++) {
        const uint8_t* r0 = wb + (mt * 16 + g) * 144;
        const uint8_t* r1 = r0 + 8 * 144;
        int c[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
#pragma unroll
        for (int ch = 0; ch < 4; ch++) {
            const uint2 w0 = *reinterpret_cast<const uint2*>(r0 + 16 + 32 * ch + 8 * t);
            const uint2 w1 = *reinterpret_cast<const uint2*>(r1 + 16 + 32 * ch + 8 * t);
            mma_u8s8_acc(c[0], w0.x & 0x0F0F0F0Fu, w1.x & 0x0F0F0F0Fu, w0.y & 0x0F0F0F0Fu, w1.y & 0x0F0F0F0Fu, B.b[0][ch][0], B.b[0][ch][1]);
            // high nibbles stay in place: the MMA sees 16 * nibble, undone in the scale
            mma_u8s8_acc(c[1], w0.x & 0xF0F0F0F0u, w1.x & 0xF0F0F0F0u, w0.y & 0xF0F0F0F0u, w1.y & 0xF0F0F0F0u, B.b[1][ch][0], B.b[1][ch][1]);
        }
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint4 hd = *reinterpret_cast<const uint4*>(h ? r1 : r0);
            const float d = half_bits_to_float(hd.x), dmin = half_bits_to_float(hd.x >> 16);
            // 6-bit scales and mins with indices t and t+4 (get_scale_min_k4, crates/engine/src/forward.rs:359-369)
            const uint32_t sa = __byte_perm(hd.y, 0u, sel), sb = __byte_perm(hd.z, 0u, sel), sc = __byte_perm(hd.w, 0u, sel);
            const float sc_lo = (float)(sa & 63u), m_lo = (float)(sb & 63u);
            const float sc_hi = (float)((sc & 15u) | ((sa >> 2) & 0x30u)), m_hi = (float)((sc >> 4) | ((sb >> 2) & 0x30u));
            const float v0 = (float)(c[0][2 * h] * 256 + c[0][2 * h + 1]), v1 = (float)(c[1][2 * h] * 256 + c[1][2 * h + 1]);
            float s = acc[2 * mt + h];
            s = fmaf(v0, (d * sc_lo) * xs.x, s);
            s = fmaf(-(dmin * m_lo), sx.x, s);
            s = fmaf(v1, (d * 0.0625f * sc_hi) * xs.y, s);
            s = fmaf(-(dmin * m_hi), sx.y, s);
            acc[2 * mt + h] = s;
        }
    }
}

// Eight Q4_0 blocks of 32 rows: formula of crates/kernels/shaders/gemv_q4_0.metal:26-49 (low nibble = even element).
__device__ __forceinline__ void unit_q4_0_mma(const uint8_t* wb, const uint8_t* xq, int lane, int nblk, float (&acc)[4]) {
    const int g = lane >> 2, t = lane & 3;
    const float* xsc = reinterpret_cast<const float*>(xq + MmaX<8>::SCALE);
    const float* xsm = reinterpret_cast<const float*>(xq + MmaX<8>::SUM);
    const MmaB B = load_mma_b<false>(xq, g, t);
#pragma unroll
    for (int mt = 0; mt < 2; mt++) {
        const uint8_t* r0 = wb + (mt * 16 + g) * 144;
        const uint8_t* r1 = r0 + 8 * 144;
#pragma unroll
        for (int grp = 0; grp < 2; grp++) {
            int c[4] = {0, 0, 0, 0};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                // block b sits at byte 18b of the row: f16 scale, then 16 bytes of nibbles; for even b the nibble words
                // straddle aligned words by two bytes
                const int b = 4 * grp + i;
                uint32_t w0, w1;
                if ((b & 1) == 0) {
                    const uint32_t* p0 = reinterpret_cast<const uint32_t*>(r0 + 18 * b) + t;
                    const uint32_t* p1 = reinterpret_cast<const uint32_t*>(r1 + 18 * b) + t;
                    w0 = __funnelshift_r(p0[0], p0[1], 16);
                    w1 = __funnelshift_r(p1[0], p1[1], 16);
                } else {
                    w0 = reinterpret_cast<const uint32_t*>(r0 + 18 * b + 2)[t];
                    w1 = reinterpret_cast<const uint32_t*>(r1 + 18 * b + 2)[t];
                }
                mma_u8s8_acc(c, w0 & 0x0F0F0F0Fu, w1 & 0x0F0F0F0Fu, (w0 >> 4) & 0x0F0F0F0Fu, (w1 >> 4) & 0x0F0F0F0Fu, B.b[grp][i][0],
                             B.b[grp][i][1]);
            }
            const int blk = 4 * grp + t;
            if (blk < nblk) {
                const float xs = xsc[blk], sx = xsm[blk];
                const float d0 = __half2float(*reinterpret_cast<const __half*>(r0 + 18 * blk));
                const float d1 = __half2float(*reinterpret_cast<const __half*>(r1 + 18 * blk));
                const float v0 = (float)(c[0] * 256 + c[1]), v1 = (float)(c[2] * 256 + c[3]);
                acc[2 * mt] = fmaf(v0, d0 * xs, fmaf(-8.0f * d0, sx, acc[2 * mt]));       // sum d (q - 8) x
                acc[2 * mt + 1] = fmaf(v1, d1 * xs, fmaf(-8.0f * d1, sx, acc[2 * mt + 1]));
            }
        }
    }
}

}  // namespace runit
