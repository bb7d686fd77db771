/*
 * runit_oracle.c — CPU oracle for the quantized decode path (TEST INFRASTRUCTURE ONLY).
 *
 * See runit_oracle.h for the role of this file and for the statement that parity for
 * the quantized operators is UNPINNED (the reference holds no golden vectors for them).
 * Paths in the citations are relative to the reference project root.
 *
 * Build: see the Makefile beside this file (-ffp-contract=off keeps the f32 tiers
 * bit-reproducible across host CPUs).
 */
#include "runit_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ───────────────────────── threads ───────────────────────── */

int ro_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void ro_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ───────────────────────── f16 <-> f32 ─────────────────────────
 * IEEE binary16, round-to-nearest-even: what the `half` crate (Cargo.lock:725-726,
 * v2.7.1) and Metal's half() conversions do. */

float ro_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { man <<= 1; e++; } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t ro_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((absx > 0x7F800000u) ? 0x200u : 0u));
    }
    if (absx >= 0x477FF000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (absx < 0x33000001u) { /* <= 2^-25 rounds to zero (tie to even = 0) */
        return (uint16_t)sign;
    }
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t m = (absx & 0x7FFFFFu) | 0x800000u;
    uint32_t shift, half_bits;
    if (e < -14) { /* subnormal half */
        shift = (uint32_t)(13 + (-14 - e));
        half_bits = 0;
    } else {
        shift = 13;
        half_bits = (uint32_t)(e + 15) << 10;
        m &= 0x7FFFFFu;
    }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) q++;
    return (uint16_t)(sign | (half_bits + q)); /* mantissa carry bumps the exponent */
}

void ro_f32_to_f16_array(const float* in, uint16_t* out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = ro_f32_to_f16(in[i]);
}

void ro_f16_to_f32_array(const uint16_t* in, float* out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = ro_f16_to_f32(in[i]);
}

static inline float rd_f16(const uint8_t* p) {
    return ro_f16_to_f32((uint16_t)(p[0] | ((uint16_t)p[1] << 8)));
}

/* ───────────────────────── block formats ─────────────────────────
 * crates/kernels/src/dispatch.rs:735-747; layouts: gemv_q8_0.metal:11-14,
 * gemv_q4_0.metal:10-15, dequant.metal:7-26. */

size_t ro_block_elems(int fmt) { return (fmt == RO_Q4K || fmt == RO_Q5K || fmt == RO_Q6K) ? 256 : 32; }
size_t ro_block_bytes(int fmt) {
    switch (fmt) {
        case RO_Q8_0: return 34;
        case RO_Q4_0: return 18;
        case RO_Q4K: return 144;
        case RO_Q5_0: return 22;    /* crates/engine/src/forward.rs:901-902 */
        case RO_Q5K: return 176;    /* forward.rs:980-981 */
        default: return 210;        /* Q6_K, forward.rs:921-922 */
    }
}
size_t ro_row_bytes(int fmt, int k) { return (size_t)k / ro_block_elems(fmt) * ro_block_bytes(fmt); }

/* crates/engine/src/forward.rs:359-369 == dequant.metal:42-51 == gemv_q4k.metal:22-34 */
void ro_q4k_get_scale_min(int j, const uint8_t* s, uint8_t* sc, uint8_t* m) {
    if (j < 4) {
        *sc = s[j] & 0x3F;
        *m = s[j + 4] & 0x3F;
    } else {
        *sc = (uint8_t)((s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4));
        *m = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

/* Tier DEQUANT row formulas.
 *   Q8_0: crates/engine/src/forward.rs:951-963   value = d * int8
 *   Q4_0: crates/engine/src/forward.rs:964-978   low nibble = element 2i, high = 2i+1
 *   Q4_K: crates/engine/src/forward.rs:1026-1057 low nibbles -> scale j, high -> j+4 */
void ro_dequant_row(int fmt, const uint8_t* row, int k, float* out) {
    if (fmt == RO_Q8_0) {
        int nb = k / 32;
        for (int b = 0; b < nb; b++) {
            const uint8_t* blk = row + (size_t)b * 34;
            float d = rd_f16(blk);
            for (int i = 0; i < 32; i++) out[b * 32 + i] = d * (float)(int8_t)blk[2 + i];
        }
    } else if (fmt == RO_Q4_0) {
        int nb = k / 32;
        for (int b = 0; b < nb; b++) {
            const uint8_t* blk = row + (size_t)b * 18;
            float d = rd_f16(blk);
            for (int i = 0; i < 16; i++) {
                uint8_t v = blk[2 + i];
                out[b * 32 + 2 * i] = d * (float)((int)(v & 0x0F) - 8);
                out[b * 32 + 2 * i + 1] = d * (float)((int)(v >> 4) - 8);
            }
        }
    } else if (fmt == RO_Q5_0) {
        /* crates/engine/src/forward.rs:900-919: {f16 d; u8 qh[4]; u8 qs[16]}; byte j holds elements j (low nibble) and
         * j + 16 (high nibble); their fifth bits are bit j%8 of qh[j/8] and of qh[j/8 + 2]; value = d * (q - 16) */
        int nb = k / 32;
        for (int b = 0; b < nb; b++) {
            const uint8_t* blk = row + (size_t)b * 22;
            float d = rd_f16(blk);
            const uint8_t* qh = blk + 2;
            const uint8_t* qs = blk + 6;
            for (int j = 0; j < 16; j++) {
                int xh0 = (qh[j / 8] >> (j % 8)) & 1, xh1 = (qh[j / 8 + 2] >> (j % 8)) & 1;
                int x0 = (qs[j] & 0x0F) | (xh0 << 4), x1 = (qs[j] >> 4) | (xh1 << 4);
                out[b * 32 + j] = d * (float)(x0 - 16);
                out[b * 32 + j + 16] = d * (float)(x1 - 16);
            }
        }
    } else if (fmt == RO_Q6K) {
        /* crates/engine/src/forward.rs:920-949: {u8 ql[128]; u8 qh[64]; i8 scales[16]; f16 d}; per half of 128 elements
         * the scale index is half/16 + {0, 2, 4, 6} for the four groups of 32 (for every l, as the reference has it) */
        int nb = k / 256;
        for (int b = 0; b < nb; b++) {
            const uint8_t* blk = row + (size_t)b * 210;
            const uint8_t* ql = blk;
            const uint8_t* qh = blk + 128;
            const int8_t* sc = (const int8_t*)(blk + 192);
            float d = rd_f16(blk + 208);
            float* o = out + (size_t)b * 256;
            for (int half = 0; half < 256; half += 128) {
                int is = half / 16;
                for (int l = 0; l < 32; l++) {
                    int a = ql[half / 2 + l], c = ql[half / 2 + l + 32], h = qh[half / 4 + l];
                    int q1 = ((a & 0x0F) | (((h >> 0) & 3) << 4)) - 32;
                    int q2 = ((c & 0x0F) | (((h >> 2) & 3) << 4)) - 32;
                    int q3 = ((a >> 4) | (((h >> 4) & 3) << 4)) - 32;
                    int q4 = ((c >> 4) | (((h >> 6) & 3) << 4)) - 32;
                    o[half + l] = d * (float)sc[is + 0] * (float)q1;
                    o[half + l + 32] = d * (float)sc[is + 2] * (float)q2;
                    o[half + l + 64] = d * (float)sc[is + 4] * (float)q3;
                    o[half + l + 96] = d * (float)sc[is + 6] * (float)q4;
                }
            }
        }
    } else if (fmt == RO_Q5K) {
        /* crates/engine/src/forward.rs:979-1012: {f16 d; f16 dmin; u8 scales[12]; u8 qh[32]; u8 qs[128]}; as Q4_K plus a
         * fifth bit per element: bit e%8 of qh[e/8] for element e */
        int nb = k / 256;
        for (int b = 0; b < nb; b++) {
            const uint8_t* blk = row + (size_t)b * 176;
            float d = rd_f16(blk), dmin = rd_f16(blk + 2);
            const uint8_t* sc = blk + 4;
            const uint8_t* qh = blk + 16;
            const uint8_t* qs = blk + 48;
            float* o = out + (size_t)b * 256;
            for (int j = 0; j < 4; j++) {
                uint8_t s_lo, m_lo, s_hi, m_hi;
                ro_q4k_get_scale_min(j, sc, &s_lo, &m_lo);
                ro_q4k_get_scale_min(j + 4, sc, &s_hi, &m_hi);
                float d_lo = d * (float)s_lo, m_lo2 = dmin * (float)m_lo;
                float d_hi = d * (float)s_hi, m_hi2 = dmin * (float)m_hi;
                for (int l = 0; l < 32; l++) {
                    uint8_t v = qs[j * 32 + l];
                    int e_lo = j * 64 + l, e_hi = j * 64 + l + 32;
                    int q_lo = (v & 0x0F) | (((qh[e_lo / 8] >> (e_lo % 8)) & 1) << 4);
                    int q_hi = (v >> 4) | (((qh[e_hi / 8] >> (e_hi % 8)) & 1) << 4);
                    o[e_lo] = d_lo * (float)q_lo - m_lo2;
                    o[e_hi] = d_hi * (float)q_hi - m_hi2;
                }
            }
        }
    } else {
        int nb = k / 256;
        for (int b = 0; b < nb; b++) {
            const uint8_t* blk = row + (size_t)b * 144;
            float d = rd_f16(blk), dmin = rd_f16(blk + 2);
            const uint8_t* sc = blk + 4;
            const uint8_t* qs = blk + 16;
            float* o = out + (size_t)b * 256;
            for (int j = 0; j < 4; j++) {
                uint8_t s_lo, m_lo, s_hi, m_hi;
                ro_q4k_get_scale_min(j, sc, &s_lo, &m_lo);
                ro_q4k_get_scale_min(j + 4, sc, &s_hi, &m_hi);
                float d_lo = d * (float)s_lo, m_lo2 = dmin * (float)m_lo;
                float d_hi = d * (float)s_hi, m_hi2 = dmin * (float)m_hi;
                for (int l = 0; l < 32; l++) {
                    uint8_t v = qs[j * 32 + l];
                    o[j * 64 + l] = d_lo * (float)(v & 0x0F) - m_lo2;
                    o[j * 64 + l + 32] = d_hi * (float)(v >> 4) - m_hi2;
                }
            }
        }
    }
}

/* crates/kernels/shaders/dequant.metal:53-98 — same values rounded to f16. */
void ro_dequant_q4k_f16(const uint8_t* in, uint16_t* out, size_t n_blocks) {
#pragma omp parallel for schedule(static)
    for (long b = 0; b < (long)n_blocks; b++) {
        float tmp[256];
        ro_dequant_row(RO_Q4K, in + (size_t)b * 144, 256, tmp);
        for (int i = 0; i < 256; i++) out[(size_t)b * 256 + i] = ro_f32_to_f16(tmp[i]);
    }
}

/* ───────────────────────── tier SHADER block dots ───────────────────────── */

/* crates/kernels/shaders/gemv_q8_0.metal:24-36 */
static inline void q8_0_block_dot(const uint8_t* blk, const float* x, float* acc) {
    float d = rd_f16(blk);
    const int8_t* qs = (const int8_t*)(blk + 2);
    for (int i = 0; i < 32; i += 4) {
        *acc += d * ((float)qs[i] * x[i] + (float)qs[i + 1] * x[i + 1] +
                     (float)qs[i + 2] * x[i + 2] + (float)qs[i + 3] * x[i + 3]);
    }
}

/* crates/kernels/shaders/gemv_q4_0.metal:26-49 */
static inline void q4_0_block_dot(const uint8_t* blk, const float* x, float* acc) {
    float d = rd_f16(blk);
    const uint8_t* qs = blk + 2;
    for (int i = 0; i < 16; i += 2) {
        uint8_t b0 = qs[i], b1 = qs[i + 1];
        *acc += d * ((float)((int)(b0 & 0x0F) - 8) * x[i * 2] +
                     (float)((int)(b0 >> 4) - 8) * x[i * 2 + 1] +
                     (float)((int)(b1 & 0x0F) - 8) * x[i * 2 + 2] +
                     (float)((int)(b1 >> 4) - 8) * x[i * 2 + 3]);
    }
}

/* crates/kernels/shaders/gemv_q4k.metal:85-122 */
static inline void q4k_block_dot(const uint8_t* blk, const float* x, float* acc) {
    float d = rd_f16(blk), dmin = rd_f16(blk + 2);
    const uint8_t* sc = blk + 4;
    const uint8_t* qs = blk + 16;
    for (int j = 0; j < 4; j++) {
        uint8_t s_lo, m_lo, s_hi, m_hi;
        ro_q4k_get_scale_min(j, sc, &s_lo, &m_lo);
        ro_q4k_get_scale_min(j + 4, sc, &s_hi, &m_hi);
        float d_lo = d * (float)s_lo, m_lo2 = dmin * (float)m_lo;
        float d_hi = d * (float)s_hi, m_hi2 = dmin * (float)m_hi;
        const float* xl = x + j * 64;
        const float* xh = x + j * 64 + 32;
        for (int i = 0; i < 32; i += 4) {
            uint8_t b0 = qs[j * 32 + i], b1 = qs[j * 32 + i + 1];
            uint8_t b2 = qs[j * 32 + i + 2], b3 = qs[j * 32 + i + 3];
            *acc += (d_lo * (float)(b0 & 0x0F) - m_lo2) * xl[i];
            *acc += (d_lo * (float)(b1 & 0x0F) - m_lo2) * xl[i + 1];
            *acc += (d_lo * (float)(b2 & 0x0F) - m_lo2) * xl[i + 2];
            *acc += (d_lo * (float)(b3 & 0x0F) - m_lo2) * xl[i + 3];
            *acc += (d_hi * (float)(b0 >> 4) - m_hi2) * xh[i];
            *acc += (d_hi * (float)(b1 >> 4) - m_hi2) * xh[i + 1];
            *acc += (d_hi * (float)(b2 >> 4) - m_hi2) * xh[i + 2];
            *acc += (d_hi * (float)(b3 >> 4) - m_hi2) * xh[i + 3];
        }
    }
}

/* One row in the lane partition of the Metal kernels.
 *   Q8_0: bpt = ceil(nb/32), lane l owns [l*bpt, min((l+1)*bpt, nb))   gemv_q8_0.metal:70-79
 *   Q4_0: same partition                                                gemv_q4_0.metal:92-100
 *   Q4_K: bpt = nb/32, lane 31 owns the remainder                       gemv_q4k.metal:140-148
 * Lane partial sums are added in lane order 0..31 (simd_sum's own order is unspecified). */
static float row_dot_shader(int fmt, const uint8_t* row, const float* x, int k) {
    int be = (int)ro_block_elems(fmt), bb = (int)ro_block_bytes(fmt);
    int nb = k / be;
    float lanes[32];
    for (int l = 0; l < 32; l++) {
        int s, e;
        if (fmt == RO_Q4K) {
            int bpt = nb / 32;
            s = l * bpt;
            e = (l == 31) ? nb : s + bpt;
        } else {
            int bpt = (nb + 31) / 32;
            s = l * bpt;
            e = s + bpt < nb ? s + bpt : nb;
        }
        float acc = 0.0f;
        for (int b = s; b < e; b++) {
            const uint8_t* blk = row + (size_t)b * bb;
            const float* xb = x + (size_t)b * be;
            if (fmt == RO_Q8_0) q8_0_block_dot(blk, xb, &acc);
            else if (fmt == RO_Q4_0) q4_0_block_dot(blk, xb, &acc);
            else q4k_block_dot(blk, xb, &acc);
        }
        lanes[l] = acc;
    }
    float r = 0.0f;
    for (int l = 0; l < 32; l++) r += lanes[l];
    return r;
}

int ro_gemv(int fmt, int tier, const uint8_t* w, const float* x, float* y, double* y64, int m,
            int k, int batch) {
    if (fmt < 0 || fmt > 5 || m < 0 || k <= 0 || batch <= 0) return -1;
    if (fmt > 2 && tier == RO_TIER_SHADER) return -1;   /* the reference has no shader for Q5_0 / Q5_K / Q6_K */
    if (k % (int)ro_block_elems(fmt)) return -1;
    size_t rb = ro_row_bytes(fmt, k);
#pragma omp parallel
    {
        float* deq = (tier == RO_TIER_SHADER) ? NULL : (float*)malloc(sizeof(float) * (size_t)k);
#pragma omp for schedule(static)
        for (long r = 0; r < m; r++) {
            const uint8_t* row = w + (size_t)r * rb;
            if (tier == RO_TIER_SHADER) {
                for (int b = 0; b < batch; b++) {
                    float v = row_dot_shader(fmt, row, x + (size_t)b * k, k);
                    y[(size_t)b * m + r] = v;
                    if (y64) y64[(size_t)b * m + r] = (double)v;
                }
            } else {
                ro_dequant_row(fmt, row, k, deq);
                for (int b = 0; b < batch; b++) {
                    const float* xb = x + (size_t)b * k;
                    if (tier == RO_TIER_DEQUANT) {
                        /* cpu_gemv: crates/kernels/src/dispatch.rs:1705-1709 */
                        float acc = 0.0f;
                        for (int c = 0; c < k; c++) acc += deq[c] * xb[c];
                        y[(size_t)b * m + r] = acc;
                        if (y64) y64[(size_t)b * m + r] = (double)acc;
                    } else {
                        double acc = 0.0;
                        for (int c = 0; c < k; c++) acc += (double)deq[c] * (double)xb[c];
                        y[(size_t)b * m + r] = (float)acc;
                        if (y64) y64[(size_t)b * m + r] = acc;
                    }
                }
            }
        }
        free(deq);
    }
    return 0;
}

/* crates/kernels/shaders/gemv.metal:82-106: lane l takes float4 groups l, l+32, ...; the
 * metal dot() of a 4-vector is evaluated here left to right; lanes summed 0..31. */
void ro_gemv_f16w_f32in(const uint16_t* w, const float* x, float* y, int m, int k) {
#pragma omp parallel for schedule(static)
    for (long r = 0; r < m; r++) {
        const uint16_t* a = w + (size_t)r * k;
        float lanes[32];
        int k4 = k >> 2;
        for (int l = 0; l < 32; l++) {
            float acc = 0.0f;
            for (int i = l; i < k4; i += 32) {
                acc += ro_f16_to_f32(a[4 * i]) * x[4 * i] + ro_f16_to_f32(a[4 * i + 1]) * x[4 * i + 1] +
                       ro_f16_to_f32(a[4 * i + 2]) * x[4 * i + 2] +
                       ro_f16_to_f32(a[4 * i + 3]) * x[4 * i + 3];
            }
            for (int i = (k4 << 2) + l; i < k; i += 32) acc += ro_f16_to_f32(a[i]) * x[i];
            lanes[l] = acc;
        }
        float s = 0.0f;
        for (int l = 0; l < 32; l++) s += lanes[l];
        y[r] = s;
    }
}

/* f32-weight router (the benchmark configuration asks for an f32 router); f64 accumulate. */
void ro_gemv_f32w(const float* w, const float* x, float* y, int m, int k) {
#pragma omp parallel for schedule(static)
    for (long r = 0; r < m; r++) {
        double acc = 0.0;
        for (int c = 0; c < k; c++) acc += (double)w[(size_t)r * k + c] * (double)x[c];
        y[r] = (float)acc;
    }
}

/* ───────────────────────── MoE glue ───────────────────────── */

/* crates/kernels/shaders/fused_ffn.metal:24-26, activation.metal:140-167,
 * crates/kernels/src/dispatch.rs:1684-1691 */
float ro_silu(float v) { return v / (1.0f + expf(-v)); }

void ro_silu_mul_f32(const float* g, const float* u, float* out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = ro_silu(g[i]) * u[i];
}

void ro_silu_mul_f16(const uint16_t* g, const uint16_t* u, uint16_t* out, size_t n) {
    for (size_t i = 0; i < n; i++)
        out[i] = ro_f32_to_f16(ro_silu(ro_f16_to_f32(g[i])) * ro_f16_to_f32(u[i]));
}

/* crates/kernels/shaders/activation.metal:120-129: acc = acc + half(float(src)*w), the sum
 * itself in half precision. */
void ro_scale_accumulate_f16(const uint16_t* src, uint16_t* acc, float weight, size_t n) {
    for (size_t i = 0; i < n; i++) {
        float t = ro_f16_to_f32(ro_f32_to_f16(ro_f16_to_f32(src[i]) * weight));
        acc[i] = ro_f32_to_f16(ro_f16_to_f32(acc[i]) + t);
    }
}

/* crates/kernels/shaders/activation.metal:187-195 */
void ro_add_f16_into_f32(const uint16_t* src, float* acc, size_t n) {
    for (size_t i = 0; i < n; i++) acc[i] += ro_f16_to_f32(src[i]);
}

/* crates/engine/src/forward.rs:2420-2448.  The reference sorts with sort_unstable_by, whose
 * order among equal probabilities is unspecified; this oracle breaks ties by lowest index. */
int ro_topk_softmax(const float* logits, int E, int top_k, int renorm, int32_t* idx, float* wts,
                    float* probs_out) {
    if (E <= 0 || top_k <= 0 || top_k > E) return -1;
    float* probs = (float*)malloc(sizeof(float) * (size_t)E);
    uint8_t* used = (uint8_t*)calloc((size_t)E, 1);
    float mx = -INFINITY;
    for (int i = 0; i < E; i++) mx = logits[i] > mx ? logits[i] : mx;
    float sum = 0.0f;
    for (int i = 0; i < E; i++) {
        probs[i] = expf(logits[i] - mx);
        sum += probs[i];
    }
    for (int i = 0; i < E; i++) probs[i] = probs[i] / sum;
    for (int s = 0; s < top_k; s++) {
        int best = -1;
        for (int i = 0; i < E; i++) {
            if (used[i]) continue;
            if (best < 0 || probs[i] > probs[best]) best = i;
        }
        used[best] = 1;
        idx[s] = best;
        wts[s] = probs[best];
    }
    if (renorm) {
        float ws = 0.0f;
        for (int s = 0; s < top_k; s++) ws += wts[s];
        if (ws > 0.0f)
            for (int s = 0; s < top_k; s++) wts[s] = wts[s] / ws;
    }
    if (probs_out) memcpy(probs_out, probs, sizeof(float) * (size_t)E);
    free(probs);
    free(used);
    return 0;
}

/* One row . x with f64 accumulation over the engine's dequant formulas. */
static double row_dot_f64(int fmt, const uint8_t* row, const float* x, int k, float* deq) {
    ro_dequant_row(fmt, row, k, deq);
    double acc = 0.0;
    for (int c = 0; c < k; c++) acc += (double)deq[c] * (double)x[c];
    return acc;
}

/* crates/engine/src/forward.rs:1644-1679 (decode) / prefill.rs:156-215 (per token).
 *  F32 mode    : logits = router.x (f32 weights), softmax/top-k, per expert in routing order:
 *                gate, up (f32) -> silu(gate)*up -> down (f32) -> out += w_i*down.
 *  REF_F16 mode: router logits rounded to f16 (forward.rs:1650), gate/up rounded to f16
 *                (forward.rs:1668-1669), act f16 (activation.metal:140-153), down f16 from
 *                the f16 act (forward.rs:1671), f16 accumulator (activation.metal:120-129),
 *                then residual add in f32 (activation.metal:187-195). */
int ro_moe_layer_q4k(int mode, int renorm, const float* router, const uint8_t* gate,
                     const uint8_t* up, const uint8_t* down, const float* x, const float* residual,
                     float* out, int32_t* idx_out, float* w_out, int T, int h, int ff, int E,
                     int top_k) {
    if (h % 256 || ff % 256 || top_k > E || top_k > 64) return -1;
    size_t rb_h = ro_row_bytes(RO_Q4K, h), rb_ff = ro_row_bytes(RO_Q4K, ff);
    size_t gate_stride = (size_t)ff * rb_h, down_stride = (size_t)h * rb_ff;
    int err = 0;
    for (int t = 0; t < T; t++) {
        const float* xt = x + (size_t)t * h;
        float* logits = (float*)malloc(sizeof(float) * (size_t)E);
        ro_gemv_f32w(router, xt, logits, E, h);
        if (mode == RO_MOE_REF_F16)
            for (int e = 0; e < E; e++) logits[e] = ro_f16_to_f32(ro_f32_to_f16(logits[e]));
        int32_t idx[64];
        float wts[64];
        if (ro_topk_softmax(logits, E, top_k, renorm, idx, wts, NULL)) err = -1;
        free(logits);
        if (err) break;
        if (idx_out) memcpy(idx_out + (size_t)t * top_k, idx, sizeof(int32_t) * (size_t)top_k);
        if (w_out) memcpy(w_out + (size_t)t * top_k, wts, sizeof(float) * (size_t)top_k);

        float* act = (float*)malloc(sizeof(float) * (size_t)ff);
        float* dn = (float*)malloc(sizeof(float) * (size_t)h);
        float* acc = (float*)calloc((size_t)h, sizeof(float));
        uint16_t* acc16 = (uint16_t*)calloc((size_t)h, sizeof(uint16_t));
        for (int s = 0; s < top_k; s++) {
            const uint8_t* wg = gate + (size_t)idx[s] * gate_stride;
            const uint8_t* wu = up + (size_t)idx[s] * gate_stride;
            const uint8_t* wd = down + (size_t)idx[s] * down_stride;
#pragma omp parallel
            {
                float* deq = (float*)malloc(sizeof(float) * (size_t)(h > ff ? h : ff));
#pragma omp for schedule(static)
                for (int r = 0; r < ff; r++) {
                    float g = (float)row_dot_f64(RO_Q4K, wg + (size_t)r * rb_h, xt, h, deq);
                    float u = (float)row_dot_f64(RO_Q4K, wu + (size_t)r * rb_h, xt, h, deq);
                    if (mode == RO_MOE_REF_F16) {
                        g = ro_f16_to_f32(ro_f32_to_f16(g));
                        u = ro_f16_to_f32(ro_f32_to_f16(u));
                        act[r] = ro_f16_to_f32(ro_f32_to_f16(ro_silu(g) * u));
                    } else {
                        act[r] = ro_silu(g) * u;
                    }
                }
#pragma omp for schedule(static)
                for (int r = 0; r < h; r++) {
                    float d = (float)row_dot_f64(RO_Q4K, wd + (size_t)r * rb_ff, act, ff, deq);
                    dn[r] = (mode == RO_MOE_REF_F16) ? ro_f16_to_f32(ro_f32_to_f16(d)) : d;
                }
                free(deq);
            }
            if (mode == RO_MOE_REF_F16) {
                uint16_t* dn16 = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)h);
                ro_f32_to_f16_array(dn, dn16, (size_t)h);
                ro_scale_accumulate_f16(dn16, acc16, wts[s], (size_t)h);
                free(dn16);
            } else {
                for (int r = 0; r < h; r++) acc[r] += wts[s] * dn[r];
            }
        }
        float* ot = out + (size_t)t * h;
        for (int r = 0; r < h; r++) {
            float base = residual ? residual[(size_t)t * h + r] : 0.0f;
            ot[r] = base + (mode == RO_MOE_REF_F16 ? ro_f16_to_f32(acc16[r]) : acc[r]);
        }
        free(act);
        free(dn);
        free(acc);
        free(acc16);
    }
    return err;
}

/* Batched MoE block with bf16 operands (the arithmetic of a tensor-core grouped GEMM; the reference's
 * analogue is the per-token loop crates/engine/src/prefill.rs:156-215 with f16 intermediates).
 *   weights  : bf16( d*sc*q - dmin*m )   (the f32 values of crates/engine/src/forward.rs:1026-1057, rounded)
 *   x        : rounded to bf16;  products exact, accumulated in f64, rounded once to f32
 *   act      : bf16( silu(g) * u );  y = Wd.act (f32);  out = residual + sum_i w_i*y_i in routing order
 * router != NULL: routing is computed here (f32 router, softmax/top-k) and returned in idx_io / w_io;
 * router == NULL: the routing in idx_io / w_io is used (ids outside [0,E) are skipped). */
float ro_bf16_round(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7F800000u) == 0x7F800000u) return f;
    u += 0x7FFFu + ((u >> 16) & 1u);
    u &= 0xFFFF0000u;
    memcpy(&f, &u, 4);
    return f;
}

int ro_moe_grouped_q4k_bf16(const float* router, int renorm, const uint8_t* gate, const uint8_t* up,
                            const uint8_t* down, const float* x, const float* residual, float* out,
                            int32_t* idx_io, float* w_io, int T, int h, int ff, int E, int top_k) {
    if (h % 256 || ff % 256 || top_k > E || top_k > 64) return -1;
    size_t rb_h = ro_row_bytes(RO_Q4K, h), rb_ff = ro_row_bytes(RO_Q4K, ff);
    size_t gate_stride = (size_t)ff * rb_h, down_stride = (size_t)h * rb_ff;
    int err = 0;
    if (router) {
        for (int t = 0; t < T && !err; t++) {
            float* logits = (float*)malloc(sizeof(float) * (size_t)E);
            ro_gemv_f32w(router, x + (size_t)t * h, logits, E, h);
            if (ro_topk_softmax(logits, E, top_k, renorm, idx_io + (size_t)t * top_k, w_io + (size_t)t * top_k, NULL)) err = -1;
            free(logits);
        }
        if (err) return err;
    }
    /* dequantise the experts that are used, once */
    char* used = (char*)calloc((size_t)E, 1);
    for (size_t s = 0; s < (size_t)T * top_k; s++)
        if (idx_io[s] >= 0 && idx_io[s] < E) used[idx_io[s]] = 1;
    float** wg = (float**)calloc((size_t)E, sizeof(float*));
    float** wu = (float**)calloc((size_t)E, sizeof(float*));
    float** wd = (float**)calloc((size_t)E, sizeof(float*));
    for (int e = 0; e < E; e++) {
        if (!used[e]) continue;
        wg[e] = (float*)malloc(sizeof(float) * (size_t)ff * h);
        wu[e] = (float*)malloc(sizeof(float) * (size_t)ff * h);
        wd[e] = (float*)malloc(sizeof(float) * (size_t)h * ff);
#pragma omp parallel for schedule(static)
        for (int r = 0; r < ff; r++) {
            ro_dequant_row(RO_Q4K, gate + e * gate_stride + (size_t)r * rb_h, h, wg[e] + (size_t)r * h);
            ro_dequant_row(RO_Q4K, up + e * gate_stride + (size_t)r * rb_h, h, wu[e] + (size_t)r * h);
            for (int c = 0; c < h; c++) {
                wg[e][(size_t)r * h + c] = ro_bf16_round(wg[e][(size_t)r * h + c]);
                wu[e][(size_t)r * h + c] = ro_bf16_round(wu[e][(size_t)r * h + c]);
            }
        }
#pragma omp parallel for schedule(static)
        for (int r = 0; r < h; r++) {
            ro_dequant_row(RO_Q4K, down + e * down_stride + (size_t)r * rb_ff, ff, wd[e] + (size_t)r * ff);
            for (int c = 0; c < ff; c++) wd[e][(size_t)r * ff + c] = ro_bf16_round(wd[e][(size_t)r * ff + c]);
        }
    }
#pragma omp parallel for schedule(dynamic, 4)
    for (int t = 0; t < T; t++) {
        float* xb = (float*)malloc(sizeof(float) * (size_t)h);
        float* act = (float*)malloc(sizeof(float) * (size_t)ff);
        float* acc = (float*)calloc((size_t)h, sizeof(float));
        for (int c = 0; c < h; c++) xb[c] = ro_bf16_round(x[(size_t)t * h + c]);
        for (int s = 0; s < top_k; s++) {
            int e = idx_io[(size_t)t * top_k + s];
            if (e < 0 || e >= E) continue;
            float wt = w_io[(size_t)t * top_k + s];
            for (int r = 0; r < ff; r++) {
                const float* g = wg[e] + (size_t)r * h;
                const float* u = wu[e] + (size_t)r * h;
                double ag = 0.0, au = 0.0;
                for (int c = 0; c < h; c++) {
                    ag += (double)g[c] * (double)xb[c];
                    au += (double)u[c] * (double)xb[c];
                }
                act[r] = ro_bf16_round(ro_silu((float)ag) * (float)au);
            }
            for (int r = 0; r < h; r++) {
                const float* d = wd[e] + (size_t)r * ff;
                double ad = 0.0;
                for (int c = 0; c < ff; c++) ad += (double)d[c] * (double)act[c];
                acc[r] += wt * (float)ad;
            }
        }
        for (int r = 0; r < h; r++) out[(size_t)t * h + r] = (residual ? residual[(size_t)t * h + r] : 0.0f) + acc[r];
        free(xb);
        free(act);
        free(acc);
    }
    for (int e = 0; e < E; e++) {
        free(wg[e]);
        free(wu[e]);
        free(wd[e]);
    }
    free(wg);
    free(wu);
    free(wd);
    free(used);
    return 0;
}

/* ───────────────────────── decode ops ───────────────────────── */

/* crates/kernels/shaders/norm.metal:125-154 (f32 gamma); cpu_rms_norm dispatch.rs:1699-1702.
 * The shader's 256-thread tree reduction is restated as an f64 sum. */
void ro_rms_norm_f32(const float* x, const float* gamma, float* y, float eps, int hidden, int rows) {
    for (int r = 0; r < rows; r++) {
        const float* xr = x + (size_t)r * hidden;
        double ss = 0.0;
        for (int i = 0; i < hidden; i++) ss += (double)xr[i] * (double)xr[i];
        float rms = 1.0f / sqrtf((float)(ss / (double)hidden) + eps);
        for (int i = 0; i < hidden; i++) y[(size_t)r * hidden + i] = xr[i] * rms * gamma[i];
    }
}

/* crates/kernels/shaders/fused_rope.metal:17-56: pairs (d, d+hd/2), freq = 1/theta^(2d/hd). */
void ro_rope_qk_f32(float* q, float* k, int hd, int q_heads, int kv_heads, int pos, float theta) {
    int half = hd / 2;
    for (int d = 0; d < half; d++) {
        float freq = 1.0f / powf(theta, (float)(2 * d) / (float)hd);
        float angle = (float)pos * freq;
        float c = cosf(angle), s = sinf(angle);
        for (int hh = 0; hh < q_heads; hh++) {
            float* p = q + (size_t)hh * hd;
            float a = p[d], b = p[d + half];
            p[d] = a * c - b * s;
            p[d + half] = a * s + b * c;
        }
        for (int hh = 0; hh < kv_heads; hh++) {
            float* p = k + (size_t)hh * hd;
            float a = p[d], b = p[d + half];
            p[d] = a * c - b * s;
            p[d + half] = a * s + b * c;
        }
    }
}

/* crates/kernels/shaders/activation.metal:13-28 with an f32 source rounded to the f16 cache;
 * cache layout [kv_heads][max_seq][head_dim] (crates/engine/src/kv_cache.rs:13-22). */
void ro_kv_copy_to_cache_f16(const float* src, uint16_t* dst, int pos, int max_seq, int hd,
                             int kv_heads) {
    for (int hh = 0; hh < kv_heads; hh++)
        for (int d = 0; d < hd; d++)
            dst[((size_t)hh * max_seq + pos) * hd + d] = ro_f32_to_f16(src[(size_t)hh * hd + d]);
}

/* crates/kernels/shaders/attention.metal:248-308 (online softmax over kv positions, scale
 * 1/sqrt(hd) from dispatch.rs:1588, GQA kv_head = q_head / (heads/kv_heads)), with the K/V
 * cache held in f16.  Lane l owns dims l, l+32, ...; lane sums added in lane order. */
void ro_decode_attention_f32q_f16kv(const float* q, const uint16_t* kc, const uint16_t* vc,
                                    float* out, int kv_len, int heads, int kv_heads, int hd,
                                    int kv_head_stride) {
    float scale = 1.0f / sqrtf((float)hd);
    int group = heads / kv_heads;
#pragma omp parallel for schedule(static)
    for (int hq = 0; hq < heads; hq++) {
        int hk = hq / group;
        const float* qh = q + (size_t)hq * hd;
        float m_i = -INFINITY, l_i = 0.0f;
        float* o = (float*)calloc((size_t)hd, sizeof(float));
        for (int p = 0; p < kv_len; p++) {
            const uint16_t* kr = kc + ((size_t)hk * kv_head_stride + p) * hd;
            const uint16_t* vr = vc + ((size_t)hk * kv_head_stride + p) * hd;
            float dot = 0.0f;
            for (int l = 0; l < 32; l++) {
                float part = 0.0f;
                for (int d = l; d < hd; d += 32) part += qh[d] * ro_f16_to_f32(kr[d]);
                dot += part;
            }
            float score = dot * scale;
            float m_new = m_i > score ? m_i : score;
            float rescale = expf(m_i - m_new);
            float e_new = expf(score - m_new);
            float l_new = rescale * l_i + e_new;
            for (int d = 0; d < hd; d++) o[d] = o[d] * rescale + e_new * ro_f16_to_f32(vr[d]);
            m_i = m_new;
            l_i = l_new;
        }
        float inv = l_i > 0.0f ? 1.0f / l_i : 0.0f;
        for (int d = 0; d < hd; d++) out[(size_t)hq * hd + d] = o[d] * inv;
        free(o);
    }
}

/* Greedy pick over f32 logits, lowest index among equal maxima.  (The reference's two argmax
 * routes disagree on ties: sampler.rs:111-116 keeps the last maximum, activation.metal:56-110
 * neither first nor last.) */
int32_t ro_argmax_f32(const float* v, size_t n) {
    size_t best = 0;
    for (size_t i = 1; i < n; i++)
        if (v[i] > v[best]) best = i;
    return (int32_t)best;
}

/* crates/engine/src/forward.rs:1795-1975 with every matrix Q4_K, an f32 router and the
 * F32 MoE mode; K/V rounded to f16 on the way into the cache. */
/* ───────────── host sampler (crates/engine/src/sampler.rs) ───────────── */
uint64_t ro_sampler_seed_state(uint64_t seed) {                     /* SimpleRng::new, sampler.rs:15-17 */
    return seed == 0 ? 0x9e3779b97f4a7c15ull : (seed ^ 0x9e3779b97f4a7c15ull);
}
float ro_sampler_next_f32(uint64_t* state) {                         /* next_u64 + next_f32, sampler.rs:18-27 */
    uint64_t x = *state;
    x ^= x << 13; x ^= x >> 7; x ^= x << 17;
    *state = x;
    return (float)(x >> 11) / (float)(1ull << 53);
}
/* max_by with partial_cmp(..).unwrap_or(Equal): a later element replaces the running maximum unless it compares Less
 * (sampler.rs:114-119); NaN compares as Equal, so it replaces too. */
int32_t ro_sampler_argmax_last(const float* v, size_t n) {
    if (n == 0) return 0;
    size_t best = 0;
    for (size_t i = 1; i < n; i++)
        if (!(v[i] < v[best])) best = i;
    return (int32_t)best;
}
static int cmp_desc_f32(const void* a, const void* b) {
    const float x = *(const float*)a, y = *(const float*)b;
    return x > y ? -1 : (x < y ? 1 : 0);
}
typedef struct { float p; uint32_t i; } ro_pi;
static int cmp_desc_pi(const void* a, const void* b) {
    const ro_pi* x = (const ro_pi*)a; const ro_pi* y = (const ro_pi*)b;
    if (x->p > y->p) return -1;
    if (x->p < y->p) return 1;
    return x->i < y->i ? -1 : (x->i > y->i ? 1 : 0);   /* the reference's unstable sort leaves equal entries open: by index here */
}
int32_t ro_sample(const float* logits, size_t n, const ro_sampler_cfg* cfg, const int32_t* context, size_t n_context,
                  const int32_t* eos_ids, size_t n_eos, uint64_t* rng_state, float* probs_out) {
    float* s = (float*)malloc(n * sizeof(float));
    int32_t result;
    memcpy(s, logits, n * sizeof(float));
    if (n_context < (size_t)cfg->min_tokens)                         /* sampler.rs:64-71 */
        for (size_t e = 0; e < n_eos; e++)
            if (eos_ids[e] >= 0 && (size_t)eos_ids[e] < n) s[eos_ids[e]] = -INFINITY;
    if (cfg->repetition_penalty != 1.0f)                             /* sampler.rs:74-76, 124-135: once per occurrence */
        for (size_t c = 0; c < n_context; c++) {
            const int32_t t = context[c];
            if (t >= 0 && (size_t)t < n) {
                if (s[t] > 0.0f) s[t] /= cfg->repetition_penalty;
                else s[t] *= cfg->repetition_penalty;
            }
        }
    if (cfg->temperature == 0.0f) {                                  /* sampler.rs:79 */
        result = ro_sampler_argmax_last(s, n);
        goto done;
    }
    for (size_t i = 0; i < n; i++) s[i] /= cfg->temperature;         /* sampler.rs:82 */
    {                                                                /* softmax_inplace, sampler.rs:137-142 */
        float mx = -INFINITY, sum = 0.0f;
        for (size_t i = 0; i < n; i++) mx = fmaxf(mx, s[i]);
        for (size_t i = 0; i < n; i++) { s[i] = expf(s[i] - mx); sum += s[i]; }
        for (size_t i = 0; i < n; i++) s[i] /= sum;
    }
    if (cfg->top_k > 0 && (size_t)cfg->top_k < n) {                  /* topk_filter, sampler.rs:144-152 */
        float* sorted = (float*)malloc(n * sizeof(float));
        memcpy(sorted, s, n * sizeof(float));
        qsort(sorted, n, sizeof(float), cmp_desc_f32);
        const float thr = sorted[cfg->top_k - 1];
        free(sorted);
        size_t kept = 0;
        for (size_t i = 0; i < n; i++) {
            if (s[i] >= thr && kept < (size_t)cfg->top_k) kept++;
            else s[i] = 0.0f;
        }
    }
    if (cfg->top_p < 1.0f) {                                         /* topp_filter, sampler.rs:154-162 */
        ro_pi* order = (ro_pi*)malloc(n * sizeof(ro_pi));
        for (size_t i = 0; i < n; i++) { order[i].p = s[i]; order[i].i = (uint32_t)i; }
        qsort(order, n, sizeof(ro_pi), cmp_desc_pi);
        float cum = 0.0f;
        for (size_t r = 0; r < n; r++) {
            if (cum >= cfg->top_p) s[order[r].i] = 0.0f;
            else cum += s[order[r].i];
        }
        free(order);
    }
    {                                                                /* sampler.rs:98-110 */
        float total = 0.0f;
        for (size_t i = 0; i < n; i++) total += s[i];
        if (total <= 0.0f) { result = ro_sampler_argmax_last(s, n); goto done; }
        const float r = ro_sampler_next_f32(rng_state) * total;
        float cum = 0.0f;
        for (size_t i = 0; i < n; i++) {
            cum += s[i];
            if (r <= cum) { result = (int32_t)i; goto done; }
        }
        result = ro_sampler_argmax_last(s, n);
    }
done:
    if (probs_out) memcpy(probs_out, s, n * sizeof(float));
    free(s);
    return result;
}

int32_t ro_decode_step(const ro_model_cfg* c, const ro_model_weights* w, uint16_t* kc, uint16_t* vc,
                       int32_t token, int32_t pos, float* logits_out) {
    int h = c->hidden, hd = c->head_dim;
    int q_dim = c->n_heads * hd, kv_dim = c->n_kv_heads * hd;
    if (token < 0 || token >= c->vocab || pos < 0 || pos >= c->max_seq) return -1;
    float* x = (float*)malloc(sizeof(float) * (size_t)h);
    float* xn = (float*)malloc(sizeof(float) * (size_t)h);
    float* q = (float*)malloc(sizeof(float) * (size_t)q_dim);
    float* k = (float*)malloc(sizeof(float) * (size_t)kv_dim);
    float* v = (float*)malloc(sizeof(float) * (size_t)kv_dim);
    float* ao = (float*)malloc(sizeof(float) * (size_t)q_dim);
    float* tmp = (float*)malloc(sizeof(float) * (size_t)h);
    float* logits = (float*)malloc(sizeof(float) * (size_t)c->vocab);
    memcpy(x, w->tok_emb + (size_t)token * h, sizeof(float) * (size_t)h);

    size_t rb_h = ro_row_bytes(RO_Q4K, h), rb_q = ro_row_bytes(RO_Q4K, q_dim);
    size_t rb_ff = ro_row_bytes(RO_Q4K, c->ff);
    size_t kv_layer = (size_t)c->n_kv_heads * c->max_seq * hd;
    for (int l = 0; l < c->n_layers; l++) {
        ro_rms_norm_f32(x, w->attn_norm + (size_t)l * h, xn, c->eps, h, 1);
        ro_gemv(RO_Q4K, RO_TIER_F64, w->wq + (size_t)l * q_dim * rb_h, xn, q, NULL, q_dim, h, 1);
        ro_gemv(RO_Q4K, RO_TIER_F64, w->wk + (size_t)l * kv_dim * rb_h, xn, k, NULL, kv_dim, h, 1);
        ro_gemv(RO_Q4K, RO_TIER_F64, w->wv + (size_t)l * kv_dim * rb_h, xn, v, NULL, kv_dim, h, 1);
        ro_rope_qk_f32(q, k, hd, c->n_heads, c->n_kv_heads, pos, c->theta);
        uint16_t* kcl = kc + (size_t)l * kv_layer;
        uint16_t* vcl = vc + (size_t)l * kv_layer;
        ro_kv_copy_to_cache_f16(k, kcl, pos, c->max_seq, hd, c->n_kv_heads);
        ro_kv_copy_to_cache_f16(v, vcl, pos, c->max_seq, hd, c->n_kv_heads);
        ro_decode_attention_f32q_f16kv(q, kcl, vcl, ao, pos + 1, c->n_heads, c->n_kv_heads, hd,
                                       c->max_seq);
        ro_gemv(RO_Q4K, RO_TIER_F64, w->wo + (size_t)l * h * rb_q, ao, tmp, NULL, h, q_dim, 1);
        for (int i = 0; i < h; i++) x[i] = tmp[i] + x[i];
        ro_rms_norm_f32(x, w->ffn_norm + (size_t)l * h, xn, c->eps, h, 1);
        size_t eg = (size_t)c->n_experts * c->ff * rb_h, ed = (size_t)c->n_experts * h * rb_ff;
        ro_moe_layer_q4k(RO_MOE_F32, c->renorm, w->router + (size_t)l * c->n_experts * h,
                         w->gate + (size_t)l * eg, w->up + (size_t)l * eg, w->down + (size_t)l * ed,
                         xn, x, tmp, NULL, NULL, 1, h, c->ff, c->n_experts, c->top_k);
        memcpy(x, tmp, sizeof(float) * (size_t)h);
    }
    ro_rms_norm_f32(x, w->out_norm, xn, c->eps, h, 1);
    ro_gemv(RO_Q4K, RO_TIER_F64, w->lm_head, xn, logits, NULL, c->vocab, h, 1);
    int32_t tok = ro_argmax_f32(logits, (size_t)c->vocab);
    if (logits_out) memcpy(logits_out, logits, sizeof(float) * (size_t)c->vocab);
    free(x); free(xn); free(q); free(k); free(v); free(ao); free(tmp); free(logits);
    return tok;
}

/* ───────────────────────── comparator ─────────────────────────
 * crates/reference/src/lib.rs:28-62 (max abs diff vs tolerance, mismatch count) and :66-96
 * (max/mean/rms of the difference), plus the relative bound used for dot products:
 * |got-ref| <= rel_tol * max(|ref|, rms(ref)). */
int64_t ro_compare(const float* ref, const float* got, size_t n, float abs_tol, float rel_tol,
                   ro_diff_stats* st) {
    double sum_abs = 0, sum_sq = 0, ref_sq = 0, max_abs = 0, max_rel = 0;
    int64_t mis_abs = 0, mis_rel = 0;
    for (size_t i = 0; i < n; i++) ref_sq += (double)ref[i] * (double)ref[i];
    double ref_rms = n ? sqrt(ref_sq / (double)n) : 0.0;
    for (size_t i = 0; i < n; i++) {
        double d = fabs((double)ref[i] - (double)got[i]);
        if (!(d == d)) d = INFINITY; /* NaN counts as a mismatch */
        if (d > max_abs) max_abs = d;
        sum_abs += d;
        sum_sq += d * d;
        if (d > (double)abs_tol) mis_abs++;
        double scale = fabs((double)ref[i]) > ref_rms ? fabs((double)ref[i]) : ref_rms;
        double rel = scale > 0 ? d / scale : (d > 0 ? INFINITY : 0.0);
        if (rel > max_rel) max_rel = rel;
        if (rel > (double)rel_tol) mis_rel++;
    }
    if (st) {
        st->max_abs = max_abs;
        st->mean_abs = n ? sum_abs / (double)n : 0.0;
        st->rms = n ? sqrt(sum_sq / (double)n) : 0.0;
        st->ref_rms = ref_rms;
        st->max_rel = max_rel;
        st->n = (int64_t)n;
        st->n_mismatch_abs = mis_abs;
        st->n_mismatch_rel = mis_rel;
    }
    return mis_rel;
}
