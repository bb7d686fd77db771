// Small bandwidth-bound operators of the MoE block and the router, plus the synthetic-data
// generators used by the benchmark and the tests.
//
// Twins of: silu_mul_f16/f32 (activation.metal:140-167), scale_accumulate_f16
// (activation.metal:120-129), add_f16_into_f32 (activation.metal:187-195), dequant_q4k_f16
// (dequant.metal:53-98), gemv_f16w_f32in (gemv.metal:82-106).  Paths under
// crates/kernels/shaders/ of the reference.
#include "gemv_common.cuh"
#include "runit_internal.h"

namespace runit {

__global__ void silu_mul_f16_kernel(const __half* __restrict__ g, const __half* __restrict__ u, __half* __restrict__ o,
                                    uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float gv = __half2float(g[i]);
    // expf, not the fast intrinsic: the f16 result must round like the reference's.
    o[i] = __float2half_rn(gv / (1.0f + expf(-gv)) * __half2float(u[i]));
}

__global__ void silu_mul_f32_kernel(const float* __restrict__ g, const float* __restrict__ u, float* __restrict__ o,
                                    uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float gv = g[i];
    o[i] = gv / (1.0f + expf(-gv)) * u[i];
}

__global__ void scale_accumulate_f16_kernel(const __half* __restrict__ src, __half* acc, float w, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    // acc = acc + half(float(src) * w), the sum itself rounded to half.
    const __half t = __float2half_rn(__half2float(src[i]) * w);
    acc[i] = __float2half_rn(__half2float(acc[i]) + __half2float(t));
}

__global__ void add_f16_into_f32_kernel(const __half* __restrict__ src, float* acc, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    acc[i] += __half2float(src[i]);
}

// One CTA of 256 threads per superblock, thread = element (same mapping as the reference).
__global__ void dequant_q4k_f16_kernel(const uint8_t* __restrict__ in, __half* __restrict__ out, uint32_t n_blocks) {
    const uint32_t blk = blockIdx.x;
    if (blk >= n_blocks) return;
    const uint8_t* p = in + (size_t)blk * 144;
    const uint32_t lid = threadIdx.x;
    const float d = half_bits_to_float(p[0] | (p[1] << 8));
    const float dmin = half_bits_to_float(p[2] | (p[3] << 8));
    const uint8_t* sc = p + 4;
    const uint32_t sub = lid >> 5, local = lid & 31, pair = sub >> 1;
    const bool hi = sub & 1;
    const uint32_t j = hi ? pair + 4 : pair;
    uint32_t s, m;
    if (j < 4) {
        s = sc[j] & 63;
        m = sc[j + 4] & 63;
    } else {
        s = (sc[j + 4] & 15) | ((sc[j - 4] >> 6) << 4);
        m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4);
    }
    const uint8_t b = p[16 + pair * 32 + local];
    const uint32_t q = hi ? (b >> 4) : (b & 15);
    out[(size_t)blk * 256 + lid] = __float2half_rn(d * (float)s * (float)q - dmin * (float)m);
}

// Router GEMV: one warp per row, 8 rows per CTA, float4 x and half4 weight loads.
__global__ void __launch_bounds__(256) gemv_f16w_f32in_kernel(const __half* __restrict__ w, const float* __restrict__ x,
                                                               __half* __restrict__ y, uint32_t m, uint32_t k) {
    const uint32_t row = blockIdx.x * 8 + (threadIdx.x >> 5);
    const uint32_t lane = threadIdx.x & 31;
    if (row >= m) return;
    const __half* a = w + (size_t)row * k;
    float acc = 0.f;
    const uint32_t k4 = k >> 2;
    const bool vec = ((reinterpret_cast<uintptr_t>(a) & 7) == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    if (vec) {
        for (uint32_t i = lane; i < k4; i += 32) {
            const uint2 hv = reinterpret_cast<const uint2*>(a)[i];
            const float4 xv = reinterpret_cast<const float4*>(x)[i];
            const float2 h01 = __half22float2(*reinterpret_cast<const __half2*>(&hv.x));
            const float2 h23 = __half22float2(*reinterpret_cast<const __half2*>(&hv.y));
            acc += h01.x * xv.x + h01.y * xv.y + h23.x * xv.z + h23.y * xv.w;
        }
    } else {
        for (uint32_t i = lane; i < k4; i += 32)
            for (uint32_t c = 0; c < 4; c++) acc += __half2float(a[4 * i + c]) * x[4 * i + c];
    }
    for (uint32_t i = (k4 << 2) + lane; i < k; i += 32) acc += __half2float(a[i]) * x[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) y[row] = __float2half_rn(acc);
}

// ───────────────────────── synthetic data ─────────────────────────
// splitmix64 as a counter-based generator: value i of stream `seed` is mix(seed + i*GOLDEN).
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__device__ __forceinline__ uint64_t rnd(uint64_t seed, uint64_t i) { return mix64(seed ^ mix64(i)); }
__device__ __forceinline__ float u01(uint64_t r) { return ((float)(r >> 40) + 0.5f) * (1.0f / 16777216.0f); }
__device__ __forceinline__ float normal(uint64_t seed, uint64_t i) {
    const uint64_t r = rnd(seed, i);
    const float u1 = u01(r), u2 = u01(r << 24 | (r >> 40));
    return sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
}

// Q8_0: qs uniform in [-127,127], d = f16(|N(0,sigma)|/127).
// Q4_0: nibbles uniform 0..15, d = f16(|N(0,sigma)|/8).
// Q4_K: d, dmin = f16(|N(0,sigma)|), 6-bit scales/mins uniform 0..63 (any 12 bytes decode to
//       that), nibbles uniform 0..15.
// zero_mean (Q4_K only): dmin = f16(7.5 d), the 6-bit min of every sub-block equals its scale.
__global__ void fill_weights_kernel(int fmt, uint8_t* dst, uint64_t n_blocks, uint64_t seed, float sigma, int zero_mean) {
    const uint64_t blk = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (blk >= n_blocks) return;
    if (fmt == RUNIT_FMT_Q8_0) {
        uint8_t* p = dst + blk * 34;
        const __half d = __float2half_rn(fabsf(normal(seed, blk * 8)) * sigma / 127.0f);
        const unsigned short db = __half_as_ushort(d);
        p[0] = db & 0xFF;
        p[1] = db >> 8;
        for (int i = 0; i < 4; i++) {
            uint64_t r = rnd(seed, blk * 8 + 1 + i);
            for (int c = 0; c < 8; c++) {
                p[2 + i * 8 + c] = (uint8_t)(int8_t)((int)((r & 0xFF) * 255 >> 8) - 127);
                r >>= 8;
            }
        }
    } else if (fmt == RUNIT_FMT_Q4_0) {
        uint8_t* p = dst + blk * 18;
        const __half d = __float2half_rn(fabsf(normal(seed, blk * 4)) * sigma / 8.0f);
        const unsigned short db = __half_as_ushort(d);
        p[0] = db & 0xFF;
        p[1] = db >> 8;
        for (int i = 0; i < 2; i++) {
            uint64_t r = rnd(seed, blk * 4 + 1 + i);
            for (int c = 0; c < 8; c++) {
                p[2 + i * 8 + c] = (uint8_t)(r & 0xFF);
                r >>= 8;
            }
        }
    } else {
        uint8_t* p = dst + blk * 144;
        const unsigned short db = __half_as_ushort(__float2half_rn(fabsf(normal(seed, blk * 24)) * sigma));
        unsigned short mb = __half_as_ushort(__float2half_rn(fabsf(normal(seed, blk * 24 + 1)) * sigma));
        if (zero_mean) mb = __half_as_ushort(__float2half_rn(7.5f * __half2float(__ushort_as_half(db))));
        p[0] = db & 0xFF; p[1] = db >> 8; p[2] = mb & 0xFF; p[3] = mb >> 8;
        for (int i = 0; i < 18; i++) {
            uint64_t r = rnd(seed, blk * 24 + 2 + i);
            const int base = 4 + i * 8;
            for (int c = 0; c < 8 && base + c < 144; c++) {
                p[base + c] = (uint8_t)(r & 0xFF);
                r >>= 8;
            }
        }
        if (zero_mean) {
            // scale bytes s[0..11] (get_scale_min_k4, crates/engine/src/forward.rs:359-369): s[j+4] = s[j] makes the low six
            // bits and the two spill bits of min j (j+4) equal those of scale j (j+4); equal nibbles in s[j+8] do the rest
            for (int j = 0; j < 4; j++) {
                p[4 + 4 + j] = p[4 + j];
                const uint8_t n = p[4 + 8 + j] & 0x0F;
                p[4 + 8 + j] = (uint8_t)(n | (n << 4));
            }
        }
    }
}

__global__ void fill_normal_kernel(float* dst, uint64_t n, uint64_t seed, float sigma) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = normal(seed, i) * sigma;
}

}  // namespace runit

using namespace runit;

extern "C" {

#define EW_CHECK(name)                                                        \
    if (!ctx) return RUNIT_ERR_BAD_ARG;                                       \
    RUNIT_REQUIRE(ctx, n > 0, name ": n == 0");

int32_t runit_silu_mul_f16(runit_ctx_t* ctx, const void* gate, const void* up, void* out, uint32_t n) {
    EW_CHECK("silu_mul_f16");
    RUNIT_REQUIRE(ctx, gate && up && out, "silu_mul_f16: null pointer");
    silu_mul_f16_kernel<<<(n + 255) / 256, 256, 0, ctx->stream>>>((const __half*)gate, (const __half*)up, (__half*)out, n);
    return runit_after_launch(ctx, "silu_mul_f16");
}

int32_t runit_silu_mul_f32(runit_ctx_t* ctx, const void* gate, const void* up, void* out, uint32_t n) {
    EW_CHECK("silu_mul_f32");
    RUNIT_REQUIRE(ctx, gate && up && out, "silu_mul_f32: null pointer");
    silu_mul_f32_kernel<<<(n + 255) / 256, 256, 0, ctx->stream>>>((const float*)gate, (const float*)up, (float*)out, n);
    return runit_after_launch(ctx, "silu_mul_f32");
}

int32_t runit_scale_accumulate_f16(runit_ctx_t* ctx, const void* src, void* acc, float weight, uint32_t n) {
    EW_CHECK("scale_accumulate_f16");
    RUNIT_REQUIRE(ctx, src && acc, "scale_accumulate_f16: null pointer");
    scale_accumulate_f16_kernel<<<(n + 255) / 256, 256, 0, ctx->stream>>>((const __half*)src, (__half*)acc, weight, n);
    return runit_after_launch(ctx, "scale_accumulate_f16");
}

int32_t runit_add_f16_into_f32(runit_ctx_t* ctx, const void* src, void* acc, uint32_t n) {
    EW_CHECK("add_f16_into_f32");
    RUNIT_REQUIRE(ctx, src && acc, "add_f16_into_f32: null pointer");
    add_f16_into_f32_kernel<<<(n + 255) / 256, 256, 0, ctx->stream>>>((const __half*)src, (float*)acc, n);
    return runit_after_launch(ctx, "add_f16_into_f32");
}

int32_t runit_dequant_q4k_f16(runit_ctx_t* ctx, const void* input, void* output, uint32_t n_blocks) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, n_blocks > 0, "dequant_q4k_f16: n_blocks == 0");
    RUNIT_REQUIRE(ctx, input && output, "dequant_q4k_f16: null pointer");
    dequant_q4k_f16_kernel<<<n_blocks, 256, 0, ctx->stream>>>((const uint8_t*)input, (__half*)output, n_blocks);
    return runit_after_launch(ctx, "dequant_q4k_f16");
}

int32_t runit_gemv_f16w_f32in(runit_ctx_t* ctx, const void* weight, const void* input, void* output, uint32_t m,
                              uint32_t k) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, m > 0 && k > 0, "gemv_f16w_f32in: empty shape %ux%u", m, k);
    RUNIT_REQUIRE(ctx, weight && input && output, "gemv_f16w_f32in: null pointer");
    gemv_f16w_f32in_kernel<<<(m + 7) / 8, 256, 0, ctx->stream>>>((const __half*)weight, (const float*)input,
                                                                   (__half*)output, m, k);
    return runit_after_launch(ctx, "gemv_f16w_f32in");
}

int32_t runit_fill_weights(runit_ctx_t* ctx, int32_t fmt, void* dst, uint64_t n_blocks, uint64_t seed, float sigma) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, fmt >= 0 && fmt <= 2 && dst && n_blocks > 0, "fill_weights: bad argument");
    RUNIT_REQUIRE(ctx, n_blocks < (1ull << 38), "fill_weights: too many blocks");
    const uint64_t grid = (n_blocks + 255) / 256;
    fill_weights_kernel<<<(unsigned)grid, 256, 0, ctx->stream>>>(fmt, (uint8_t*)dst, n_blocks, seed, sigma, 0);
    return runit_after_launch(ctx, "fill_weights");
}

int32_t runit_fill_weights_q4k_zero_mean(runit_ctx_t* ctx, void* dst, uint64_t n_blocks, uint64_t seed, float sigma) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, dst && n_blocks > 0 && n_blocks < (1ull << 38), "fill_weights_q4k_zero_mean: bad argument");
    const uint64_t grid = (n_blocks + 255) / 256;
    fill_weights_kernel<<<(unsigned)grid, 256, 0, ctx->stream>>>(RUNIT_FMT_Q4K, (uint8_t*)dst, n_blocks, seed, sigma, 1);
    return runit_after_launch(ctx, "fill_weights_q4k_zero_mean");
}

int32_t runit_fill_normal_f32(runit_ctx_t* ctx, void* dst, uint64_t n, uint64_t seed, float sigma) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, dst && n > 0, "fill_normal_f32: bad argument");
    const uint64_t grid = (n + 255) / 256;
    RUNIT_REQUIRE(ctx, grid < (1ull << 31), "fill_normal_f32: too many elements");
    fill_normal_kernel<<<(unsigned)grid, 256, 0, ctx->stream>>>((float*)dst, n, seed, sigma);
    return runit_after_launch(ctx, "fill_normal_f32");
}

}  // extern "C"
