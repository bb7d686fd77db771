// Fused-dequant GEMVs for the formats the reference only dequantises on the CPU at load time: Q5_0, Q5_K and Q6_K
// (crates/engine/src/forward.rs:900-949, 979-1012; files quantised as "Q4_K_M" mix them in: Q6_K for ffn_down and the
// output matrix, Q5_0 / Q5_K in some attention matrices, docs/STATUS_REPORT.md:19-27).  The reference expands such
// tensors to f32 or f16 and runs its f16 GEMV on them; here they stay packed in HBM (0.69 / 0.69 / 0.82 bytes per weight
// instead of 2) and are decoded in registers, so a decode step streams 2.4 - 2.9 times fewer bytes for them.
//
// Kernel: one warp per row, lane l decodes 8 of the 256 weights of a unit (a Q5_K / Q6_K superblock, or 8 Q5_0 blocks)
// exactly as the reference's loops index them; the packed bytes of 4 units at a time arrive through a per-warp ring of
// three cp.async stages that runs across the warp's rows (rows are only 2- or 4-byte aligned in these formats, so the
// copies are 4-byte ones from the aligned word below); f32 accumulation, shuffle reduction, optional f32 residual.
// HBM-bound in principle; at ~7 instructions per weight it is issue-bound at roughly half the HBM rate on B200.
#include "gemv_common.cuh"
#include "runit_internal.h"
#include "tma.cuh"

namespace runit {
namespace kq {

constexpr int kWarps = 8;       // per CTA
constexpr int kChunk = 4;       // units per stage
constexpr int kStages = 3;

template <int FMT> struct KTraits;
template <> struct KTraits<RUNIT_FMT_Q5_0> { static constexpr int UB = 176; };   // 8 blocks of 22 bytes
template <> struct KTraits<RUNIT_FMT_Q5K>  { static constexpr int UB = 176; };
template <> struct KTraits<RUNIT_FMT_Q6K>  { static constexpr int UB = 210; };

// Partial dot product of this lane's 8 weights of one unit with x (xu = the unit's 256 activations in global memory).
template <int FMT>
__device__ __forceinline__ float unit_dot(const uint8_t* u, const float* __restrict__ xu, int lane, int nblk) {
    float acc = 0.f;
    if (FMT == RUNIT_FMT_Q6K) {
        // forward.rs:920-949: {ql[128]; qh[64]; i8 scales[16]; f16 d}
        const float d = half_bits_to_float((uint32_t)u[208] | ((uint32_t)u[209] << 8));
        const int8_t* sc = reinterpret_cast<const int8_t*>(u + 192);
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const int a = u[64 * half + lane], c = u[64 * half + lane + 32], h = u[128 + 32 * half + lane];
            const int q1 = ((a & 15) | ((h & 3) << 4)) - 32, q2 = ((c & 15) | (((h >> 2) & 3) << 4)) - 32;
            const int q3 = ((a >> 4) | (((h >> 4) & 3) << 4)) - 32, q4 = ((c >> 4) | (((h >> 6) & 3) << 4)) - 32;
            const float* xh = xu + 128 * half + lane;
            float s = (float)sc[8 * half + 0] * ((float)q1 * xh[0]);
            s = fmaf((float)sc[8 * half + 2], (float)q2 * xh[32], s);
            s = fmaf((float)sc[8 * half + 4], (float)q3 * xh[64], s);
            s = fmaf((float)sc[8 * half + 6], (float)q4 * xh[96], s);
            acc = fmaf(d, s, acc);
        }
    } else if (FMT == RUNIT_FMT_Q5K) {
        // forward.rs:979-1012: {f16 d; f16 dmin; scales[12]; qh[32]; qs[128]}; fifth bit of element e = bit e%8 of qh[e/8]
        const uint32_t h0 = *reinterpret_cast<const uint16_t*>(u) | ((uint32_t)*reinterpret_cast<const uint16_t*>(u + 2) << 16);
        const float d = half_bits_to_float(h0), dmin = half_bits_to_float(h0 >> 16);
        const uint8_t* s = u + 4;
        const uint8_t* qh = u + 16;
        const uint8_t* qs = u + 48;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            // get_scale_min_k4 (forward.rs:359-369) for indices j and j + 4
            const float sc_lo = (float)(s[j] & 63), m_lo = (float)(s[j + 4] & 63);
            const float sc_hi = (float)((s[j + 8] & 15) | ((s[j] >> 6) << 4)), m_hi = (float)((s[j + 8] >> 4) | ((s[j + 4] >> 6) << 4));
            const int v = qs[32 * j + lane];
            const int e_lo = 64 * j + lane, e_hi = e_lo + 32;
            const int q_lo = (v & 15) | (((qh[e_lo >> 3] >> (e_lo & 7)) & 1) << 4);
            const int q_hi = (v >> 4) | (((qh[e_hi >> 3] >> (e_hi & 7)) & 1) << 4);
            const float x_lo = xu[e_lo], x_hi = xu[e_hi];
            acc = fmaf(d * sc_lo * (float)q_lo - dmin * m_lo, x_lo, acc);
            acc = fmaf(d * sc_hi * (float)q_hi - dmin * m_hi, x_hi, acc);
        }
    } else {
        // forward.rs:900-919: blocks {f16 d; qh[4]; qs[16]}; lane l: block l / 4, bytes 4 (l % 4) .. + 3
        const int b = lane >> 2, j0 = (lane & 3) * 4;
        if (b < nblk) {
            const uint8_t* blk = u + 22 * b;
            const float d = half_bits_to_float((uint32_t)blk[0] | ((uint32_t)blk[1] << 8));
            const uint32_t qh = (uint32_t)blk[2] | ((uint32_t)blk[3] << 8) | ((uint32_t)blk[4] << 16) | ((uint32_t)blk[5] << 24);
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int j = j0 + i, v = blk[6 + j];
                const int x0 = (v & 15) | (((qh >> j) & 1) << 4), x1 = (v >> 4) | (((qh >> (j + 16)) & 1) << 4);
                s = fmaf((float)(x0 - 16), xu[32 * b + j], s);
                s = fmaf((float)(x1 - 16), xu[32 * b + j + 16], s);
            }
            acc = d * s;
        }
    }
    return acc;
}

struct Args {
    const uint8_t* w;
    const float* x;
    float* y;
    const float* res;
    uint32_t m, k, n_units, row_bytes, nb;   // nb: 32-blocks per row (Q5_0: the last unit may hold fewer than 8)
};

template <int FMT>
__global__ void __launch_bounds__(kWarps * 32) gemv_kquant_kernel(const Args a) {
    constexpr int UB = KTraits<FMT>::UB;
    constexpr int SB = (kChunk * UB + 4 + 15) / 16 * 16;   // stage bytes: the chunk plus the alignment shift
    __shared__ __align__(16) uint8_t ring[kWarps][kStages][SB];
    grid_dependency_wait();
    grid_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t gw = blockIdx.x * kWarps + warp, n_warps = gridDim.x * kWarps;
    if (gw >= a.m) return;
    const uint32_t n_chunks = (a.n_units + kChunk - 1) / kChunk;
    const uint32_t my_rows = (a.m - gw + n_warps - 1) / n_warps;
    const uint32_t n_steps = my_rows * n_chunks;   // (row, chunk) pairs of this warp, in order

    // chunk t of this warp: row gw + (t / n_chunks) * n_warps, units [c * kChunk, ...)
    auto issue = [&](uint32_t t) {
        if (t < n_steps) {
            const uint32_t row = gw + (t / n_chunks) * n_warps, c = t % n_chunks;
            const uint32_t units = min((uint32_t)kChunk, a.n_units - c * kChunk);
            const size_t start = (size_t)row * a.row_bytes + (size_t)c * kChunk * UB;
            const size_t bytes = FMT == RUNIT_FMT_Q5_0 ? min((size_t)units * UB, (size_t)a.row_bytes - (size_t)c * kChunk * UB) : (size_t)units * UB;
            const uint32_t shift = (uint32_t)((reinterpret_cast<uintptr_t>(a.w) + start) & 3u);
            const uint8_t* src = a.w + start - shift;
            const uint32_t words = (uint32_t)((shift + bytes + 3) / 4);
            const uint32_t dst = smem_u32(&ring[warp][t % kStages][0]);
            for (uint32_t wd = lane; wd < words; wd += 32) cp_async4(dst + 4 * wd, src + 4 * (size_t)wd);
        }
        cp_async_commit();
    };
#pragma unroll
    for (int s = 0; s < kStages - 1; s++) issue(s);
    float acc = 0.f;
    for (uint32_t t = 0; t < n_steps; t++) {
        issue(t + kStages - 1);
        cp_async_wait<kStages - 1>();
        __syncwarp();
        const uint32_t row = gw + (t / n_chunks) * n_warps, c = t % n_chunks;
        const uint32_t units = min((uint32_t)kChunk, a.n_units - c * kChunk);
        const size_t start = (size_t)row * a.row_bytes + (size_t)c * kChunk * UB;
        const uint32_t shift = (uint32_t)((reinterpret_cast<uintptr_t>(a.w) + start) & 3u);
        const uint8_t* base = &ring[warp][t % kStages][shift];
        for (uint32_t i = 0; i < units; i++) {
            const uint32_t u = c * kChunk + i;
            const int nblk = FMT == RUNIT_FMT_Q5_0 ? min(8, (int)(a.nb - u * 8u)) : 8;
            acc += unit_dot<FMT>(base + i * UB, a.x + (size_t)u * 256, lane, nblk);
        }
        __syncwarp();   // the stage may be refilled by the next issue
        if (c + 1 == n_chunks) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (lane == 0) a.y[row] = a.res ? a.res[row] + acc : acc;
            acc = 0.f;
        }
    }
    cp_async_wait<0>();
}

template <int FMT>
static int32_t launch(runit_ctx* ctx, const char* name, const void* w, const void* x, void* y, const void* res, uint32_t m, uint32_t k) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, w && x && y, "%s: null pointer", name);
    RUNIT_REQUIRE(ctx, m > 0 && m <= (1u << 28), "%s: m=%u out of range", name, m);
    const uint32_t be = FMT == RUNIT_FMT_Q5_0 ? 32u : 256u;
    RUNIT_REQUIRE(ctx, k > 0 && k % be == 0 && k <= (1u << 24), "%s: k=%u is not a positive multiple of %u", name, k, be);
    RUNIT_REQUIRE(ctx, runit_aligned(w, 16) && runit_aligned(x, 16) && runit_aligned(y, 4) && (!res || runit_aligned(res, 4)),
                  "%s: weights and input 16-byte aligned, output 4-byte aligned", name);
    Args a;
    a.w = (const uint8_t*)w;
    a.x = (const float*)x;
    a.y = (float*)y;
    a.res = (const float*)res;
    a.m = m;
    a.k = k;
    a.nb = k / 32;
    a.n_units = (k + 255) / 256;
    a.row_bytes = FMT == RUNIT_FMT_Q5_0 ? (k / 32) * 22 : (k / 256) * (uint32_t)KTraits<FMT>::UB;
    uint32_t grid = (m + kWarps - 1) / kWarps;
    const uint32_t cap = (uint32_t)ctx->sm_count * 8u;   // 64 warps per SM
    if (grid > cap) grid = cap;
    runit_launch_chain(ctx, gemv_kquant_kernel<FMT>, dim3(grid), dim3(kWarps * 32), a);
    return runit_after_launch(ctx, name);
}

}  // namespace kq
}  // namespace runit

using namespace runit;

extern "C" {

int32_t runit_gemv_q5_0_f32in_f32out(runit_ctx_t* ctx, const void* w, const void* x, void* y, uint32_t m, uint32_t k) {
    return kq::launch<RUNIT_FMT_Q5_0>(ctx, "gemv_q5_0_f32in_f32out", w, x, y, nullptr, m, k);
}
int32_t runit_gemv_q5_0_add_f32_f32in(runit_ctx_t* ctx, const void* w, const void* x, void* y, const void* r, uint32_t m, uint32_t k) {
    if (ctx) RUNIT_REQUIRE(ctx, r, "gemv_q5_0_add_f32_f32in: null residual");
    return kq::launch<RUNIT_FMT_Q5_0>(ctx, "gemv_q5_0_add_f32_f32in", w, x, y, r, m, k);
}
int32_t runit_gemv_q5k_f32in_f32out(runit_ctx_t* ctx, const void* w, const void* x, void* y, uint32_t m, uint32_t k) {
    return kq::launch<RUNIT_FMT_Q5K>(ctx, "gemv_q5k_f32in_f32out", w, x, y, nullptr, m, k);
}
int32_t runit_gemv_q5k_add_f32_f32in(runit_ctx_t* ctx, const void* w, const void* x, void* y, const void* r, uint32_t m, uint32_t k) {
    if (ctx) RUNIT_REQUIRE(ctx, r, "gemv_q5k_add_f32_f32in: null residual");
    return kq::launch<RUNIT_FMT_Q5K>(ctx, "gemv_q5k_add_f32_f32in", w, x, y, r, m, k);
}
int32_t runit_gemv_q6k_f32in_f32out(runit_ctx_t* ctx, const void* w, const void* x, void* y, uint32_t m, uint32_t k) {
    return kq::launch<RUNIT_FMT_Q6K>(ctx, "gemv_q6k_f32in_f32out", w, x, y, nullptr, m, k);
}
int32_t runit_gemv_q6k_add_f32_f32in(runit_ctx_t* ctx, const void* w, const void* x, void* y, const void* r, uint32_t m, uint32_t k) {
    if (ctx) RUNIT_REQUIRE(ctx, r, "gemv_q6k_add_f32_f32in: null residual");
    return kq::launch<RUNIT_FMT_Q6K>(ctx, "gemv_q6k_add_f32_f32in", w, x, y, r, m, k);
}

}  // extern "C"
