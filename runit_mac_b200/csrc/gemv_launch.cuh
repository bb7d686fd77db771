// Template launchers of the staged and simple GEMV kernels; instantiated once per weight
// format in gemv_q8_0.cu / gemv_q4_0.cu / gemv_q4k.cu so the formats compile in parallel.
#pragma once

#include "gemv_kernels.cuh"
#include "runit_internal.h"

namespace runit {

template <int FMT, int B, bool XF16, int CPB, int S, bool DUAL, int LD>
static inline int32_t launch_staged(runit_ctx* ctx, const GemvArgs& a, const GemvMaps& maps, uint32_t tiles,
                                    const char* name) {
    using L = WarpStage<FMT, B, XF16>;
    constexpr int smem = kKS * S * L::BYTES + 128;   // + slack to align the rings to 128 bytes
    static_assert(smem <= 227 * 1024, "stage rings exceed shared memory");
    auto kern = gemv_staged_kernel<FMT, B, XF16, CPB, S, DUAL, LD>;
    static bool configured[16] = {false};
    if (ctx->device < 16 && !configured[ctx->device]) {
        RUNIT_CUDA_TRY(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured[ctx->device] = true;
    }
    kern<<<tiles, kNT, smem, ctx->stream>>>(a, maps);
    return runit_after_launch(ctx, name);
}

template <int FMT, int B, bool XF16, int CPB, int LD>
static inline int32_t pick_stages(runit_ctx* ctx, const GemvArgs& a, const GemvMaps& maps, uint32_t tiles,
                                  const char* name) {
    if constexpr (B == 1 && !XF16) {
        if (a.dual) {
            if constexpr (FMT != RUNIT_FMT_Q4K)
                return launch_staged<FMT, 1, false, CPB, 3, true, LD>(ctx, a, maps, tiles, name);
            else
                return runit_fail(ctx, RUNIT_ERR_UNSUPPORTED, "%s: no fused gate/up kernel for Q4_K", name);
        }
        if (ctx->tune.gemv_stages == 4) return launch_staged<FMT, 1, false, CPB, 4, false, LD>(ctx, a, maps, tiles, name);
    }
    if (a.dual) return runit_fail(ctx, RUNIT_ERR_UNSUPPORTED, "%s: fused gate/up is batch 1, f32 input", name);
    return launch_staged<FMT, B, XF16, CPB, 3, false, LD>(ctx, a, maps, tiles, name);
}

template <int FMT, int B, bool XF16>
static inline int32_t pick_copy(runit_ctx* ctx, const GemvArgs& a, const GemvMaps& maps, uint32_t tiles, int cpb,
                                bool tma, const char* name) {
    if constexpr (FMT == RUNIT_FMT_Q8_0) {
        // Q8_0 rows (34-byte blocks) are only 8- or 4-byte aligned in general and the unit (136 bytes)
        // is not a multiple of 16, so Q8_0 uses per-thread 8- or 4-byte cp.async copies.
        (void)tma;
        if (cpb >= 8) return pick_stages<FMT, B, XF16, 8, 0>(ctx, a, maps, tiles, name);
        return pick_stages<FMT, B, XF16, 4, 0>(ctx, a, maps, tiles, name);
    } else {
        (void)cpb;   // the 4-bit formats take the staged path only with 16-byte aligned rows
        if (tma) return pick_stages<FMT, B, XF16, 16, 1>(ctx, a, maps, tiles, name);
        return pick_stages<FMT, B, XF16, 16, 0>(ctx, a, maps, tiles, name);
    }
}

// Batches other than 1, 2, 4, 8 are issued as several launches over sub-batches.
template <int FMT>
static inline int32_t launch_fmt(runit_ctx* ctx, const GemvArgs& a, const GemvMaps& maps, uint32_t tiles, int cpb,
                                 bool tma, uint32_t batch, bool xf16, const char* name) {
    if (xf16) {
        if (batch != 1) return runit_fail(ctx, RUNIT_ERR_UNSUPPORTED, "%s: f16 input supports batch 1 only", name);
        return pick_copy<FMT, 1, true>(ctx, a, maps, tiles, cpb, tma, name);
    }
    switch (batch) {
        case 1: return pick_copy<FMT, 1, false>(ctx, a, maps, tiles, cpb, tma, name);
        case 2: return pick_copy<FMT, 2, false>(ctx, a, maps, tiles, cpb, tma, name);
        case 4: return pick_copy<FMT, 4, false>(ctx, a, maps, tiles, cpb, tma, name);
        case 8: return pick_copy<FMT, 8, false>(ctx, a, maps, tiles, cpb, tma, name);
        default: return runit_fail(ctx, RUNIT_ERR_UNSUPPORTED, "%s: batch %u not in {1,2,4,8}", name, batch);
    }
}

template <int FMT>
static inline int32_t launch_simple(runit_ctx* ctx, const GemvArgs& a, uint32_t total_rows, uint32_t batch, bool xf16,
                             const char* name) {
    const uint32_t grid = (total_rows + 3) / 4;
    if (xf16) gemv_simple_kernel<FMT, true><<<grid, 128, 0, ctx->stream>>>(a, (int)batch);
    else gemv_simple_kernel<FMT, false><<<grid, 128, 0, ctx->stream>>>(a, (int)batch);
    return runit_after_launch(ctx, name);
}


// Per-format entry points (defined in gemv_<fmt>.cu).
int32_t gemv_launch_q8_0(runit_ctx* ctx, const GemvArgs& a, const GemvMaps& maps, uint32_t tiles, uint32_t total_rows,
                         int cpb, bool tma, uint32_t batch, bool xf16, bool simple, const char* name);
int32_t gemv_launch_q4_0(runit_ctx* ctx, const GemvArgs& a, const GemvMaps& maps, uint32_t tiles, uint32_t total_rows,
                         int cpb, bool tma, uint32_t batch, bool xf16, bool simple, const char* name);
int32_t gemv_launch_q4k(runit_ctx* ctx, const GemvArgs& a, const GemvMaps& maps, uint32_t tiles, uint32_t total_rows,
                         int cpb, bool tma, uint32_t batch, bool xf16, bool simple, const char* name);

}  // namespace runit
