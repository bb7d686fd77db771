// Template launchers of the staged and simple GEMV kernels; instantiated once per weight
// format in gemv_q8_0.cu / gemv_q4_0.cu / gemv_q4k.cu so the formats compile in parallel.
#pragma once

#include "gemv_kernels.cuh"
#include "gemv_stream_host.h"
#include "runit_internal.h"

namespace runit {

template <int FMT, int B, bool XF16, int CPB, int S, bool DUAL, int LD, int KSL, int MATH>
static inline int32_t launch_staged(runit_ctx* ctx, const GemvArgs& a, const GemvMaps& maps, const char* name) {
    using L = WarpStage<FMT, B, XF16>;
    constexpr int smem = kKS * S * L::BYTES + 128;   // + slack to align the rings to 128 bytes
    static_assert(smem <= 227 * 1024, "stage rings exceed shared memory");
    auto kern = gemv_staged_kernel<FMT, B, XF16, CPB, S, DUAL, LD, KSL, MATH>;
    static bool configured[16] = {false};
    if (ctx->device < 16 && !configured[ctx->device]) {
        RUNIT_CUDA_TRY(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured[ctx->device] = true;
    }
    constexpr uint32_t tpc = kKS / KSL;
    GemvArgs args = a;
    // Few-tile shapes (fewer CTAs than ~2 per SM) with a long K: split K over a thread-block cluster of 2 or 4
    // CTAs per tile so that every SM has warps to run; partial sums meet through distributed shared memory.
    uint32_t csplit = 1;
    if (KSL == 4 && !ctx->tune.gemv_no_cluster) {
        const uint32_t ctas = a.n_tiles;
        if (ctx->tune.gemv_csplit == 2 || ctx->tune.gemv_csplit == 4) csplit = ctx->tune.gemv_csplit;
        else if (ctas < 2u * (uint32_t)ctx->sm_count) csplit = a.n_units >= 24 ? 4 : (a.n_units >= 12 ? 2 : 1);
        if (4 * csplit > a.n_units) csplit = 1;
    }
    args.csplit = csplit;
    const uint32_t grid = ((a.n_tiles + tpc - 1) / tpc) * csplit;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kNT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    // Dependent launch pays except for grids of about one CTA per SM, which were measured 15-25% slower with it
    // (the early CTAs of the next grid double up on busy SMs instead of spreading out).
    const uint32_t sms = (uint32_t)ctx->sm_count;
    const bool pdl = ctx->tune.pdl == 1 || (ctx->tune.pdl == 2 && (grid < (2 * sms) / 3 || grid > (4 * sms) / 3));
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    if (csplit > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = csplit;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        na++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, args, maps);
    if (e != cudaSuccess) return runit_fail(ctx, RUNIT_ERR_LAUNCH, "launch of %s failed: %s", name, cudaGetErrorString(e));
    // While a command list is recorded, launches of this kind are noted: when the recording ends, runs of consecutive
    // ones are folded into one persistent launch (gemv_stream.cu).
    if constexpr (FMT != RUNIT_FMT_Q8_0 && B == 1 && !XF16 && LD == 1 && MATH == 2) {
        if (ctx->capturing && ctx->tune.stream_fuse && a.grp_expert == nullptr && a.n_peer == 0 && a.res_kind != RES_F16 &&
            a.norm_gamma == nullptr && a.am_part == nullptr) {
            StreamRec r;
            memset(&r, 0, sizeof(r));
            r.func = reinterpret_cast<const void*>(kern);
            r.w0 = a.seg[0].w;
            r.x = a.x;
            r.fmt = FMT;
            r.dual = DUAL ? 1 : 0;
            r.nseg = a.nseg;
            for (int i = 0; i < a.nseg && i < 3; i++) {
                r.map[i] = maps.m[i];
                r.y[i] = a.seg[i].y;
                r.res[i] = a.seg[i].res;
                r.bias[i] = a.seg[i].bias;
                r.rows[i] = a.seg[i].rows;
            }
            if (DUAL) r.map[3] = maps.m[3];
            r.k = a.k;
            r.nb = a.nb;
            r.n_units = a.n_units;
            r.out_f16 = a.out_f16;
            r.res_kind = a.res_kind;
            r.bias_kind = a.bias_kind;
            stream_rec_push(ctx, r);
        }
    }
    return runit_after_launch(ctx, name);
}

// K-slices per tile: the largest of 4, 2, 1 that divides the unit count evenly among the warps
// (e.g. k=3584 has 14 units: 2 warps x 7 units instead of 4 warps with 4,4,3,3), unless there are
// too few tiles to fill the GPU, in which case 4 slices keep more warps busy.
template <int FMT, int B, bool XF16, int CPB, int S, bool DUAL, int LD, int MATH>
static inline int32_t pick_slices(runit_ctx* ctx, const GemvArgs& a, const GemvMaps& maps, const char* name) {
    int ksl = 4;
    if (ctx->tune.gemv_ksl == 1 || ctx->tune.gemv_ksl == 2 || ctx->tune.gemv_ksl == 4) ksl = ctx->tune.gemv_ksl;
    else if (a.n_units % 4 != 0 && a.n_tiles >= (uint32_t)ctx->sm_count * 4) ksl = (a.n_units % 2 == 0) ? 2 : 1;
    if constexpr (B == 1) {
        if (ksl == 2) return launch_staged<FMT, B, XF16, CPB, S, DUAL, LD, 2, MATH>(ctx, a, maps, name);
        if constexpr (!DUAL) {
            if (ksl == 1) return launch_staged<FMT, B, XF16, CPB, S, DUAL, LD, 1, MATH>(ctx, a, maps, name);
        }
    }
    return launch_staged<FMT, B, XF16, CPB, S, DUAL, LD, 4, MATH>(ctx, a, maps, name);
}

// Batch 1: integer tensor-core MMAs for the 4-bit formats, dp4a for Q8_0 (tuning knob gemv_math: 1 = packed f32,
// 2 = dp4a for every format).
template <int FMT, int B, bool XF16, int CPB, int S, bool DUAL, int LD>
static inline int32_t pick_math(runit_ctx* ctx, const GemvArgs& a, const GemvMaps& maps, const char* name) {
    if constexpr (B == 1) {
        if constexpr (FMT != RUNIT_FMT_Q8_0) {
            if (ctx->tune.gemv_math == 0 || ctx->tune.gemv_math == 3) return pick_slices<FMT, B, XF16, CPB, S, DUAL, LD, 2>(ctx, a, maps, name);
        }
        if (ctx->tune.gemv_math != 1) return pick_slices<FMT, B, XF16, CPB, S, DUAL, LD, 1>(ctx, a, maps, name);
    }
    return pick_slices<FMT, B, XF16, CPB, S, DUAL, LD, 0>(ctx, a, maps, name);
}

template <int FMT, int B, bool XF16, int CPB, int LD>
static inline int32_t pick_stages(runit_ctx* ctx, const GemvArgs& a, const GemvMaps& maps, const char* name) {
    if constexpr (B == 1 && !XF16) {
        if (a.dual) return pick_math<FMT, 1, false, CPB, 2, true, LD>(ctx, a, maps, name);
        // Two stages per warp leave room for 4 CTAs (16 warps) per SM, which hides more latency than a
        // deeper ring with 12 warps; measured best on every large shape.
        if (ctx->tune.gemv_stages == 3) return pick_math<FMT, 1, false, CPB, 3, false, LD>(ctx, a, maps, name);
        return pick_math<FMT, 1, false, CPB, 2, false, LD>(ctx, a, maps, name);
    }
    if (a.dual) return runit_fail(ctx, RUNIT_ERR_UNSUPPORTED, "%s: fused gate/up is batch 1, f32 input", name);
    if constexpr (B == 1) return pick_math<FMT, B, XF16, CPB, 2, false, LD>(ctx, a, maps, name);
    else return pick_slices<FMT, B, XF16, CPB, 3, false, LD, 0>(ctx, a, maps, name);
}

template <int FMT, int B, bool XF16>
static inline int32_t pick_copy(runit_ctx* ctx, const GemvArgs& a, const GemvMaps& maps, uint32_t tiles, int cpb,
                                bool tma, const char* name) {
    if constexpr (FMT == RUNIT_FMT_Q8_0) {
        // Q8_0 rows (34-byte blocks) are only 8- or 4-byte aligned in general and the unit (136 bytes)
        // is not a multiple of 16, so Q8_0 uses per-thread 8- or 4-byte cp.async copies.
        (void)tma;
        if (cpb >= 8) return pick_stages<FMT, B, XF16, 8, 0>(ctx, a, maps, name);
        return pick_stages<FMT, B, XF16, 4, 0>(ctx, a, maps, name);
    } else {
        (void)cpb;   // the 4-bit formats take the staged path only with 16-byte aligned rows
        if (tma) return pick_stages<FMT, B, XF16, 16, 1>(ctx, a, maps, name);
        return pick_stages<FMT, B, XF16, 16, 0>(ctx, a, maps, name);
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
