// Internal definitions shared by the translation units of librunit_cuda.so.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>

#include <cstdint>
#include <cstdio>
#include <cstring>

#include "runit_cuda.h"

struct runit_tuning {
    int32_t gemv_variant = 0;   // 0 = staged kernel, 1 = simple warp-per-row kernel
    int32_t gemv_stages = 0;    // 0 = default
    int32_t moe_variant = 0;
    int32_t pdl = 0;            // programmatic dependent launch between ops
};

// One per GPU; replaces the reference's MetalContext (crates/kernels/src/context.rs:137-160).
struct runit_ctx {
    int32_t device = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int32_t sm_count = 0;
    int32_t max_smem_optin = 0;
    uint64_t launches = 0;
    int32_t sticky_status = RUNIT_OK;   // first error since the last flush
    char err[512] = {0};
    runit_tuning tune;
    // Device scratch owned by the context (allocated at creation; ops never allocate).
    int32_t* d_status = nullptr;        // status word written by kernels with bounded waits
};

const char* runit_status_name(int32_t st);

// Record an error in the context (first one sticks) and return its status.
int32_t runit_fail(runit_ctx* ctx, int32_t st, const char* fmt, ...);

#define RUNIT_CUDA_TRY(ctx, expr)                                                              \
    do {                                                                                       \
        cudaError_t e__ = (expr);                                                              \
        if (e__ != cudaSuccess)                                                                \
            return runit_fail((ctx), RUNIT_ERR_LAUNCH, "%s: %s (%s:%d)", #expr,                \
                              cudaGetErrorString(e__), __FILE__, __LINE__);                    \
    } while (0)

#define RUNIT_REQUIRE(ctx, cond, ...)                                                          \
    do {                                                                                       \
        if (!(cond)) return runit_fail((ctx), RUNIT_ERR_BAD_ARG, __VA_ARGS__);                 \
    } while (0)

// Checks the launch that was just issued and counts it.
static inline int32_t runit_after_launch(runit_ctx* ctx, const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return runit_fail(ctx, RUNIT_ERR_LAUNCH, "launch of %s failed: %s", what, cudaGetErrorString(e));
    ctx->launches++;
    return RUNIT_OK;
}

static inline bool runit_aligned(const void* p, size_t a) {
    return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0;
}

static inline size_t runit_block_elems(int fmt) { return fmt == RUNIT_FMT_Q4K ? 256 : 32; }
static inline size_t runit_block_bytes(int fmt) {
    return fmt == RUNIT_FMT_Q8_0 ? 34 : (fmt == RUNIT_FMT_Q4_0 ? 18 : 144);
}
static inline size_t runit_row_bytes(int fmt, uint32_t k) {
    return (size_t)k / runit_block_elems(fmt) * runit_block_bytes(fmt);
}
