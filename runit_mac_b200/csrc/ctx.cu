// Context, buffers, flush and error reporting.
//
// Replaces MetalContext::{new, new_buffer, encode, flush} of the reference
// (crates/kernels/src/context.rs:163-296): one in-order CUDA stream instead of a Metal
// command buffer; runit_flush == commit + wait_until_completed.
#include "runit_internal.h"

#include <cstdarg>
#include <cstdlib>
#include <new>

const char* runit_status_name(int32_t st) {
    switch (st) {
        case RUNIT_OK: return "RUNIT_OK";
        case RUNIT_ERR_NO_DEVICE: return "RUNIT_ERR_NO_DEVICE";
        case RUNIT_ERR_BAD_ARG: return "RUNIT_ERR_BAD_ARG";
        case RUNIT_ERR_BUFFER_SIZE: return "RUNIT_ERR_BUFFER_SIZE";
        case RUNIT_ERR_LAUNCH: return "RUNIT_ERR_LAUNCH";
        case RUNIT_ERR_NCCL: return "RUNIT_ERR_NCCL";
        case RUNIT_ERR_TIMEOUT: return "RUNIT_ERR_TIMEOUT";
        case RUNIT_ERR_UNSUPPORTED: return "RUNIT_ERR_UNSUPPORTED";
        case RUNIT_ERR_ALLOC: return "RUNIT_ERR_ALLOC";
        default: return "RUNIT_ERR_UNKNOWN";
    }
}

int32_t runit_fail(runit_ctx* ctx, int32_t st, const char* fmt, ...) {
    if (ctx) {
        if (ctx->sticky_status == RUNIT_OK) ctx->sticky_status = st;
        va_list ap;
        va_start(ap, fmt);
        int n = snprintf(ctx->err, sizeof(ctx->err), "%s: ", runit_status_name(st));
        if (n < 0) n = 0;
        vsnprintf(ctx->err + n, sizeof(ctx->err) - (size_t)n, fmt, ap);
        va_end(ap);
    }
    return st;
}

static int32_t ctx_init(int32_t device, cudaStream_t adopt, bool adopt_stream, runit_ctx_t** out) {
    if (!out) return RUNIT_ERR_BAD_ARG;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) return RUNIT_ERR_NO_DEVICE;
    if (device < 0 || device >= n) return RUNIT_ERR_NO_DEVICE;
    if (cudaSetDevice(device) != cudaSuccess) return RUNIT_ERR_NO_DEVICE;
    runit_ctx* c = new (std::nothrow) runit_ctx();
    if (!c) return RUNIT_ERR_ALLOC;
    c->device = device;
    cudaDeviceProp p;
    if (cudaGetDeviceProperties(&p, device) != cudaSuccess) {
        delete c;
        return RUNIT_ERR_NO_DEVICE;
    }
    if (p.major != 10) {
        // Kernels are built for sm_100a only; there is no other code path.
        delete c;
        return RUNIT_ERR_UNSUPPORTED;
    }
    c->sm_count = p.multiProcessorCount;
    c->max_smem_optin = (int32_t)p.sharedMemPerBlockOptin;
    if (adopt_stream) {
        c->stream = adopt;
        c->owns_stream = false;
    } else {
        if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) {
            delete c;
            return RUNIT_ERR_LAUNCH;
        }
        c->owns_stream = true;
    }
    if (cudaMalloc(&c->d_status, 64) != cudaSuccess) {
        if (c->owns_stream) cudaStreamDestroy(c->stream);
        delete c;
        return RUNIT_ERR_ALLOC;
    }
    cudaMemsetAsync(c->d_status, 0, 64, c->stream);
    const char* v = getenv("RUNIT_GEMV_VARIANT");
    if (v) c->tune.gemv_variant = atoi(v);
    *out = c;
    return RUNIT_OK;
}

extern "C" {

int32_t runit_ctx_create(int32_t device, runit_ctx_t** out) { return ctx_init(device, nullptr, false, out); }

int32_t runit_ctx_create_on_stream(int32_t device, void* cuda_stream, runit_ctx_t** out) {
    return ctx_init(device, (cudaStream_t)cuda_stream, true, out);
}

int32_t runit_ctx_destroy(runit_ctx_t* ctx) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);   // Drop flushes, context.rs:299-304
    if (ctx->d_status) cudaFree(ctx->d_status);
    if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return RUNIT_OK;
}

void* runit_ctx_stream(runit_ctx_t* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

int32_t runit_flush(runit_ctx_t* ctx) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) runit_fail(ctx, RUNIT_ERR_LAUNCH, "stream synchronize: %s", cudaGetErrorString(e));
    int32_t st = ctx->sticky_status;
    ctx->sticky_status = RUNIT_OK;   // the message stays readable until the next error
    return st;
}

const char* runit_last_error_string(runit_ctx_t* ctx) { return ctx ? ctx->err : "null context"; }

const char* runit_status_string(int32_t status) { return runit_status_name(status); }

uint64_t runit_launch_count(runit_ctx_t* ctx) { return ctx ? ctx->launches : 0; }

int32_t runit_set_tuning(runit_ctx_t* ctx, const char* key, int32_t value) {
    if (!ctx || !key) return RUNIT_ERR_BAD_ARG;
    if (!strcmp(key, "gemv_variant")) ctx->tune.gemv_variant = value;
    else if (!strcmp(key, "gemv_stages")) ctx->tune.gemv_stages = value;
    else if (!strcmp(key, "moe_variant")) ctx->tune.moe_variant = value;
    else if (!strcmp(key, "pdl")) ctx->tune.pdl = value;
    else return runit_fail(ctx, RUNIT_ERR_BAD_ARG, "unknown tuning key '%s'", key);
    return RUNIT_OK;
}

int32_t runit_buf_alloc(runit_ctx_t* ctx, size_t bytes, int32_t flags, void** dptr) {
    if (!ctx || !dptr) return RUNIT_ERR_BAD_ARG;
    *dptr = nullptr;
    if (bytes == 0) return runit_fail(ctx, RUNIT_ERR_BAD_ARG, "runit_buf_alloc: zero bytes");
    RUNIT_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    cudaError_t e;
    if (flags & RUNIT_BUF_HOST_VISIBLE) {
        // Pinned, device-mapped host memory: readable and writable from the CPU between
        // flushes, like the reference's StorageModeShared buffers (context.rs:215-220).
        e = cudaHostAlloc(dptr, bytes, cudaHostAllocMapped | cudaHostAllocPortable);
    } else {
        e = cudaMalloc(dptr, bytes);
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        return runit_fail(ctx, RUNIT_ERR_ALLOC, "allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    }
    return RUNIT_OK;
}

int32_t runit_buf_free(runit_ctx_t* ctx, void* dptr) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    if (!dptr) return RUNIT_OK;
    cudaPointerAttributes a;
    cudaError_t e = cudaPointerGetAttributes(&a, dptr);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return runit_fail(ctx, RUNIT_ERR_BAD_ARG, "runit_buf_free: not a buffer of this library");
    }
    cudaStreamSynchronize(ctx->stream);
    if (a.type == cudaMemoryTypeHost) RUNIT_CUDA_TRY(ctx, cudaFreeHost(dptr));
    else RUNIT_CUDA_TRY(ctx, cudaFree(dptr));
    return RUNIT_OK;
}

int32_t runit_memcpy_h2d(runit_ctx_t* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, dst && src, "runit_memcpy_h2d: null pointer");
    if (bytes == 0) return RUNIT_OK;
    RUNIT_CUDA_TRY(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return RUNIT_OK;
}

int32_t runit_memcpy_d2h(runit_ctx_t* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, dst && src, "runit_memcpy_d2h: null pointer");
    if (bytes == 0) return RUNIT_OK;
    RUNIT_CUDA_TRY(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return RUNIT_OK;
}

int32_t runit_memset(runit_ctx_t* ctx, void* dst, int32_t byte, size_t bytes) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, dst, "runit_memset: null pointer");
    if (bytes == 0) return RUNIT_OK;
    RUNIT_CUDA_TRY(ctx, cudaMemsetAsync(dst, byte, bytes, ctx->stream));
    return RUNIT_OK;
}

}  // extern "C"
