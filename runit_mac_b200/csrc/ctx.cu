// Context, buffers, flush and error reporting.
//
// Replaces MetalContext::{new, new_buffer, encode, flush} of the reference
// (crates/kernels/src/context.rs:163-296): one in-order CUDA stream instead of a Metal
// command buffer; runit_flush == commit + wait_until_completed.
#include "gemv_stream_host.h"
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
        // Argument errors are reported to the caller at once and launch nothing; only failures of
        // work that was already accepted are kept for the next flush.
        const bool async_kind = st == RUNIT_ERR_LAUNCH || st == RUNIT_ERR_NCCL || st == RUNIT_ERR_TIMEOUT;
        if (async_kind && ctx->sticky_status == RUNIT_OK) ctx->sticky_status = st;
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
    // Status word for kernels with bounded waits: pinned host memory mapped into the device, so
    // the host reads it after a flush without a copy.
    if (cudaHostAlloc((void**)&c->h_status, 64, cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer((void**)&c->d_status, c->h_status, 0) != cudaSuccess) {
        cudaGetLastError();
        if (c->owns_stream) cudaStreamDestroy(c->stream);
        delete c;
        return RUNIT_ERR_ALLOC;
    }
    memset(c->h_status, 0, 64);
    if (cudaMalloc((void**)&c->d_abort, 64) != cudaSuccess || cudaMemset(c->d_abort, 0, 64) != cudaSuccess) {
        cudaGetLastError();
        cudaFreeHost(c->h_status);
        if (c->owns_stream) cudaStreamDestroy(c->stream);
        delete c;
        return RUNIT_ERR_ALLOC;
    }
    // Staging area of the batched GEMV (its activations, quantised once per call): 4 MiB = K up to 232,960.
    // Greedy epilogue of the GEMV: 65536 tile pairs (2,097,152 rows) behind a zeroed ticket word.
    if (cudaMalloc(&c->d_am, 256 + 65536 * 8) == cudaSuccess) cudaMemset(c->d_am, 0, 256);
    else { c->d_am = nullptr; cudaGetLastError(); }
    if (cudaMalloc((void**)&c->d_xq_ctl, 4096) == cudaSuccess) cudaMemset(c->d_xq_ctl, 0, 4096);
    else { c->d_xq_ctl = nullptr; cudaGetLastError(); }
    if (cudaMalloc(&c->d_kq, 8192 + (1u << 20)) == cudaSuccess) cudaMemset(c->d_kq, 0, 8192);
    else { c->d_kq = nullptr; cudaGetLastError(); }
    if (cudaMalloc(&c->d_xq, 4u << 20) == cudaSuccess) c->xq_bytes = 4u << 20;
    else { c->d_xq = nullptr; cudaGetLastError(); }
    {
        cudaDriverEntryPointQueryResult qres;
        void* fn = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            c->encode_tiled = fn;
        else
            cudaGetLastError();
    }
    c->tune.pdl = 2;   // dependent launch where it was measured to pay (see gemv_launch.cuh)
    const char* v = getenv("RUNIT_GEMV_VARIANT");
    if (v) c->tune.gemv_variant = atoi(v);
    *out = c;
    return RUNIT_OK;
}

int32_t runit_get_tmap(runit_ctx* ctx, const void* ptr, uint64_t rows, uint64_t row_bytes, uint32_t box_rows,
                       uint32_t box_bytes, CUtensorMap* out, uint32_t swizzle128) {
    if (!ctx->encode_tiled) return runit_fail(ctx, RUNIT_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled is not available");
    uint64_t h = (reinterpret_cast<uintptr_t>(ptr) >> 8) * 0x9E3779B97F4A7C15ull ^ (rows * 31 + row_bytes * 7 + box_rows + swizzle128 * 131);
    runit_tmap_entry& e = ctx->tmaps[(h >> 32) & 255];
    if (e.ptr == ptr && e.rows == rows && e.row_bytes == row_bytes && e.box_rows == box_rows && e.box_bytes == box_bytes &&
        e.swizzle128 == swizzle128) {
        *out = e.map;
        return RUNIT_OK;
    }
    auto encode = reinterpret_cast<CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill)>(
        ctx->encode_tiled);
    const cuuint64_t gdim[2] = {row_bytes, rows};
    const cuuint64_t gstride[1] = {row_bytes};
    const cuuint32_t box[2] = {box_bytes, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap m;
    CUresult r = encode(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return runit_fail(ctx, RUNIT_ERR_LAUNCH, "cuTensorMapEncodeTiled failed with %d", (int)r);
    e.ptr = ptr; e.rows = rows; e.row_bytes = row_bytes; e.box_rows = box_rows; e.box_bytes = box_bytes; e.swizzle128 = swizzle128; e.map = m;
    *out = m;
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
    if (ctx->h_status) cudaFreeHost(ctx->h_status);
    if (ctx->d_xq) cudaFree(ctx->d_xq);
    if (ctx->d_am) cudaFree(ctx->d_am);
    if (ctx->d_xq_ctl) cudaFree(ctx->d_xq_ctl);
    if (ctx->d_kq) cudaFree(ctx->d_kq);
    if (ctx->d_abort) cudaFree(ctx->d_abort);
    if (ctx->stream_rec) delete static_cast<std::vector<runit::StreamRec>*>(ctx->stream_rec);
    if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return RUNIT_OK;
}

void* runit_ctx_stream(runit_ctx_t* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

int32_t runit_flush(runit_ctx_t* ctx) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) runit_fail(ctx, RUNIT_ERR_LAUNCH, "stream synchronize: %s", cudaGetErrorString(e));
    if (ctx->h_status && ctx->h_status[0] != 0) {
        const int32_t why = ctx->h_status[0];
        ctx->h_status[0] = 0;
        if (ctx->d_abort) cudaMemset(ctx->d_abort, 0, 4);   // the stream is idle: barriers wait again after this report
        if (why == 4) {
            runit_fail(ctx, RUNIT_ERR_UNSUPPORTED, "sampler: top-k is off and the nucleus is wider than the 1024 most probable tokens (code %d)", why);
            if (ctx->sticky_status == RUNIT_OK) ctx->sticky_status = RUNIT_ERR_UNSUPPORTED;   // reported by this flush
        } else
        runit_fail(ctx, RUNIT_ERR_TIMEOUT, why == 3 ? "a peer barrier gave up: a rank never announced its epoch (code %d)"
                                                    : "a kernel gave up a bounded wait (a copy or a dependency never completed; code %d)", why);
    }
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
    else if (!strcmp(key, "pdl")) ctx->tune.pdl = value;
    else if (!strcmp(key, "gemv_load")) ctx->tune.gemv_load = value;
    else if (!strcmp(key, "gemv_ksl")) ctx->tune.gemv_ksl = value;
    else if (!strcmp(key, "gemv_csplit")) ctx->tune.gemv_csplit = value;
    else if (!strcmp(key, "gemv_math")) ctx->tune.gemv_math = value;
    else if (!strcmp(key, "gemv_no_cluster")) ctx->tune.gemv_no_cluster = value;
    else if (!strcmp(key, "stream_fuse")) ctx->tune.stream_fuse = value;
    else if (!strcmp(key, "stream_cfg")) ctx->tune.stream_cfg = value;
    else if (!strcmp(key, "stream_ksl")) ctx->tune.stream_ksl = value;
    else if (!strcmp(key, "stream_dynamic")) ctx->tune.stream_dynamic = value;
    else if (!strcmp(key, "router_variant")) ctx->tune.router_variant = value;
    else if (!strcmp(key, "ep_fused_exchange")) ctx->tune.ep_fused_exchange = value;
    else if (!strcmp(key, "imma_fold")) ctx->tune.imma_fold = value;
    else if (!strcmp(key, "imma_rw")) ctx->tune.imma_rw = value;
    else if (!strcmp(key, "imma_csplit")) ctx->tune.imma_csplit = value;
    else if (!strcmp(key, "imma_stages")) ctx->tune.imma_stages = value;
    else if (!strcmp(key, "kquant_variant")) ctx->tune.kquant_variant = value;
    else if (!strcmp(key, "kquant_split")) ctx->tune.kquant_split = value;
    else return runit_fail(ctx, RUNIT_ERR_BAD_ARG, "unknown tuning key '%s'", key);
    return RUNIT_OK;
}

// CUDA graphs stand in for the reference's encoded command buffer: record once, replay per token.  Runs of consecutive
// batch-1 GEMVs of a recording are folded into one persistent launch (gemv_stream.cu) before the graph is instantiated.
struct runit_graph {
    cudaGraphExec_t exec = nullptr;
    std::vector<void*> allocs;      // device memory of the fused GEMV programs
    uint32_t fused_launches = 0;
    uint32_t kernel_nodes = 0;      // kernel launches one replay performs
};

int32_t runit_graph_begin(runit_ctx_t* ctx) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, !ctx->capturing, "runit_graph_begin: a recording is already open");
    RUNIT_CUDA_TRY(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    ctx->capturing = true;
    runit::stream_rec_begin(ctx);
    return RUNIT_OK;
}

int32_t runit_graph_end(runit_ctx_t* ctx, runit_graph_t** out) {
    if (!ctx || !out) return RUNIT_ERR_BAD_ARG;
    *out = nullptr;
    RUNIT_REQUIRE(ctx, ctx->capturing, "runit_graph_end: no recording is open");
    ctx->capturing = false;
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &g);
    if (e != cudaSuccess || !g) {
        cudaGetLastError();
        runit::stream_rec_discard(ctx);
        return runit_fail(ctx, RUNIT_ERR_LAUNCH, "cudaStreamEndCapture: %s", cudaGetErrorString(e));
    }
    runit_graph* gr = new (std::nothrow) runit_graph();
    if (!gr) {
        cudaGraphDestroy(g);
        runit::stream_rec_discard(ctx);
        return RUNIT_ERR_ALLOC;
    }
    int32_t st = runit::stream_rec_fuse(ctx, g, &gr->allocs, &gr->fused_launches);
    runit::stream_rec_discard(ctx);
    if (st == RUNIT_OK) {
        size_t n_nodes = 0;
        if (cudaGraphGetNodes(g, nullptr, &n_nodes) == cudaSuccess && n_nodes > 0) {
            std::vector<cudaGraphNode_t> nodes(n_nodes);
            if (cudaGraphGetNodes(g, nodes.data(), &n_nodes) == cudaSuccess)
                for (size_t i = 0; i < n_nodes; i++) {
                    cudaGraphNodeType ty;
                    if (cudaGraphNodeGetType(nodes[i], &ty) == cudaSuccess && ty == cudaGraphNodeTypeKernel) gr->kernel_nodes++;
                }
        }
        cudaGetLastError();
        e = cudaGraphInstantiate(&gr->exec, g, 0);
        if (e != cudaSuccess) st = runit_fail(ctx, RUNIT_ERR_LAUNCH, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
    }
    cudaGraphDestroy(g);
    if (st != RUNIT_OK) {
        for (void* p : gr->allocs) cudaFree(p);
        delete gr;
        return st;
    }
    *out = gr;
    return RUNIT_OK;
}

int32_t runit_graph_launch(runit_ctx_t* ctx, runit_graph_t* graph) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, graph && graph->exec, "runit_graph_launch: null graph");
    RUNIT_CUDA_TRY(ctx, cudaGraphLaunch(graph->exec, ctx->stream));
    return RUNIT_OK;
}

int32_t runit_graph_destroy(runit_ctx_t* ctx, runit_graph_t* graph) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    if (!graph) return RUNIT_OK;
    cudaStreamSynchronize(ctx->stream);   // a replay may still be running on the program memory
    if (graph->exec) cudaGraphExecDestroy(graph->exec);
    for (void* p : graph->allocs) cudaFree(p);
    delete graph;
    return RUNIT_OK;
}

uint32_t runit_graph_fused_launches(runit_graph_t* graph) { return graph ? graph->fused_launches : 0; }
uint32_t runit_graph_kernel_launches(runit_graph_t* graph) { return graph ? graph->kernel_nodes : 0; }

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
