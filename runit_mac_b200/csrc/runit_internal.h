// Internal definitions shared by the translation units of librunit_cuda.so.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_fp16.h>

#include <cstdint>
#include <cstdio>
#include <cstring>

#include "runit_cuda.h"

struct runit_tuning {
    int32_t gemv_variant = 0;   // 0 = staged kernel, 1 = simple warp-per-row kernel
    int32_t gemv_stages = 0;    // 0 = default
    int32_t pdl = 0;            // programmatic dependent launch between ops
    int32_t gemv_math = 0;      // batch 1: 0 = tensor-core MMAs (4-bit) / dp4a (Q8_0), 1 = packed f32, 2 = dp4a
    int32_t gemv_csplit = 0;    // 0 = automatic cluster split of K, else 2 or 4
    int32_t gemv_no_cluster = 0;
    int32_t gemv_ksl = 0;       // 0 = automatic K-slices per tile, else 1, 2 or 4
    int32_t gemv_load = 0;      // 0 = tiled bulk loads (TMA) where rows allow, 1 = cp.async everywhere
    int32_t stream_fuse = 0;    // recorded command lists: 1 = runs of consecutive GEMVs become one persistent launch
    int32_t stream_cfg = 0;     // warps per SM x ring stages of that launch: 0 = default, 1..3 = alternatives
    int32_t stream_ksl = 0;     // 0 = warps per tile chosen per GEMV, else forced (experiments)
    int32_t stream_dynamic = 0;
    int32_t kquant_split = 0;        // K-quant tile kernels: 0 = shares of K chosen from the shape, 1..16 = this many (power of two)
    int32_t kquant_variant = 0;      // Q6_K / Q5_K / Q5_0 GEMV: 0 = tile kernel (lane = row, dp4a), 1 = one warp per row (the first kernel; cross-check)
    int32_t imma_rw = 0, imma_csplit = 0, imma_stages = 0;   // batched 4-bit GEMV: rows per warp (16 / 32), cluster size over K, ring depth; 0 = chosen from the shape
    int32_t imma_fold = 0;           // batched 4-bit GEMV: 1 = activation pre-pass inside the GEMV launch where the grid allows (measured slower:
                                     // 950 against 1331 GB/s over the 7B set at batch 8), 0 = a launch of its own
    int32_t ep_fused_exchange = 0;   // expert-parallel decoder: 1 = exchange inside the GEMVs (no launches of its own; measured slower)
    int32_t router_variant = 0;   // batched f32 router: 0 = by size, 1 = one warp per expert, 2 = tiled GEMM, 3 = GEMM with K split over the warps of a CTA (tests force each)
};

// Cached tensor map of one weight matrix view (encoding costs ~1 us on the host).
struct runit_tmap_entry {
    const void* ptr = nullptr;
    uint64_t rows = 0, row_bytes = 0;
    uint32_t box_rows = 0, box_bytes = 0, swizzle128 = 0;
    CUtensorMap map;
};

// One per GPU; replaces the reference's MetalContext (crates/kernels/src/context.rs:137-160).
struct runit_ctx {
    int32_t device = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int32_t sm_count = 0;
    int32_t max_smem_optin = 0;
    uint64_t launches = 0;
    bool capturing = false;             // a command list is being recorded on the stream
    int32_t sticky_status = RUNIT_OK;   // first error since the last flush
    char err[512] = {0};
    runit_tuning tune;
    // Device scratch owned by the context (allocated at creation; ops never allocate).
    int32_t* d_status = nullptr;        // device address of the status word written by kernels with bounded waits
    int32_t* h_status = nullptr;        // the same word, host side (pinned, mapped)
    uint32_t* d_abort = nullptr;        // device word: set by the first peer barrier that gave up; later barriers skip their wait
    void* d_am = nullptr;               // greedy epilogue of the GEMV: ticket word at 0, result pair at 16, per-tile pairs from 256
    uint32_t* d_xq_ctl = nullptr;       // batched GEMV with the pre-pass inside: launch number, exit tickets, one flag per unit (from word 64)
    void* d_kq = nullptr;               // Q6_K GEMV with K split over CTAs: 2048 tile tickets (zero at rest), then 1 MiB of partial sums
    void* d_xq = nullptr;               // staging area of the batched GEMV's quantised activations
    size_t xq_bytes = 0;
    void* encode_tiled = nullptr;       // cuTensorMapEncodeTiled, resolved at context creation
    runit_tmap_entry tmaps[256];
    void* stream_rec = nullptr;         // std::vector<runit::StreamRec>* while a command list is being recorded
    uint64_t fused_launches = 0;        // GEMV launches that recorded command lists folded into persistent launches
};

// Tensor map of a [rows][row_bytes] byte matrix with a [box_rows][box_bytes] box (cached per context).
// swizzle128 != 0: the box (at most 128 bytes wide) lands in shared memory in the 128-byte swizzled layout the
// tensor cores read (16-byte chunk c of row r at chunk position c ^ (r % 8)); the destination must be 1024-byte
// aligned.
int32_t runit_get_tmap(runit_ctx* ctx, const void* ptr, uint64_t rows, uint64_t row_bytes, uint32_t box_rows,
                       uint32_t box_bytes, CUtensorMap* out, uint32_t swizzle128 = 0);

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

// Launch of a small kernel of an operator chain.  With dependent launch enabled (tune.pdl != 0) the kernel may be
// scheduled while its predecessor on the stream is still draining; every kernel launched through this helper
// therefore begins with griddepcontrol.wait (grid_dependency_wait) before it touches memory.
template <typename... KArgs, typename... Args>
static inline void runit_launch_chain(runit_ctx* ctx, void (*kern)(KArgs...), dim3 grid, dim3 block, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->tune.pdl != 0 ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);   // errors surface in runit_after_launch
}

// The same with dynamic shared memory.
template <typename... KArgs, typename... Args>
static inline void runit_launch_chain_smem(runit_ctx* ctx, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem_bytes, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->tune.pdl != 0 ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);   // errors surface in runit_after_launch
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

namespace runit {
// Expert-parallel decode without launches of its own (GemvArgs::ep_* / epw_* in gemv_kernels.cuh).
struct EpPush {          // producer: the grouped down projection of a rank
    void* const* partial_all;    // every rank's partial buffer f32 [2][world][rows]
    void* const* pads;           // every rank's flag pad
    uint32_t world, rank;
    uint32_t* epoch;             // device word, advanced by the launch
    uint32_t* done;              // zeroed device word (ticket over the row tiles)
};
struct EpWait {          // consumer: the next GEMV that reads the hidden state
    const float* partial;        // this rank's partial buffer
    const uint32_t* pad;         // this rank's flag pad
    const float* residual;       // hidden state before the block
    float* copies;               // scratch f32 [copies_rows][k]: one copy of the summed state per CTA of the consuming launch
    uint32_t copies_rows;
    uint32_t world;
    const uint32_t* epoch;
};
// gemv_imma.cu: batched GEMV of the 4-bit formats on the integer tensor-core path.
bool gemv_imma_applies(const runit_ctx* ctx, int fmt, uint32_t k, uint32_t batch);
int32_t gemv_imma(runit_ctx* ctx, int fmt, const void* w, const float* x, float* y, const float* res, uint32_t m, uint32_t k,
                  uint32_t batch);
int32_t gemv_imma_multi(runit_ctx* ctx, int fmt, uint32_t n_mats, const void* const* w, const float* x, float* const* y,
                        const float* const* res, const uint32_t* m, uint32_t k, uint32_t batch);
// gemv.cu: grouped GEMVs over stacked expert matrices (MoE block).  Slot s uses expert slot_expert[s] - expert_lo of the
// n_experts stacked ones; an id outside that range marks an unused slot.
int32_t gemv_grouped(runit_ctx* ctx, const char* name, int fmt, const void* w, const void* w2, uint32_t n_experts,
                     uint32_t rows, uint32_t k, const void* x, uint32_t xdiv, void* y, const int32_t* slot_expert,
                     uint32_t n_slots, int32_t expert_lo = 0,
                     // cmb_out != nullptr (one token): out = res + sum_i cmb_w[i] * y[i], written by the last tile of every
                     // 32-row tile; cmb_cnt = rows / 32 (rounded up) zeroed words, zero again when the launch ends
                     const float* cmb_w = nullptr, const float* cmb_res = nullptr, float* cmb_out = nullptr,
                     uint32_t* cmb_cnt = nullptr,
                     // dependent-launch ordering of a gate/up + down pair whose expert ids come from the kernel before the
                     // pair: 1 = first of the pair (releases its successor only after its own wait), 2 = second of the pair
                     // (reads the ids and requests weights before its wait); 0 = neither
                     int order = 0,
                     // expert parallelism: the weighted sum of this rank's slots goes to every rank's partial buffer (cmb_out unused)
                     const EpPush* ep = nullptr);
// gemv.cu: the one-kernel barrier over peer memory behind runit_peer_barrier.
int32_t peer_barrier_launch(runit_ctx* ctx, void* const* signal_pads, uint32_t world, uint32_t rank, uint32_t epoch,
                            uint32_t* epoch_ptr, const void* pairs = nullptr, int32_t* pair_result = nullptr);
// moe.cu: the same block for one token with the exchange inside the down projection's epilogue (see there)
int32_t moe_layer_q4k_ep_push_impl(runit_ctx* ctx, const void* router_w, const void* gate_local, const void* up_local,
                                   const void* down_local, float* xn, const float* pre_x, const float* pre_gamma, float pre_eps,
                                   void* scratch, size_t scratch_bytes, uint32_t h, uint32_t ff, uint32_t E, uint32_t k, int32_t renorm,
                                   uint32_t* counters, const EpPush* push);
// moe.cu: expert-parallel decode block (runit_moe_layer_q4k_ep); epoch_ptr != nullptr keeps the epoch in a device word.
int32_t moe_layer_q4k_ep_impl(runit_ctx* ctx, const void* router_w, const void* gate_local, const void* up_local,
                              const void* down_local, const void* x, const void* residual, void* out, void* idx_out, void* w_out,
                              void* scratch, size_t scratch_bytes, void* const* partial_all, void* const* signal_pads,
                              uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k, int32_t renorm, uint32_t world,
                              uint32_t rank, uint32_t epoch, uint32_t* epoch_ptr, uint32_t* route_counter, const float* pre_x,
                              const float* pre_gamma, float pre_eps);
}  // namespace runit
