// Expert-parallel MoE block for prefill-sized batches: tokens are data-parallel (T per rank), experts are split over the
// ranks, and the token rows travel to the experts' owners and back by plain stores into peer memory; no host read, no
// collective library on the data path.  (The reference is single-device; its prefill runs the block token by token,
// crates/engine/src/prefill.rs:153-215.)
//
// One call on every rank, all launches on the context's stream:
//   1 route        the replicated f32 router and top-k on this rank's tokens (the batched block's own kernels)
//   2 dispatch     one warp per slot (token, expert): the owner d of the expert gives the next free row j of the region
//                  this rank owns in d's receive buffer (a counter in this rank's memory), the token row is rounded to
//                  bf16 (the operand type of the expert GEMMs) and stored there together with (local expert id, slot)
//   3 counts       the rows this rank used in every owner's region, stored into the owners' count tables
//   4 barrier      peer_barrier_kernel (bounded wait, sticky give-up)
//   5 fix up       the owner turns the count tables into one expert id per receive row (-1 past a region's count)
//   6 experts      the two grouped tcgen05 GEMMs of the batched block over the receive rows
//   7 return       fused into the second GEMM: its epilogue stores every f32 expert output straight into the slot it came
//                  from, in the memory of the rank that sent it (a table of row destinations, built from 5), so the
//                  transfer runs under the GEMM
//   8 barrier
//   9 weighted sum out[t] = residual[t] + sum_i w[t][i] * y[t*k+i] in routing order (the batched block's kernel)
// A receive buffer is only written between a rank's barrier 8 of one call and barrier 4 of the next, and only read
// between its barrier 4 and its announcement of barrier 8, so one buffer suffices; the same holds for the return buffer
// (written between barriers 4 and 8, read after 8 and before the announcement of the next 4).
// Every rank owns a fixed region of T*k rows in every owner's buffer (all its slots could go to one owner), so no count
// has to be known before the rows are stored.  The result is bit-identical to the single-GPU batched block: an expert
// output does not depend on which other rows share its tile, and the sum runs in the same order.
#include <cuda_bf16.h>

#include "runit_internal.h"
#include "tma.cuh"

namespace runit {

// moe.cu / moe_grouped.cu
int32_t moe_router(runit_ctx* ctx, const float* router_w, const float* x, float* logits, uint32_t E, uint32_t h, uint32_t T);
int32_t moe_topk(runit_ctx* ctx, const float* logits, uint32_t E, uint32_t k, int32_t renorm, uint32_t T, int32_t* idx, float* w);
int32_t moe_grouped_slots_bf16(runit_ctx* ctx, const void* gate, const void* up, const void* down, const void* x_bf16,
                               const int32_t* idx, void* scratch, size_t scratch_bytes, uint32_t S, uint32_t h, uint32_t ff, uint32_t E,
                               const float** y_out, const int32_t** pos_out, const void* ret_meta, const int32_t* ret_cnt,
                               void* const* ret_rows_all, uint32_t world, uint32_t cap_src);
int32_t moe_grouped_combine(runit_ctx* ctx, const float* y, const int32_t* pos_of_slot, const float* w, const float* residual, float* out,
                            uint32_t T, uint32_t h, uint32_t k);

namespace epp {

struct Peers {
    void* p[8];
};

__device__ __forceinline__ uint32_t bf2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// placement 0: expert e lives on rank e / n_local as local expert e % n_local; 1: on rank e % world as e / world.
__global__ void __launch_bounds__(256) dispatch_kernel(const float* __restrict__ x, const int32_t* __restrict__ idx, const Peers rx,
                                                        const Peers rmeta, uint32_t* __restrict__ cursor, uint32_t rank, uint32_t world,
                                                        uint32_t n_local, uint32_t cap_src, uint32_t S, uint32_t h, uint32_t k,
                                                        int placement) {
    const uint32_t s = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (s >= S) return;
    const int32_t e = idx[s];
    if (e < 0 || (uint32_t)e >= n_local * world) return;
    const uint32_t d = placement ? (uint32_t)e % world : (uint32_t)e / n_local;
    const uint32_t le = placement ? (uint32_t)e / world : (uint32_t)e % n_local;
    uint32_t j = 0;
    if (lane == 0) j = atomicAdd(&cursor[d], 1u);
    j = __shfl_sync(0xffffffffu, j, 0);
    const size_t row = (size_t)rank * cap_src + j;
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)(s / k) * h);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(rx.p[d]) + row * h);
    for (uint32_t c = lane; c < h / 8; c += 32) {
        const float4 a0 = __ldg(src + 2 * c), a1 = __ldg(src + 2 * c + 1);
        uint4 o;
        o.x = bf2(a0.x, a0.y); o.y = bf2(a0.z, a0.w); o.z = bf2(a1.x, a1.y); o.w = bf2(a1.z, a1.w);
        dst[c] = o;
    }
    if (lane == 0) reinterpret_cast<int2*>(rmeta.p[d])[row] = make_int2((int)le, (int)s);
}

// The rows this rank used in every owner's region; the cursors go back to zero for the next call.
__global__ void counts_kernel(uint32_t* __restrict__ cursor, const Peers rcnt, uint32_t rank, uint32_t world) {
    const uint32_t d = threadIdx.x;
    if (d >= world) return;
    reinterpret_cast<int32_t*>(rcnt.p[d])[rank] = (int32_t)cursor[d];
    cursor[d] = 0;
}

// idx_local[r * cap_src + j] = local expert of that receive row, or -1 past the count of region r.
__global__ void __launch_bounds__(256) fixup_kernel(const int2* __restrict__ meta, const int32_t* __restrict__ cnt, int32_t* __restrict__ idx_local,
                                                     uint32_t cap_src, uint32_t total) {
    const uint32_t i = blockIdx.x * 256 + threadIdx.x;
    if (i >= total) return;
    const uint32_t r = i / cap_src, j = i - r * cap_src;
    idx_local[i] = j < (uint32_t)cnt[r] ? meta[i].x : -1;
}

__global__ void __launch_bounds__(256) iota_kernel(int32_t* p, uint32_t n) {
    const uint32_t i = blockIdx.x * 256 + threadIdx.x;
    if (i < n) p[i] = (int32_t)i;
}

struct Local {
    float* logits;       // [T][E]
    int32_t* idx;        // [T][k]
    float* w;            // [T][k]
    uint32_t* cursor;    // [8]
    int32_t* idx_local;  // [world * cap_src]
    int32_t* iota;       // [T * k]
    void* grouped;       // scratch of the grouped GEMMs
    size_t grouped_bytes, bytes;
};

static Local carve(void* base, uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k, uint32_t world) {
    Local l{};
    const size_t S = (size_t)T * k, total = S * world;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        void* p = base ? (void*)((uint8_t*)base + off) : nullptr;
        off += (bytes + 1023) & ~(size_t)1023;
        return p;
    };
    l.logits = (float*)take(4 * (size_t)T * E);
    l.idx = (int32_t*)take(4 * S);
    l.w = (float*)take(4 * S);
    l.cursor = (uint32_t*)take(64);
    l.idx_local = (int32_t*)take(4 * total);
    l.iota = (int32_t*)take(4 * S);
    l.grouped_bytes = runit_moe_grouped_scratch_bytes((uint32_t)total, h, ff, E / world, 1);
    l.grouped = take(l.grouped_bytes);
    l.bytes = off;
    return l;
}

}  // namespace epp
}  // namespace runit

using namespace runit;

extern "C" {

size_t runit_moe_ep_prefill_scratch_bytes(uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k, uint32_t world) {
    if (world == 0 || E % world) return 0;
    return epp::carve(nullptr, T, h, ff, E, k, world).bytes;
}

int32_t runit_moe_layer_q4k_bf16_ep(runit_ctx_t* ctx, const void* router_w, const void* gate_local, const void* up_local,
                                    const void* down_local, const void* x, const void* residual, void* out, void* idx_out, void* w_out,
                                    void* scratch, size_t scratch_bytes, void* const* recv_rows_all, void* const* recv_meta_all,
                                    void* const* recv_counts_all, void* const* return_rows_all, void* const* signal_pads, uint32_t T,
                                    uint32_t h, uint32_t ff, uint32_t E, uint32_t k, int32_t renorm, uint32_t world, uint32_t rank,
                                    uint32_t epoch, int32_t placement) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, router_w && gate_local && up_local && down_local && x && out && scratch && recv_rows_all && recv_meta_all &&
                           recv_counts_all && return_rows_all && signal_pads,
                  "moe_layer_q4k_bf16_ep: null pointer");
    RUNIT_REQUIRE(ctx, world >= 1 && world <= 8 && rank < world && E > 0 && E % world == 0 && E <= 256 && epoch > 0,
                  "moe_layer_q4k_bf16_ep: world=%u rank=%u E=%u unsupported (1..8 ranks, experts divisible, epoch from 1)", world, rank, E);
    RUNIT_REQUIRE(ctx, T > 0 && k > 0 && k <= 32 && k <= E && h % 256 == 0 && ff % 256 == 0 && (uint64_t)T * k * world < (1ull << 30),
                  "moe_layer_q4k_bf16_ep: bad shape");
    RUNIT_REQUIRE(ctx, runit_aligned(scratch, 1024) && runit_aligned(x, 16) && runit_aligned(out, 16) && (!residual || runit_aligned(residual, 16)),
                  "moe_layer_q4k_bf16_ep: scratch must be 1024-byte aligned, tensors 16-byte aligned");
    const epp::Local l = epp::carve(scratch, T, h, ff, E, k, world);
    if (l.bytes > scratch_bytes)
        return runit_fail(ctx, RUNIT_ERR_BUFFER_SIZE, "moe_layer_q4k_bf16_ep: scratch has %zu bytes, needs %zu", scratch_bytes, l.bytes);
    epp::Peers rx{}, rmeta{}, rcnt{}, ry{};
    for (uint32_t p = 0; p < world; p++) {
        RUNIT_REQUIRE(ctx, recv_rows_all[p] && recv_meta_all[p] && recv_counts_all[p] && return_rows_all[p] && runit_aligned(recv_rows_all[p], 16) &&
                               runit_aligned(recv_meta_all[p], 8) && runit_aligned(return_rows_all[p], 16),
                      "moe_layer_q4k_bf16_ep: null or misaligned peer buffer %u", p);
        rx.p[p] = recv_rows_all[p]; rmeta.p[p] = recv_meta_all[p]; rcnt.p[p] = recv_counts_all[p]; ry.p[p] = return_rows_all[p];
    }
    const uint32_t S = T * k, cap_src = S, total = S * world, n_local = E / world;
    int32_t* idx = idx_out ? (int32_t*)idx_out : l.idx;
    float* w = w_out ? (float*)w_out : l.w;
    int32_t st;
    if (epoch == 1) {
        RUNIT_CUDA_TRY(ctx, cudaMemsetAsync(l.cursor, 0, 64, ctx->stream));
        epp::iota_kernel<<<(S + 255) / 256, 256, 0, ctx->stream>>>(l.iota, S);
        if ((st = runit_after_launch(ctx, "moe_ep_prefill_iota"))) return st;
    }
    if ((st = moe_router(ctx, (const float*)router_w, (const float*)x, l.logits, E, h, T))) return st;
    if ((st = moe_topk(ctx, l.logits, E, k, renorm, T, idx, w))) return st;
    epp::dispatch_kernel<<<(S + 7) / 8, 256, 0, ctx->stream>>>((const float*)x, idx, rx, rmeta, l.cursor, rank, world, n_local, cap_src, S, h, k,
                                                               placement ? 1 : 0);
    if ((st = runit_after_launch(ctx, "moe_ep_prefill_dispatch"))) return st;
    epp::counts_kernel<<<1, 32, 0, ctx->stream>>>(l.cursor, rcnt, rank, world);
    if ((st = runit_after_launch(ctx, "moe_ep_prefill_counts"))) return st;
    if ((st = peer_barrier_launch(ctx, signal_pads, world, rank, 2 * epoch - 1, nullptr))) return st;
    const int2* meta = (const int2*)rmeta.p[rank];
    const int32_t* cnt = (const int32_t*)rcnt.p[rank];
    epp::fixup_kernel<<<(total + 255) / 256, 256, 0, ctx->stream>>>(meta, cnt, l.idx_local, cap_src, total);
    if ((st = runit_after_launch(ctx, "moe_ep_prefill_fixup"))) return st;
    const float* y = nullptr;
    const int32_t* pos = nullptr;
    // the down GEMM's epilogue stores every expert output straight into the slot of the rank it came from
    if ((st = moe_grouped_slots_bf16(ctx, gate_local, up_local, down_local, rx.p[rank], l.idx_local, l.grouped, l.grouped_bytes, total, h, ff,
                                     n_local, &y, &pos, meta, cnt, return_rows_all, world, cap_src)))
        return st;
    if ((st = peer_barrier_launch(ctx, signal_pads, world, rank, 2 * epoch, nullptr))) return st;
    return moe_grouped_combine(ctx, (const float*)ry.p[rank], l.iota, w, (const float*)residual, (float*)out, T, h, k);
}

}  // extern "C"
