// One persistent launch for a run of consecutive fused-dequant GEMVs (batch 1, 4-bit formats).
//
// A decode token is a chain of dependent GEMVs (crates/engine/src/forward.rs:1523-1765: fused Q|K|V, o-proj + residual,
// fused gate/up + SiLU, down + residual per layer, then lm_head).  As separate launches each of them pays the drain of
// its predecessor, the dependency release and the refill of its own load pipeline (about 3.4 us against 5.9 us of HBM
// time for a 38 MB matrix).  Here the whole run is ONE kernel:
//   * the grid is one CTA per SM, NW warps each; the unit of work is a warp-item = one 32-row tile x one K-slice of one
//     GEMV (the tile/unit/MMA arithmetic is that of gemv_staged_kernel, integer tensor-core path);
//   * the items of all GEMVs form one list in launch order, dealt into NW interleaved classes; warp w of every CTA
//     takes the items of class w from that class's counter, lowest index first (SMs differ in speed by about 10 %: a
//     fixed split leaves the fast ones idle, and one counter for all warps saturates).  An item only ever waits for
//     items with lower indices, and the lowest unfinished item is always some warp's current one, so no wait can last;
//     which warp computes an item has no influence on the result;
//   * every warp keeps its own ring of S weight stages (TMA boxes of 32 rows x 144 bytes) and its load cursor runs S
//     stages ahead of its compute cursor ACROSS item and GEMV boundaries: weights do not depend on anything, so the
//     stream from HBM never stops at a boundary;
//   * activations are read with plain L2 loads (8 floats per lane and stage, one stage ahead, held in registers) once
//     the GEMVs that produce them have completed: every GEMV has a completion counter (tiles done), and a warp that
//     reaches the first item of a GEMV waits, with a time bound, until the counters of the GEMVs it depends on are full;
//   * K-slices of a tile meet through a scratch array in global memory: each slice stores its 32 partial sums and takes
//     a ticket; the slice that draws the last ticket adds the partials in slice order (bit-reproducible) and runs the
//     epilogue (bias, residual, SiLU(gate)*up, f16 output), then counts the tile as done.
// The host side (gemv_stream.cu) builds the item list, the dependency lists (read/write overlap of the recorded calls)
// and rewrites a recorded command list so that each run of such GEMVs becomes one launch of this kernel.
#pragma once

#include "gemv_kernels.cuh"

namespace runit {
namespace gs {

constexpr uint32_t kMaxOps = 128;         // GEMVs per launch (a 28-layer token has 113)
constexpr uint32_t kMaxDeps = 4;
constexpr uint32_t kNoDep = 0xFFFFu;
constexpr uint32_t kNoSeg = 0xFFFFFFFFu;
constexpr uint32_t kMaxSlices = 17;       // K-slices per tile: 16 partial sums + the adder's own
constexpr int kStageBytes = kRT * 144;    // one warp stage: 32 rows x one 256-weight unit
constexpr int kXqBytes = 640;             // prepared activations of one unit (MmaX<8>::BYTES = 576), padded to 128

// Everything a warp needs about one GEMV except its tensor maps; copied to shared memory at kernel start.
struct alignas(16) OpLite {
    uint32_t item_begin, n_items;     // this GEMV's range in the global item list
    uint32_t n_slices, n_units, n_tiles;
    uint32_t tile_begin1, tile_begin2;   // first tile of segments 1 and 2 (Q|K|V launches), kNoSeg if absent
    uint32_t dual;                    // fused gate/up: a tile is 16 gate rows + 16 up rows
    uint32_t k, nb;
    const float* x;
    uint16_t dep[kMaxDeps];           // GEMVs (indices in this launch) that must be complete first; kNoDep = none
    uint32_t partial_off;             // floats: [tile][slice][32] partial sums of this GEMV
    uint32_t ticket_off;              // words: one arrival counter per tile
    // epilogue
    void* y[3];
    const void* res[3];
    const void* bias[3];
    uint32_t rows[3];
    uint8_t out_f16, res_kind, bias_kind, pad;
};
static_assert(sizeof(OpLite) == 160, "OpLite is copied as 16-byte words");

// Tensor maps of one GEMV; stay in global memory (the bulk-load unit reads them there).
struct alignas(64) OpFull {
    CUtensorMap map[4];               // per segment; [3] = the up matrix of a fused gate/up launch
};

struct Params {
    const OpFull* full;
    const OpLite* lite;
    uint32_t n_ops, total_items;
    float* partial;
    uint32_t* tickets;
    uint32_t n_tickets;
    uint32_t* done;      // [n_ops] tiles completed; zero at rest
    uint32_t* ctl;       // [0] exit ticket, [1] abort flag, [2 + w] items of class w handed out beyond the CTAs' first; zero at rest
    int32_t* status;     // host-visible status word of the context
};

struct Cursor {
    uint32_t g;          // global item index; >= total_items: past the end
    uint32_t ord;        // how many items this warp has taken before this one
    uint32_t op, tile, slice, nsl;
    uint32_t it, n_it;   // stage inside the item
    uint32_t stage;      // running stage number of this warp: ring slot = stage % S, barrier phase = (stage / S) & 1
};

// Which GEMV, tile and K-slice item c.g is.  A warp's items come in increasing order, so c.op only moves forward.
__device__ __forceinline__ void locate(Cursor& c, const OpLite* lite, uint32_t total) {
    c.it = 0;
    if (c.g >= total) { c.n_it = 0; return; }
    while (c.g >= lite[c.op].item_begin + lite[c.op].n_items) c.op++;
    const uint32_t local = c.g - lite[c.op].item_begin, nsl = lite[c.op].n_slices;
    c.tile = local / nsl;
    c.slice = local - c.tile * nsl;
    c.nsl = nsl;
    c.n_it = (lite[c.op].n_units - c.slice + nsl - 1) / nsl;
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

template <int FMT, int NW, int S>
__global__ void __launch_bounds__(NW * 32, 1) gemv_stream_kernel(const Params p) {
    static_assert(FMT == RUNIT_FMT_Q4K || FMT == RUNIT_FMT_Q4_0, "4-bit formats");
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ OpLite lite[kMaxOps];
    __shared__ __align__(8) uint64_t mbar[NW][S];
    __shared__ uint32_t s_last;
    __shared__ uint32_t s_ok[kMaxOps], s_lock[kMaxOps];
    __shared__ uint32_t s_taken[NW][8];   // the item indices a warp has taken, by ordinal modulo 8 (load cursor -> compute cursor)

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    {
        const uint4* src = reinterpret_cast<const uint4*>(p.lite);
        uint4* dst = reinterpret_cast<uint4*>(lite);
        for (uint32_t i = threadIdx.x; i < p.n_ops * (uint32_t)(sizeof(OpLite) / 16); i += NW * 32) dst[i] = src[i];
    }
    for (uint32_t i = threadIdx.x; i < kMaxOps; i += NW * 32) s_ok[i] = s_lock[i] = 0u;
    const uint32_t bar0 = smem_u32(&mbar[warp][0]);
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < S; s++) mbar_init(bar0 + 8 * s, 1);
        fence_mbar_init();
    }
    __syncthreads();

    uint8_t* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    uint8_t* ring = smem + warp * (S * kStageBytes + kXqBytes);
    uint8_t* xq = ring + S * kStageBytes;
    const uint32_t ring_u32 = smem_u32(ring);
    const uint32_t total = p.total_items;

    // Weight boxes of the stage the cursor points at (lane 0 issues; everything it needs is in shared memory).
    uint32_t issued_end = 0;    // stages [0, issued_end) of this warp carry a bulk-load transaction
    auto issue_w = [&](const Cursor& c) {
        if (c.g >= total) return;
        issued_end = c.stage + 1;
        if (lane != 0) return;
        const OpLite& o = lite[c.op];
        uint32_t si = 0, tb = 0;
        if (c.tile >= o.tile_begin2) { si = 2; tb = o.tile_begin2; }
        else if (c.tile >= o.tile_begin1) { si = 1; tb = o.tile_begin1; }
        const uint32_t u = c.slice + c.nsl * c.it;
        const uint32_t slot = ring_u32 + (c.stage % S) * kStageBytes, bar = bar0 + 8 * (c.stage % S);
        const OpFull* f = p.full + c.op;
        fence_proxy_async();   // the warp's generic-proxy reads of this slot precede the bulk writes
        mbar_expect_tx(bar, kStageBytes);
        if (o.dual) {
            const int32_t row0 = (int32_t)((c.tile - tb) * (kRT / 2));
            tma_load_2d(slot, &f->map[0], (int32_t)(u * 144), row0, bar);
            tma_load_2d(slot + (kRT / 2) * 144, &f->map[3], (int32_t)(u * 144), row0, bar);
        } else {
            tma_load_2d(slot, &f->map[si], (int32_t)(u * 144), (int32_t)((c.tile - tb) * kRT), bar);
        }
    };
    // This lane's 8 activations of the stage (L2 loads: the vector may have been written by another SM a moment ago).
    auto load_x = [&](const Cursor& c, float (&v)[8]) {
        const OpLite& o = lite[c.op];
        const uint32_t e0 = (c.slice + c.nsl * c.it) * 256 + lane * 8;
        if (e0 < o.k) {
            const float4 a = __ldcg(reinterpret_cast<const float4*>(o.x + e0));
            const float4 b = __ldcg(reinterpret_cast<const float4*>(o.x + e0) + 1);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = 0.f;
        }
    };

    bool dead = false;          // a bounded wait ran out (here or in another warp): stop, drain, leave
    // Polls a counter in global memory (gpu-scope acquire) until it reaches `want`.  Returns false if another warp has
    // raised the abort flag or after about half a second, which it reports through the status word.
    auto poll_counter = [&](const uint32_t* ctr, uint32_t want, int code) -> bool {
        if (ld_acquire_gpu(ctr) >= want) return true;
        const long long t0 = clock64();
        uint32_t spins = 0;
        while (true) {
            __nanosleep(100);
            if (ld_acquire_gpu(ctr) >= want) return true;
            if ((++spins & 31u) == 0u) {
                if (*reinterpret_cast<volatile uint32_t*>(p.ctl + 1) != 0u) return false;
                if (clock64() - t0 > (1ll << 30)) {
                    atomicExch(p.ctl + 1, 1u);
                    if (p.status) atomicExch(p.status, code);
                    return false;
                }
            }
        }
    };
    // Wait until every GEMV that `op` depends on is complete.  One warp per CTA polls the completion counters in global
    // memory (s_lock), the others wait for its verdict in shared memory (s_ok: 1 = complete, 2 = gave up), so a counter
    // sees one poller per SM instead of one per warp.  Returns false on time-out / abort.
    // A counter this warp still has to bump (a tile's arrival count or a GEMV's completion count) once its earlier
    // stores are visible.  The fence that makes them visible costs a round trip to L2 right after the stores and next
    // to nothing a little later, so the bump is put off until the next stage's activations are prepared — unless the warp is
    // about to wait for somebody else, in which case it goes out first (a waiting warp never holds a signal back).
    uint32_t* pending = nullptr;
    auto flush_pending = [&]() {
        if (pending != nullptr) {
            __syncwarp();
            if (lane == 0) {
                __threadfence();
                atomicAdd(pending, 1u);
            }
            pending = nullptr;
        }
    };
    uint32_t checked_op = 0xFFFFFFFFu;
    auto ensure_deps = [&](uint32_t op) -> bool {
        if (op == checked_op) return true;
        if (*reinterpret_cast<volatile uint32_t*>(&s_ok[op]) != 1u && lite[op].dep[0] != kNoDep) flush_pending();
        int ok = 1;
        if (lane == 0) {
            volatile uint32_t* okf = &s_ok[op];
            if (*okf == 0u) {
                const OpLite& o = lite[op];
                if (o.dep[0] == kNoDep) {
                    *okf = 1u;
                } else if (atomicExch(&s_lock[op], 1u) == 0u) {
#pragma unroll
                    for (int d = 0; d < (int)kMaxDeps; d++) {
                        const uint32_t dop = o.dep[d];
                        if (dop != kNoDep && ok) ok = poll_counter(p.done + dop, lite[dop].n_tiles, 4) ? 1 : 0;
                    }
                    __threadfence_block();
                    *okf = ok ? 1u : 2u;
                } else {
                    const long long t0 = clock64();
                    while (*okf == 0u) {
                        __nanosleep(40);
                        if (clock64() - t0 > (3ll << 29)) break;   // the polling warp itself gives up after 2^30 cycles
                    }
                }
            }
            if (*okf != 1u) ok = 0;
            __threadfence_block();
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        __syncwarp();           // lane 0's acquire is ordered before the other lanes' loads of the produced vectors
        if (ok) checked_op = op;
        return ok != 0;
    };

    // Item sequence of this warp: the first item is fixed, every later one comes from the counter of the warp's class.  The load cursor takes items; the request for the item after the next is in flight while
    // the next one is being loaded, so the counter's latency stays hidden.  The compute cursor follows through s_taken.
    uint32_t take_raw = 0;      // lane 0: reply of the outstanding request
    auto request_item = [&]() {   // class `warp`: items warp, warp + NW, ...; the first gridDim.x of them are the CTAs' first items
        if (lane == 0) take_raw = (uint32_t)warp + (uint32_t)NW * (gridDim.x + atomicAdd(p.ctl + 2 + warp, 1u));
    };
    auto advance_load = [&](Cursor& c) {
        c.stage++;
        if (++c.it >= c.n_it) {
            if (c.g >= total) { c.it = 0; return; }          // past the end: stay there
            c.ord++;
            c.g = __shfl_sync(0xffffffffu, take_raw, 0);
            if (lane == 0) s_taken[warp][c.ord & 7u] = c.g;
            if (c.g < total) request_item();
            locate(c, lite, total);
        }
    };
    auto advance_follow = [&](Cursor& c) {
        c.stage++;
        if (++c.it >= c.n_it) {
            c.ord++;
            c.g = *reinterpret_cast<volatile uint32_t*>(&s_taken[warp][c.ord & 7u]);
            locate(c, lite, total);
        }
    };
    Cursor cur;
    cur.g = (uint32_t)warp + (uint32_t)NW * blockIdx.x;
    cur.ord = 0;
    cur.op = 0;
    cur.stage = 0;
    cur.tile = cur.slice = cur.nsl = 0;
    locate(cur, lite, total);
    if (lane == 0) s_taken[warp][0] = cur.g;
    if (cur.g < total) request_item();
    Cursor lc = cur;
#pragma unroll
    for (int s = 0; s < S; s++) {
        issue_w(lc);
        advance_load(lc);
    }
    __syncwarp();

    float macc[4] = {0.f, 0.f, 0.f, 0.f};
    float v[8];
    bool have_x = false;
    const int g8 = lane >> 2, t4 = lane & 3;
    const uint32_t rit = 8u * (uint32_t)t4 + (uint32_t)g8;   // row of the tile this lane files after the K loop

    while (cur.g < total) {
        if (!have_x) {
            if (!ensure_deps(cur.op)) { dead = true; break; }
            load_x(cur, v);
        }
        if (!mbar_wait(bar0 + 8 * (cur.stage % S), (cur.stage / S) & 1u)) {
            if (p.status) atomicExch(p.status, 1);
            atomicExch(p.ctl + 1, 1u);
            dead = true;
            break;
        }
        __syncwarp();
        const OpLite& o = lite[cur.op];
        const uint32_t u = cur.slice + cur.nsl * cur.it;
        const int nblk = FMT == RUNIT_FMT_Q4K ? 8 : min(8, (int)(o.nb - u * 8u));
        prep_mma_block<8, FMT == RUNIT_FMT_Q4_0 ? 1 : 0>(xq, v, lane, nblk);
        __syncwarp();
        flush_pending();        // the signal of the item that ended a moment ago: its stores have had time to land
        // activations of the next stage travel while this one is multiplied (only if their producers are known complete)
        Cursor nxt = cur;
        advance_follow(nxt);
        have_x = false;
        if (nxt.g < total && (nxt.op == checked_op || *reinterpret_cast<volatile uint32_t*>(&s_ok[nxt.op]) == 1u)) {
            __threadfence_block();
            load_x(nxt, v);
            have_x = true;
            checked_op = nxt.op;
        }
        const uint8_t* slot = ring + (cur.stage % S) * kStageBytes;
        if (FMT == RUNIT_FMT_Q4K) unit_q4k_mma(slot, xq, lane, macc);
        else unit_q4_0_mma(slot, xq, lane, nblk, macc);
        __syncwarp();           // every lane is done with the slot and with xq
        issue_w(lc);
        advance_load(lc);

        if (cur.it + 1 == cur.n_it) {
            // ── end of the item: fold the four lanes of a row group, meet the other K-slices, epilogue ──
#pragma unroll
            for (int j = 0; j < 4; j++) {
                macc[j] += __shfl_xor_sync(0xffffffffu, macc[j], 1);
                macc[j] += __shfl_xor_sync(0xffffffffu, macc[j], 2);
            }
            float r = t4 == 0 ? macc[0] : (t4 == 1 ? macc[1] : (t4 == 2 ? macc[2] : macc[3]));
            macc[0] = macc[1] = macc[2] = macc[3] = 0.f;
            // K-slices of a tile: every slice but the last one of the tile files its partial sums and counts itself in
            // (no reply awaited); the last slice of the tile, which is also the last of them in the item list, waits
            // for that count, adds the partial sums in slice order with its own at the end, and runs the epilogue.
            bool last = true;
            if (cur.nsl > 1) {
                float* part = p.partial + o.partial_off + (size_t)cur.tile * cur.nsl * 32;
                uint32_t* ticket = p.tickets + o.ticket_off + cur.tile;
                if (cur.slice + 1 != cur.nsl) {
                    last = false;
                    __stcg(part + cur.slice * 32 + rit, r);
                    pending = ticket;
                } else {
                    flush_pending();
                    int ok = 1;
                    if (lane == 0) ok = poll_counter(ticket, cur.nsl - 1, 5) ? 1 : 0;
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    __syncwarp();
                    if (!ok) { dead = true; break; }
                    float acc = 0.f;
                    for (uint32_t s0 = 0; s0 + 1 < cur.nsl; s0 += 16) {   // 16 loads in flight per round trip
                        float pv[16];
#pragma unroll
                        for (int q = 0; q < 16; q++) pv[q] = s0 + q + 1 < cur.nsl ? __ldcg(part + (s0 + q) * 32 + rit) : 0.f;
#pragma unroll
                        for (int q = 0; q < 16; q++) acc += pv[q];
                    }
                    r = acc + r;
                    if (lane == 0) *ticket = 0;   // at rest again for the next launch
                }
            }
            if (last) {
                const OpLite* f = &o;
                uint32_t si = 0, tb = 0;
                if (cur.tile >= o.tile_begin2) { si = 2; tb = o.tile_begin2; }
                else if (cur.tile >= o.tile_begin1) { si = 1; tb = o.tile_begin1; }
                bool writer = true;
                uint32_t row = (cur.tile - tb) * kRT + rit;
                if (o.dual) {
                    // lanes t = 0, 1 hold gate rows 8t + g, lanes t + 2 the matching up rows:
                    // act = silu(gate) * up  (crates/kernels/shaders/fused_ffn.metal:24-26,89-92)
                    const float up_v = __shfl_down_sync(0xffffffffu, r, 2);
                    r = silu(r) * up_v;
                    writer = t4 < 2;
                    row = (cur.tile - tb) * (kRT / 2) + rit;
                }
                if (writer && row < f->rows[si]) {
                    if (f->bias_kind == BIAS_F16) r += __half2float(reinterpret_cast<const __half*>(f->bias[si])[row]);
                    else if (f->bias_kind == BIAS_F32) r += reinterpret_cast<const float*>(f->bias[si])[row];
                    if (f->res_kind == RES_F32) r += __ldcg(reinterpret_cast<const float*>(f->res[si]) + row);
                    if (f->out_f16) reinterpret_cast<__half*>(f->y[si])[row] = __float2half_rn(r);
                    else reinterpret_cast<float*>(f->y[si])[row] = r;
                }
                pending = p.done + cur.op;   // the tile counts as done once its results are visible
                // nothing else of this warp is ready to run: the consumers should not wait for a later stage of ours
                if (!have_x) flush_pending();
            }
        }
        cur = nxt;
    }
    flush_pending();

    if (dead) {
        // stages already requested still land in this CTA's shared memory: wait for them (bounded) before leaving
        for (uint32_t st = cur.stage; st < issued_end; st++) mbar_wait(bar0 + 8 * (st % S), (st / S) & 1u);
    }

    // The CTA that leaves last puts the counters back to rest for the next launch of this program.
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        s_last = atomicAdd(p.ctl, 1u) == gridDim.x - 1 ? 1u : 0u;
    }
    __syncthreads();
    if (s_last) {
        __threadfence();
        const bool aborted = *reinterpret_cast<volatile uint32_t*>(p.ctl + 1) != 0u;
        for (uint32_t i = threadIdx.x; i < p.n_ops; i += NW * 32) p.done[i] = 0;
        if (aborted)
            for (uint32_t i = threadIdx.x; i < p.n_tickets; i += NW * 32) p.tickets[i] = 0;
        __syncthreads();
        if (threadIdx.x == 0) {
            p.ctl[1] = 0;
            for (int w = 0; w < NW; w++) p.ctl[2 + w] = 0;
            __threadfence();
            p.ctl[0] = 0;
        }
    }
}

}  // namespace gs
}  // namespace runit
