// One persistent launch for a run of consecutive fused-dequant GEMVs (batch 1, 4-bit formats).
//
// A decode token is a chain of dependent GEMVs (crates/engine/src/forward.rs:1523-1765: fused Q|K|V, o-proj + residual,
// fused gate/up + SiLU, down + residual per layer, then lm_head).  As separate launches each of them pays the drain of
// its predecessor, the dependency release and the refill of its own load pipeline (about 3.4 us against 5.9 us of HBM
// time for a 38 MB matrix).  Here the whole run is ONE kernel:
//   * the grid is one CTA per SM, NW warps each.  The unit of work is a CTA-item: a group of TPC tiles (32 rows each) of
//     one GEMV, every tile shared by a team of KSL warps that split its K range (KSL * TPC <= NW; the host picks KSL per
//     GEMV so that the items fill the SMs: 2 for an 18944-row gate/up pair, 16 for a 3584 x 18944 down projection).  The
//     tile/unit/MMA arithmetic is that of gemv_staged_kernel (integer tensor-core path);
//   * the items of all GEMVs form one list in launch order; CTA b takes items b, b + CTAs, ... (a shared counter that
//     hands items out lowest index first is there as an experiment: it evens out the 10 % speed differences between SMs
//     on long GEMVs but piles the items of a dependent GEMV onto the CTAs that happen to be free).  An item only ever
//     waits for items with lower indices, and the lowest unfinished item is always some CTA's current one, so no wait
//     can last; which CTA computes an item has no influence on the result;
//   * every warp keeps its own ring of S weight stages (TMA boxes of 32 rows x 144 bytes) and its load cursor runs S
//     stages ahead of its compute cursor ACROSS item and GEMV boundaries: weights do not depend on anything, so the
//     stream from HBM never stops at a boundary;
//   * activations are read with plain L2 loads (8 floats per lane and stage, one stage ahead, held in registers) once
//     the GEMVs that produce them have completed: every GEMV has a completion counter (tiles done); one warp per CTA
//     polls the counters a GEMV depends on, with a time bound, and the others wait for its verdict in shared memory;
//   * the K-slices of a tile meet in shared memory: each warp of the team files its 32 partial sums, the team's last
//     warp adds them in slice order (bit-reproducible) and runs the epilogue (bias, residual, SiLU(gate)*up, f16
//     output), then counts the tile as done.
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
constexpr int kStageBytes = kRT * 144;    // one warp stage: 32 rows x one 256-weight unit
constexpr int kXqBytes = 640;             // prepared activations of one unit (MmaX<8>::BYTES = 576), padded to 128
constexpr uint32_t kItemRing = 16;        // per-ordinal slots of a CTA's item sequence (power of two)
constexpr uint32_t kItemLag = 6;          // an ordinal is published once every warp has left the one kItemLag back

// Everything a warp needs about one GEMV except its tensor maps; copied to shared memory at kernel start.
struct alignas(16) OpLite {
    uint32_t item_begin, n_items;     // this GEMV's range in the global list of CTA-items
    uint32_t ksl, tpc;                // warps per tile (K-slices), tiles per item
    uint32_t n_units, n_tiles;
    uint32_t tile_begin1, tile_begin2;   // first tile of segments 1 and 2 (Q|K|V launches), kNoSeg if absent
    uint32_t dual;                    // fused gate/up: a tile is 16 gate rows + 16 up rows
    uint32_t k, nb;
    uint32_t pad0;
    const float* x;
    uint16_t dep[kMaxDeps];           // GEMVs (indices in this launch) that must be complete first; kNoDep = none
    // epilogue
    void* y[3];
    const void* res[3];
    const void* bias[3];
    uint32_t rows[3];
    uint8_t out_f16, res_kind, bias_kind, pad1;
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
    uint32_t* done;      // [n_ops] tiles completed; zero at rest
    uint32_t* ctl;       // [0] exit ticket, [1] abort flag, [2] items handed out beyond the CTAs' first; zero at rest
    int32_t* status;     // host-visible status word of the context
    int32_t dynamic;     // 1: items beyond a CTA's first come from the shared counter; 0: fixed split (item + k * CTAs)
};

// A position in a warp's walk over its CTA's item sequence.
struct Cursor {
    uint32_t ord;        // ordinal of the item in the CTA's sequence
    uint32_t c;          // its index in the global item list; >= total_items: past the end
    uint32_t op, tile, slice, ksl;
    uint32_t it, n_it;   // stage inside the item; n_it == 0: this warp has no part in the item
    uint32_t stage;      // running count of this warp's stages: ring slot = stage % S, barrier phase = (stage / S) & 1
};

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_vs(const uint32_t* p) { return *reinterpret_cast<const volatile uint32_t*>(p); }
__device__ __forceinline__ void st_vs(uint32_t* p, uint32_t v) { *reinterpret_cast<volatile uint32_t*>(p) = v; }

template <int FMT, int NW, int S>
__global__ void __launch_bounds__(NW * 32, 1) gemv_stream_kernel(const Params p) {
    static_assert(FMT == RUNIT_FMT_Q4K || FMT == RUNIT_FMT_Q4_0, "4-bit formats");
    static_assert(S + 2 <= (int)kItemLag, "warp 0's compute cursor trails the newest published ordinal by at most S + 1 items");
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ OpLite lite[kMaxOps];
    __shared__ __align__(8) uint64_t mbar[NW][S];
    __shared__ uint32_t s_last;
    __shared__ uint32_t s_ok[kMaxOps], s_lock[kMaxOps];   // dependency verdicts (1 = complete, 2 = gave up) and who polls
    __shared__ uint32_t s_item[kItemRing];                // global index of the CTA's item with ordinal o, at o % kItemRing
    __shared__ uint32_t s_item_ready;                     // ordinals [0, s_item_ready) are published (by warp 0)
    __shared__ uint32_t s_fin[kItemRing];                 // warps that have left the item of that ordinal
    __shared__ uint32_t s_arr[kItemRing][NW];             // per ordinal and team: warps whose partial sums are filed
    __shared__ float s_red[NW][kRT];                      // the partial sums a warp has filed last
    __shared__ uint32_t s_red_seq[NW];                    // how many of a warp's filings a team's adder has read

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    {
        const uint4* src = reinterpret_cast<const uint4*>(p.lite);
        uint4* dst = reinterpret_cast<uint4*>(lite);
        for (uint32_t i = threadIdx.x; i < p.n_ops * (uint32_t)(sizeof(OpLite) / 16); i += NW * 32) dst[i] = src[i];
    }
    for (uint32_t i = threadIdx.x; i < kMaxOps; i += NW * 32) s_ok[i] = s_lock[i] = 0u;
    for (uint32_t i = threadIdx.x; i < kItemRing * NW; i += NW * 32) (&s_arr[0][0])[i] = 0u;
    if (threadIdx.x < kItemRing) { s_fin[threadIdx.x] = 0u; s_item[threadIdx.x] = 0u; }
    if (threadIdx.x < NW) s_red_seq[threadIdx.x] = 0u;
    if (threadIdx.x == 0) {
        s_item[0] = blockIdx.x;
        s_item_ready = 1u;
    }
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

    bool dead = false;          // a bounded wait ran out (here or in another warp): stop, drain, leave

    // A completion counter this warp still has to bump once its earlier stores are visible.  The fence that makes them
    // visible costs a round trip to L2 right after the stores and next to nothing a little later, so the bump is put off
    // until the next stage's activations are prepared — unless the warp is about to wait for somebody else, in which case
    // it goes out first (a waiting warp never holds a signal back).
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
    // Whole-warp wait on a word in shared memory until pred(value): a quick look first; if that fails the warp's pending
    // signal goes out and lane 0 polls, for about 0.4 s at most (abort flag checked on the way).
    auto wait_shared = [&](const uint32_t* w, auto pred, int site = 6) -> bool {
        int ok = 0;
        if (lane == 0) ok = pred(ld_vs(w)) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
            flush_pending();
            if (lane == 0) {
                const long long t0 = clock64();
                uint32_t spins = 0;
                while (true) {
                    if (pred(ld_vs(w))) { ok = 1; break; }
                    __nanosleep(32);
                    if ((++spins & 255u) == 0u) {
                        if (*reinterpret_cast<volatile uint32_t*>(p.ctl + 1) != 0u) break;
                        if (clock64() - t0 > (3ll << 28)) {
                            atomicExch(p.ctl + 1, 1u);
                            if (p.status) atomicCAS(p.status, 0, site);
                            break;
                        }
                    }
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
        }
        __threadfence_block();
        __syncwarp();
        return ok != 0;
    };
    // Lane 0: polls a counter in global memory (gpu-scope acquire) until it reaches `want`.  False if another warp has
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
                    if (p.status) atomicCAS(p.status, 0, code);
                    return false;
                }
            }
        }
    };

    // ── the CTA's item sequence ──
    // Ordinal 0 is the CTA's own number; warp 0 (which has work in every item) publishes each later one when its load
    // cursor gets there: the next value of the shared counter (dynamic) or blockIdx + ordinal * CTAs (fixed split).  It
    // publishes an ordinal only once every warp has left the item kItemLag ordinals back, so the per-ordinal slots
    // (kItemRing of them) are never reused while in use.  The other warps read what is published; a warp whose ring still
    // holds stages does not wait for a publication (it comes back later), a warp with nothing left to compute does.
    auto get_item = [&](uint32_t ord, bool may_block, uint32_t& c_out) -> bool {
        if (warp == 0) {
            // everything up to `ord`, and one ordinal more if that needs no waiting: the other warps then know their next
            // item an item ahead and keep their rings full across the boundary
            while (true) {
                const uint32_t o = ld_vs(&s_item_ready);   // warp-uniform: only this warp writes the word
                if (o > ord + 1u) break;
                if (o >= kItemLag) {
                    uint32_t* fin = &s_fin[(o - kItemLag) % kItemRing];
                    if (o <= ord) {
                        if (!wait_shared(fin, [&](uint32_t v) { return v >= (uint32_t)NW; }, 10)) { dead = true; return false; }
                    } else {
                        int full = 0;
                        if (lane == 0) full = ld_vs(fin) >= (uint32_t)NW ? 1 : 0;
                        if (!__shfl_sync(0xffffffffu, full, 0)) break;
                    }
                    if (lane == 0) st_vs(fin, 0u);   // the slot serves ordinal o - kItemLag + kItemRing next
                }
                if (lane == 0) {
                    const uint32_t prev = s_item[(o - 1u) % kItemRing];
                    uint32_t g = prev;               // past the end stays past the end
                    if (prev < total) g = p.dynamic ? gridDim.x + atomicAdd(p.ctl + 2, 1u) : blockIdx.x + o * gridDim.x;
                    st_vs(&s_item[o % kItemRing], g);
                    __threadfence_block();
                    st_vs(&s_item_ready, o + 1u);
                }
                __syncwarp();
            }
        } else {
            int ready = 0;
            if (lane == 0) ready = ld_vs(&s_item_ready) > ord ? 1 : 0;
            ready = __shfl_sync(0xffffffffu, ready, 0);
            if (!ready) {
                if (!may_block) return false;
                if (!wait_shared(&s_item_ready, [&](uint32_t v) { return v > ord; }, 11)) { dead = true; return false; }
            }
        }
        __threadfence_block();
        c_out = ld_vs(&s_item[ord % kItemRing]);
        return true;
    };
    // Which GEMV, tile and K-slice of item c.c this warp has.  A CTA's items come in increasing order: c.op only moves on.
    auto locate = [&](Cursor& c) {
        c.it = 0;
        c.n_it = 0;
        if (c.c >= total) return;
        while (c.c >= lite[c.op].item_begin + lite[c.op].n_items) c.op++;
        const OpLite& o = lite[c.op];
        const uint32_t team = (uint32_t)warp / o.ksl;
        c.ksl = o.ksl;
        c.slice = (uint32_t)warp - team * o.ksl;
        c.tile = (c.c - o.item_begin) * o.tpc + team;
        if (team < o.tpc && c.tile < o.n_tiles && c.slice < o.n_units) c.n_it = (o.n_units - c.slice + o.ksl - 1) / o.ksl;
    };
    // Moves the cursor on to the next stage this warp has work for (skipping items it has no part in), or past the end.
    // count_fin: the cursor is the compute cursor, which reports every item it leaves.  False: the next item is not
    // published yet and may_block was false (the cursor stays where it was, at the end of its item).
    auto seek = [&](Cursor& c, bool may_block, bool count_fin) -> bool {
        while (c.c < total && c.it >= c.n_it) {
            uint32_t g;
            if (!get_item(c.ord + 1u, may_block, g)) return false;
            if (count_fin && lane == 0) atomicAdd(&s_fin[c.ord % kItemRing], 1u);
            c.ord++;
            c.c = g;
            locate(c);
        }
        return true;
    };

    // Weight boxes of the stage the cursor points at (lane 0 issues; everything it needs is in shared memory).
    auto issue_w = [&](const Cursor& c) {
        if (lane != 0) return;
        const OpLite& o = lite[c.op];
        uint32_t si = 0, tb = 0;
        if (c.tile >= o.tile_begin2) { si = 2; tb = o.tile_begin2; }
        else if (c.tile >= o.tile_begin1) { si = 1; tb = o.tile_begin1; }
        const uint32_t u = c.slice + c.ksl * c.it;
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
        const uint32_t e0 = (c.slice + c.ksl * c.it) * 256 + lane * 8;
        if (e0 < o.k) {
            const float4 a = __ldcg(reinterpret_cast<const float4*>(o.x + e0));
            const float4 b = __ldcg(reinterpret_cast<const float4*>(o.x + e0) + 1);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = 0.f;
        }
    };

    // Wait until every GEMV that `op` depends on is complete.  One warp per CTA polls the completion counters in global
    // memory (s_lock), the others wait for its verdict in shared memory (s_ok), so a counter sees one poller per SM
    // instead of one per warp.  Returns false on time-out / abort.
    uint32_t checked_op = 0xFFFFFFFFu;
    auto ensure_deps = [&](uint32_t op) -> bool {
        if (op == checked_op) return true;
        if (lite[op].dep[0] == kNoDep) { checked_op = op; return true; }
        int state = 0;   // 0: unknown, 1: complete, 2: gave up, 3: this warp polls
        if (lane == 0) {
            state = (int)ld_vs(&s_ok[op]);
            if (state == 0 && atomicExch(&s_lock[op], 1u) == 0u) state = 3;
        }
        state = __shfl_sync(0xffffffffu, state, 0);
        if (state == 3) {
            flush_pending();
            int ok = 1;
            if (lane == 0) {
                const OpLite& o = lite[op];
#pragma unroll
                for (int d = 0; d < (int)kMaxDeps; d++) {
                    const uint32_t dop = o.dep[d];
                    if (dop != kNoDep && ok) ok = poll_counter(p.done + dop, lite[dop].n_tiles, 4) ? 1 : 0;
                }
                __threadfence_block();
                st_vs(&s_ok[op], ok ? 1u : 2u);
            }
            state = __shfl_sync(0xffffffffu, ok, 0) ? 1 : 2;
        } else if (state == 0) {
            if (!wait_shared(&s_ok[op], [&](uint32_t v) { return v != 0u; }, 12)) return false;
            state = (int)ld_vs(&s_ok[op]);
        }
        __threadfence_block();
        __syncwarp();           // the poller's acquire is ordered before every lane's loads of the produced vectors
        if (state == 1) checked_op = op;
        return state == 1;
    };

    Cursor cur;
    cur.ord = 0;
    cur.c = blockIdx.x;
    cur.op = 0;
    cur.stage = 0;
    cur.tile = cur.slice = 0;
    cur.ksl = 1;
    locate(cur);
    Cursor lc = cur;            // load cursor: the next stage to request
    if (!seek(cur, true, true)) dead = true;     // the compute cursor waits at the first stage this warp has work for
    // Requests stages until the ring is full (S stages beyond the compute cursor) or the next item is not known yet.
    // A warp may wait for an item to be published only when it owes nothing to anybody: its ring is empty AND the item it
    // just computed has been handed in (may_wait is false between the last MMA of an item and its filing / epilogue).
    auto refill = [&](bool may_wait) {
        while (!dead && lc.stage < cur.stage + S) {
            const bool ring_empty = lc.stage == cur.stage;
            if (!seek(lc, ring_empty && may_wait, false)) break;
            if (lc.c >= total) break;
            issue_w(lc);
            lc.it++;
            lc.stage++;
        }
    };
    refill(true);
    __syncwarp();

    float macc[4] = {0.f, 0.f, 0.f, 0.f};
    float v[8];
    bool have_x = false;
    uint32_t filed = 0;         // partial sums this warp has filed in s_red so far
    const int g8 = lane >> 2, t4 = lane & 3;
    const uint32_t rit = 8u * (uint32_t)t4 + (uint32_t)g8;   // row of the tile this lane files after the K loop

    while (cur.c < total && !dead) {
        if (!have_x) {
            if (!ensure_deps(cur.op)) { dead = true; break; }
            load_x(cur, v);
        }
        if (lc.stage == cur.stage) {   // the stage was never requested (the item became known only now)
            refill(true);
            if (dead) break;
        }
        if (!mbar_wait(bar0 + 8 * (cur.stage % S), (cur.stage / S) & 1u)) {
            if (p.status) atomicExch(p.status, 1);
            atomicExch(p.ctl + 1, 1u);
            dead = true;
            break;
        }
        __syncwarp();
        const OpLite& o = lite[cur.op];
        const uint32_t u = cur.slice + cur.ksl * cur.it;
        const int nblk = FMT == RUNIT_FMT_Q4K ? 8 : min(8, (int)(o.nb - u * 8u));
        prep_mma_block<8, FMT == RUNIT_FMT_Q4_0 ? 1 : 0>(xq, v, lane, nblk);
        __syncwarp();
        flush_pending();        // the signal of the item that ended a moment ago: its stores have had time to land
        // activations of the item's next stage travel while this one is multiplied
        const bool item_ends = cur.it + 1 == cur.n_it;
        have_x = false;
        {
            Cursor nxt = cur;
            nxt.it++;
            bool known = true;
            if (item_ends) {
                // the first stage of the warp's next item, if that item is published and its inputs are known complete
                known = seek(nxt, false, false) && nxt.c < total &&
                        (nxt.op == checked_op || lite[nxt.op].dep[0] == kNoDep || ld_vs(&s_ok[nxt.op]) == 1u);
                if (known) {
                    __threadfence_block();
                    checked_op = nxt.op;
                }
            }
            if (known) {
                load_x(nxt, v);
                have_x = true;
            }
        }
        const uint8_t* slot = ring + (cur.stage % S) * kStageBytes;
        if (FMT == RUNIT_FMT_Q4K) unit_q4k_mma(slot, xq, lane, macc);
        else unit_q4_0_mma(slot, xq, lane, nblk, macc);
        __syncwarp();           // every lane is done with the slot and with xq
        cur.it++;
        cur.stage++;
        refill(!item_ends);

        if (item_ends) {
            // ── end of the item: fold the four lanes of a row group, meet the team's other K-slices, epilogue ──
#pragma unroll
            for (int j = 0; j < 4; j++) {
                macc[j] += __shfl_xor_sync(0xffffffffu, macc[j], 1);
                macc[j] += __shfl_xor_sync(0xffffffffu, macc[j], 2);
            }
            float r = t4 == 0 ? macc[0] : (t4 == 1 ? macc[1] : (t4 == 2 ? macc[2] : macc[3]));
            macc[0] = macc[1] = macc[2] = macc[3] = 0.f;
            bool last = true;
            const uint32_t live = min(cur.ksl, o.n_units);   // warps of the team that have a K-slice
            if (live > 1) {
                const uint32_t team = (uint32_t)warp / cur.ksl, w0 = team * cur.ksl;
                uint32_t* arr = &s_arr[cur.ord % kItemRing][team];
                // the previous filing of this warp must have been read before its slot is written again
                if (!wait_shared(&s_red_seq[warp], [&](uint32_t q) { return q == filed; }, 13)) { dead = true; break; }
                s_red[warp][rit] = r;
                filed++;
                __syncwarp();
                if (lane == 0) {
                    __threadfence_block();
                    atomicAdd(arr, 1u);
                }
                last = cur.slice + 1 == live;
                if (last) {
                    if (!wait_shared(arr, [&](uint32_t q) { return q >= live; }, 14)) { dead = true; break; }
                    float acc = 0.f;
                    for (uint32_t j = 0; j < live; j++) acc += *reinterpret_cast<volatile float*>(&s_red[w0 + j][rit]);
                    r = acc;
                    __syncwarp();
                    if ((uint32_t)lane < live) atomicAdd(&s_red_seq[w0 + lane], 1u);
                    if (lane == 0) st_vs(arr, 0u);
                }
            }
            if (last) {
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
                if (writer && row < o.rows[si]) {
                    if (o.bias_kind == BIAS_F16) r += __half2float(reinterpret_cast<const __half*>(o.bias[si])[row]);
                    else if (o.bias_kind == BIAS_F32) r += reinterpret_cast<const float*>(o.bias[si])[row];
                    if (o.res_kind == RES_F32) r += __ldcg(reinterpret_cast<const float*>(o.res[si]) + row);
                    if (o.out_f16) reinterpret_cast<__half*>(o.y[si])[row] = __float2half_rn(r);
                    else reinterpret_cast<float*>(o.y[si])[row] = r;
                }
                pending = p.done + cur.op;   // the tile counts as done once its results are visible
            }
            // on to this warp's next item: known already if the load cursor has been there, else wait for it
            if (!seek(cur, true, true)) { dead = true; break; }
            // nothing of this warp can run right away: its signal should not wait for a later stage
            if (cur.c >= total || (cur.op != checked_op && lite[cur.op].dep[0] != kNoDep && ld_vs(&s_ok[cur.op]) != 1u)) flush_pending();
        }
    }
    flush_pending();

    if (dead) {
        // stages already requested still land in this CTA's shared memory: wait for them (bounded) before leaving
        for (uint32_t st = cur.stage; st < lc.stage; st++) mbar_wait(bar0 + 8 * (st % S), (st / S) & 1u);
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
        for (uint32_t i = threadIdx.x; i < p.n_ops; i += NW * 32) p.done[i] = 0;
        __syncthreads();
        if (threadIdx.x == 0) {
            p.ctl[1] = 0;
            p.ctl[2] = 0;
            __threadfence();
            p.ctl[0] = 0;
        }
    }
}

}  // namespace gs
}  // namespace runit
