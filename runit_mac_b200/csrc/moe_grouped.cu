// Batched (prefill-sized) MoE block on the tensor cores: token permutation by expert, then two grouped GEMMs whose
// weight operand is dequantised from Q4_K to bf16 tiles and multiplied with tcgen05.mma into f32 accumulators in
// tensor memory.
//
// The reference has no batched MoE kernel: its prefill runs the decode block once per token
// (crates/engine/src/prefill.rs:156-215: per token a router GEMV, a flush, CPU top-k, and per selected expert
// gate/up/silu/down/accumulate launches).  The arithmetic here is the same block with bf16 operands:
//   act[s] = bf16( silu(Wg[e].bf16(x[t])) * (Wu[e].bf16(x[t])) ),  y[s] = Wd[e].act[s],  out[t] = res[t] + sum_i w_i*y[s_i]
// with every weight the bf16 rounding of the Q4_K value d*sc*q - dmin*m (crates/engine/src/forward.rs:1026-1057),
// f32 accumulation, and the weighted sum taken in routing order.
//
// Layout of one grouped GEMM (weight rows ride the M of the MMA, token slots ride N):
//   * slots (token, expert) are sorted by expert; every expert's slots start at a multiple of 128 rows of the
//     permuted order and are cut into token tiles of up to 256 slots, so a tile never mixes experts;
//   * work item = (token tile, block of 256 weight rows); persistent clusters of two CTAs (cta_group::2) take items
//     round-robin, each CTA owning 128 of the rows and half of the token tile;
//   * per 128-wide K step: the weight operand is dequantised by 16 warps from raw Q4_K superblocks (TMA ring in shared
//     memory) straight into tensor memory (tcgen05.st), the token tile arrives by TMA into 128-byte-swizzled shared
//     memory, and the leader CTA issues 8 MMAs of M = 256, N <= 256, K = 16;
//   * 23 warps per CTA: 0 = token-tile producer (+ tensor-memory allocation), 1 = MMA issuer (leader CTA), 2-5 =
//     epilogue (tensor memory -> registers -> global), 6-21 = dequantisers, 22 = raw-superblock producer.
// The reasons for each of these choices, with the measurements behind them, are in the comment above the kernel.
// Every wait is bounded in time; a wait that gives up raises the CTA's abort flag, all roles leave their loops,
// tensor memory is freed and the host sees RUNIT_ERR_TIMEOUT at the next flush.
#include <cuda_bf16.h>

#include "gemv_common.cuh"
#include "runit_internal.h"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace runit {
namespace gg {

constexpr int kTok = 128;                  // token slots per tile (MMA N, at most)
constexpr int kRows = 128;                 // weight rows per tile (MMA M)
constexpr int kKC = 64;                    // K elements per pipeline stage: one 128-byte row of bf16
constexpr int kTileBytes = kRows * 128;    // 16 KiB
constexpr int kEpiWarp0 = 2;                // first of the four epilogue warps

struct Args {
    const uint8_t* w0;            // stacked expert matrices [E][rows][K/256 * 144]
    const uint8_t* w1;            // second matrix (up) when gate and up are fused
    uint32_t rows;                // rows per expert
    uint32_t K;
    uint32_t nb;                  // rows / 128
    const int32_t* tile_expert;   // per token tile
    const int32_t* tile_nvalid;   // valid slots of the tile (1..tile size)
    const int32_t* tile_row0;     // first row of the tile in the permuted order
    const int32_t* n_tok_tiles;   // device-resident count
    void* out;                    // bf16 [rows_padded][ld] (fused gate/up) or f32 [rows_padded][ld]
    uint32_t ld;
    // f32 output only: when not null, row r of the permuted order is stored at row_ptr[r] instead of out + r * ld.  The
    // pointers may lie in another GPU's memory (plain stores): the expert outputs of an expert-parallel block go straight
    // back to the ranks that sent the tokens while the GEMM is still running.
    float* const* row_ptr;
    int32_t* status;
};

// ── dequantisation of one 64-element K chunk of one weight row ──
// q: the 8 words (32 bytes) of the chunk; low nibbles are elements 0..31 (scale pair lo), high nibbles elements
// 32..63 (scale pair hi).  A field at bit p becomes 2^23 + nibble*2^p with one LOP3, the magic is subtracted, and one
// FMA with (scale * 2^-p, -min) gives exactly fl(scale*nibble - min); pairs are rounded to bf16 with one cvt.
__device__ __forceinline__ uint32_t bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float lo_f(uint64_t v) { return __uint_as_float((uint32_t)v); }
__device__ __forceinline__ float hi_f(uint64_t v) { return __uint_as_float((uint32_t)(v >> 32)); }

// silu without the IEEE division: v / (1 + exp(-v)) takes the division's slow path whenever the denominator is
// huge or infinite (v below about -87), and gate values that far out are common at these weight scales.
// __fdividef returns 0 for an infinite or very large denominator, which is the limit of silu there; error <= 2 ulp.
__device__ __forceinline__ float silu_fast(float v) { return __fdividef(v, 1.0f + __expf(-v)); }

// The 32 values of one nibble half (low nibbles: elements 0..31, high: 32..63 of the chunk)
// packed as 16 bf16 pairs in registers, in K order: out[i] = (element 2i, element 2i+1).
template <bool HI>
__device__ __forceinline__ void dequant_half(const uint32_t* q, float sc, float mn, uint32_t (&out)[16]) {
    const uint64_t neg_magic = packf(-kTwo23), nm = packf(-mn);
#pragma unroll
    for (int c = 0; c < 4; c++) {
        const uint64_t P = pack2(q[2 * c], q[2 * c + 1]);
        const uint64_t P12 = pack2(q[2 * c] >> 12, q[2 * c + 1] >> 12);
        uint64_t o0, o1, o2, o3;
        if (!HI) {
            o0 = ffma2(fadd2(field_or_magic<0xFu << 0>(P), neg_magic), packf(sc), nm);
            o1 = ffma2(fadd2(field_or_magic<0xFu << 8>(P), neg_magic), packf(sc * exp2_neg(8)), nm);
            o2 = ffma2(fadd2(field_or_magic<0xFu << 16>(P), neg_magic), packf(sc * exp2_neg(16)), nm);
            o3 = ffma2(fadd2(field_or_magic<0xFu << 12>(P12), neg_magic), packf(sc * exp2_neg(12)), nm);
        } else {
            o0 = ffma2(fadd2(field_or_magic<0xFu << 4>(P), neg_magic), packf(sc * exp2_neg(4)), nm);
            o1 = ffma2(fadd2(field_or_magic<0xFu << 12>(P), neg_magic), packf(sc * exp2_neg(12)), nm);
            o2 = ffma2(fadd2(field_or_magic<0xFu << 8>(P12), neg_magic), packf(sc * exp2_neg(8)), nm);
            o3 = ffma2(fadd2(field_or_magic<0xFu << 16>(P12), neg_magic), packf(sc * exp2_neg(16)), nm);
        }
        out[4 * c + 0] = bf16x2(lo_f(o0), lo_f(o1));
        out[4 * c + 1] = bf16x2(lo_f(o2), lo_f(o3));
        out[4 * c + 2] = bf16x2(hi_f(o0), hi_f(o1));
        out[4 * c + 3] = bf16x2(hi_f(o2), hi_f(o3));
    }
}

// ───────────────────────── CTA-pair kernel (cta_group::2) ─────────────────────────
// Two CTAs of one cluster share a work item of 256 weight rows x up to 256 token slots.  Each CTA dequantises 128
// of the rows and loads half of the token tile; the leader CTA issues M = 256 MMAs that write 128 accumulator rows
// into each CTA's tensor memory.  What shaped it (all measured on B200):
//   * one thread can issue a tcgen05.mma about every 110-130 cycles, whatever its size: only M = 256, N = 256 MMAs
//     (128 cycles of tensor work) keep the pipe busy, and barrier waits, the fence and the commits are all paid by
//     that same thread, so a pipeline step covers 128 K (8 MMAs) rather than 64;
//   * with the weight operand in shared memory the dequantisers' stores, the TMA writes and the MMAs' operand reads
//     need more than the 128 B/clk an SM's shared memory delivers: the dequantiser warps write their bf16 rows
//     straight into tensor memory (tcgen05.st) and the MMA takes A from there; shared memory carries the token
//     tiles and the raw superblocks only;
//   * the commit -> refill -> arrive round trip between the two CTAs costs about 2400 cycles of signalling: 4
//     weight stages (64 tensor-memory columns each) and 5 token-tile stages (32 KiB each) cover it;
//   * Q4_K rows arrive by TMA (box 128 rows x 144 bytes = one superblock per row) into a 3-deep raw ring, issued
//     by a warp of their own so that they never queue behind the token-tile loads;
//   * 16 dequantiser warps in two groups, each taking one of the two 64-wide chunks of a step;
//   * fused gate/up: the CTA's 128 tile rows are 64 gate rows followed by the 64 up rows of the same
//     intermediate indices; gate and up warps of the epilogue swap half of their columns through shared memory, so
//     all four warps compute, and the bf16 results leave through a shared-memory transpose as 16-byte stores
//     (two-byte stores cost 60 cycles each);
//   * one 256-column accumulator (the other 256 columns hold the weight stages): the epilogue of an item is not
//     overlapped with the MMAs of the next, but both rings refill during it.
// Barriers: a_full[s], b_full[s] and acc_empty live in the leader and also take arrivals from the peer;
// a_empty[s], b_empty[s] and acc_full are signalled in both CTAs at once by the leader's tcgen05.commit.
namespace pair {

constexpr int kThreads = 736;              // 23 warps: token-tile producer, MMA, 4 epilogue, 16 dequantisers, raw producer
constexpr int kRawWarp = 22;
constexpr int kDeqWarp0 = 6, kGroupWarps = 8;
constexpr int kNS = 4;                     // pipeline stages: token tile (shared memory, two 64-wide K chunks = 32 KiB) +
                                           // weight tile (tensor memory, 64 columns); one full / one empty barrier each, so
                                           // the MMA thread pays one wait and one commit per step
constexpr int kNR = 3;                     // raw superblock ring
constexpr int kStageB = 2 * kTileBytes;
constexpr int kRawBytes = 128 * 144;
constexpr int kXchgBytes = 2 * 2 * 32 * 17 * 4;
constexpr int kOffRaw = kNS * kStageB;
constexpr int kOffXchg = kOffRaw + kNR * kRawBytes;
constexpr int kOffCtrl = kOffXchg + kXchgBytes;
constexpr int kSmem = kOffCtrl + 512 + 1024;
constexpr int kTmemCols = 512, kACol0 = 256;
constexpr int kTokPair = 256;

template <bool DUAL>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_w0,
                         const __grid_constant__ CUtensorMap map_w1, const Args a) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_p = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t ctrl = base + kOffCtrl;
    const uint32_t bar_full = ctrl, bar_empty = bar_full + 8 * kNS, bar_rawf = bar_empty + 8 * kNS, bar_rawe = bar_rawf + 8 * kNR,
                   bar_accf = bar_rawe + 8 * kNR, bar_acce = bar_accf + 8, holder = bar_acce + 8;
    volatile uint32_t* holder_p = reinterpret_cast<volatile uint32_t*>(base_p + kOffCtrl + (holder - ctrl));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_p + kOffCtrl + (holder - ctrl) + 4);
    float* xchg = reinterpret_cast<float*>(base_p + kOffXchg);

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_ctarank();
    const uint32_t pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    if (tid == 0) {
        for (int s = 0; s < kNS; s++) {
            // full: both dequantiser groups of each CTA (one K chunk each) + the leader's expect_tx (bytes from both CTAs' loads)
            mbar_init(bar_full + 8 * s, 4 * kGroupWarps + 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int u = 0; u < kNR; u++) {
            mbar_init(bar_rawf + 8 * u, 1);
            mbar_init(bar_rawe + 8 * u, 2 * kGroupWarps);
        }
        mbar_init(bar_accf, 1);
        mbar_init(bar_acce, 8);                                 // 4 epilogue warps of each CTA
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc_pair(holder, kTmemCols);
        tmem_relinquish_pair();
    }
    __syncwarp();
    tc_fence_before_sync();
    cluster_sync();
    tc_fence_after_sync();
    const uint32_t tmem_base = *holder_p;

    const uint32_t nb = DUAL ? a.rows / 128 : a.rows / 256;
    const uint32_t n_items = (uint32_t)(*a.n_tok_tiles) * nb;
    const uint32_t units = a.K / 256;
    const uint32_t leader_full = cluster_map(bar_full, 0), leader_acce = cluster_map(bar_acce, 0);

    auto tile_cols = [&](int32_t nvalid) -> uint32_t { return nvalid <= 32 ? 32u : (uint32_t)((nvalid + 31) & ~31); };

    if (warp == 0) {
        // ───────── TMA producer: the token tile of every step (128 K = two 64-wide swizzled sub-tiles) ─────────
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t item = pair_id; item < n_items && ok && !*abort_flag; item += n_pairs) {
                const uint32_t tt = item / nb;
                const uint32_t ncols = tile_cols(a.tile_nvalid[tt]);
                const int32_t row_b = a.tile_row0[tt] + (int32_t)(rank * (ncols / 2));
                for (uint32_t st = 0; st < units * 2; st++, it++) {
                    const uint32_t s = it % kNS, ph = (it / kNS) & 1;
                    if (!mbar_wait_timed(bar_empty + 8 * s, ph ^ 1, abort_flag)) { ok = false; break; }
                    if (rank == 0) mbar_expect_tx(bar_full + 8 * s, 2 * kStageB);
                    tma_load_2d_pair(base + s * kStageB, &map_b, (int32_t)(st * 256), row_b, leader_full + 8 * s);
                    tma_load_2d_pair(base + s * kStageB + kTileBytes, &map_b, (int32_t)(st * 256 + 128), row_b, leader_full + 8 * s);
                }
            }
        }
    } else if (warp == kRawWarp) {
        // ───────── TMA producer: raw Q4_K superblocks, one unit (256 K) of the CTA's 128 rows per ring slot ─────────
        if (lane == 0) {
            uint32_t uc = 0;
            bool ok = true;
            for (uint32_t item = pair_id; item < n_items && ok && !*abort_flag; item += n_pairs) {
                const uint32_t tt = item / nb, rb = item % nb;
                const uint32_t e = (uint32_t)a.tile_expert[tt];
                for (uint32_t u = 0; u < units; u++, uc++) {
                    const uint32_t ur = uc % kNR;
                    if (!mbar_wait_timed(bar_rawe + 8 * ur, ((uc / kNR) & 1) ^ 1, abort_flag)) { ok = false; break; }
                    const uint32_t dst = base + kOffRaw + ur * kRawBytes;
                    mbar_expect_tx(bar_rawf + 8 * ur, kRawBytes);
                    if (DUAL) {
                        const int32_t row = (int32_t)(e * a.rows + rb * 128 + rank * 64);
                        tma_load_2d(dst, &map_w0, (int32_t)(u * 144), row, bar_rawf + 8 * ur);
                        tma_load_2d(dst + 64 * 144, &map_w1, (int32_t)(u * 144), row, bar_rawf + 8 * ur);
                    } else {
                        tma_load_2d(dst, &map_w0, (int32_t)(u * 144), (int32_t)(e * a.rows + rb * 256 + rank * 128), bar_rawf + 8 * ur);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ───────── MMA issuer (leader CTA only) ─────────
        if (lane == 0 && rank == 0) {
            uint32_t it = 0, n = 0;
            bool ok = true;
            for (uint32_t item = pair_id; item < n_items && ok && !*abort_flag; item += n_pairs, n++) {
                const uint32_t idesc = umma_idesc_bf16(256, tile_cols(a.tile_nvalid[item / nb]));
                if (!mbar_wait_timed_cluster(bar_acce, (n & 1) ^ 1, abort_flag)) break;   // the epilogue has drained the accumulator
                for (uint32_t st = 0; st < units * 2; st++, it++) {
                    const uint32_t sa = it % kNS, sb = sa, pa = (it / kNS) & 1;
                    if (!mbar_wait_timed_cluster(bar_full + 8 * sa, pa, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t at = tmem_base + kACol0 + 64 * sa;
#pragma unroll
                    for (uint32_t c = 0; c < 2; c++) {
                        const uint64_t db = umma_desc_sw128(base + sb * kStageB + c * kTileBytes);
#pragma unroll
                        for (uint32_t k4 = 0; k4 < 4; k4++)
                            umma_bf16_pair_ts(tmem_base, at + 32 * c + 8 * k4, db + 2 * k4, idesc, (st | c | k4) != 0);
                    }
                    umma_commit_pair(bar_empty + 8 * sa, 3);
                }
                if (ok) umma_commit_pair(bar_accf, 3);
            }
        }
    } else if (warp < kDeqWarp0) {
        // ───────── epilogue ─────────
        // The four warps meet on a named barrier inside the loop, so they must leave it together: one thread waits
        // for the accumulator and publishes the outcome (also on abort) to the other 127.
        const uint32_t quarter = warp & 3;
        volatile int* go = reinterpret_cast<volatile int*>(base_p + kOffCtrl + (holder - ctrl) + 8);
        uint32_t n = 0;
        for (uint32_t item = pair_id; item < n_items; item += n_pairs, n++) {
            const uint32_t tt = item / nb, rb = item % nb;
            const int32_t nvalid = a.tile_nvalid[tt];
            const size_t row0 = (size_t)a.tile_row0[tt];
            if (warp == kEpiWarp0 && lane == 0)
                *go = (mbar_wait_timed(bar_accf, n & 1, abort_flag) && !*abort_flag) ? 1 : 0;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const int ready = *go;
            asm volatile("bar.sync 1, 128;" ::: "memory");   // everyone has read it before the next item overwrites it
            if (!ready) break;
            tc_fence_after_sync();
            const uint32_t taddr0 = tmem_base + ((quarter * 32) << 16);
#pragma unroll 1
            for (int cg = 0; cg * 32 < nvalid; cg++) {
                uint32_t v[32];
                tmem_ld32(taddr0 + cg * 32, v);
                tmem_ld_wait();
                if (DUAL) {
                    // tile rows 0..63 = gate (quarters 0, 1), 64..127 = up of the same intermediate indices (quarters
                    // 2, 3).  Each side hands half of its 32 columns to the other: the gate warp finishes tokens
                    // 0..15 of the group, the up warp tokens 16..31.
                    float* xg = xchg + (quarter & 1) * (2 * 32 * 17) + lane * 17;   // gate values 16..31 of my row
                    float* xu = xg + 32 * 17;                                       // up values 0..15 of my row
                    const bool is_gate = quarter < 2;
                    if (is_gate) {
#pragma unroll
                        for (int i = 0; i < 16; i++) xg[i] = __uint_as_float(v[16 + i]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; i++) xu[i] = __uint_as_float(v[i]);
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    float gv[16], uv[16];
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        gv[i] = is_gate ? __uint_as_float(v[i]) : xg[i];
                        uv[i] = is_gate ? xu[i] : __uint_as_float(v[16 + i]);
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");   // the exchange area may be rewritten
                    // 16 tokens x 32 intermediate indices of bf16 go through the warp's own (now idle) exchange array so
                    // that every lane stores 16 bytes: 2 stores per lane instead of 16 two-byte ones.
                    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.out);
                    const uint32_t col0 = rb * 128 + rank * 64 + (quarter & 1) * 32;
                    const int tok0 = cg * 32 + (is_gate ? 0 : 16);
                    uint8_t* stage = reinterpret_cast<uint8_t*>(is_gate ? (xg - lane * 17) : (xu - lane * 17));
#pragma unroll
                    for (int i = 0; i < 16; i++)
                        *reinterpret_cast<__nv_bfloat16*>(stage + i * 64 + lane * 2) = __float2bfloat16_rn(silu_fast(gv[i]) * uv[i]);
                    __syncwarp();
#pragma unroll
                    for (int hh = 0; hh < 2; hh++) {
                        const int tk = (lane >> 2) + 8 * hh, ch = lane & 3;
                        const uint4 pk = *reinterpret_cast<const uint4*>(stage + tk * 64 + ch * 16);
                        if (tok0 + tk < nvalid) *reinterpret_cast<uint4*>(out + (row0 + tok0 + tk) * a.ld + col0 + 8 * ch) = pk;
                    }
                    __syncwarp();
                } else {
                    float* out = reinterpret_cast<float*>(a.out);
                    const uint32_t col = rb * 256 + rank * 128 + quarter * 32 + lane;
                    if (a.row_ptr != nullptr) {
#pragma unroll
                        for (int i = 0; i < 32; i++)
                            if (cg * 32 + i < nvalid) a.row_ptr[row0 + cg * 32 + i][col] = __uint_as_float(v[i]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; i++)
                            if (cg * 32 + i < nvalid) out[(row0 + cg * 32 + i) * a.ld + col] = __uint_as_float(v[i]);
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0) mbar_arrive(bar_acce);
                else mbar_arrive_cluster(leader_acce);
            }
        }
    } else if (warp < kRawWarp) {
        // ───────── dequantisers: raw ring -> bf16 rows in tensor memory.  Group g takes chunk g of every step (the
        //            chunks j of a unit with j % 2 == g).  A warp may only write the tensor-memory lanes
        //            32 * (warp % 4) .. + 31: those are its rows. ─────────
        const uint32_t dw = warp - kDeqWarp0;
        const uint32_t g = dw / kGroupWarps, part = (dw % kGroupWarps) / 4;   // part 0: low nibbles (K 0..31 of the chunk), 1: high
        const uint32_t quarter = warp & 3, r = quarter * 32 + lane;
        uint32_t uc = 0;
        bool ok = true;
        for (uint32_t item = pair_id; item < n_items && ok && !*abort_flag; item += n_pairs) {
            for (uint32_t u = 0; u < units && ok; u++, uc++) {
                const uint32_t ur = uc % kNR;
                if (!mbar_wait_timed(bar_rawf + 8 * ur, (uc / kNR) & 1, abort_flag)) { ok = false; break; }
                const uint32_t raw_row = base + kOffRaw + ur * kRawBytes + r * 144;
                uint32_t h0, h1, h2, h3;
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(h0), "=r"(h1), "=r"(h2), "=r"(h3) : "r"(raw_row) : "memory");
                const float dd = half_bits_to_float(h0), dmin = half_bits_to_float(h0 >> 16);
                const Q4KScales sc = q4k_unpack_scales(h1, h2, h3);
#pragma unroll
                for (int jj = 0; jj < 2; jj++) {
                    const uint32_t j = 2 * jj + g;               // chunk of the unit; step 2 * unit + jj holds chunks 2jj, 2jj + 1
                    const uint32_t it = uc * 2 + jj;
                    const uint32_t s = it % kNS, ph = (it / kNS) & 1;
                    uint32_t q[8];
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(q[0]), "=r"(q[1]), "=r"(q[2]), "=r"(q[3]) : "r"(raw_row + 16 + 32 * j) : "memory");
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(q[4]), "=r"(q[5]), "=r"(q[6]), "=r"(q[7]) : "r"(raw_row + 32 + 32 * j) : "memory");
                    const uint32_t sh = 8 * j;
                    uint32_t out[16];
                    if (part == 0) dequant_half<false>(q, dd * (float)((sc.sl >> sh) & 0xFFu), dmin * (float)((sc.ml >> sh) & 0xFFu), out);
                    else dequant_half<true>(q, dd * (float)((sc.sh >> sh) & 0xFFu), dmin * (float)((sc.mh >> sh) & 0xFFu), out);
                    uint32_t got = 1;
                    if (lane == 0) got = mbar_wait_timed(bar_empty + 8 * s, ph ^ 1, abort_flag);
                    got = __shfl_sync(0xffffffffu, got, 0);
                    if (!got) { ok = false; break; }
                    tc_fence_after_sync();
                    tmem_st16(tmem_base + ((quarter * 32) << 16) + kACol0 + 64 * s + 32 * g + 16 * part, out);
                    tmem_st_wait();
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) {
                        if (rank == 0) mbar_arrive(bar_full + 8 * s);
                        else mbar_arrive_cluster(leader_full + 8 * s);
                    }
                }
                __syncwarp();
                if (lane == 0 && ok) mbar_arrive(bar_rawe + 8 * ur);
            }
        }
    }

    __syncwarp();            // the single-lane roles rejoin their warps before the aligned cluster barrier
    tc_fence_before_sync();
    cluster_sync();
    if (warp == 0) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, kTmemCols);
    }
    if (tid == 0 && *abort_flag && a.status) atomicExch(a.status, 2);
}

}  // namespace pair

// ───────────────────────── token permutation ─────────────────────────

// counts[e] = slots routed to expert e; slots with an id outside [0, E) get position -1.
__global__ void __launch_bounds__(256) count_kernel(const int32_t* __restrict__ idx, uint32_t S, uint32_t E,
                                                     int32_t* __restrict__ counts, int32_t* __restrict__ pos_of_slot) {
    __shared__ int hist[256];
    hist[threadIdx.x] = 0;
    __syncthreads();
    for (uint32_t s = blockIdx.x * 4096 + threadIdx.x, i = 0; i < 16 && s < S; i++, s += 256) {
        const int32_t e = idx[s];
        if (e >= 0 && (uint32_t)e < E) atomicAdd(&hist[e], 1);
        else pos_of_slot[s] = -1;
    }
    __syncthreads();
    if (threadIdx.x < E && hist[threadIdx.x]) atomicAdd(&counts[threadIdx.x], hist[threadIdx.x]);
}

// One CTA per expert: first row of the expert in the permuted order (experts in index order, each padded to a
// multiple of 128 rows), the token-tile table (tiles of `tile_tok` slots, 128 or 256, never across experts), and the
// position of each of its slots (slot order kept).
__global__ void __launch_bounds__(1024) place_kernel(const int32_t* __restrict__ idx, uint32_t S, uint32_t E,
                                                      const int32_t* __restrict__ counts, int tile_tok,
                                                      int32_t* __restrict__ pos_of_slot, int32_t* __restrict__ tile_expert,
                                                      int32_t* __restrict__ tile_nvalid, int32_t* __restrict__ tile_row0,
                                                      int32_t* __restrict__ n_tok_tiles) {
    __shared__ int s_cnt[256];
    __shared__ int s_warp[32];
    __shared__ int s_off, s_tile0, s_chunk;
    const uint32_t e = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < 256) s_cnt[tid] = tid < E ? counts[tid] : 0;
    __syncthreads();
    if (tid == 0) {
        int off = 0, tiles = 0;
        for (uint32_t i = 0; i < E; i++) {
            if (i == e) { s_off = off; s_tile0 = tiles; }
            off += ((s_cnt[i] + kTok - 1) / kTok) * kTok;
            tiles += (s_cnt[i] + tile_tok - 1) / tile_tok;
        }
        if (e == 0) n_tok_tiles[0] = tiles;
    }
    __syncthreads();
    const int cnt = s_cnt[e], off = s_off, tile0 = s_tile0;
    for (int i = tid; i * tile_tok < cnt; i += 1024) {
        tile_expert[tile0 + i] = (int32_t)e;
        tile_nvalid[tile0 + i] = min(tile_tok, cnt - i * tile_tok);
        tile_row0[tile0 + i] = off + i * tile_tok;
    }
    // every thread takes 4 consecutive slots per round, so a round covers 4096 slots in slot order
    int running = 0;
    for (uint32_t s0 = 0; s0 < S; s0 += 4096) {
        const uint32_t s = s0 + 4 * tid;
        bool hit[4];
        int mine = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            hit[i] = s + i < S && idx[s + i] == (int32_t)e;
            mine += hit[i];
        }
        int incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, o);
            if ((int)lane >= o) incl += t;
        }
        if (lane == 31) s_warp[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int v = s_warp[lane], wi = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, wi, o);
                if ((int)lane >= o) wi += t;
            }
            s_warp[lane] = wi - v;   // exclusive prefix over the warps
            if (lane == 31) s_chunk = wi;
        }
        __syncthreads();
        int p = off + running + s_warp[warp] + incl - mine;
#pragma unroll
        for (int i = 0; i < 4; i++)
            if (hit[i]) pos_of_slot[s + i] = p++;
        running += s_chunk;
        __syncthreads();
    }
}

// xperm[pos(s)][:] = bf16(x[s / k][:]); one warp per slot, 8 slots per CTA.
__global__ void __launch_bounds__(256) gather_kernel(const float* __restrict__ x, const int32_t* __restrict__ pos_of_slot,
                                                      __nv_bfloat16* __restrict__ xperm, uint32_t S, uint32_t h, uint32_t k) {
    const uint32_t s = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (s >= S) return;
    const int32_t pos = pos_of_slot[s];
    if (pos < 0) return;
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)(s / k) * h);
    uint4* dst = reinterpret_cast<uint4*>(xperm + (size_t)pos * h);
#pragma unroll 4
    for (uint32_t c = lane; c < h / 8; c += 32) {
        const float4 a0 = __ldg(src + 2 * c), a1 = __ldg(src + 2 * c + 1);
        uint4 o;
        o.x = bf16x2(a0.x, a0.y); o.y = bf16x2(a0.z, a0.w); o.z = bf16x2(a1.x, a1.y); o.w = bf16x2(a1.z, a1.w);
        dst[c] = o;
    }
}

// The same permutation for rows that are bf16 already (slots received from other ranks): xperm[pos(s)][:] = x[s][:].
__global__ void __launch_bounds__(256) gather_bf16_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ pos_of_slot,
                                                           __nv_bfloat16* __restrict__ xperm, uint32_t S, uint32_t h) {
    const uint32_t s = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (s >= S) return;
    const int32_t pos = pos_of_slot[s];
    if (pos < 0) return;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)s * h);
    uint4* dst = reinterpret_cast<uint4*>(xperm + (size_t)pos * h);
    for (uint32_t c = lane; c < h / 8; c += 32) dst[c] = src[c];
}

// Destination of every permuted row of an expert-parallel block: receive row i (region r = i / cap_src of rank r, used
// while i % cap_src < cnt[r]) came from slot meta[i].y of rank r and goes back to row meta[i].y of that rank's return buffer.
struct ReturnPeers {
    float* p[8];
};
__global__ void __launch_bounds__(256) row_ptr_kernel(const int32_t* __restrict__ pos_of_slot, const int2* __restrict__ meta,
                                                       const int32_t* __restrict__ cnt, const ReturnPeers ry, float** __restrict__ table,
                                                       uint32_t cap_src, uint32_t total, uint32_t h) {
    const uint32_t i = blockIdx.x * 256 + threadIdx.x;
    if (i >= total) return;
    const uint32_t r = i / cap_src, j = i - r * cap_src;
    if (j >= (uint32_t)cnt[r]) return;
    const int32_t pos = pos_of_slot[i];
    if (pos >= 0) table[pos] = ry.p[r] + (size_t)meta[i].y * h;
}

// out[t] = (residual ? residual[t] : 0) + sum_i w[t][i] * y[pos(t, i)]   (routing order; product and sum rounded
// separately, like the reference's scale-accumulate followed by the residual add).
__global__ void __launch_bounds__(256) combine_kernel(const float* __restrict__ y, const int32_t* __restrict__ pos_of_slot,
                                                       const float* __restrict__ w, const float* __restrict__ residual,
                                                       float* __restrict__ out, uint32_t h, uint32_t k) {
    const uint32_t t = blockIdx.y, c = blockIdx.x * 256 + threadIdx.x;
    if (c >= h / 4) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t i = 0; i < k; i++) {
        const int32_t pos = pos_of_slot[t * k + i];
        if (pos < 0) continue;
        const float wi = w[t * k + i];
        const float4 v = __ldg(reinterpret_cast<const float4*>(y + (size_t)pos * h) + c);
        acc.x = __fadd_rn(acc.x, __fmul_rn(wi, v.x)); acc.y = __fadd_rn(acc.y, __fmul_rn(wi, v.y));
        acc.z = __fadd_rn(acc.z, __fmul_rn(wi, v.z)); acc.w = __fadd_rn(acc.w, __fmul_rn(wi, v.w));
    }
    float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
    if (residual) b = reinterpret_cast<const float4*>(residual + (size_t)t * h)[c];
    reinterpret_cast<float4*>(out + (size_t)t * h)[c] = make_float4(b.x + acc.x, b.y + acc.y, b.z + acc.z, b.w + acc.w);
}

// ───────────────────────── host side ─────────────────────────

struct Scratch {
    int32_t *counts, *n_tok_tiles, *tile_expert, *tile_nvalid, *tile_row0, *pos_of_slot, *idx;
    float *logits, *w, *y;
    __nv_bfloat16 *xperm, *act;
    uint32_t max_tiles;
    size_t bytes;
};

static Scratch carve(void* base, uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k) {
    Scratch s{};
    const size_t S = (size_t)T * k;
    s.max_tiles = (uint32_t)((S + kTok - 1) / kTok) + E;
    const size_t rows = (size_t)s.max_tiles * kTok + 256;   // + slack: a tile's load may reach past its last valid row
    size_t off = 0;
    auto take = [&](size_t bytes) {
        void* p = base ? (void*)((uint8_t*)base + off) : nullptr;
        off += (bytes + 1023) & ~(size_t)1023;
        return p;
    };
    s.counts = (int32_t*)take(4 * 256);
    s.n_tok_tiles = (int32_t*)take(16);
    s.tile_expert = (int32_t*)take(4 * (size_t)s.max_tiles);
    s.tile_nvalid = (int32_t*)take(4 * (size_t)s.max_tiles);
    s.tile_row0 = (int32_t*)take(4 * (size_t)s.max_tiles);
    s.pos_of_slot = (int32_t*)take(4 * S);
    s.idx = (int32_t*)take(4 * S);
    s.w = (float*)take(4 * S);
    s.logits = (float*)take(4 * (size_t)T * E);
    s.xperm = (__nv_bfloat16*)take(2 * rows * h);
    s.act = (__nv_bfloat16*)take(2 * rows * ff);
    s.y = (float*)take(4 * rows * h);
    s.bytes = off;
    return s;
}

template <bool DUAL>
static int32_t launch_pair(runit_ctx* ctx, const char* name, const Args& a, const void* b_ptr, uint32_t b_rows, uint32_t n_experts,
                           uint32_t max_items) {
    static bool attr_set[64] = {false};
    if (ctx->device >= 0 && ctx->device < 64 && !attr_set[ctx->device]) {
        RUNIT_CUDA_TRY(ctx, cudaFuncSetAttribute(pair::grouped_gemm_pair_kernel<DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, pair::kSmem));
        attr_set[ctx->device] = true;
    }
    CUtensorMap map_b, map_w0, map_w1;
    int32_t st = runit_get_tmap(ctx, b_ptr, b_rows, (uint64_t)a.K * 2, kTok, 128, &map_b, 1);
    if (st != RUNIT_OK) return st;
    const uint64_t w_rows = (uint64_t)n_experts * a.rows, row_bytes = (uint64_t)a.K / 256 * 144;
    st = runit_get_tmap(ctx, a.w0, w_rows, row_bytes, DUAL ? 64 : 128, 144, &map_w0);
    if (st != RUNIT_OK) return st;
    map_w1 = map_w0;
    if (DUAL && (st = runit_get_tmap(ctx, a.w1, w_rows, row_bytes, 64, 144, &map_w1)) != RUNIT_OK) return st;
    uint32_t pairs = (uint32_t)ctx->sm_count / 2;
    if (pairs > max_items) pairs = max_items;
    if (pairs == 0) pairs = 1;
    pair::grouped_gemm_pair_kernel<DUAL><<<2 * pairs, pair::kThreads, pair::kSmem, ctx->stream>>>(map_b, map_w0, map_w1, a);
    return runit_after_launch(ctx, name);
}

// The expert part of the block for given routing (idx int32 [T][k], w f32 [T][k]).
// x_bf16 != nullptr: the rows are bf16 already, one per slot (k == 1); out == nullptr: the weighted sum is left to the
// caller, who finds the expert outputs in s.y at row s.pos_of_slot[slot].
static int32_t experts_impl(runit_ctx* ctx, const Scratch& s, const void* gate, const void* up, const void* down,
                            const float* x, const int32_t* idx, const float* w, const float* residual, float* out,
                            uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k, const void* x_bf16 = nullptr,
                            // expert-parallel return fused into the down GEMM: see row_ptr_kernel (cap_src > 0 turns it on)
                            const int2* ret_meta = nullptr, const int32_t* ret_cnt = nullptr, const ReturnPeers* ret_peers = nullptr,
                            uint32_t cap_src = 0) {
    const uint32_t S = T * k;
    RUNIT_CUDA_TRY(ctx, cudaMemsetAsync(s.counts, 0, 4 * 256, ctx->stream));
    count_kernel<<<(S + 4095) / 4096, 256, 0, ctx->stream>>>(idx, S, E, s.counts, s.pos_of_slot);
    int32_t st = runit_after_launch(ctx, "moe_grouped_count");
    if (st != RUNIT_OK) return st;
    place_kernel<<<E, 1024, 0, ctx->stream>>>(idx, S, E, s.counts, pair::kTokPair, s.pos_of_slot, s.tile_expert,
                                              s.tile_nvalid, s.tile_row0, s.n_tok_tiles);
    if ((st = runit_after_launch(ctx, "moe_grouped_place")) != RUNIT_OK) return st;
    if (x_bf16) gather_bf16_kernel<<<(S + 7) / 8, 256, 0, ctx->stream>>>((const __nv_bfloat16*)x_bf16, s.pos_of_slot, s.xperm, S, h);
    else gather_kernel<<<(S + 7) / 8, 256, 0, ctx->stream>>>(x, s.pos_of_slot, s.xperm, S, h, k);
    if ((st = runit_after_launch(ctx, "moe_grouped_gather")) != RUNIT_OK) return st;

    const uint32_t rows = s.max_tiles * kTok + 256;
    Args a1{};
    a1.w0 = (const uint8_t*)gate; a1.w1 = (const uint8_t*)up; a1.rows = ff; a1.K = h; a1.nb = ff / kRows;
    a1.tile_expert = s.tile_expert; a1.tile_nvalid = s.tile_nvalid; a1.tile_row0 = s.tile_row0; a1.n_tok_tiles = s.n_tok_tiles;
    a1.out = s.act; a1.ld = ff; a1.status = ctx->d_status;
    Args a2{};
    a2.w0 = (const uint8_t*)down; a2.w1 = nullptr; a2.rows = h; a2.K = ff; a2.nb = h / kRows;
    a2.tile_expert = s.tile_expert; a2.tile_nvalid = s.tile_nvalid; a2.tile_row0 = s.tile_row0; a2.n_tok_tiles = s.n_tok_tiles;
    a2.out = s.y; a2.ld = h; a2.status = ctx->d_status;
    if (cap_src > 0) {
        // the table of row destinations lives in the output area the GEMM no longer writes (8 bytes per row of 4*h)
        float** table = reinterpret_cast<float**>(s.y);
        row_ptr_kernel<<<(S + 255) / 256, 256, 0, ctx->stream>>>(s.pos_of_slot, ret_meta, ret_cnt, *ret_peers, table, cap_src, S, h);
        if ((st = runit_after_launch(ctx, "moe_grouped_row_ptr")) != RUNIT_OK) return st;
        a2.row_ptr = table;
    }
    if ((st = launch_pair<true>(ctx, "moe_grouped_gate_up", a1, s.xperm, rows, E, s.max_tiles * (ff / 128))) != RUNIT_OK) return st;
    if ((st = launch_pair<false>(ctx, "moe_grouped_down", a2, s.act, rows, E, s.max_tiles * (h / 256))) != RUNIT_OK) return st;
    if (!out) return RUNIT_OK;
    combine_kernel<<<dim3((h / 4 + 255) / 256, T), 256, 0, ctx->stream>>>(s.y, s.pos_of_slot, w, residual, out, h, k);
    return runit_after_launch(ctx, "moe_grouped_combine");
}

static int32_t check_shapes(runit_ctx* ctx, const char* who, uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k) {
    RUNIT_REQUIRE(ctx, T > 0 && h > 0 && ff > 0 && E > 0 && k > 0, "%s: empty shape", who);
    RUNIT_REQUIRE(ctx, h % 256 == 0 && ff % 256 == 0, "%s: hidden %u and intermediate %u must be multiples of 256", who, h, ff);
    RUNIT_REQUIRE(ctx, E <= 256 && k <= E && k <= 32, "%s: E=%u k=%u unsupported (E <= 256, k <= min(E, 32))", who, E, k);
    RUNIT_REQUIRE(ctx, (uint64_t)T * k < (1ull << 30), "%s: too many slots", who);
    return RUNIT_OK;
}

// ── dense use of the same kernels: one "expert" that owns the whole matrix, tokens in their own order ──
__global__ void dense_tiles_kernel(uint32_t T, int32_t* tile_expert, int32_t* tile_nvalid, int32_t* tile_row0, int32_t* n_tok_tiles) {
    const uint32_t n = (T + pair::kTokPair - 1) / pair::kTokPair;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        tile_expert[i] = 0;
        tile_nvalid[i] = (int32_t)min((uint32_t)pair::kTokPair, T - i * pair::kTokPair);
        tile_row0[i] = (int32_t)(i * pair::kTokPair);
    }
    if (threadIdx.x == 0) n_tok_tiles[0] = (int32_t)n;
}

}  // namespace gg

// Expert outputs of S slots whose rows are bf16 already (slot s: expert idx[s] of the E local ones, or an id outside
// [0, E) for an unused slot): the two grouped GEMMs without the weighted sum.  *y_out is the f32 output [rows][h] in the
// permuted order, *pos_out the row of every slot (-1 for unused slots); both live inside `scratch`
// (runit_moe_grouped_scratch_bytes(S, h, ff, E, 1) bytes, 1024-byte aligned).
// ret_*: the outputs go straight into the return buffers of the ranks the rows came from (row_ptr_kernel), *y_out is
// then unused.
int32_t moe_grouped_slots_bf16(runit_ctx* ctx, const void* gate, const void* up, const void* down, const void* x_bf16,
                               const int32_t* idx, void* scratch, size_t scratch_bytes, uint32_t S, uint32_t h, uint32_t ff, uint32_t E,
                               const float** y_out, const int32_t** pos_out, const void* ret_meta, const int32_t* ret_cnt,
                               void* const* ret_rows_all, uint32_t world, uint32_t cap_src) {
    int32_t st = gg::check_shapes(ctx, "moe_grouped_slots_bf16", S, h, ff, E, 1);
    if (st != RUNIT_OK) return st;
    const gg::Scratch s = gg::carve(scratch, S, h, ff, E, 1);
    if (s.bytes > scratch_bytes)
        return runit_fail(ctx, RUNIT_ERR_BUFFER_SIZE, "moe_grouped_slots_bf16: scratch has %zu bytes, needs %zu", scratch_bytes, s.bytes);
    *y_out = s.y;
    *pos_out = s.pos_of_slot;
    if (ret_rows_all) {
        gg::ReturnPeers rp{};
        for (uint32_t p = 0; p < world && p < 8; p++) rp.p[p] = (float*)ret_rows_all[p];
        return gg::experts_impl(ctx, s, gate, up, down, nullptr, idx, nullptr, nullptr, nullptr, S, h, ff, E, 1, x_bf16, (const int2*)ret_meta,
                                ret_cnt, &rp, cap_src);
    }
    return gg::experts_impl(ctx, s, gate, up, down, nullptr, idx, nullptr, nullptr, nullptr, S, h, ff, E, 1, x_bf16);
}

// The weighted sum of the batched block by itself: out[t] = residual[t] + sum_i w[t][i] * y[pos_of_slot[t*k+i]].
int32_t moe_grouped_combine(runit_ctx* ctx, const float* y, const int32_t* pos_of_slot, const float* w, const float* residual, float* out,
                            uint32_t T, uint32_t h, uint32_t k) {
    gg::combine_kernel<<<dim3((h / 4 + 255) / 256, T), 256, 0, ctx->stream>>>(y, pos_of_slot, w, residual, out, h, k);
    return runit_after_launch(ctx, "moe_grouped_combine");
}

// Tile tables for dense_gemm_q4k_bf16 over T tokens: `tables` holds 3 * ceil(T / 256) + 4 int32.
int32_t dense_tiles_prepare(runit_ctx* ctx, int32_t* tables, uint32_t T) {
    const uint32_t n = (T + gg::pair::kTokPair - 1) / gg::pair::kTokPair;
    gg::dense_tiles_kernel<<<1, 256, 0, ctx->stream>>>(T, tables + 4, tables + 4 + n, tables + 4 + 2 * n, tables);
    return runit_after_launch(ctx, "dense_tiles");
}

// out[t][r] = sum_k bf16(W[r][k]) * x[t][k] (f32 out, w_up == nullptr), or out[t][r] = bf16(silu(W.x) * (W_up.x)) (bf16 out):
// the grouped tensor-core GEMM with every token tile on expert 0.  x_bf16 has x_rows rows allocated, at least
// ceil(T / 256) * 256 + 256 (a tile's load may reach past its last valid row; what it reads there is never stored).
int32_t dense_gemm_q4k_bf16(runit_ctx* ctx, const char* name, const void* w, const void* w_up, uint32_t rows, uint32_t K,
                            const void* x_bf16, uint32_t x_rows, void* out, uint32_t ld, uint32_t T, const int32_t* tables) {
    RUNIT_REQUIRE(ctx, w && x_bf16 && out && tables && T > 0, "%s: null pointer", name);
    RUNIT_REQUIRE(ctx, K % 256 == 0 && rows % 256 == 0, "%s: rows %u and K %u must be multiples of 256", name, rows, K);
    const uint32_t n = (T + gg::pair::kTokPair - 1) / gg::pair::kTokPair;
    RUNIT_REQUIRE(ctx, x_rows >= n * gg::pair::kTokPair + 256, "%s: activation buffer too short", name);
    gg::Args a{};
    a.w0 = (const uint8_t*)w;
    a.w1 = (const uint8_t*)w_up;
    a.rows = rows;
    a.K = K;
    a.nb = rows / gg::kRows;
    a.tile_expert = tables + 4;
    a.tile_nvalid = tables + 4 + n;
    a.tile_row0 = tables + 4 + 2 * n;
    a.n_tok_tiles = tables;
    a.out = out;
    a.ld = ld;
    a.status = ctx->d_status;
    if (w_up) return gg::launch_pair<true>(ctx, name, a, x_bf16, x_rows, 1, n * (rows / 128));
    return gg::launch_pair<false>(ctx, name, a, x_bf16, x_rows, 1, n * (rows / 256));
}

// moe.cu
int32_t moe_router(runit_ctx* ctx, const float* router_w, const float* x, float* logits, uint32_t E, uint32_t h, uint32_t T);
int32_t moe_topk(runit_ctx* ctx, const float* logits, uint32_t E, uint32_t k, int32_t renorm, uint32_t T, int32_t* idx, float* w);

}  // namespace runit

using namespace runit;

extern "C" {

size_t runit_moe_grouped_scratch_bytes(uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k) {
    return gg::carve(nullptr, T, h, ff, E, k).bytes;
}

int32_t runit_moe_experts_grouped_q4k_bf16(runit_ctx_t* ctx, const void* gate, const void* up, const void* down, const void* x,
                                           const void* idx, const void* w, const void* residual, void* out, void* scratch,
                                           size_t scratch_bytes, uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    int32_t st = gg::check_shapes(ctx, "moe_experts_grouped_q4k_bf16", T, h, ff, E, k);
    if (st != RUNIT_OK) return st;
    RUNIT_REQUIRE(ctx, gate && up && down && x && idx && w && out && scratch, "moe_experts_grouped_q4k_bf16: null pointer");
    RUNIT_REQUIRE(ctx, runit_aligned(scratch, 1024) && runit_aligned(gate, 16) && runit_aligned(up, 16) && runit_aligned(down, 16) &&
                           runit_aligned(x, 16) && runit_aligned(out, 16) && (!residual || runit_aligned(residual, 16)),
                  "moe_experts_grouped_q4k_bf16: scratch must be 1024-byte aligned, tensors 16-byte aligned");
    const gg::Scratch s = gg::carve(scratch, T, h, ff, E, k);
    if (s.bytes > scratch_bytes)
        return runit_fail(ctx, RUNIT_ERR_BUFFER_SIZE, "moe_experts_grouped_q4k_bf16: scratch has %zu bytes, needs %zu", scratch_bytes, s.bytes);
    return gg::experts_impl(ctx, s, gate, up, down, (const float*)x, (const int32_t*)idx, (const float*)w, (const float*)residual,
                            (float*)out, T, h, ff, E, k);
}

int32_t runit_moe_layer_q4k_bf16(runit_ctx_t* ctx, const void* router_w, const void* gate, const void* up, const void* down,
                                 const void* x, const void* residual, void* out, void* idx_out, void* w_out, void* scratch,
                                 size_t scratch_bytes, uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k, int32_t renorm) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    int32_t st = gg::check_shapes(ctx, "moe_layer_q4k_bf16", T, h, ff, E, k);
    if (st != RUNIT_OK) return st;
    RUNIT_REQUIRE(ctx, router_w && gate && up && down && x && out && scratch, "moe_layer_q4k_bf16: null pointer");
    RUNIT_REQUIRE(ctx, runit_aligned(scratch, 1024) && runit_aligned(gate, 16) && runit_aligned(up, 16) && runit_aligned(down, 16) &&
                           runit_aligned(x, 16) && runit_aligned(out, 16) && runit_aligned(router_w, 16) &&
                           (!residual || runit_aligned(residual, 16)),
                  "moe_layer_q4k_bf16: scratch must be 1024-byte aligned, tensors 16-byte aligned");
    const gg::Scratch s = gg::carve(scratch, T, h, ff, E, k);
    if (s.bytes > scratch_bytes)
        return runit_fail(ctx, RUNIT_ERR_BUFFER_SIZE, "moe_layer_q4k_bf16: scratch has %zu bytes, needs %zu", scratch_bytes, s.bytes);
    st = moe_router(ctx, (const float*)router_w, (const float*)x, s.logits, E, h, T);
    if (st != RUNIT_OK) return st;
    int32_t* idx = idx_out ? (int32_t*)idx_out : s.idx;
    float* w = w_out ? (float*)w_out : s.w;
    st = moe_topk(ctx, s.logits, E, k, renorm, T, idx, w);
    if (st != RUNIT_OK) return st;
    return gg::experts_impl(ctx, s, gate, up, down, (const float*)x, idx, w, (const float*)residual, (float*)out, T, h, ff, E, k);
}

}  // extern "C"
