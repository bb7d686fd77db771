// Fused-dequant GEMV kernels for sm_100a: y = dequant(W) . x with W in Q8_0 / Q4_0 / Q4_K.
//
// Replaces the Metal kernels of crates/kernels/shaders/{gemv_q8_0,gemv_q4_0,gemv_q4k,
// fused_qkv,fused_ffn}.metal.  Design (HBM-bound streaming kernel):
//   * a CTA of 4 warps owns a tile of 32 rows; warp w dots the rows with the K "units"
//     w, w+4, w+8, ... (a unit = 256 weights of a row for the 4-bit formats, 128 for Q8_0);
//   * every warp runs its OWN cp.async ring (3 stages of 32 rows x 1 unit + the matching slice
//     of the activations), synchronised with __syncwarp only: there is no CTA barrier in the
//     K loop, so the bytes in flight per SM depend neither on registers nor on the slowest warp;
//   * lane l owns row l: it reads its unit from the shared tile with 128-bit loads (row pitch is
//     an odd multiple of the load width: conflict-free), the activation slice is a warp-wide
//     broadcast, and no cross-lane reduction is needed until the end;
//   * the activation slice of the next stage is permuted, pre-scaled and (Q4_K) block-summed by
//     the warp one stage ahead, which removes integer->float conversions, per-weight scale
//     multiplies and register-pair shuffles from the inner loop (see gemv_common.cuh);
//   * the four K-slices of a row are added in a fixed order (deterministic results).
#pragma once

#include <type_traits>

#include "gemv_common.cuh"
#include "gemv_int8.cuh"
#include "runit_cuda.h"
#include "tma.cuh"

namespace runit {

constexpr int kNT = 128;   // threads per CTA
constexpr int kRT = 32;    // rows per tile (one per lane)
constexpr int kKS = 4;     // K-slices (one per warp)

template <int FMT> struct Traits;
template <> struct Traits<RUNIT_FMT_Q8_0> { static constexpr int UE = 128, UB = 136, BPU = 4; };
template <> struct Traits<RUNIT_FMT_Q4_0> { static constexpr int UE = 256, UB = 144, BPU = 8; };
template <> struct Traits<RUNIT_FMT_Q4K>  { static constexpr int UE = 256, UB = 144, BPU = 1; };

// One stage of one warp's ring.
template <int FMT, int B, bool XF16>
struct WarpStage {
    using T = Traits<FMT>;
    static constexpr int W_BYTES = kRT * T::UB;                    // dense rows, pitch UB
    static constexpr int XR_OFF = W_BYTES;                         // raw f16 activations (XF16 only)
    static constexpr int XR_BYTES = XF16 ? B * T::UE * 2 : 0;
    static constexpr int XP_OFF = XR_OFF + XR_BYTES;               // prepared f32 activations
    static constexpr int XP_BYTES = B * T::UE * 4;
    static constexpr int XS_OFF = XP_OFF + XP_BYTES;               // 32-element block sums (Q4_K)
    static constexpr int XS_BYTES = (FMT == RUNIT_FMT_Q4K) ? B * 8 * 4 : 0;
    // padded to 128 bytes: the destination of a tiled bulk load must be 128-byte aligned
    static constexpr int BYTES = (XS_OFF + XS_BYTES + 127) / 128 * 128;
    static_assert(W_BYTES % 16 == 0 && XP_OFF % 16 == 0 && XS_OFF % 16 == 0, "regions stay 16-byte aligned");
};

enum { RES_NONE = 0, RES_F32 = 1, RES_F16 = 2 };
enum { BIAS_NONE = 0, BIAS_F16 = 1, BIAS_F32 = 2 };

struct GemvSeg {
    const uint8_t* w;     // weight rows of this segment
    const uint8_t* w2;    // second matrix (fused gate/up), else null
    void* y;
    const void* res;
    const void* bias;
    uint32_t rows;
    uint32_t tile_begin;  // first tile index of this segment in the grid
};

struct GemvArgs {
    GemvSeg seg[3];
    int32_t nseg;
    const void* x;
    uint32_t k, nb, row_bytes, n_units, n_tiles;
    uint32_t csplit;       // CTAs per tile (thread-block cluster size along K): 1, 2 or 4
    uint32_t ldy;          // elements between batch rows of y / residual
    int32_t out_f16, res_kind, bias_kind, dual;
    int32_t* status;       // host-visible word: set non-zero if a bounded wait ran out
    // Grouped (mixture-of-experts) mode, active when grp_expert != nullptr: the launch covers
    // n_slots independent GEMVs; slot s uses the weight rows of expert grp_expert[s] inside the
    // stacked matrix seg[0].w ([E][grp_rows][row_bytes]), the input row s / grp_xdiv and the
    // output row s.
    const int32_t* grp_expert;
    uint32_t grp_rows, grp_tiles, grp_xdiv;
    int32_t grp_lo;        // slot s uses expert grp_expert[s] - grp_lo; ids outside [0, grp_cnt) mark unused slots
    uint32_t grp_cnt;
    // Row-sharded launch with the all-gather fused into the epilogue: every f32 result of segment 0 is also
    // stored at the same index of these vectors, which live in the memory of the other GPUs (plain peer stores).
    float* peer_y[7];
    uint32_t n_peer;
    // RMSNorm prologue (batch 1, f32 input), active when norm_gamma != nullptr: x is the un-normalised hidden state and the
    // kernel multiplies with x * rsqrt(mean(x^2) + eps) * gamma (crates/kernels/shaders/norm.metal:95-154 feeding the
    // GEMV, crates/engine/src/forward.rs:1528-1569).  Every CTA computes the scale itself from the k inputs.
    const float* norm_gamma;
    float norm_eps;
    // Grouped mode with the weighted sum of the slots fused in (one token), active when cmb_out != nullptr: after storing
    // its rows of y[slot], every tile takes a ticket on cmb_cnt[row tile]; the tile that takes the last of the cmb_slots
    // tickets writes cmb_out[r] = cmb_res[r] + sum_i cmb_w[i] * y[i][r] (i ascending, as moe_combine_kernel does) for the
    // rows of the tile and puts the counter back to zero.
    // Dependent-launch ordering for two grouped launches in a row (gate/up, then down) whose expert ids were written by the
    // kernel BEFORE the first one.  late_trigger: this kernel lets its successor start only after its own dependency wait
    // returned, i.e. once everything older than itself has completed.  grp_early: the predecessor was launched with
    // late_trigger, so the expert ids are final when this kernel starts: it requests its first weight stages before
    // its own wait (the activations come from the predecessor and follow the wait).
    int32_t late_trigger, grp_early;
    const float* cmb_w;
    const float* cmb_res;
    float* cmb_out;
    uint32_t* cmb_cnt;
    uint32_t cmb_slots;
    // Greedy epilogue (batch 1, f32 results of one segment; argmax_f16 after lm_head, crates/engine/src/forward.rs:1967-1973),
    // active when am_part != nullptr: every 32-row tile files (largest result, its row index + am_base) in am_part[tile]
    // and takes a ticket on *am_cnt; the tile with the last ticket reduces the n_tiles pairs (the lowest index wins among
    // equal values), stores the pair into every am_dst[i] (own memory or a peer's: plain stores), the index into *am_token
    // when that is not null, and puts the counter back to zero.
    // Expert-parallel decode without launches of its own.
    // Producer (grouped down projection with cmb_*, ep_npeer > 0): the weighted sum over THIS rank's slots goes, instead of
    // cmb_out, into slot ep_rank of every rank's partial buffer ep_peer[p] (f32 [2][world][rows], the half chosen by the
    // parity of the epoch = *ep_epoch + 1; plain peer stores); the warp that completes the last row tile (ticket on
    // *ep_done) makes everything visible system-wide, stores the epoch into word ep_rank of every rank's flag pad and
    // advances *ep_epoch.
    // Consumer (batch-1 GEMV with epw_partial != nullptr): after its dependency wait every CTA waits (bounded) until all
    // ranks' flags have reached *epw_epoch, adds residual + the world partials in rank order for all k inputs, stores
    // them to epw_out (= this launch's x: every CTA writes the same bits) and goes on from there.
    float* ep_peer[8];
    uint32_t* ep_pad[8];
    uint32_t ep_npeer, ep_rank;
    uint32_t* ep_epoch;
    uint32_t* ep_done;
    const float* epw_partial;
    const uint32_t* epw_pad;
    const float* epw_res;
    float* epw_out;
    float* epw_copies;           // [grid][k]: one copy of the summed state per CTA
    const uint32_t* epw_epoch;
    uint32_t* epw_abort;
    uint32_t epw_world;
    uint2* am_part;
    uint32_t* am_cnt;
    uint32_t am_base;
    uint2* am_dst[8];
    uint32_t am_ndst;
    int32_t* am_token;
};

// (value, index) pairs of the greedy epilogue: the larger value wins, the lower index among equal values; a NaN never
// replaces a number.
__device__ __forceinline__ void am_better(float& bv, uint32_t& bi, float ov, uint32_t oi) {
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
}
__device__ __forceinline__ void am_warp_reduce(float& bv, uint32_t& bi) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
        am_better(bv, bi, ov, oi);
    }
}

// Tensor maps of the weight matrices (bulk-load path): one per segment, plus the second matrix of
// a fused gate/up launch in slot 3.
struct GemvMaps {
    CUtensorMap m[4];
};

// ───────────────────────── unit dot products ─────────────────────────
// All take: up = this lane's unit in shared memory, xp = the unit's prepared activations
// (batch stride XPS floats), and add the dot products into the running accumulators.
//
// Accumulation is organised for instruction-level parallelism: every bit-field position has its
// own packed accumulator (short dependency chains), and block scales are applied with packed
// FMAs into two running packed sums per batch row, which are only folded to a scalar at the very
// end of the K loop.

struct RowAcc {
    uint64_t t0, t1;   // packed partial sums
    float s;           // scalar part (Q4_K min terms)
};

__device__ __forceinline__ float magic_byte(uint32_t w, int j) {
    // float value of byte j of w without an int->float conversion instruction
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7440u | (uint32_t)j)) - kTwo23;
}

// One Q4_K superblock (144 bytes).  Formula: crates/kernels/shaders/gemv_q4k.metal:85-122
// (sum over pairs j of (d*sc_j*q - dmin*m_j)*x for the low nibbles, index j+4 for the high ones).
template <int B, int XPS, int XSS>
__device__ __forceinline__ void unit_q4k(const uint8_t* up, const float* xp, const float* xs, RowAcc (&acc)[B]) {
    const ulonglong2* u = reinterpret_cast<const ulonglong2*>(up);
    const ulonglong2 h = u[0];
    const uint32_t h0 = (uint32_t)h.x;
    const float d = half_bits_to_float(h0), dmin = half_bits_to_float(h0 >> 16);
    const Q4KScales s = q4k_unpack_scales((uint32_t)(h.x >> 32), (uint32_t)h.y, (uint32_t)(h.y >> 32));
    const uint64_t neg = packf(-kTwo23);
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float dl = d * magic_byte(s.sl, j), ml = dmin * magic_byte(s.ml, j);
        const float dh = d * magic_byte(s.sh, j), mh = dmin * magic_byte(s.mh, j);
        uint64_t al[B][4], ah[B][4];
#pragma unroll
        for (int b = 0; b < B; b++)
#pragma unroll
            for (int f = 0; f < 4; f++) al[b][f] = ah[b][f] = 0ull;
#pragma unroll
        for (int n2 = 0; n2 < 2; n2++) {
            const ulonglong2 q = u[1 + 2 * j + n2];
#pragma unroll
            for (int t = 0; t < 2; t++) {
                const uint64_t P = t ? q.y : q.x, P12 = P >> 12;
                const int n = 2 * n2 + t;   // 8-element group of the sub-block
                const uint64_t l0 = fadd2(field_or_magic<0xFu << 0>(P), neg);
                const uint64_t l1 = fadd2(field_or_magic<0xFu << 8>(P), neg);
                const uint64_t l2 = fadd2(field_or_magic<0xFu << 16>(P), neg);
                const uint64_t l3 = fadd2(field_or_magic<0xFu << 12>(P12), neg);
                const uint64_t g0 = fadd2(field_or_magic<0xFu << 4>(P), neg);
                const uint64_t g1 = fadd2(field_or_magic<0xFu << 12>(P), neg);
                const uint64_t g2 = fadd2(field_or_magic<0xFu << 8>(P12), neg);
                const uint64_t g3 = fadd2(field_or_magic<0xFu << 16>(P12), neg);
#pragma unroll
                for (int b = 0; b < B; b++) {
                    const float* xb = xp + b * XPS + 64 * j + 8 * n;
                    const ulonglong2 xa = *reinterpret_cast<const ulonglong2*>(xb);
                    const ulonglong2 xc = *reinterpret_cast<const ulonglong2*>(xb + 4);
                    const ulonglong2 ya = *reinterpret_cast<const ulonglong2*>(xb + 32);
                    const ulonglong2 yc = *reinterpret_cast<const ulonglong2*>(xb + 36);
                    al[b][0] = ffma2(l0, xa.x, al[b][0]);
                    al[b][1] = ffma2(l1, xa.y, al[b][1]);
                    al[b][2] = ffma2(l2, xc.x, al[b][2]);
                    al[b][3] = ffma2(l3, xc.y, al[b][3]);
                    ah[b][0] = ffma2(g0, ya.x, ah[b][0]);
                    ah[b][1] = ffma2(g1, ya.y, ah[b][1]);
                    ah[b][2] = ffma2(g2, yc.x, ah[b][2]);
                    ah[b][3] = ffma2(g3, yc.y, ah[b][3]);
                }
            }
        }
        const uint64_t dl2 = packf(dl), dh2 = packf(dh);
#pragma unroll
        for (int b = 0; b < B; b++) {
            acc[b].t0 = ffma2(dl2, fadd2(al[b][0], al[b][1]), acc[b].t0);
            acc[b].t1 = ffma2(dl2, fadd2(al[b][2], al[b][3]), acc[b].t1);
            acc[b].t0 = ffma2(dh2, fadd2(ah[b][0], ah[b][1]), acc[b].t0);
            acc[b].t1 = ffma2(dh2, fadd2(ah[b][2], ah[b][3]), acc[b].t1);
            acc[b].s = fmaf(-ml, xs[b * XSS + 2 * j], acc[b].s);
            acc[b].s = fmaf(-mh, xs[b * XSS + 2 * j + 1], acc[b].s);
        }
    }
}

// Eight Q4_0 blocks (144 bytes).  Formula: crates/kernels/shaders/gemv_q4_0.metal:26-49
// (d * sum((nib-8)*x), low nibble = element 2i, high nibble = element 2i+1).
template <int B, int XPS>
__device__ __forceinline__ void unit_q4_0(const uint8_t* up, const float* xp, int nblk, RowAcc (&acc)[B]) {
    const uint4* u4 = reinterpret_cast<const uint4*>(up);
    uint32_t w[36];
#pragma unroll
    for (int i = 0; i < 9; i++) {
        const uint4 q = u4[i];
        w[4 * i] = q.x; w[4 * i + 1] = q.y; w[4 * i + 2] = q.z; w[4 * i + 3] = q.w;
    }
#pragma unroll
    for (int blk = 0; blk < 8; blk++) {
        if (blk < nblk) {
            const int o0 = 18 * blk, s = (o0 + 2) >> 2;
            const uint32_t dw = w[o0 >> 2];
            const uint64_t d2 = packf(half_bits_to_float((o0 & 2) ? (dw >> 16) : dw));
            uint32_t Q[4];
#pragma unroll
            for (int i = 0; i < 4; i++)   // the 16 quant bytes start 2 bytes into a word in even blocks
                Q[i] = ((o0 + 2) & 2) ? __funnelshift_r(w[s + i], w[s + i + 1], 16) : w[s + i];
            uint64_t a[B][8];
#pragma unroll
            for (int g = 0; g < 2; g++) {
                const uint64_t P = pack2(Q[2 * g], Q[2 * g + 1]), P12 = P >> 12;
                // field i = nibble at bit 4i of both words (bits above 16 are read from P >> 12)
                uint64_t f[8];
                f[0] = fadd2(field_or_magic<0xFu << 0>(P), packf(-(kTwo23 + 8.0f)));
                f[1] = fadd2(field_or_magic<0xFu << 4>(P), packf(-(kTwo23 + 128.0f)));
                f[2] = fadd2(field_or_magic<0xFu << 8>(P), packf(-(kTwo23 + 2048.0f)));
                f[3] = fadd2(field_or_magic<0xFu << 12>(P), packf(-(kTwo23 + 32768.0f)));
                f[4] = fadd2(field_or_magic<0xFu << 16>(P), packf(-(kTwo23 + 524288.0f)));
                f[5] = fadd2(field_or_magic<0xFu << 8>(P12), packf(-(kTwo23 + 2048.0f)));
                f[6] = fadd2(field_or_magic<0xFu << 12>(P12), packf(-(kTwo23 + 32768.0f)));
                f[7] = fadd2(field_or_magic<0xFu << 16>(P12), packf(-(kTwo23 + 524288.0f)));
#pragma unroll
                for (int b = 0; b < B; b++) {
                    const float* xb = xp + b * XPS + 32 * blk + 16 * g;
#pragma unroll
                    for (int k4 = 0; k4 < 4; k4++) {
                        const ulonglong2 xv = *reinterpret_cast<const ulonglong2*>(xb + 4 * k4);
                        a[b][2 * k4] = ffma2(f[2 * k4], xv.x, g ? a[b][2 * k4] : 0ull);
                        a[b][2 * k4 + 1] = ffma2(f[2 * k4 + 1], xv.y, g ? a[b][2 * k4 + 1] : 0ull);
                    }
                }
            }
#pragma unroll
            for (int b = 0; b < B; b++) {
                const uint64_t s01 = fadd2(fadd2(a[b][0], a[b][1]), fadd2(a[b][2], a[b][3]));
                const uint64_t s23 = fadd2(fadd2(a[b][4], a[b][5]), fadd2(a[b][6], a[b][7]));
                acc[b].t0 = ffma2(d2, s01, acc[b].t0);
                acc[b].t1 = ffma2(d2, s23, acc[b].t1);
            }
        }
    }
}

// Four Q8_0 blocks (136 bytes, 8-byte aligned).  Formula:
// crates/kernels/shaders/gemv_q8_0.metal:24-36 (d * sum(int8 * x)).
template <int B, int XPS>
__device__ __forceinline__ void unit_q8_0(const uint8_t* up, const float* xp, int nblk, RowAcc (&acc)[B]) {
    const uint2* u2 = reinterpret_cast<const uint2*>(up);
    uint32_t w[34];
#pragma unroll
    for (int i = 0; i < 17; i++) {
        const uint2 q = u2[i];
        w[2 * i] = q.x; w[2 * i + 1] = q.y;
    }
    // int8 -> biased uint8 and magic in one LOP3: ((v & mask) ^ c), c = (0x80<<p | 2^23 bits)
    const uint64_t n0 = packf(-(kTwo23 + 128.0f)), n8 = packf(-(kTwo23 + 32768.0f));
#pragma unroll
    for (int blk = 0; blk < 4; blk++) {
        if (blk < nblk) {
            const int o0 = 34 * blk, s = (o0 + 2) >> 2;
            const uint32_t dw = w[o0 >> 2];
            const uint64_t d2 = packf(half_bits_to_float((o0 & 2) ? (dw >> 16) : dw));
            uint64_t a[B][4];
#pragma unroll
            for (int n = 0; n < 4; n++) {
                uint32_t q0, q1;
                if ((o0 + 2) & 2) {
                    q0 = __funnelshift_r(w[s + 2 * n], w[s + 2 * n + 1], 16);
                    q1 = __funnelshift_r(w[s + 2 * n + 1], w[s + 2 * n + 2], 16);
                } else {
                    q0 = w[s + 2 * n];
                    q1 = w[s + 2 * n + 1];
                }
                const uint64_t P = pack2(q0, q1), P16 = P >> 16;
                const uint64_t f0 = fadd2(field_xor<0xFFu, 0x4B000080u>(P), n0);
                const uint64_t f1 = fadd2(field_xor<0xFF00u, 0x4B008000u>(P), n8);
                const uint64_t f2 = fadd2(field_xor<0xFFu, 0x4B000080u>(P16), n0);
                const uint64_t f3 = fadd2(field_xor<0xFF00u, 0x4B008000u>(P16), n8);
#pragma unroll
                for (int b = 0; b < B; b++) {
                    const float* xb = xp + b * XPS + 32 * blk + 8 * n;
                    const ulonglong2 xa = *reinterpret_cast<const ulonglong2*>(xb);
                    const ulonglong2 xc = *reinterpret_cast<const ulonglong2*>(xb + 4);
                    a[b][0] = ffma2(f0, xa.x, n ? a[b][0] : 0ull);
                    a[b][1] = ffma2(f1, xa.y, n ? a[b][1] : 0ull);
                    a[b][2] = ffma2(f2, xc.x, n ? a[b][2] : 0ull);
                    a[b][3] = ffma2(f3, xc.y, n ? a[b][3] : 0ull);
                }
            }
#pragma unroll
            for (int b = 0; b < B; b++) {
                acc[b].t0 = ffma2(d2, fadd2(a[b][0], a[b][1]), acc[b].t0);
                acc[b].t1 = ffma2(d2, fadd2(a[b][2], a[b][3]), acc[b].t1);
            }
        }
    }
}

// ───────────────────────── staged kernel ─────────────────────────
// LD = 0: weights and activations arrive with per-thread cp.async copies (any row alignment >= 4).
// LD = 1: one elected lane per warp issues a 2-D tiled bulk load (TMA) of the 32-row x 1-unit box
//         and a 1-D bulk copy of the activation slice; completion is tracked by one mbarrier per
//         stage and warp.  Needs 16-byte aligned rows (always true for the 4-bit formats here).

//
// KSL = number of warps that share one 32-row tile (each takes every KSL-th unit of K); a CTA
// holds 4/KSL tiles.  The host picks KSL so that the units divide evenly among the warps.
// MATH = 0: packed f32 arithmetic (any batch); MATH = 1: integer dot products (dp4a) on 8-bit limbs of the activations
// (batch 1); MATH = 2: integer tensor-core MMAs on 16-bit activations (batch 1, 4-bit formats).  See gemv_int8.cuh.
template <int FMT, int B, bool XF16, int CPB, int S, bool DUAL, int LD, int KSL, int MATH>
__global__ void __launch_bounds__(kNT, S <= 2 ? 4 : 3) gemv_staged_kernel(const GemvArgs a, const __grid_constant__ GemvMaps maps) {
    using T = Traits<FMT>;
    using L = WarpStage<FMT, B, XF16>;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ float red[kKS][kRT][B];
    __shared__ __align__(8) uint64_t mbar[kKS][4];
    __shared__ float s_norm[kKS + 1];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint8_t* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    uint8_t* ring = smem + warp * (S * L::BYTES);
    const uint32_t ring_u32 = smem_u32(ring);
    const uint32_t bar0 = smem_u32(&mbar[warp][0]);

    if (!a.late_trigger) grid_launch_dependents();   // let the next kernel of the stream begin its own prologue
    const bool early_weights = LD == 1 && (a.grp_expert == nullptr || a.grp_early);
    if (!early_weights) {
        grid_dependency_wait();
        if (a.late_trigger) grid_launch_dependents();
    }
    constexpr int TPC = kKS / KSL;              // tiles per CTA
    // With csplit > 1 (host guarantees KSL == 4) a cluster of csplit CTAs shares one tile: CTA c of the
    // cluster and warp w take K-slice w*csplit + c of 4*csplit slices; partial sums meet in CTA 0 through
    // distributed shared memory.
    const uint32_t csplit = a.csplit, crank = csplit > 1 ? cluster_ctarank() : 0u;
    const int slice = (warp % KSL) * (int)csplit + (int)crank;
    const int n_slices = KSL * (int)csplit;
    const uint32_t tile = (blockIdx.x / csplit) * TPC + warp / KSL;   // global tile index over all segments
    int si = 0;
#pragma unroll
    for (int i = 1; i < 3; i++)
        if (i < a.nseg && tile >= a.seg[i].tile_begin) si = i;
    GemvSeg sg = a.seg[si];
    constexpr int RPT = DUAL ? kRT / 2 : kRT;   // real rows per tile
    const bool tile_ok = tile < a.n_tiles;
    uint32_t row0 = (tile - sg.tile_begin) * RPT;
    uint32_t wrow0 = row0;                       // row of the tile inside the weight matrix
    const uint8_t* xbase = reinterpret_cast<const uint8_t*>(a.x);
    bool slot_live = true;   // grouped mode: an expert id outside the stacked matrix marks an unused slot (nothing is computed or written)
    if (a.grp_expert != nullptr && tile_ok) {
        const uint32_t slot = tile / a.grp_tiles;
        row0 = (tile - slot * a.grp_tiles) * RPT;
        const int32_t eid = a.grp_expert[slot] - a.grp_lo;
        slot_live = eid >= 0 && (uint32_t)eid < a.grp_cnt;
        wrow0 = (uint32_t)(slot_live ? eid : 0) * a.grp_rows + row0;
        xbase += (size_t)(slot / a.grp_xdiv) * a.k * (XF16 ? 2 : 4);
        sg.y = reinterpret_cast<uint8_t*>(sg.y) + (size_t)slot * a.ldy * (a.out_f16 ? 2 : 4);
    }
    const uint32_t rows_here = (tile_ok && slot_live) ? min((uint32_t)RPT, sg.rows - row0) : 0u;
    const bool row_ok = (uint32_t)(DUAL ? (lane & 15) : lane) < rows_here;
    const int n_it = (tile_ok && slot_live) ? ((int)a.n_units - slice + n_slices - 1) / n_slices : 0;   // units slice, slice+n_slices, ...

    if (LD == 1) {
        if (lane == 0) {
#pragma unroll
            for (int s = 0; s < S; s++) mbar_init(bar0 + 8 * s, 1);
            fence_mbar_init();
        }
        __syncwarp();
    }

    constexpr int CPR = T::UB / CPB;        // copy chunks per row of one unit
    constexpr int DR = 32 / CPR, DC = 32 % CPR;
    const int c_row0 = lane / CPR, c_col0 = lane % CPR;

    // part: 0 = weights and activations, 1 = weights only (arms the barrier for both), 2 = activations only.
    // The split lets the prologue prefetch weights before it waits for the producer of the activations.
    auto issue = [&](int it, int part = 0) {
        if (LD == 1) {
            if (it < n_it && lane == 0) {
                const uint32_t u = slice + n_slices * it;
                const uint32_t slot = ring_u32 + (it % S) * L::BYTES;
                const uint32_t bar = bar0 + 8 * (it % S);
                const uint32_t e0 = u * T::UE;
                const uint32_t nx = min((uint32_t)T::UE, a.k - e0);   // activations of this unit
                const uint32_t xbytes = nx * (XF16 ? 2u : 4u);
                if (part != 2) {
                    fence_proxy_async();   // earlier generic-proxy accesses to this slot precede the bulk writes
                    mbar_expect_tx(bar, (uint32_t)L::W_BYTES + B * xbytes);
                    if (DUAL) {
                        tma_load_2d(slot, &maps.m[0], (int32_t)(u * T::UB), (int32_t)wrow0, bar);
                        tma_load_2d(slot + 16 * T::UB, &maps.m[3], (int32_t)(u * T::UB), (int32_t)wrow0, bar);
                    } else {
                        tma_load_2d(slot, &maps.m[si], (int32_t)(u * T::UB), (int32_t)wrow0, bar);
                    }
                }
                if (part != 1) {
#pragma unroll
                    for (int b = 0; b < B; b++) {
                        if (XF16)
                            bulk_load_1d(slot + L::XR_OFF + b * T::UE * 2,
                                         reinterpret_cast<const __half*>(xbase) + (size_t)b * a.k + e0, xbytes, bar);
                        else
                            bulk_load_1d(slot + L::XP_OFF + b * T::UE * 4,
                                         reinterpret_cast<const float*>(xbase) + (size_t)b * a.k + e0, xbytes, bar);
                    }
                }
            }
            return;
        }
        if (it < n_it) {
            const uint32_t u = slice + n_slices * it;
            const uint32_t slot = ring_u32 + (it % S) * L::BYTES;
            const uint32_t uoff = u * T::UB;
            const int vb = min((int)T::UB, (int)(a.row_bytes - uoff));
            int row = c_row0, col = c_col0;
#pragma unroll
            for (int j = 0; j < CPR; j++) {
                const int rr = DUAL ? (row & 15) : row;
                if (row < kRT && (uint32_t)rr < rows_here && col * CPB < vb) {
                    const uint8_t* base = (DUAL && row >= 16) ? sg.w2 : sg.w;
                    cp_async<CPB>(slot + row * T::UB + col * CPB,
                                  base + (size_t)(wrow0 + rr) * a.row_bytes + uoff + col * CPB);
                }
                row += DR;
                col += DC;
                if (col >= CPR) { col -= CPR; row++; }
            }
            const uint32_t e0 = u * T::UE;
            if (XF16) {
                const __half* xg = reinterpret_cast<const __half*>(xbase);
#pragma unroll
                for (int b = 0; b < B; b++)
#pragma unroll
                    for (int c = lane; c < T::UE / 8; c += 32)
                        if (e0 + c * 8 < a.k)
                            cp_async16(slot + L::XR_OFF + (b * T::UE + c * 8) * 2, xg + (size_t)b * a.k + e0 + c * 8);
            } else {
                const float* xg = reinterpret_cast<const float*>(xbase);
#pragma unroll
                for (int b = 0; b < B; b++)
#pragma unroll
                    for (int c = lane; c < T::UE / 4; c += 32)
                        if (e0 + c * 4 < a.k)
                            cp_async16(slot + L::XP_OFF + (b * T::UE + c * 4) * 4, xg + (size_t)b * a.k + e0 + c * 4);
            }
        }
        cp_async_commit();
    };

    // Wait until stage `it` has landed for this lane (`pending` = cp.async groups that may stay open).
    bool timed_out = false;
    float norm_r = 1.f;      // RMSNorm prologue: scale of the input vector (set after the dependency wait)
    auto wait_stage = [&](int it, auto pending) {
        if (LD == 1) {
            // after one failed wait the warp stops waiting (its results are reported as invalid)
            if (it < n_it && !timed_out && !mbar_wait(bar0 + 8 * (it % S), (uint32_t)(it / S) & 1u)) timed_out = true;
        } else {
            cp_async_wait<decltype(pending)::value>();
        }
    };

    // Prepare the activations of stage `it` (warp-private): f16 -> f32, permutation into the pair
    // order of the weight words, pre-scaling by the nibble position, 32-element block sums.
    auto prep = [&](int it) {
        if (it >= n_it) return;
        uint8_t* slot = ring + (it % S) * L::BYTES;
        constexpr int EPL = T::UE / 32;   // 8 (4-bit formats) or 4 (Q8_0) consecutive elements per lane
        float v[B][EPL];
#pragma unroll
        for (int b = 0; b < B; b++) {
            if (XF16) {
                const __half* xr = reinterpret_cast<const __half*>(slot + L::XR_OFF) + b * T::UE + lane * EPL;
#pragma unroll
                for (int i = 0; i < EPL; i++) v[b][i] = __half2float(xr[i]);
            } else {
                const float4* xr = reinterpret_cast<const float4*>(slot + L::XP_OFF) + (b * T::UE + lane * EPL) / 4;
#pragma unroll
                for (int i = 0; i < EPL / 4; i++) {
                    const float4 t4 = xr[i];
                    v[b][4 * i] = t4.x; v[b][4 * i + 1] = t4.y; v[b][4 * i + 2] = t4.z; v[b][4 * i + 3] = t4.w;
                }
            }
        }
        __syncwarp();   // in-place: every lane has read its inputs before anyone overwrites them
        if constexpr (B == 1 && !XF16) {
            if (a.norm_gamma != nullptr) {
                const uint32_t e0 = (slice + n_slices * it) * T::UE + lane * EPL;
#pragma unroll
                for (int i = 0; i < EPL; i++)
                    if (e0 + i < a.k) v[0][i] = v[0][i] * norm_r * a.norm_gamma[e0 + i];
            }
        }
        if (MATH == 1) {
            prep_int_block<EPL, T::UE / 32, FMT == RUNIT_FMT_Q4_0 ? 1 : 0, FMT == RUNIT_FMT_Q8_0 ? 2 : 3>(slot + L::XP_OFF, v[0], lane);
            return;
        }
        if constexpr (MATH == 2) {
            const uint32_t u = slice + n_slices * it;
            const int nblk = FMT == RUNIT_FMT_Q4K ? 8 : min(8, (int)(a.nb - u * T::BPU));
            prep_mma_block<8, FMT == RUNIT_FMT_Q4_0 ? 1 : 0>(slot + L::XP_OFF, v[0], lane, nblk);
            return;
        }
#pragma unroll
        for (int b = 0; b < B; b++) {
            float* xp = reinterpret_cast<float*>(slot + L::XP_OFF) + b * T::UE;
            if (FMT == RUNIT_FMT_Q4K) {
                float sum = 0.f;
#pragma unroll
                for (int i = 0; i < EPL; i++) sum += v[b][i];
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                if ((lane & 3) == 0) reinterpret_cast<float*>(slot + L::XS_OFF)[b * 8 + (lane >> 2)] = sum;
                // elements 8*lane .. 8*lane+7: sub-block half = (lane>>2)&1, byte position = i%4.
                // low half: 2^-{0,8,16,12}; high half: 2^-{4,12,8,16}: the high-half exponent is the
                // low-half one + 4 for byte positions 0,1,3... except position 2 (16 -> 8)
                const bool hi = (lane >> 2) & 1;
                float o[8];
#pragma unroll
                for (int i = 0; i < 8; i++)
                    o[pos8(i)] = v[b][i] * (hi ? exp2_neg(q4k_shift(i & 3, true)) : exp2_neg(q4k_shift(i & 3, false)));
                float4* dst = reinterpret_cast<float4*>(xp + 8 * lane);
                dst[0] = make_float4(o[0], o[1], o[2], o[3]);
                dst[1] = make_float4(o[4], o[5], o[6], o[7]);
            } else if (FMT == RUNIT_FMT_Q4_0) {
                // element t of this lane: field 2*(t/2)+(t%2) = t of its word; stored as pair member lane&1
#pragma unroll
                for (int i = 0; i < 8; i++)
                    xp[16 * (lane >> 1) + 2 * i + (lane & 1)] = v[b][i] * exp2_neg(q4_0_shift(i >> 1, i & 1));
            } else {
#pragma unroll
                for (int i = 0; i < 4; i++)
                    xp[8 * (lane >> 1) + 2 * i + (lane & 1)] = v[b][i] * exp2_neg(q8_0_shift(i));
            }
        }
    };

    RowAcc acc[B];
#pragma unroll
    for (int b = 0; b < B; b++) { acc[b].t0 = 0ull; acc[b].t1 = 0ull; acc[b].s = 0.f; }
    float macc[4] = {0.f, 0.f, 0.f, 0.f};   // MATH == 2: rows g, g+8, 16+g, 24+g of the tile (g = lane / 4)

    // Programmatic dependent launch: this grid may start while its predecessor in the stream is still
    // draining.  Weights do not depend on the predecessor, so (outside grouped mode, where the expert id does)
    // their first stages are requested before the dependency wait; activations, residual and every store
    // come after it.
    if (early_weights) {
#pragma unroll
        for (int s = 0; s < S; s++) issue(s, 1);
        grid_dependency_wait();
        if (a.late_trigger) grid_launch_dependents();
        if constexpr (B == 1 && !XF16 && !DUAL) {
            if (a.epw_partial != nullptr) {
                const uint32_t epoch = *a.epw_epoch;     // advanced by the launch that pushed this rank's partial sums
                if (warp == 0 && (uint32_t)lane < a.epw_world) {
                    const bool aborted = a.epw_abort && *reinterpret_cast<volatile uint32_t*>(a.epw_abort) != 0u;
                    const long long t0 = clock64();
                    while (!aborted) {
                        uint32_t v;
                        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(a.epw_pad + lane) : "memory");
                        if ((int32_t)(v - epoch) >= 0) break;
                        if (clock64() - t0 > (1ll << 30)) {   // about half a second: a rank never raised its flag
                            if (a.status) atomicExch(a.status, 3);
                            if (a.epw_abort) atomicExch(a.epw_abort, 1u);
                            break;
                        }
                        __nanosleep(100);
                    }
                }
                __syncthreads();
                // every CTA forms the summed hidden state in a copy of its own (192 CTAs storing the same 8 KB would queue up on
                // the same lines); CTA 0 also stores the copy that later launches read
                const float* part = a.epw_partial + (size_t)(epoch & 1u) * a.epw_world * a.k;
                float* mine = a.epw_copies + (size_t)blockIdx.x * a.k;
                for (uint32_t i = threadIdx.x; i < a.k; i += kNT) {
                    float v = a.epw_res[i];
                    for (uint32_t r = 0; r < a.epw_world; r++) v += __ldcg(part + (size_t)r * a.k + i);   // rank order, as ep_reduce_kernel
                    mine[i] = v;
                    if (blockIdx.x == 0) a.epw_out[i] = v;
                }
                xbase = reinterpret_cast<const uint8_t*>(mine);
                fence_proxy_async();     // the bulk loads of x below read what this CTA has just stored
                __syncthreads();
            }
        }
#pragma unroll
        for (int s = 0; s < S; s++) issue(s, 2);
    } else {
#pragma unroll
        for (int s = 0; s < S; s++) issue(s);
    }
    // RMSNorm prologue: the scale of the whole input vector, computed by this CTA while its first stages are in flight
    // (summation order of the stand-alone kernel's warps differs: the scale agrees to rounding)
    if constexpr (B == 1 && !XF16) {
        if (a.norm_gamma != nullptr) {
            const float* xg = reinterpret_cast<const float*>(xbase);
            float sq = 0.f;
            for (uint32_t i = threadIdx.x; i < a.k; i += kNT) {
                const float t = xg[i];
                sq = fmaf(t, t, sq);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            if (lane == 0) s_norm[warp] = sq;
            __syncthreads();
            float tot = 0.f;
#pragma unroll
            for (int i = 0; i < kKS; i++) tot += s_norm[i];
            norm_r = rsqrtf(tot / (float)a.k + a.norm_eps);
        }
    }

    for (int it = 0; it < n_it; it++) {
        wait_stage(it, std::integral_constant<int, S - 1>());   // this lane's copies of stage `it` have landed
        __syncwarp();                                           // ... and every lane's
        prep(it);
        __syncwarp();                                           // prepared activations visible to the warp
        if constexpr (MATH == 2) {
            // whole-warp MMAs: rows past the end of the matrix are zero-filled boxes (or stale bytes that only reach
            // their own, unwritten, rows)
            const uint32_t u = slice + n_slices * it;
            const uint8_t* slot = ring + (it % S) * L::BYTES;
            if (FMT == RUNIT_FMT_Q4K) unit_q4k_mma(slot, slot + L::XP_OFF, lane, macc);
            else unit_q4_0_mma(slot, slot + L::XP_OFF, lane, min(8, (int)(a.nb - u * T::BPU)), macc);
        } else if (row_ok) {
            const uint32_t u = slice + n_slices * it;
            const uint8_t* slot = ring + (it % S) * L::BYTES;
            const uint8_t* up = slot + lane * T::UB;
            const float* xp = reinterpret_cast<const float*>(slot + L::XP_OFF);
            if (MATH == 1) {
                if (FMT == RUNIT_FMT_Q4K) acc[0].s += unit_q4k_i8(up, slot + L::XP_OFF);
                else if (FMT == RUNIT_FMT_Q4_0) acc[0].s += unit_q4_0_i8(up, slot + L::XP_OFF, min(T::BPU, (int)(a.nb - u * T::BPU)));
                else acc[0].s += unit_q8_0_i8(up, slot + L::XP_OFF, min(T::BPU, (int)(a.nb - u * T::BPU)));
            } else if (FMT == RUNIT_FMT_Q4K) {
                unit_q4k<B, T::UE, 8>(up, xp, reinterpret_cast<const float*>(slot + L::XS_OFF), acc);
            } else if (FMT == RUNIT_FMT_Q4_0) {
                unit_q4_0<B, T::UE>(up, xp, min(T::BPU, (int)(a.nb - u * T::BPU)), acc);
            } else {
                unit_q8_0<B, T::UE>(up, xp, min(T::BPU, (int)(a.nb - u * T::BPU)), acc);
            }
        }
        __syncwarp();             // every lane is done with slot it%S: refill it with stage it+S
        issue(it + S);
    }
    if (LD == 0) cp_async_wait<0>();
    if (timed_out && a.status) atomicExch(a.status, 1);

    // Add the K-slices of each row in slice order, then the epilogue (first warp of each tile).
    if constexpr (MATH == 2) {
        // the four lanes of a row group hold the blocks t, 4+t of their rows: add them, then lane (g, t) files row 8t + g
#pragma unroll
        for (int j = 0; j < 4; j++) {
            macc[j] += __shfl_xor_sync(0xffffffffu, macc[j], 1);
            macc[j] += __shfl_xor_sync(0xffffffffu, macc[j], 2);
        }
        const int t = lane & 3;
        red[warp][8 * t + (lane >> 2)][0] = t == 0 ? macc[0] : (t == 1 ? macc[1] : (t == 2 ? macc[2] : macc[3]));
    } else {
#pragma unroll
        for (int b = 0; b < B; b++) red[warp][lane][b] = (sum2(acc[b].t0) + sum2(acc[b].t1)) + acc[b].s;
    }
    __syncthreads();
    if (csplit > 1) {
        // CTA-local sum of the four warps (warp 0), published in red[0]; then CTA 0 of the cluster adds the
        // other CTAs' sums in rank order.  The second cluster barrier keeps every CTA alive until it was read.
        if (warp == 0) {
#pragma unroll
            for (int b = 0; b < B; b++)
                red[0][lane][b] = ((red[0][lane][b] + red[1][lane][b]) + red[2][lane][b]) + red[3][lane][b];
        }
        cluster_sync();
        if (crank == 0 && warp == 0) {
#pragma unroll
            for (int b = 0; b < B; b++) {
                float v = red[0][lane][b];
                for (uint32_t c = 1; c < csplit; c++) v += ld_cluster_f32(&red[0][lane][b], c);
                red[1][lane][b] = v;   // own slot, nobody reads red[1] remotely
            }
        }
        cluster_sync();
    }
    if ((warp % KSL) == 0 && crank == 0) {
        float r[B];
#pragma unroll
        for (int b = 0; b < B; b++) {
            if (csplit > 1) {
                r[b] = red[1][lane][b];
            } else {
                r[b] = red[warp][lane][b];
#pragma unroll
                for (int k = 1; k < KSL; k++) r[b] += red[warp + k][lane][b];
            }
        }
        if (DUAL) {
            // lanes 0..15 hold gate rows, lanes 16..31 the matching up rows:
            // act = silu(gate) * up  (crates/kernels/shaders/fused_ffn.metal:24-26,89-92)
#pragma unroll
            for (int b = 0; b < B; b++) {
                const float up_v = __shfl_down_sync(0xffffffffu, r[b], 16);
                r[b] = silu(r[b]) * up_v;
            }
        }
        const uint32_t row = row0 + (DUAL ? (lane & 15) : lane);
        const bool writer = DUAL ? (lane < 16 && row_ok) : row_ok;
        float v_first = -INFINITY;   // this lane's final result of batch row 0 (greedy epilogue)
        if (writer) {
#pragma unroll
            for (int b = 0; b < B; b++) {
                float v = r[b];
                if (a.bias_kind == BIAS_F16) v += __half2float(reinterpret_cast<const __half*>(sg.bias)[row]);
                else if (a.bias_kind == BIAS_F32) v += reinterpret_cast<const float*>(sg.bias)[row];
                const size_t o = (size_t)b * a.ldy + row;
                if (a.res_kind == RES_F32) v += reinterpret_cast<const float*>(sg.res)[o];
                else if (a.res_kind == RES_F16) v += __half2float(reinterpret_cast<const __half*>(sg.res)[o]);
                if (a.out_f16) reinterpret_cast<__half*>(sg.y)[o] = __float2half_rn(v);
                else reinterpret_cast<float*>(sg.y)[o] = v;
                for (uint32_t p = 0; p < a.n_peer; p++) a.peer_y[p][o] = v;
                if (b == 0) v_first = v;
            }
        }
        if constexpr (B == 1 && !DUAL && !XF16) {
            if (a.am_part != nullptr && tile_ok) {
                float bv = writer ? v_first : -INFINITY;
                uint32_t bi = writer ? a.am_base + row : 0xFFFFFFFFu;
                am_warp_reduce(bv, bi);
                uint32_t ticket = 0;
                if (lane == 0) {
                    __stcg(&a.am_part[tile], make_uint2(__float_as_uint(bv), bi));
                    __threadfence();                     // the pair is visible before the ticket is
                    ticket = atomicAdd(a.am_cnt, 1u);
                }
                ticket = __shfl_sync(0xffffffffu, ticket, 0);
                if (ticket == a.n_tiles - 1) {
                    __threadfence();
                    bv = -INFINITY;
                    bi = 0xFFFFFFFFu;
                    for (uint32_t i = lane; i < a.n_tiles; i += 32) {
                        const uint2 pr = __ldcg(&a.am_part[i]);
                        am_better(bv, bi, __uint_as_float(pr.x), pr.y);
                    }
                    am_warp_reduce(bv, bi);
                    if (lane == 0) {
                        const uint2 pr = make_uint2(__float_as_uint(bv), bi);
                        for (uint32_t d = 0; d < a.am_ndst; d++) *a.am_dst[d] = pr;
                        if (a.am_token) *a.am_token = (int32_t)bi;
                        *a.am_cnt = 0;                   // at rest again for the next launch
                    }
                }
            }
            if ((a.cmb_out != nullptr || a.ep_npeer != 0) && tile_ok) {
                const uint32_t t = tile % a.grp_tiles;   // row tile, shared by the slots
                __threadfence();                         // this lane's row of y[slot] is visible before the ticket is
                __syncwarp();
                uint32_t ticket = 0;
                if (lane == 0) ticket = atomicAdd(&a.cmb_cnt[t], 1u);
                ticket = __shfl_sync(0xffffffffu, ticket, 0);
                if (ticket == a.cmb_slots - 1) {
                    __threadfence();                     // the other slots' rows, published before their tickets
                    if (lane == 0) a.cmb_cnt[t] = 0;     // at rest again for the next launch
                    const uint32_t r = t * RPT + lane;
                    if (r < sg.rows) {
                        const float* y0 = reinterpret_cast<const float*>(a.seg[0].y);
                        float acc = 0.f;
                        for (uint32_t i = 0; i < a.cmb_slots; i++) {
                            const int32_t eid = a.grp_expert[i] - a.grp_lo;
                            if (eid >= 0 && (uint32_t)eid < a.grp_cnt)
                                acc = fmaf(a.cmb_w[i], __ldcg(y0 + (size_t)i * a.ldy + r), acc);
                        }
                        if (a.ep_npeer == 0) {
                            a.cmb_out[r] = (a.cmb_res ? a.cmb_res[r] : 0.f) + acc;
                        } else {
                            const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(a.ep_epoch) + 1u;
                            const size_t o = ((size_t)(epoch & 1u) * a.ep_npeer + a.ep_rank) * sg.rows + r;
                            for (uint32_t p = 0; p < a.ep_npeer; p++) a.ep_peer[p][o] = acc;
                        }
                    }
                    if (a.ep_npeer != 0) {
                        // the partial sums of this row tile are out: the warp that files the last row tile raises the flags
                        const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(a.ep_epoch) + 1u;
                        __syncwarp();                    // the lanes' peer stores are ordered before lane 0's fence
                        uint32_t done = 0;
                        if (lane == 0) {
                            __threadfence_system();
                            done = atomicAdd(a.ep_done, 1u);
                        }
                        done = __shfl_sync(0xffffffffu, done, 0);
                        if (done == a.grp_tiles - 1) {
                            if (lane == 0) __threadfence_system();
                            __syncwarp();
                            if ((uint32_t)lane < a.ep_npeer)
                                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.ep_pad[lane] + a.ep_rank), "r"(epoch) : "memory");
                            __syncwarp();
                            if (lane == 0) {
                                *a.ep_done = 0;
                                *a.ep_epoch = epoch;     // read by the kernels that follow in the stream
                            }
                        }
                    }
                }
            }
        }
    }
}

// ───────────────────────── simple kernel (any alignment) ─────────────────────────
// One warp per row, scalar byte loads, lanes take blocks round-robin, shuffle reduction.
// Used when the rows of W are not 4-byte aligned in memory, and as an independent second
// implementation for cross-checking the staged kernel.
template <int FMT, bool XF16>
__global__ void __launch_bounds__(128) gemv_simple_kernel(const GemvArgs a, int batch) {
    const int lane = threadIdx.x & 31;
    const uint32_t grow = blockIdx.x * 4 + (threadIdx.x >> 5);
    int si = 0;
    uint32_t base = 0;
    {
        uint32_t acc_rows = 0;
        for (int i = 0; i < a.nseg; i++) {
            const uint32_t nr = a.seg[i].rows;
            if (grow >= acc_rows && grow < acc_rows + nr) { si = i; base = acc_rows; }
            acc_rows += nr;
        }
        if (grow >= acc_rows) return;
    }
    const GemvSeg sg = a.seg[si];
    const uint32_t row = grow - base;
    const int nmat = a.dual ? 2 : 1;
    float norm_r = 1.f;
    if (!XF16 && a.norm_gamma != nullptr) {   // RMSNorm prologue (batch 1): every warp computes the scale itself
        float sq = 0.f;
        for (uint32_t i = lane; i < a.k; i += 32) {
            const float t = reinterpret_cast<const float*>(a.x)[i];
            sq = fmaf(t, t, sq);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        norm_r = rsqrtf(sq / (float)a.k + a.norm_eps);
    }
    for (int b = 0; b < batch; b++) {
        float res2[2] = {0.f, 0.f};
        for (int mi = 0; mi < nmat; mi++) {
            const uint8_t* rp = (mi ? sg.w2 : sg.w) + (size_t)row * a.row_bytes;
            float acc = 0.f;
            for (uint32_t blk = lane; blk < a.nb; blk += 32) {
                auto X = [&](uint32_t i) -> float {
                    const size_t o = (size_t)b * a.k + i;
                    if (XF16) return __half2float(reinterpret_cast<const __half*>(a.x)[o]);
                    const float xv = reinterpret_cast<const float*>(a.x)[o];
                    return a.norm_gamma != nullptr ? xv * norm_r * a.norm_gamma[i] : xv;
                };
                if (FMT == RUNIT_FMT_Q8_0) {
                    const uint8_t* p = rp + (size_t)blk * 34;
                    const float d = half_bits_to_float(p[0] | (p[1] << 8));
                    float s = 0.f;
                    for (int i = 0; i < 32; i++) s += (float)(int8_t)p[2 + i] * X(blk * 32 + i);
                    acc += d * s;
                } else if (FMT == RUNIT_FMT_Q4_0) {
                    const uint8_t* p = rp + (size_t)blk * 18;
                    const float d = half_bits_to_float(p[0] | (p[1] << 8));
                    float s = 0.f;
                    for (int i = 0; i < 16; i++) {
                        s += (float)((int)(p[2 + i] & 15) - 8) * X(blk * 32 + 2 * i);
                        s += (float)((int)(p[2 + i] >> 4) - 8) * X(blk * 32 + 2 * i + 1);
                    }
                    acc += d * s;
                } else {
                    const uint8_t* p = rp + (size_t)blk * 144;
                    const float d = half_bits_to_float(p[0] | (p[1] << 8));
                    const float dmin = half_bits_to_float(p[2] | (p[3] << 8));
                    const uint8_t* sc = p + 4;
                    const uint8_t* qs = p + 16;
                    for (int j = 0; j < 4; j++) {
                        const float s_lo = (float)(sc[j] & 63), m_lo = (float)(sc[j + 4] & 63);
                        const float s_hi = (float)((sc[j + 8] & 15) | ((sc[j] >> 6) << 4));
                        const float m_hi = (float)((sc[j + 8] >> 4) | ((sc[j + 4] >> 6) << 4));
                        float ql = 0.f, qh = 0.f, xl = 0.f, xh = 0.f;
                        for (int l = 0; l < 32; l++) {
                            const float x0 = X(blk * 256 + j * 64 + l), x1 = X(blk * 256 + j * 64 + 32 + l);
                            ql += (float)(qs[j * 32 + l] & 15) * x0;
                            qh += (float)(qs[j * 32 + l] >> 4) * x1;
                            xl += x0;
                            xh += x1;
                        }
                        acc += (d * s_lo * ql - dmin * m_lo * xl) + (d * s_hi * qh - dmin * m_hi * xh);
                    }
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            res2[mi] = acc;
        }
        if (lane == 0) {
            float v = a.dual ? silu(res2[0]) * res2[1] : res2[0];
            if (a.bias_kind == BIAS_F16) v += __half2float(reinterpret_cast<const __half*>(sg.bias)[row]);
            else if (a.bias_kind == BIAS_F32) v += reinterpret_cast<const float*>(sg.bias)[row];
            const size_t o = (size_t)b * a.ldy + row;
            if (a.res_kind == RES_F32) v += reinterpret_cast<const float*>(sg.res)[o];
            else if (a.res_kind == RES_F16) v += __half2float(reinterpret_cast<const __half*>(sg.res)[o]);
            if (a.out_f16) reinterpret_cast<__half*>(sg.y)[o] = __float2half_rn(v);
            else reinterpret_cast<float*>(sg.y)[o] = v;
            for (uint32_t p = 0; p < a.n_peer; p++) a.peer_y[p][o] = v;
        }
    }
}

}  // namespace runit
