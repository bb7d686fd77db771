// Fused-dequant GEMV kernels for sm_100a: y = dequant(W) . x with W in Q8_0 / Q4_0 / Q4_K.
//
// Replaces the Metal kernels of crates/kernels/shaders/{gemv_q8_0,gemv_q4_0,gemv_q4k,
// fused_qkv,fused_ffn}.metal.  Design (HBM-bound streaming kernel):
//   * a CTA of 128 threads owns a tile of 32 rows and walks K in stages; a stage holds, per
//     row, the bytes of 4 "units" (a unit = 256 weights for the 4-bit formats, 128 for Q8_0);
//   * weights move HBM -> shared memory with 16-byte cp.async copies in a 3- or 4-deep ring,
//     so the bytes in flight per SM do not depend on register pressure or occupancy;
//   * thread (lane, warp) dots row `lane` with unit `warp` of the stage: weights are read
//     from the padded, conflict-free shared tile with 128-bit loads, the activation slice is
//     a warp-wide broadcast read, and no cross-lane reduction is needed until the end;
//   * the activation slice of the next stage is pre-scaled (and, for Q4_K, block-summed) by
//     all threads one stage ahead, which removes the per-weight scale multiply and the
//     integer->float conversion (see gemv_common.cuh);
//   * the four K-slices of a row are added in a fixed order (deterministic results).
#pragma once

#include "gemv_common.cuh"
#include "runit_cuda.h"

namespace runit {

constexpr int kNT = 128;   // threads per CTA
constexpr int kRT = 32;    // rows per tile (one per lane)
constexpr int kKS = 4;     // K-slices per stage (one per warp)

template <int FMT> struct Traits;
template <> struct Traits<RUNIT_FMT_Q8_0> { static constexpr int UE = 128, UB = 136, BPU = 4, BE = 32; };
template <> struct Traits<RUNIT_FMT_Q4_0> { static constexpr int UE = 256, UB = 144, BPU = 8, BE = 32; };
template <> struct Traits<RUNIT_FMT_Q4K>  { static constexpr int UE = 256, UB = 144, BPU = 1, BE = 256; };

template <int FMT, int B, bool XF16>
struct StageLayout {
    using T = Traits<FMT>;
    // Row pitch in shared memory: an odd multiple of the unit's load width (16 bytes for the
    // 4-bit formats, 8 for Q8_0), so that the 32 lanes of a warp hit distinct banks.
    static constexpr int ROW_STRIDE = kKS * T::UB + (FMT == RUNIT_FMT_Q8_0 ? 8 : 16);
    static constexpr int W_BYTES = kRT * ROW_STRIDE;
    static constexpr int XE = kKS * T::UE;                         // activations per stage per batch row
    static constexpr int XR_OFF = W_BYTES;                         // raw f16 activations (XF16 only)
    static constexpr int XR_BYTES = XF16 ? B * XE * 2 : 0;
    static constexpr int XP_OFF = XR_OFF + XR_BYTES;               // prepared f32 activations
    static constexpr int XP_BYTES = B * XE * 4;
    static constexpr int XS_OFF = XP_OFF + XP_BYTES;               // 32-element block sums (Q4_K)
    static constexpr int XS_BYTES = (FMT == RUNIT_FMT_Q4K) ? B * kKS * 8 * 4 : 0;
    static constexpr int BYTES = XS_OFF + XS_BYTES;
    static_assert(BYTES % 16 == 0, "stage must stay 16-byte aligned");
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
    uint32_t k, nb, row_bytes, n_units, n_stages;
    uint32_t ldy;          // elements between batch rows of y / residual
    int32_t out_f16, res_kind, bias_kind, dual;
};

// ───────────────────────── unit dot products ─────────────────────────

// One Q4_K superblock (144 bytes in shared memory) against B prepared activation slices.
// Formula: crates/kernels/shaders/gemv_q4k.metal:85-122 (sum over pairs j of
// (d*sc_j*q - dmin*m_j)*x for the low nibbles and the same with index j+4 for the high ones).
template <int B, int XPS, int XSS>
__device__ __forceinline__ void unit_q4k(const uint8_t* up, const float* xp, const float* xs, float (&acc)[B]) {
    const uint4* u4 = reinterpret_cast<const uint4*>(up);
    const uint4 h = u4[0];
    const float d = half_bits_to_float(h.x), dmin = half_bits_to_float(h.x >> 16);
    const Q4KScales s = q4k_unpack_scales(h);
    const float2 m2 = make_float2(-kTwo23, -kTwo23);
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float dl = d * byte_to_float(s.sl, j), ml = dmin * byte_to_float(s.ml, j);
        const float dh = d * byte_to_float(s.sh, j), mh = dmin * byte_to_float(s.mh, j);
        float2 al0[B], al1[B], ah0[B], ah1[B];
#pragma unroll
        for (int b = 0; b < B; b++) al0[b] = al1[b] = ah0[b] = ah1[b] = make_float2(0.f, 0.f);
#pragma unroll
        for (int c4 = 0; c4 < 2; c4++) {
            const uint4 q = u4[1 + 2 * j + c4];
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const uint32_t v = w[c], v12 = v >> 12;
                const float2 l01 = fadd2(bits2((v & 0xFu) | kMagic, (v & 0xF00u) | kMagic), m2);
                const float2 l23 = fadd2(bits2((v & 0xF0000u) | kMagic, (v12 & 0xF000u) | kMagic), m2);
                const float2 h01 = fadd2(bits2((v & 0xF0u) | kMagic, (v & 0xF000u) | kMagic), m2);
                const float2 h23 = fadd2(bits2((v12 & 0xF00u) | kMagic, (v12 & 0xF0000u) | kMagic), m2);
#pragma unroll
                for (int b = 0; b < B; b++) {
                    const float4 xl = *reinterpret_cast<const float4*>(xp + b * XPS + 64 * j + 16 * c4 + 4 * c);
                    const float4 xh = *reinterpret_cast<const float4*>(xp + b * XPS + 64 * j + 32 + 16 * c4 + 4 * c);
                    al0[b] = ffma2(l01, make_float2(xl.x, xl.y), al0[b]);
                    al1[b] = ffma2(l23, make_float2(xl.z, xl.w), al1[b]);
                    ah0[b] = ffma2(h01, make_float2(xh.x, xh.y), ah0[b]);
                    ah1[b] = ffma2(h23, make_float2(xh.z, xh.w), ah1[b]);
                }
            }
        }
#pragma unroll
        for (int b = 0; b < B; b++) {
            const float sl = (al0[b].x + al0[b].y) + (al1[b].x + al1[b].y);
            const float sh = (ah0[b].x + ah0[b].y) + (ah1[b].x + ah1[b].y);
            const float Xl = xs[b * XSS + 2 * j], Xh = xs[b * XSS + 2 * j + 1];
            acc[b] += (dl * sl - ml * Xl) + (dh * sh - mh * Xh);
        }
    }
}

// Eight Q4_0 blocks (144 bytes) against B prepared slices.  Formula:
// crates/kernels/shaders/gemv_q4_0.metal:26-49 (d * sum((nib-8)*x), interleaved nibbles).
template <int B, int XPS>
__device__ __forceinline__ void unit_q4_0(const uint8_t* up, const float* xp, int nblk, float (&acc)[B]) {
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
            const int o0 = 18 * blk;
            const uint32_t dw = w[o0 >> 2];
            const float d = half_bits_to_float((o0 & 2) ? (dw >> 16) : dw);
            float2 a0[B], a1[B];
#pragma unroll
            for (int b = 0; b < B; b++) a0[b] = a1[b] = make_float2(0.f, 0.f);
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
                // bytes i and i+1 of the block: element pairs (2i, 2i+1) and (2i+2, 2i+3)
                float2 q2[2];
#pragma unroll
                for (int t = 0; t < 2; t++) {
                    const int o = o0 + 2 + i + t, bp = o & 3;
                    const uint32_t v = w[o >> 2], v12 = v >> 12;
                    uint32_t lo, hi;
                    float cl, ch;
                    if (bp == 0)      { lo = v & 0xFu;       hi = v & 0xF0u;       cl = 8.f;      ch = 128.f; }
                    else if (bp == 1) { lo = v & 0xF00u;     hi = v & 0xF000u;     cl = 2048.f;   ch = 32768.f; }
                    else if (bp == 2) { lo = v & 0xF0000u;   hi = v12 & 0xF00u;    cl = 524288.f; ch = 2048.f; }
                    else              { lo = v12 & 0xF000u;  hi = v12 & 0xF0000u;  cl = 32768.f;  ch = 524288.f; }
                    q2[t] = fadd2(bits2(lo | kMagic, hi | kMagic), make_float2(-(kTwo23 + cl), -(kTwo23 + ch)));
                }
#pragma unroll
                for (int b = 0; b < B; b++) {
                    const float4 x4 = *reinterpret_cast<const float4*>(xp + b * XPS + 32 * blk + 2 * i);
                    a0[b] = ffma2(q2[0], make_float2(x4.x, x4.y), a0[b]);
                    a1[b] = ffma2(q2[1], make_float2(x4.z, x4.w), a1[b]);
                }
            }
#pragma unroll
            for (int b = 0; b < B; b++) acc[b] += d * ((a0[b].x + a0[b].y) + (a1[b].x + a1[b].y));
        }
    }
}

// Four Q8_0 blocks (136 bytes, 8-byte aligned) against B slices.  Formula:
// crates/kernels/shaders/gemv_q8_0.metal:24-36 (d * sum(int8 * x)).
template <int B, int XPS>
__device__ __forceinline__ void unit_q8_0(const uint8_t* up, const float* xp, int nblk, float (&acc)[B]) {
    const uint2* u2 = reinterpret_cast<const uint2*>(up);
    uint32_t w[34];
#pragma unroll
    for (int i = 0; i < 17; i++) {
        const uint2 q = u2[i];
        w[2 * i] = q.x; w[2 * i + 1] = q.y;
    }
    const float2 m2 = make_float2(-(kTwo23 + 128.f), -(kTwo23 + 128.f));
#pragma unroll
    for (int blk = 0; blk < 4; blk++) {
        if (blk < nblk) {
            const int o0 = 34 * blk;
            const uint32_t dw = w[o0 >> 2];
            const float d = half_bits_to_float((o0 & 2) ? (dw >> 16) : dw);
            float2 a0[B], a1[B];
#pragma unroll
            for (int b = 0; b < B; b++) a0[b] = a1[b] = make_float2(0.f, 0.f);
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                float2 q2[2];
#pragma unroll
                for (int t = 0; t < 2; t++) {
                    const int o = o0 + 2 + i + 2 * t, bp = o & 3;   // o is even: bytes o, o+1 share a word
                    const uint32_t wx = w[o >> 2] ^ 0x80808080u;    // int8 -> biased uint8
                    q2[t] = fadd2(bits2(__byte_perm(wx, kMagic, 0x7540 | bp), __byte_perm(wx, kMagic, 0x7540 | (bp + 1))), m2);
                }
#pragma unroll
                for (int b = 0; b < B; b++) {
                    const float4 x4 = *reinterpret_cast<const float4*>(xp + b * XPS + 32 * blk + i);
                    a0[b] = ffma2(q2[0], make_float2(x4.x, x4.y), a0[b]);
                    a1[b] = ffma2(q2[1], make_float2(x4.z, x4.w), a1[b]);
                }
            }
#pragma unroll
            for (int b = 0; b < B; b++) acc[b] += d * ((a0[b].x + a0[b].y) + (a1[b].x + a1[b].y));
        }
    }
}

// ───────────────────────── staged kernel ─────────────────────────

template <int FMT, int B, bool XF16, int CPB, int S>
__global__ void __launch_bounds__(kNT) gemv_staged_kernel(const GemvArgs a) {
    using T = Traits<FMT>;
    using L = StageLayout<FMT, B, XF16>;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float red[kKS][kRT][B];

    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;

    // Which segment / tile is this CTA?
    int si = 0;
#pragma unroll
    for (int i = 1; i < 3; i++)
        if (i < a.nseg && blockIdx.x >= a.seg[i].tile_begin) si = i;
    const GemvSeg sg = a.seg[si];
    const int rows_per_tile = a.dual ? kRT / 2 : kRT;
    const uint32_t row0 = (blockIdx.x - sg.tile_begin) * rows_per_tile;

    // Copy role: thread <-> (virtual row, quarter of the row's stage bytes).
    const int crow = t >> 2, cq = t & 3;
    const int crow_real = a.dual ? (crow & 15) : crow;
    const bool crow_ok = row0 + crow_real < sg.rows;
    const uint8_t* cw = (a.dual && crow >= 16) ? sg.w2 : sg.w;
    const uint8_t* gsrc = cw + (size_t)(row0 + (crow_ok ? crow_real : 0)) * a.row_bytes + cq * CPB;
    const uint32_t sdst = smem_u32(smem) + crow * L::ROW_STRIDE + cq * CPB;

    auto issue = [&](int st) {
        if (st < (int)a.n_stages) {
            const uint32_t slot = (st % S) * L::BYTES;
            const uint32_t off = (uint32_t)st * (kKS * T::UB);
            const int vb = min((int)(kKS * T::UB), (int)(a.row_bytes - off));
            if (crow_ok) {
                const uint8_t* g = gsrc + off;
                const uint32_t sd = sdst + slot;
                constexpr int NCH = (kKS * T::UB / CPB + 3) / 4;
#pragma unroll
                for (int j = 0; j < NCH; j++) {
                    const int bo = (cq + 4 * j) * CPB;
                    if (bo < vb) {
                        if (CPB == 16) cp_async16(sd + 4 * j * CPB, g + 4 * j * CPB);
                        else if (CPB == 8) cp_async8(sd + 4 * j * CPB, g + 4 * j * CPB);
                        else cp_async4(sd + 4 * j * CPB, g + 4 * j * CPB);
                    }
                }
            }
            // activations of this stage
            const uint32_t e0 = (uint32_t)st * L::XE;
            if (XF16) {
                const __half* xg = reinterpret_cast<const __half*>(a.x);
                constexpr int NX = L::XE / 8;   // 16-byte chunks per batch row
#pragma unroll
                for (int b = 0; b < B; b++)
                    for (int c = t; c < NX; c += kNT)
                        if (e0 + c * 8 < a.k)
                            cp_async16(smem_u32(smem) + slot + L::XR_OFF + (b * L::XE + c * 8) * 2,
                                       xg + (size_t)b * a.k + e0 + c * 8);
            } else {
                const float* xg = reinterpret_cast<const float*>(a.x);
                constexpr int NX = L::XE / 4;
#pragma unroll
                for (int b = 0; b < B; b++)
#pragma unroll
                    for (int c = t; c < NX; c += kNT)
                        if (e0 + c * 4 < a.k)
                            cp_async16(smem_u32(smem) + slot + L::XP_OFF + (b * L::XE + c * 4) * 4,
                                       xg + (size_t)b * a.k + e0 + c * 4);
            }
        }
        cp_async_commit();
    };

    // Prepare the activations of stage st: f16 -> f32, nibble-position pre-scaling, block sums.
    auto prep = [&](int st) {
        if (st >= (int)a.n_stages) return;
        if (FMT == RUNIT_FMT_Q8_0 && !XF16) return;
        uint8_t* slot = smem + (st % S) * L::BYTES;
        constexpr int EPT = L::XE / kNT;   // 8 (4-bit formats) or 4 (Q8_0) consecutive elements
        const int e = t * EPT;             // stage-local element index
        const int eu = e % T::UE;          // unit-local
#pragma unroll
        for (int b = 0; b < B; b++) {
            float v[EPT];
            float* xp = reinterpret_cast<float*>(slot + L::XP_OFF) + b * L::XE + e;
            if (XF16) {
                const __half* xr = reinterpret_cast<const __half*>(slot + L::XR_OFF) + b * L::XE + e;
#pragma unroll
                for (int i = 0; i < EPT; i++) v[i] = __half2float(xr[i]);
            } else {
#pragma unroll
                for (int i = 0; i < EPT; i++) v[i] = xp[i];
            }
            // e is a multiple of EPT (8 for the 4-bit formats), so the position inside a qs
            // word depends only on i; the half of the pair (Q4_K) or the block parity (Q4_0)
            // is uniform over the thread's elements.
            const int par = (eu >> 5) & 1;
            if (FMT == RUNIT_FMT_Q4K) {
                float s = 0.f;
#pragma unroll
                for (int i = 0; i < EPT; i++) s += v[i];
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                if ((t & 3) == 0) reinterpret_cast<float*>(slot + L::XS_OFF)[b * (kKS * 8) + (e >> 5)] = s;
#pragma unroll
                for (int i = 0; i < EPT; i++) v[i] *= par ? q4k_xscale(32 + i) : q4k_xscale(i);
            } else if (FMT == RUNIT_FMT_Q4_0) {
#pragma unroll
                for (int i = 0; i < EPT; i++) v[i] *= par ? q4_0_xscale(32 + i) : q4_0_xscale(i);
            }
#pragma unroll
            for (int i = 0; i < EPT; i++) xp[i] = v[i];
        }
    };

    float acc[B];
#pragma unroll
    for (int b = 0; b < B; b++) acc[b] = 0.f;

    const bool row_ok = a.dual ? (row0 + (lane & 15) < sg.rows) : (row0 + lane < sg.rows);

#pragma unroll
    for (int s = 0; s < S - 1; s++) issue(s);
    cp_async_wait<S - 2>();
    __syncthreads();
    prep(0);

    for (int st = 0; st < (int)a.n_stages; st++) {
        cp_async_wait<S - 3>();          // stages <= st+1 have landed
        __syncthreads();                 // slot (st-1)%S is free; prep(st) is visible
        issue(st + S - 1);
        prep(st + 1);
        const uint32_t u = (uint32_t)st * kKS + warp;
        if (row_ok && u < a.n_units) {
            const uint8_t* slot = smem + (st % S) * L::BYTES;
            const uint8_t* up = slot + lane * L::ROW_STRIDE + warp * T::UB;
            const float* xp = reinterpret_cast<const float*>(slot + L::XP_OFF) + warp * T::UE;
            if (FMT == RUNIT_FMT_Q4K) {
                const float* xs = reinterpret_cast<const float*>(slot + L::XS_OFF) + warp * 8;
                unit_q4k<B, L::XE, kKS * 8>(up, xp, xs, acc);
            } else if (FMT == RUNIT_FMT_Q4_0) {
                unit_q4_0<B, L::XE>(up, xp, min(T::BPU, (int)(a.nb - u * T::BPU)), acc);
            } else {
                unit_q8_0<B, L::XE>(up, xp, min(T::BPU, (int)(a.nb - u * T::BPU)), acc);
            }
        }
    }
    cp_async_wait<0>();

    // Add the four K-slices of each row in slice order, then the epilogue.
#pragma unroll
    for (int b = 0; b < B; b++) red[warp][lane][b] = acc[b];
    __syncthreads();
    if (warp == 0) {
        float r[B];
#pragma unroll
        for (int b = 0; b < B; b++) r[b] = ((red[0][lane][b] + red[1][lane][b]) + red[2][lane][b]) + red[3][lane][b];
        if (a.dual) {
            // lanes 0..15 hold gate rows, lanes 16..31 the matching up rows:
            // act = silu(gate) * up  (crates/kernels/shaders/fused_ffn.metal:24-26,89-92)
#pragma unroll
            for (int b = 0; b < B; b++) {
                const float up_v = __shfl_down_sync(0xffffffffu, r[b], 16);
                r[b] = silu(r[b]) * up_v;
            }
        }
        const uint32_t row = row0 + (a.dual ? (lane & 15) : lane);
        const bool writer = a.dual ? (lane < 16 && row < sg.rows) : (row < sg.rows);
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
            const uint32_t nr = a.dual ? a.seg[i].rows : a.seg[i].rows;
            if (grow >= acc_rows && grow < acc_rows + nr) { si = i; base = acc_rows; }
            acc_rows += nr;
        }
        if (grow >= acc_rows) return;
    }
    const GemvSeg sg = a.seg[si];
    const uint32_t row = grow - base;
    const int nmat = a.dual ? 2 : 1;
    for (int b = 0; b < batch; b++) {
        float res2[2] = {0.f, 0.f};
        for (int mi = 0; mi < nmat; mi++) {
            const uint8_t* rp = (mi ? sg.w2 : sg.w) + (size_t)row * a.row_bytes;
            float acc = 0.f;
            for (uint32_t blk = lane; blk < a.nb; blk += 32) {
                auto X = [&](uint32_t i) -> float {
                    const size_t o = (size_t)b * a.k + i;
                    return XF16 ? __half2float(reinterpret_cast<const __half*>(a.x)[o])
                                : reinterpret_cast<const float*>(a.x)[o];
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
        }
    }
}

}  // namespace runit
