// Fused-dequant GEMVs for the formats the reference only dequantises on the CPU at load time: Q5_0, Q5_K and Q6_K
// (crates/engine/src/forward.rs:900-949, 979-1012; files quantised as "Q4_K_M" mix them in: Q6_K for ffn_down and the
// output matrix, Q5_0 / Q5_K in some attention matrices, docs/STATUS_REPORT.md:19-27).  The reference expands such
// tensors to f32 or f16 and runs its f16 GEMV on them; here they stay packed in HBM (0.69 / 0.69 / 0.82 bytes per weight
// instead of 2) and are decoded in registers, so a decode step streams 2.4 - 2.9 times fewer bytes for them.
//
// Kernel: one warp per row, lane l decodes 8 of the 256 weights of a unit (a Q5_K / Q6_K superblock, or 8 Q5_0 blocks)
// exactly as the reference's loops index them; the packed bytes of 4 units at a time arrive through a per-warp ring of
// three cp.async stages that runs across the warp's rows (rows are only 2- or 4-byte aligned in these formats, so the
// copies are 4-byte ones from the aligned word below); f32 accumulation, shuffle reduction, optional f32 residual.
// HBM-bound in principle; at ~7 instructions per weight it is issue-bound at roughly half the HBM rate on B200.
#include "gemv_common.cuh"
#include "gemv_int8.cuh"
#include "runit_internal.h"
#include "tma.cuh"

namespace runit {
namespace kq {

constexpr int kWarps = 8;       // per CTA
constexpr int kChunk = 4;       // units per stage
constexpr int kStages = 3;

template <int FMT> struct KTraits;
template <> struct KTraits<RUNIT_FMT_Q5_0> { static constexpr int UB = 176; };   // 8 blocks of 22 bytes
template <> struct KTraits<RUNIT_FMT_Q5K>  { static constexpr int UB = 176; };
template <> struct KTraits<RUNIT_FMT_Q6K>  { static constexpr int UB = 210; };

// Partial dot product of this lane's 8 weights of one unit with x (xu = the unit's 256 activations in global memory).
template <int FMT>
__device__ __forceinline__ float unit_dot(const uint8_t* u, const float* __restrict__ xu, int lane, int nblk) {
    float acc = 0.f;
    if (FMT == RUNIT_FMT_Q6K) {
        // forward.rs:920-949: {ql[128]; qh[64]; i8 scales[16]; f16 d}
        const float d = half_bits_to_float((uint32_t)u[208] | ((uint32_t)u[209] << 8));
        const int8_t* sc = reinterpret_cast<const int8_t*>(u + 192);
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const int a = u[64 * half + lane], c = u[64 * half + lane + 32], h = u[128 + 32 * half + lane];
            const int q1 = ((a & 15) | ((h & 3) << 4)) - 32, q2 = ((c & 15) | (((h >> 2) & 3) << 4)) - 32;
            const int q3 = ((a >> 4) | (((h >> 4) & 3) << 4)) - 32, q4 = ((c >> 4) | (((h >> 6) & 3) << 4)) - 32;
            const float* xh = xu + 128 * half + lane;
            float s = (float)sc[8 * half + 0] * ((float)q1 * xh[0]);
            s = fmaf((float)sc[8 * half + 2], (float)q2 * xh[32], s);
            s = fmaf((float)sc[8 * half + 4], (float)q3 * xh[64], s);
            s = fmaf((float)sc[8 * half + 6], (float)q4 * xh[96], s);
            acc = fmaf(d, s, acc);
        }
    } else if (FMT == RUNIT_FMT_Q5K) {
        // forward.rs:979-1012: {f16 d; f16 dmin; scales[12]; qh[32]; qs[128]}; fifth bit of element e = bit e%8 of qh[e/8]
        const uint32_t h0 = *reinterpret_cast<const uint16_t*>(u) | ((uint32_t)*reinterpret_cast<const uint16_t*>(u + 2) << 16);
        const float d = half_bits_to_float(h0), dmin = half_bits_to_float(h0 >> 16);
        const uint8_t* s = u + 4;
        const uint8_t* qh = u + 16;
        const uint8_t* qs = u + 48;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            // get_scale_min_k4 (forward.rs:359-369) for indices j and j + 4
            const float sc_lo = (float)(s[j] & 63), m_lo = (float)(s[j + 4] & 63);
            const float sc_hi = (float)((s[j + 8] & 15) | ((s[j] >> 6) << 4)), m_hi = (float)((s[j + 8] >> 4) | ((s[j + 4] >> 6) << 4));
            const int v = qs[32 * j + lane];
            const int e_lo = 64 * j + lane, e_hi = e_lo + 32;
            const int q_lo = (v & 15) | (((qh[e_lo >> 3] >> (e_lo & 7)) & 1) << 4);
            const int q_hi = (v >> 4) | (((qh[e_hi >> 3] >> (e_hi & 7)) & 1) << 4);
            const float x_lo = xu[e_lo], x_hi = xu[e_hi];
            acc = fmaf(d * sc_lo * (float)q_lo - dmin * m_lo, x_lo, acc);
            acc = fmaf(d * sc_hi * (float)q_hi - dmin * m_hi, x_hi, acc);
        }
    } else {
        // forward.rs:900-919: blocks {f16 d; qh[4]; qs[16]}; lane l: block l / 4, bytes 4 (l % 4) .. + 3
        const int b = lane >> 2, j0 = (lane & 3) * 4;
        if (b < nblk) {
            const uint8_t* blk = u + 22 * b;
            const float d = half_bits_to_float((uint32_t)blk[0] | ((uint32_t)blk[1] << 8));
            const uint32_t qh = (uint32_t)blk[2] | ((uint32_t)blk[3] << 8) | ((uint32_t)blk[4] << 16) | ((uint32_t)blk[5] << 24);
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int j = j0 + i, v = blk[6 + j];
                const int x0 = (v & 15) | (((qh >> j) & 1) << 4), x1 = (v >> 4) | (((qh >> (j + 16)) & 1) << 4);
                s = fmaf((float)(x0 - 16), xu[32 * b + j], s);
                s = fmaf((float)(x1 - 16), xu[32 * b + j + 16], s);
            }
            acc = d * s;
        }
    }
    return acc;
}

struct Args {
    const uint8_t* w;
    const float* x;
    float* y;
    const float* res;
    uint32_t m, k, n_units, row_bytes, nb;   // nb: 32-blocks per row (Q5_0: the last unit may hold fewer than 8)
};

template <int FMT>
__global__ void __launch_bounds__(kWarps * 32) gemv_kquant_kernel(const Args a) {
    constexpr int UB = KTraits<FMT>::UB;
    constexpr int SB = (kChunk * UB + 4 + 15) / 16 * 16;   // stage bytes: the chunk plus the alignment shift
    __shared__ __align__(16) uint8_t ring[kWarps][kStages][SB];
    grid_dependency_wait();
    grid_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t gw = blockIdx.x * kWarps + warp, n_warps = gridDim.x * kWarps;
    if (gw >= a.m) return;
    const uint32_t n_chunks = (a.n_units + kChunk - 1) / kChunk;
    const uint32_t my_rows = (a.m - gw + n_warps - 1) / n_warps;
    const uint32_t n_steps = my_rows * n_chunks;   // (row, chunk) pairs of this warp, in order

    // chunk t of this warp: row gw + (t / n_chunks) * n_warps, units [c * kChunk, ...)
    auto issue = [&](uint32_t t) {
        if (t < n_steps) {
            const uint32_t row = gw + (t / n_chunks) * n_warps, c = t % n_chunks;
            const uint32_t units = min((uint32_t)kChunk, a.n_units - c * kChunk);
            const size_t start = (size_t)row * a.row_bytes + (size_t)c * kChunk * UB;
            const size_t bytes = FMT == RUNIT_FMT_Q5_0 ? min((size_t)units * UB, (size_t)a.row_bytes - (size_t)c * kChunk * UB) : (size_t)units * UB;
            const uint32_t shift = (uint32_t)((reinterpret_cast<uintptr_t>(a.w) + start) & 3u);
            const uint8_t* src = a.w + start - shift;
            const uint32_t words = (uint32_t)((shift + bytes + 3) / 4);
            const uint32_t dst = smem_u32(&ring[warp][t % kStages][0]);
            for (uint32_t wd = lane; wd < words; wd += 32) cp_async4(dst + 4 * wd, src + 4 * (size_t)wd);
        }
        cp_async_commit();
    };
#pragma unroll
    for (int s = 0; s < kStages - 1; s++) issue(s);
    float acc = 0.f;
    for (uint32_t t = 0; t < n_steps; t++) {
        issue(t + kStages - 1);
        cp_async_wait<kStages - 1>();
        __syncwarp();
        const uint32_t row = gw + (t / n_chunks) * n_warps, c = t % n_chunks;
        const uint32_t units = min((uint32_t)kChunk, a.n_units - c * kChunk);
        const size_t start = (size_t)row * a.row_bytes + (size_t)c * kChunk * UB;
        const uint32_t shift = (uint32_t)((reinterpret_cast<uintptr_t>(a.w) + start) & 3u);
        const uint8_t* base = &ring[warp][t % kStages][shift];
        for (uint32_t i = 0; i < units; i++) {
            const uint32_t u = c * kChunk + i;
            const int nblk = FMT == RUNIT_FMT_Q5_0 ? min(8, (int)(a.nb - u * 8u)) : 8;
            acc += unit_dot<FMT>(base + i * UB, a.x + (size_t)u * 256, lane, nblk);
        }
        __syncwarp();   // the stage may be refilled by the next issue
        if (c + 1 == n_chunks) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (lane == 0) a.y[row] = a.res ? a.res[row] + acc : acc;
            acc = 0.f;
        }
    }
    cp_async_wait<0>();
}

// ───────────────────────── Q6_K, tile kernel ─────────────────────────
// Lane = row.  Every warp owns a tile of 32 rows and walks all superblocks of K (4 tiles per CTA, no reduction across
// warps).  Per superblock the warp copies the 32 rows' 210 bytes into its own two-stage ring (4-byte cp.async from the aligned word
// below each row's start: a row's superblock starts on a 2-byte boundary only) together with the 256 activations, which
// it then turns into three signed 8-bit limbs per element with one power-of-two scale per 32 (prep_int_block: 23 bits,
// exact to f32 rounding).  Every lane decodes its own row: a word of ql low nibbles, a word of ql high nibbles and a word
// of qh give four weights each of the reference's four groups q1..q4 (forward.rs:920-949) as 6-bit fields in bytes,
// which meet the limbs in dp4a; the "- 32" is taken through the blocks' sums.  About 1.7 instructions per weight instead
// of 7, and scales, d and the activations are read once per row-lane instead of once per weight.
namespace q6t {

constexpr int kPitch = 220;                       // bytes per row in a stage: 53 words + 2 (an odd number of words)
constexpr int kXOff = 32 * kPitch;                // activations of the unit: 1024 bytes raw, prepared in place
constexpr int kStage = kXOff + 1024;
constexpr int kS = 2;

__device__ __forceinline__ int dp4a_u8s8(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

struct Args {
    const uint8_t* w;
    const float* x;
    float* y;
    const float* res;
    uint32_t m, nb, row_bytes;
    // split > 0 (matrices with few rows): a CTA owns ONE tile and one of `split` shares of K; its 4 warps take every
    // 4 * split-th superblock each, the CTA files one partial sum per row in part[share][row], and the CTA that takes the
    // last of the tile's tickets adds the shares in order (deterministic) and stores the rows.
    uint32_t split;
    float* part;
    uint32_t* tickets;       // one word per tile, zero at rest
};

__global__ void __launch_bounds__(128) gemv_q6k_tile_kernel(const Args a) {
    extern __shared__ __align__(16) uint8_t q6_smem[];
    __shared__ float red[4][32];
    __shared__ uint32_t s_last;
    grid_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint8_t* ring = q6_smem + warp * (kS * kStage);
    // split == 0: every warp owns a tile of 32 rows and walks all of K; else the CTA owns tile blockIdx.x
    const uint32_t row0 = a.split ? blockIdx.x * 32 : (blockIdx.x * 4 + warp) * 32;
    if (row0 >= a.m) return;
    const uint32_t rows_here = min(32u, a.m - row0);
    const uint32_t u0 = a.split ? blockIdx.y * 4 + warp : 0u, ustep = a.split ? 4u * a.split : 1u;
    const int n_it = u0 < a.nb ? (int)((a.nb - u0 + ustep - 1) / ustep) : 0;

    auto issue = [&](int it) {
        if (it < n_it) {
            const uint32_t u = u0 + ustep * (uint32_t)it;
            const uint32_t st = smem_u32(ring + (it % kS) * kStage);
            // row r: 53 words from the aligned word below its superblock; lane l copies words l and l + 32 (l < 21).  With
            // shift 0 the last word holds only two bytes of the row (its f16 d): that copy takes two bytes from memory
            // (the rest is filled with zeros), so nothing is read past the row.  Branch-free: the size is an operand.
            const uint8_t* p = a.w + (size_t)row0 * a.row_bytes + (size_t)u * 210;
            uint32_t dst = st + 4 * lane;
#pragma unroll 4
            for (uint32_t r = 0; r < rows_here; r++) {
                const uint32_t shift = (uint32_t)(reinterpret_cast<uintptr_t>(p) & 3u);      // 0 or 2
                const uint8_t* src = p - shift + 4 * lane;
                cp_async4(dst, src);
                if (lane < 21) {
                    const uint32_t nbytes = (lane == 20 && shift == 0) ? 2u : 4u;
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(dst + 128), "l"(src + 128), "r"(nbytes) : "memory");
                }
                p += a.row_bytes;
                dst += kPitch;
            }
            const float* xu = a.x + (size_t)u * 256;
            cp_async16(st + kXOff + 16 * lane, xu + 4 * lane);
            cp_async16(st + kXOff + 16 * (32 + lane), xu + 4 * (32 + lane));
        }
        cp_async_commit();
    };
    grid_dependency_wait();      // x (and the residual) may come from the previous kernel of the chain
#pragma unroll
    for (int s = 0; s < kS; s++) issue(s);
    float acc = 0.f;
    for (int it = 0; it < n_it; it++) {
        cp_async_wait<kS - 1>();
        __syncwarp();
        uint8_t* stg = ring + (it % kS) * kStage;
        {   // activations of the unit -> limbs, scales, block sums (in place)
            float v[8];
            const float4* xr = reinterpret_cast<const float4*>(stg + kXOff) + 2 * lane;
            const float4 t0 = xr[0], t1 = xr[1];
            v[0] = t0.x; v[1] = t0.y; v[2] = t0.z; v[3] = t0.w; v[4] = t1.x; v[5] = t1.y; v[6] = t1.z; v[7] = t1.w;
            __syncwarp();
            prep_int_block<8, 8, 0>(stg + kXOff, v, lane);
            __syncwarp();
        }
        if ((uint32_t)lane < rows_here) {
            const uint32_t u = u0 + ustep * (uint32_t)it;
            const uint32_t sh8 = (uint32_t)((((size_t)(row0 + lane) * a.row_bytes + (size_t)u * 210) & 3u) * 8u);   // 0 or 16
            const uint32_t* rw = reinterpret_cast<const uint32_t*>(stg + lane * kPitch);
            uint32_t rv[54];                     // the row's words, once; word 53 is never part of a result
#pragma unroll
            for (int j = 0; j < 53; j++) rv[j] = rw[j];
            rv[53] = 0;
            auto W = [&](int j) -> uint32_t { return __funnelshift_r(rv[j], rv[j + 1], sh8); };
            const uint8_t* xq = stg + kXOff;
            const float* sx = reinterpret_cast<const float*>(xq + IntX<8>::SCALE);
            const int* sv = reinterpret_cast<const int*>(xq + IntX<8>::VSUM);
            const uint32_t sc_w[4] = {W(48), W(49), W(50), W(51)};           // 16 signed scales
            const float d = half_bits_to_float(W(52) & 0xFFFFu);
            float unit_acc = 0.f;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                // the 128 weights of this half as 6-bit fields in bytes: q[j][g] = elements 32 j + 4 g .. + 3 of the half
                uint32_t q[4][8];
#pragma unroll
                for (int g = 0; g < 8; g++) {
                    const uint32_t wa = W(16 * h + g), wc = W(16 * h + 8 + g), wh = W(32 + 8 * h + g);
                    q[0][g] = (wa & 0x0F0F0F0Fu) | ((wh & 0x03030303u) << 4);
                    q[1][g] = (wc & 0x0F0F0F0Fu) | ((wh & 0x0C0C0C0Cu) << 2);
                    q[2][g] = ((wa >> 4) & 0x0F0F0F0Fu) | (wh & 0x30303030u);
                    q[3][g] = ((wc >> 4) & 0x0F0F0F0Fu) | ((wh >> 2) & 0x30303030u);
                }
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int b = 4 * h + j;
                    const uint4* xl = reinterpret_cast<const uint4*>(xq + b * 96);     // limb l of the block: xl[2 l], xl[2 l + 1]
                    int s0 = 0, s1 = 0, s2 = 0;
#pragma unroll
                    for (int hf = 0; hf < 2; hf++) {
                        const uint4 l0 = xl[hf], l1 = xl[2 + hf], l2 = xl[4 + hf];
                        const uint32_t x0[4] = {l0.x, l0.y, l0.z, l0.w}, x1[4] = {l1.x, l1.y, l1.z, l1.w}, x2[4] = {l2.x, l2.y, l2.z, l2.w};
#pragma unroll
                        for (int c = 0; c < 4; c++) {
                            s0 = dp4a_u8s8(q[j][4 * hf + c], x0[c], s0);
                            s1 = dp4a_u8s8(q[j][4 * hf + c], x1[c], s1);
                            s2 = dp4a_u8s8(q[j][4 * hf + c], x2[c], s2);
                        }
                    }
                    // sum q * v over the block, exact in every limb; the reference's q - 32 through the block's sum of v
                    const float dot = fmaf((float)s2, 65536.f, fmaf((float)s1, 256.f, (float)s0)) - 32.f * (float)sv[b];
                    const int scb = (int)(int8_t)((sc_w[(2 * b) >> 2] >> (8 * ((2 * b) & 3))) & 0xFFu);   // scales[8 half + 2 group]
                    unit_acc = fmaf((float)scb * sx[b], dot, unit_acc);
                }
            }
            acc = fmaf(d, unit_acc, acc);
        }
        __syncwarp();
        issue(it + kS);
    }
    cp_async_wait<0>();
    if (a.split == 0) {
        if ((uint32_t)lane < rows_here) {
            const uint32_t row = row0 + lane;
            a.y[row] = a.res ? a.res[row] + acc : acc;
        }
        return;
    }
    red[warp][lane] = acc;
    __syncthreads();
    if (warp == 0) {
        const float v = ((red[0][lane] + red[1][lane]) + red[2][lane]) + red[3][lane];
        if ((uint32_t)lane < rows_here) __stcg(&a.part[(size_t)blockIdx.y * a.m + row0 + lane], v);
        __threadfence();
        __syncwarp();
        if (lane == 0) s_last = atomicAdd(&a.tickets[blockIdx.x], 1u) == a.split - 1;
    }
    __syncthreads();
    if (s_last && warp == 0) {
        __threadfence();
        if ((uint32_t)lane < rows_here) {
            const uint32_t row = row0 + lane;
            float v = a.res ? a.res[row] : 0.f;
            for (uint32_t sp = 0; sp < a.split; sp++) v += __ldcg(&a.part[(size_t)sp * a.m + row]);
            a.y[row] = v;
        }
        if (lane == 0) a.tickets[blockIdx.x] = 0;
    }
}

}  // namespace q6t

// ───────────────────────── Q5_K, tile kernel ─────────────────────────
// The same arrangement for Q5_K: superblocks are 176 bytes and rows 16-byte aligned, so a tile's unit arrives by 16-byte
// cp.async (11 per row) at a pitch of 176 bytes (an odd multiple of 16: lane = row reads 128 bits without bank conflicts).
// A word of qs gives four low-nibble weights of block 2j and four high-nibble weights of block 2j + 1; their fifth bits
// are a nibble of qh (bit e % 8 of qh[e / 8], forward.rs:979-1012), spread into bit 4 of four bytes by one multiply.
namespace q5t {

constexpr int kPitch = 176;
constexpr int kXOff = 32 * kPitch;
constexpr int kStage = kXOff + 1024;
constexpr int kS = 2;

__global__ void __launch_bounds__(128) gemv_q5k_tile_kernel(const q6t::Args a) {
    extern __shared__ __align__(16) uint8_t q5_smem[];
    __shared__ float red[4][32];
    __shared__ uint32_t s_last;
    grid_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint8_t* ring = q5_smem + warp * (kS * kStage);
    const uint32_t row0 = a.split ? blockIdx.x * 32 : (blockIdx.x * 4 + warp) * 32;
    if (row0 >= a.m) return;
    const uint32_t rows_here = min(32u, a.m - row0);
    const uint32_t u0 = a.split ? blockIdx.y * 4 + warp : 0u, ustep = a.split ? 4u * a.split : 1u;
    const int n_it = u0 < a.nb ? (int)((a.nb - u0 + ustep - 1) / ustep) : 0;

    auto issue = [&](int it) {
        if (it < n_it) {
            const uint32_t u = u0 + ustep * (uint32_t)it;
            const uint32_t st = smem_u32(ring + (it % kS) * kStage);
            const uint8_t* base = a.w + (size_t)row0 * a.row_bytes + (size_t)u * 176;
#pragma unroll
            for (int i = 0; i < 11; i++) {
                const uint32_t c = (uint32_t)lane + 32u * i, r = c / 11u, col = c - 11u * r;      // 352 chunks of 16 bytes
                if (r < rows_here) cp_async16(st + r * kPitch + 16 * col, base + (size_t)r * a.row_bytes + 16 * col);
            }
            const float* xu = a.x + (size_t)u * 256;
            cp_async16(st + kXOff + 16 * lane, xu + 4 * lane);
            cp_async16(st + kXOff + 16 * (32 + lane), xu + 4 * (32 + lane));
        }
        cp_async_commit();
    };
    grid_dependency_wait();
#pragma unroll
    for (int s = 0; s < kS; s++) issue(s);
    float acc = 0.f;
    for (int it = 0; it < n_it; it++) {
        cp_async_wait<kS - 1>();
        __syncwarp();
        uint8_t* stg = ring + (it % kS) * kStage;
        {
            float v[8];
            const float4* xr = reinterpret_cast<const float4*>(stg + kXOff) + 2 * lane;
            const float4 t0 = xr[0], t1 = xr[1];
            v[0] = t0.x; v[1] = t0.y; v[2] = t0.z; v[3] = t0.w; v[4] = t1.x; v[5] = t1.y; v[6] = t1.z; v[7] = t1.w;
            __syncwarp();
            prep_int_block<8, 8, 0>(stg + kXOff, v, lane);
            __syncwarp();
        }
        if ((uint32_t)lane < rows_here) {
            const uint4* ru = reinterpret_cast<const uint4*>(stg + lane * kPitch);
            const uint8_t* xq = stg + kXOff;
            const float* sx = reinterpret_cast<const float*>(xq + IntX<8>::SCALE);
            const int* sv = reinterpret_cast<const int*>(xq + IntX<8>::VSUM);
            const uint4 hd = ru[0];                                   // d, dmin, 12 bytes of packed 6-bit scales and mins
            const float d = half_bits_to_float(hd.x), dmin = half_bits_to_float(hd.x >> 16);
            const Q4KScales sc = q4k_unpack_scales(hd.y, hd.z, hd.w);   // get_scale_min_k4 for j (sl, ml) and j + 4 (sh, mh)
            const uint4 h0 = ru[1], h1 = ru[2];
            const uint32_t qh[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
            float unit_acc = 0.f;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint4 qa = ru[3 + 2 * j], qb = ru[4 + 2 * j];
                const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
                uint32_t lo[8], hi[8];
#pragma unroll
                for (int g = 0; g < 8; g++) {
                    const int sh = 8 * (g >> 1) + 4 * (g & 1);
                    const uint32_t nl = (qh[2 * j] >> sh) & 15u, nh = (qh[2 * j + 1] >> sh) & 15u;
                    lo[g] = (w[g] & 0x0F0F0F0Fu) | (((nl * 0x00204081u) & 0x01010101u) << 4);
                    hi[g] = ((w[g] >> 4) & 0x0F0F0F0Fu) | (((nh * 0x00204081u) & 0x01010101u) << 4);
                }
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    const int b = 2 * j + half;
                    const uint32_t* q = half ? hi : lo;
                    const uint4* xl = reinterpret_cast<const uint4*>(xq + b * 96);
                    int s0 = 0, s1 = 0, s2 = 0;
#pragma unroll
                    for (int hf = 0; hf < 2; hf++) {
                        const uint4 l0 = xl[hf], l1 = xl[2 + hf], l2 = xl[4 + hf];
                        const uint32_t x0[4] = {l0.x, l0.y, l0.z, l0.w}, x1[4] = {l1.x, l1.y, l1.z, l1.w}, x2[4] = {l2.x, l2.y, l2.z, l2.w};
#pragma unroll
                        for (int c = 0; c < 4; c++) {
                            s0 = q6t::dp4a_u8s8(q[4 * hf + c], x0[c], s0);
                            s1 = q6t::dp4a_u8s8(q[4 * hf + c], x1[c], s1);
                            s2 = q6t::dp4a_u8s8(q[4 * hf + c], x2[c], s2);
                        }
                    }
                    const float dot = fmaf((float)s2, 65536.f, fmaf((float)s1, 256.f, (float)s0));
                    const float scw = (float)(((half ? sc.sh : sc.sl) >> (8 * j)) & 0xFFu), mnw = (float)(((half ? sc.mh : sc.ml) >> (8 * j)) & 0xFFu);
                    unit_acc = fmaf(sx[b], d * scw * dot - dmin * mnw * (float)sv[b], unit_acc);
                }
            }
            acc += unit_acc;
        }
        __syncwarp();
        issue(it + kS);
    }
    cp_async_wait<0>();
    if (a.split == 0) {
        if ((uint32_t)lane < rows_here) {
            const uint32_t row = row0 + lane;
            a.y[row] = a.res ? a.res[row] + acc : acc;
        }
        return;
    }
    red[warp][lane] = acc;
    __syncthreads();
    if (warp == 0) {
        const float v = ((red[0][lane] + red[1][lane]) + red[2][lane]) + red[3][lane];
        if ((uint32_t)lane < rows_here) __stcg(&a.part[(size_t)blockIdx.y * a.m + row0 + lane], v);
        __threadfence();
        __syncwarp();
        if (lane == 0) s_last = atomicAdd(&a.tickets[blockIdx.x], 1u) == a.split - 1;
    }
    __syncthreads();
    if (s_last && warp == 0) {
        __threadfence();
        if ((uint32_t)lane < rows_here) {
            const uint32_t row = row0 + lane;
            float v = a.res ? a.res[row] : 0.f;
            for (uint32_t sp = 0; sp < a.split; sp++) v += __ldcg(&a.part[(size_t)sp * a.m + row]);
            a.y[row] = v;
        }
        if (lane == 0) a.tickets[blockIdx.x] = 0;
    }
}

}  // namespace q5t

// ───────────────────────── Q5_0, tile kernel ─────────────────────────
// Q5_0 with K a multiple of 256: a unit is eight 22-byte blocks (176 bytes, 256 weights), rows are then multiples of
// 176 bytes and the copy is the Q5_K one (16-byte cp.async, pitch 176).  Inside the unit the blocks alternate between
// word-aligned and two bytes off, which a compile-time funnel shift takes care of.  A word of qs gives four low-nibble weights (elements 4 g ..) and four
// high-nibble weights (elements 16 + 4 g ..); their fifth bits are nibbles g and 4 + g of qh (forward.rs:900-918); the
// "- 16" is taken through the block's sum of activations.
namespace q50t {

constexpr int kPitch = 176;
constexpr int kXOff = 32 * kPitch;
constexpr int kStage = kXOff + 1024;
constexpr int kS = 2;

__global__ void __launch_bounds__(128) gemv_q5_0_tile_kernel(const q6t::Args a) {
    extern __shared__ __align__(16) uint8_t q50_smem[];
    __shared__ float red[4][32];
    __shared__ uint32_t s_last;
    grid_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint8_t* ring = q50_smem + warp * (kS * kStage);
    const uint32_t row0 = a.split ? blockIdx.x * 32 : (blockIdx.x * 4 + warp) * 32;
    if (row0 >= a.m) return;
    const uint32_t rows_here = min(32u, a.m - row0);
    const uint32_t u0 = a.split ? blockIdx.y * 4 + warp : 0u, ustep = a.split ? 4u * a.split : 1u;
    const int n_it = u0 < a.nb ? (int)((a.nb - u0 + ustep - 1) / ustep) : 0;

    auto issue = [&](int it) {
        if (it < n_it) {
            const uint32_t u = u0 + ustep * (uint32_t)it;
            const uint32_t st = smem_u32(ring + (it % kS) * kStage);
            const uint8_t* base = a.w + (size_t)row0 * a.row_bytes + (size_t)u * 176;
#pragma unroll
            for (int i = 0; i < 11; i++) {
                const uint32_t c = (uint32_t)lane + 32u * i, r = c / 11u, col = c - 11u * r;
                if (r < rows_here) cp_async16(st + r * kPitch + 16 * col, base + (size_t)r * a.row_bytes + 16 * col);
            }
            const float* xu = a.x + (size_t)u * 256;
            cp_async16(st + kXOff + 16 * lane, xu + 4 * lane);
            cp_async16(st + kXOff + 16 * (32 + lane), xu + 4 * (32 + lane));
        }
        cp_async_commit();
    };
    grid_dependency_wait();
#pragma unroll
    for (int s = 0; s < kS; s++) issue(s);
    float acc = 0.f;
    for (int it = 0; it < n_it; it++) {
        cp_async_wait<kS - 1>();
        __syncwarp();
        uint8_t* stg = ring + (it % kS) * kStage;
        {
            float v[8];
            const float4* xr = reinterpret_cast<const float4*>(stg + kXOff) + 2 * lane;
            const float4 t0 = xr[0], t1 = xr[1];
            v[0] = t0.x; v[1] = t0.y; v[2] = t0.z; v[3] = t0.w; v[4] = t1.x; v[5] = t1.y; v[6] = t1.z; v[7] = t1.w;
            __syncwarp();
            prep_int_block<8, 8, 0>(stg + kXOff, v, lane);
            __syncwarp();
        }
        if ((uint32_t)lane < rows_here) {
            const uint4* ru = reinterpret_cast<const uint4*>(stg + lane * kPitch);
            uint32_t al[45];                         // the unit's 44 words (al[44] only feeds discarded bytes)
#pragma unroll
            for (int j = 0; j < 11; j++) {
                const uint4 t = ru[j];
                al[4 * j] = t.x; al[4 * j + 1] = t.y; al[4 * j + 2] = t.z; al[4 * j + 3] = t.w;
            }
            al[44] = 0;
            // 32 bits at the (even, compile-time) byte offset e of the unit
            auto F = [&](int e) -> uint32_t { return (e & 3) ? __funnelshift_r(al[e >> 2], al[(e >> 2) + 1], 16) : al[e >> 2]; };
            const uint8_t* xq = stg + kXOff;
            const float* sx = reinterpret_cast<const float*>(xq + IntX<8>::SCALE);
            const int* sv = reinterpret_cast<const int*>(xq + IntX<8>::VSUM);
#pragma unroll
            for (int b = 0; b < 8; b++) {
                const float d = half_bits_to_float(F(22 * b) & 0xFFFFu);
                const uint32_t qh = F(22 * b + 2);
                const uint4* xl = reinterpret_cast<const uint4*>(xq + b * 96);
                int s0 = 0, s1 = 0, s2 = 0;
                uint32_t w[4];
#pragma unroll
                for (int g = 0; g < 4; g++) w[g] = F(22 * b + 6 + 4 * g);
#pragma unroll
                for (int hf = 0; hf < 2; hf++) {
                    const uint4 l0 = xl[hf], l1 = xl[2 + hf], l2 = xl[4 + hf];
                    const uint32_t x0[4] = {l0.x, l0.y, l0.z, l0.w}, x1[4] = {l1.x, l1.y, l1.z, l1.w}, x2[4] = {l2.x, l2.y, l2.z, l2.w};
#pragma unroll
                    for (int g = 0; g < 4; g++) {
                        const uint32_t nib = (qh >> (16 * hf + 4 * g)) & 15u;
                        const uint32_t q = ((hf ? (w[g] >> 4) : w[g]) & 0x0F0F0F0Fu) | (((nib * 0x00204081u) & 0x01010101u) << 4);
                        s0 = q6t::dp4a_u8s8(q, x0[g], s0);
                        s1 = q6t::dp4a_u8s8(q, x1[g], s1);
                        s2 = q6t::dp4a_u8s8(q, x2[g], s2);
                    }
                }
                const float dot = fmaf((float)s2, 65536.f, fmaf((float)s1, 256.f, (float)s0)) - 16.f * (float)sv[b];
                acc = fmaf(d * sx[b], dot, acc);
            }
        }
        __syncwarp();
        issue(it + kS);
    }
    cp_async_wait<0>();
    if (a.split == 0) {
        if ((uint32_t)lane < rows_here) {
            const uint32_t row = row0 + lane;
            a.y[row] = a.res ? a.res[row] + acc : acc;
        }
        return;
    }
    red[warp][lane] = acc;
    __syncthreads();
    if (warp == 0) {
        const float v = ((red[0][lane] + red[1][lane]) + red[2][lane]) + red[3][lane];
        if ((uint32_t)lane < rows_here) __stcg(&a.part[(size_t)blockIdx.y * a.m + row0 + lane], v);
        __threadfence();
        __syncwarp();
        if (lane == 0) s_last = atomicAdd(&a.tickets[blockIdx.x], 1u) == a.split - 1;
    }
    __syncthreads();
    if (s_last && warp == 0) {
        __threadfence();
        if ((uint32_t)lane < rows_here) {
            const uint32_t row = row0 + lane;
            float v = a.res ? a.res[row] : 0.f;
            for (uint32_t sp = 0; sp < a.split; sp++) v += __ldcg(&a.part[(size_t)sp * a.m + row]);
            a.y[row] = v;
        }
        if (lane == 0) a.tickets[blockIdx.x] = 0;
    }
}

}  // namespace q50t

template <int FMT>
static int32_t launch(runit_ctx* ctx, const char* name, const void* w, const void* x, void* y, const void* res, uint32_t m, uint32_t k) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, w && x && y, "%s: null pointer", name);
    RUNIT_REQUIRE(ctx, m > 0 && m <= (1u << 28), "%s: m=%u out of range", name, m);
    const uint32_t be = FMT == RUNIT_FMT_Q5_0 ? 32u : 256u;
    RUNIT_REQUIRE(ctx, k > 0 && k % be == 0 && k <= (1u << 24), "%s: k=%u is not a positive multiple of %u", name, k, be);
    RUNIT_REQUIRE(ctx, runit_aligned(w, 16) && runit_aligned(x, 16) && runit_aligned(y, 4) && (!res || runit_aligned(res, 4)),
                  "%s: weights and input 16-byte aligned, output 4-byte aligned", name);
    // the tile kernel needs a tile of 32 rows per warp: with fewer than two warps' worth of tiles per scheduler the first
    // kernel (one warp per row) keeps more of the machine busy
    if ((FMT != RUNIT_FMT_Q5_0 || k % 256 == 0) && ctx->tune.kquant_variant != 1) {
        q6t::Args t;
        const uint32_t tiles = (m + 31) / 32, sms = (uint32_t)ctx->sm_count, nbk = k / 256;
        // few tiles: shares of K go to different CTAs (2..16 shares, about one superblock per warp at least, fewer than 8 CTAs
        // per SM; measured on 3584 x 3584: 4 shares 15 -> 9 us, and on 18944 x 3584 two shares gain nothing)
        uint32_t split = 0;
        if (tiles < 8 * sms && ctx->d_kq && tiles <= 2048 && nbk >= 8) {
            split = 1;
            while (split < 16 && tiles * split * 2 < 8 * sms && 4 * split * 2 <= nbk + 2) split *= 2;
            if (ctx->tune.kquant_split > 0) split = (uint32_t)min(16, ctx->tune.kquant_split);
            if ((size_t)split * m * 4 > (1u << 20)) split = 0;
        }
        if (tiles < 8 * sms && split == 0 && ctx->tune.kquant_variant != 2) goto first_kernel;
        t.split = split;
        t.part = reinterpret_cast<float*>((uint8_t*)ctx->d_kq + 8192);
        t.tickets = reinterpret_cast<uint32_t*>(ctx->d_kq);
        t.w = (const uint8_t*)w;
        t.x = (const float*)x;
        t.y = (float*)y;
        t.res = (const float*)res;
        t.m = m;
        t.nb = k / 256;
        t.row_bytes = (k / 256) * (FMT == RUNIT_FMT_Q6K ? 210u : 176u);
        constexpr int smem = FMT == RUNIT_FMT_Q6K ? 4 * q6t::kS * q6t::kStage : FMT == RUNIT_FMT_Q5K ? 4 * q5t::kS * q5t::kStage : 4 * q50t::kS * q50t::kStage;
        auto kern = FMT == RUNIT_FMT_Q6K ? q6t::gemv_q6k_tile_kernel : FMT == RUNIT_FMT_Q5K ? q5t::gemv_q5k_tile_kernel : q50t::gemv_q5_0_tile_kernel;
        static bool configured[64] = {false};
        if (ctx->device >= 0 && ctx->device < 64 && !configured[ctx->device]) {
            RUNIT_CUDA_TRY(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            configured[ctx->device] = true;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = split ? dim3(tiles, split) : dim3((m + 127) / 128);
        cfg.blockDim = dim3(128);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = ctx->tune.pdl ? 1 : 0;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, kern, t);
        if (e != cudaSuccess) return runit_fail(ctx, RUNIT_ERR_LAUNCH, "launch of %s failed: %s", name, cudaGetErrorString(e));
        return runit_after_launch(ctx, name);
    }
first_kernel:
    Args a;
    a.w = (const uint8_t*)w;
    a.x = (const float*)x;
    a.y = (float*)y;
    a.res = (const float*)res;
    a.m = m;
    a.k = k;
    a.nb = k / 32;
    a.n_units = (k + 255) / 256;
    a.row_bytes = FMT == RUNIT_FMT_Q5_0 ? (k / 32) * 22 : (k / 256) * (uint32_t)KTraits<FMT>::UB;
    uint32_t grid = (m + kWarps - 1) / kWarps;
    const uint32_t cap = (uint32_t)ctx->sm_count * 8u;   // 64 warps per SM
    if (grid > cap) grid = cap;
    runit_launch_chain(ctx, gemv_kquant_kernel<FMT>, dim3(grid), dim3(kWarps * 32), a);
    return runit_after_launch(ctx, name);
}

}  // namespace kq
}  // namespace runit

using namespace runit;

extern "C" {

int32_t runit_gemv_q5_0_f32in_f32out(runit_ctx_t* ctx, const void* w, const void* x, void* y, uint32_t m, uint32_t k) {
    return kq::launch<RUNIT_FMT_Q5_0>(ctx, "gemv_q5_0_f32in_f32out", w, x, y, nullptr, m, k);
}
int32_t runit_gemv_q5_0_add_f32_f32in(runit_ctx_t* ctx, const void* w, const void* x, void* y, const void* r, uint32_t m, uint32_t k) {
    if (ctx) RUNIT_REQUIRE(ctx, r, "gemv_q5_0_add_f32_f32in: null residual");
    return kq::launch<RUNIT_FMT_Q5_0>(ctx, "gemv_q5_0_add_f32_f32in", w, x, y, r, m, k);
}
int32_t runit_gemv_q5k_f32in_f32out(runit_ctx_t* ctx, const void* w, const void* x, void* y, uint32_t m, uint32_t k) {
    return kq::launch<RUNIT_FMT_Q5K>(ctx, "gemv_q5k_f32in_f32out", w, x, y, nullptr, m, k);
}
int32_t runit_gemv_q5k_add_f32_f32in(runit_ctx_t* ctx, const void* w, const void* x, void* y, const void* r, uint32_t m, uint32_t k) {
    if (ctx) RUNIT_REQUIRE(ctx, r, "gemv_q5k_add_f32_f32in: null residual");
    return kq::launch<RUNIT_FMT_Q5K>(ctx, "gemv_q5k_add_f32_f32in", w, x, y, r, m, k);
}
int32_t runit_gemv_q6k_f32in_f32out(runit_ctx_t* ctx, const void* w, const void* x, void* y, uint32_t m, uint32_t k) {
    return kq::launch<RUNIT_FMT_Q6K>(ctx, "gemv_q6k_f32in_f32out", w, x, y, nullptr, m, k);
}
int32_t runit_gemv_q6k_add_f32_f32in(runit_ctx_t* ctx, const void* w, const void* x, void* y, const void* r, uint32_t m, uint32_t k) {
    if (ctx) RUNIT_REQUIRE(ctx, r, "gemv_q6k_add_f32_f32in: null residual");
    return kq::launch<RUNIT_FMT_Q6K>(ctx, "gemv_q6k_add_f32_f32in", w, x, y, r, m, k);
}

}  // extern "C"
