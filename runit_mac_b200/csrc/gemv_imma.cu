// Batched (2..8 activation rows) fused-dequant GEMV for the 4-bit formats on the integer tensor-core path.
//
// With 8 activation rows a weight takes part in 8 multiply-adds; on the CUDA cores that is 8 FMAs (or 6 dp4a) per
// weight and the kernel is arithmetic-bound far below the HBM roofline.  Here the 4-bit weights go into
// mma.sync.m16n8k32 (8-bit integer operands, one MMA = 16 rows x 8 activation rows x 32 K = exactly one Q4_0 block or
// one Q4_K sub-block), so the per-block scale is applied to an int32 tile in registers and nothing else has to be
// dequantised:
//   * a pre-pass quantises the activations once per call: per 256-element unit and activation row a scale
//     s = max|x| / 32767 and 16-bit integers q = rint(x / s), stored as a signed high byte and an unsigned low byte in the
//     order the MMA's B fragments want them, plus the integer block sums of q (for the "- min" / "- 8" terms).  Error of an
//     activation <= 2^-16 of its unit's maximum, far inside the 1e-3 bar; products and block sums are exact integers.
//     With one scale per unit Q4_K's 6-bit block scales stay integer factors (prepare_row<Q4_K>), and Q4_0's "- 8" is an
//     integer multiply-add.
//   * the weight nibbles are the MMA's A operand after one mask (low nibbles) or shift+mask (high nibbles; Q4_K feeds
//     the high nibbles unshifted, as 16 * nibble, and gives the low-nibble tiles 16 * scale instead).
//   * Q4_0, per k32 tile: 2 MMAs (high and low activation byte), v = 256 * hi + lo - 8 * sum(q), unit sum += d_w * v; per
//     unit acc += s * unit sum.
//   * Q4_K, per k32 tile: 2 MMAs and 8 integer multiply-adds (sc_j times the two limbs' tiles, summed over the unit's eight
//     blocks in int32); per unit: three more MMAs give sum_j m_j * (block sum of the activation integers) exactly, then one
//     conversion and acc += s * (d * V - dmin * M).  4.2 -> 2.8 thread instructions per weight.
//   * CTA = 4 consumer warps on the same K range (a fifth warp issues the copies), each with its own rows (RW = 16 or 32 per warp); the activation unit of a stage
//     is shared by the 4 warps, the CTA's weight box arrives by TMA (4 RW rows x 144 bytes), 3 stages (2..8 by a knob), mbarrier pipeline.
//     Few-tile shapes split K over a thread-block cluster and reduce through distributed shared memory.
// Reference formulas: Q4_0 value d * (nibble - 8), low nibble = element 2i, high = 2i + 1
// (crates/kernels/shaders/gemv_q4_0.metal:26-49); Q4_K value d*sc*q - dmin*m (crates/engine/src/forward.rs:1026-1057).
#include "gemv_common.cuh"
#include "runit_internal.h"
#include "tma.cuh"

namespace runit {
namespace imma {

constexpr int kUnitBytes = 4608;   // activations of one 256-K unit: 4096 bytes of limbs + 256 scales + 256 block sums
constexpr int kMaxStages = 8;       // ring depth is a launch argument (Args::stages, 2..8)

// ───────────────────────── activation pre-pass ─────────────────────────
// Slot of element e (0..31) of a block in the MMA's K order.  Q4_K: natural.  Q4_0: word t of the block holds
// elements 8t..8t+7 as (low, high) nibble pairs, low nibbles feed K slots 4t..4t+3, high nibbles 16+4t..16+4t+3.
template <int FMT>
__device__ __forceinline__ int k_slot(int e) {
    if (FMT == RUNIT_FMT_Q4K) return e;
    return 16 * (e & 1) + 4 * (e >> 3) + ((e & 7) >> 1);
}

// Activation row n of unit u by one warp (rows >= batch are written as zeros).  ONE scale per unit and activation row:
// s = max|x| over the 256 elements / 32767, q = rint(x / s) as a signed high byte and an unsigned low byte in the order
// the MMA's B fragments want them.  Q4_0 (this template): behind the limbs
//   [4096, 4128)   s of the 8 activation rows (f32)
//   [4128, 4384)   block sums of q as int32, [block][activation row] (for the "- 8" of the weights: exact integers)
template <int FMT>
__device__ __forceinline__ void prepare_row(const float* __restrict__ x, uint8_t* __restrict__ dst, uint32_t k, uint32_t batch, uint32_t u,
                                            uint32_t n, uint32_t lane) {
    float v[8];
    float amax = 0.f;
    bool bad = false;
#pragma unroll
    for (int bt = 0; bt < 8; bt++) {
        v[bt] = n < batch ? x[(size_t)n * k + (size_t)u * 256 + bt * 32 + lane] : 0.f;
        amax = fmaxf(amax, fabsf(v[bt]));
        bad |= !(fabsf(v[bt]) <= 3.0e38f);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    // an Inf or a NaN in the unit gives a NaN scale: every row's result of that activation row becomes NaN, as a
    // non-finite activation does (to +-Inf or NaN) in the reference's f32 multiply-add chain
    bad = __any_sync(0xffffffffu, bad);
    const float s = bad ? __uint_as_float(0x7FC00000u) : amax * (1.0f / 32767.0f);
    const float inv = (amax > 0.f && !bad) ? 32767.0f / amax : 0.f;
    const int slot = k_slot<FMT>((int)lane);
#pragma unroll
    for (int bt = 0; bt < 8; bt++) {
        const int q = __float2int_rn(v[bt] * inv);
        int qs = q;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) qs += __shfl_xor_sync(0xffffffffu, qs, o);
        uint8_t* p = dst + ((bt * 8 + n) * 4 + ((slot & 15) >> 2)) * 16 + (slot >> 4) * 4 + (slot & 3);
        p[0] = (uint8_t)(q >> 8);      // signed high byte
        p[8] = (uint8_t)(q & 255);     // unsigned low byte
        if (lane == 0) reinterpret_cast<int*>(dst + 4128)[bt * 8 + n] = qs;
    }
    if (lane == 0) reinterpret_cast<float*>(dst + 4096)[n] = s;
}

// Q4_K: ONE scale per unit and activation row (s = max|x| over the 256 elements / 32767, q = rint(x / s) as a signed high
// byte and an unsigned low byte, in the same fragment order).  With a common scale the weights' 6-bit block scales stay
// integers: the kernel adds sc_j * (q . xq) over the unit's eight blocks in int32 and converts once per unit.  The block
// sums of xq (for the "- dmin * m_j" term) are kept exactly as three bytes each (signed high, two unsigned), laid out as
// the B fragments of one more MMA per limb whose A operand is the row's eight 6-bit minimums:
//   [4096, 4128)        s of the 8 activation rows (f32)
//   [4128 + 64 l, ...)  limb l (0 = bits 16.., 1 = bits 8..15, 2 = bits 0..7) of the block sums: [activation row][8 bytes in
//                       the order blocks 0, 2, 4, 6, 1, 3, 5, 7] (the order of the unpacked minimums ml | mh)
template <>
__device__ __forceinline__ void prepare_row<RUNIT_FMT_Q4K>(const float* __restrict__ x, uint8_t* __restrict__ dst, uint32_t k, uint32_t batch,
                                                           uint32_t u, uint32_t n, uint32_t lane) {
    float v[8];
    float amax = 0.f;
    bool bad = false;
#pragma unroll
    for (int bt = 0; bt < 8; bt++) {
        v[bt] = n < batch ? x[(size_t)n * k + (size_t)u * 256 + bt * 32 + lane] : 0.f;
        amax = fmaxf(amax, fabsf(v[bt]));
        bad |= !(fabsf(v[bt]) <= 3.0e38f);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    // an Inf or a NaN in the unit gives a NaN scale: every row's result of that activation row becomes NaN, as a
    // non-finite activation does (to +-Inf or NaN) in the reference's f32 multiply-add chain
    bad = __any_sync(0xffffffffu, bad);
    const float s = bad ? __uint_as_float(0x7FC00000u) : amax * (1.0f / 32767.0f);
    const float inv = (amax > 0.f && !bad) ? 32767.0f / amax : 0.f;
#pragma unroll
    for (int bt = 0; bt < 8; bt++) {
        const int q = __float2int_rn(v[bt] * inv);
        int qs = q;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) qs += __shfl_xor_sync(0xffffffffu, qs, o);
        uint8_t* p = dst + ((bt * 8 + n) * 4 + ((lane & 15) >> 2)) * 16 + (lane >> 4) * 4 + (lane & 3);
        p[0] = (uint8_t)(q >> 8);      // signed high byte
        p[8] = (uint8_t)(q & 255);     // unsigned low byte
        if (lane == 0) {
            uint8_t* sp = dst + 4128 + n * 8 + (bt >> 1) + 4 * (bt & 1);
            sp[0] = (uint8_t)(qs >> 16);
            sp[64] = (uint8_t)((qs >> 8) & 255);
            sp[128] = (uint8_t)(qs & 255);
        }
    }
    if (lane == 0) reinterpret_cast<float*>(dst + 4096)[n] = s;
}

// One CTA per unit, one warp per activation row: the pre-pass as a launch of its own (launches too small to carry it).
template <int FMT>
__global__ void __launch_bounds__(256) xq_prepare_kernel(const float* __restrict__ x, uint8_t* __restrict__ xq, uint32_t k,
                                                          uint32_t batch) {
    grid_launch_dependents();   // the consumer may start fetching its weights; it waits for this grid before reading xq
    prepare_row<FMT>(x, xq + (size_t)blockIdx.x * kUnitBytes, k, batch, blockIdx.x, threadIdx.x >> 5, threadIdx.x & 31);
}

// ───────────────────────── main kernel ─────────────────────────
// Up to three matrices that share the activations (q | k | v, gate | up) ride one launch: segment i owns the row tiles
// [tile0[i], tile0[i+1]) and has its own tensor map, row count, output and residual.
struct Args {
    const uint8_t* xq;
    float* y[3];
    const float* res[3];
    uint32_t m[3], tile0[3];
    uint32_t nseg, units, batch, csplit, stages;
    int32_t* status;
    // The pre-pass inside this launch (ctl != nullptr): CTA u < units quantises unit u of x first and publishes the number
    // of this launch in ctl[64 + u]; a CTA asks for a unit's quantised activations only once its word shows that number.
    // ctl[0] = number of the last finished launch (advanced by the CTA that leaves last), ctl[1] = exit tickets.
    const float* x;
    uint32_t k;
    uint32_t* ctl;
};
struct Maps {
    CUtensorMap m[3];
};

__device__ __forceinline__ void mma_u8s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}
__device__ __forceinline__ void mma_u8u8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}
// Shared-memory reads are plain C++ loads through generic pointers: the compiler may reorder them among themselves and
// around the MMAs (instruction-level parallelism inside a warp), while the "memory" clobber of the barrier wait keeps
// them behind the wait.
__device__ __forceinline__ uint32_t lds32(const uint8_t* p) { return *reinterpret_cast<const uint32_t*>(p); }

// One k32 tile of the Q4_K path: the two limbs' int32 tiles times the rows' integer block scales, into the unit's sums.
__device__ __forceinline__ void tile_mma_int(int (&ih)[4], int (&il)[4], const uint32_t (&a)[4], const uint8_t* xaddr, int sc0, int sc1) {
    const uint4 bf = *reinterpret_cast<const uint4*>(xaddr);
    int ch[4], cl[4];
    mma_u8s8(ch, a, bf.x, bf.y);
    mma_u8u8(cl, a, bf.z, bf.w);
    ih[0] += sc0 * ch[0]; ih[1] += sc0 * ch[1]; ih[2] += sc1 * ch[2]; ih[3] += sc1 * ch[3];
    il[0] += sc0 * cl[0]; il[1] += sc0 * cl[1]; il[2] += sc1 * cl[2]; il[3] += sc1 * cl[3];
}

template <int FMT, int RW>
__global__ void __launch_bounds__(160) gemv_imma_kernel(const __grid_constant__ Maps wmaps, const Args a) {
    constexpr int WBYTES = RW * 144;                       // one warp's weight box
    constexpr int STAGE = kUnitBytes + 4 * WBYTES;
    constexpr int MT = RW / 16;                            // m16 tiles per warp
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * kMaxStages];
    __shared__ float red[4 * RW][8];
    const uint32_t base = (smem_u32(smem_raw) + 127u) & ~127u;
    const uint8_t* base_p = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const uint32_t crank = a.csplit > 1 ? cluster_ctarank() : 0;
    const uint32_t tile = blockIdx.x / a.csplit;
    int si = 0;
#pragma unroll
    for (int i = 1; i < 3; i++)
        if (i < (int)a.nseg && tile >= a.tile0[i]) si = i;
    const CUtensorMap* wmap = &wmaps.m[si];
    const uint32_t row_tile0 = (tile - a.tile0[si]) * (4 * RW);
    const uint32_t seg_m = a.m[si];
    float* const seg_y = a.y[si];
    const float* const seg_res = a.res[si];
    const uint32_t u_begin = (uint32_t)(((uint64_t)a.units * crank) / a.csplit), u_end = (uint32_t)(((uint64_t)a.units * (crank + 1)) / a.csplit);
    const uint32_t nu = u_end - u_begin;
    const uint32_t kStages = a.stages;
    const uint32_t bar_full = smem_u32(&bars[0]), bar_empty = smem_u32(&bars[kMaxStages]);
    if (tid == 0) {
        for (uint32_t s = 0; s < kStages; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 4);
        }
        fence_mbar_init();
    }
    __syncthreads();
    bool timed_out = false;
    auto issue_w = [&](uint32_t i) {   // weight boxes of the i-th unit of this CTA (thread 0 only)
        const uint32_t s = i % kStages, u = u_begin + i;
        const uint32_t sb = base + s * STAGE;
        mbar_expect_tx(bar_full + 8 * s, STAGE);
        tma_load_2d(sb + kUnitBytes, wmap, (int32_t)(u * 144), (int32_t)row_tile0, bar_full + 8 * s);   // one box: the four warps' rows
    };
    uint32_t launch_no = 0;
    auto issue_x = [&](uint32_t i) {   // its quantised activations
        const uint32_t s = i % kStages, u = u_begin + i;
        if (a.ctl != nullptr) {
            // wait (bounded) until the CTA that quantises unit u has published this launch's number
            const long long t0 = clock64();
            while (true) {
                uint32_t v;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(a.ctl + 64 + u) : "memory");
                if (v == launch_no) break;
                if (clock64() - t0 > (1ll << 28)) { timed_out = true; break; }
                __nanosleep(40);
            }
            fence_proxy_async();       // the bulk load below reads what another CTA stored with ordinary stores
        }
        bulk_load_1d(base + s * STAGE, a.xq + (size_t)u * kUnitBytes, kUnitBytes, bar_full + 8 * s);
    };
    auto issue = [&](uint32_t i) { issue_w(i); issue_x(i); };
    // The weights do not depend on the activation pre-pass: their first loads go out before the dependency wait
    // (programmatic dependent launch), the activations after it.
    const bool producer = tid == 128;      // lane 0 of warp 4 issues every copy; warps 0..3 consume
    if (producer)
        for (uint32_t i = 0; i < kStages && i < nu; i++) issue_w(i);
    grid_dependency_wait();
    if (a.ctl != nullptr) {
        // the launch number is read after the wait: the launch before this one has advanced it by then
        launch_no = *reinterpret_cast<volatile uint32_t*>(a.ctl) + 1u;
        if (blockIdx.x < a.units) {
            uint8_t* dst = const_cast<uint8_t*>(a.xq) + (size_t)blockIdx.x * kUnitBytes;
            if (warp < 4) {
                prepare_row<FMT>(a.x, dst, a.k, a.batch, blockIdx.x, warp, lane);
                prepare_row<FMT>(a.x, dst, a.k, a.batch, blockIdx.x, warp + 4, lane);
            }
            __threadfence();
            __syncthreads();
            if (tid == 0) atomicExch(&a.ctl[64 + blockIdx.x], launch_no);
        }
    }
    if (producer) {
        for (uint32_t i = 0; i < kStages && i < nu; i++) issue_x(i);
        // the ring's later rounds: stage j % kStages is free once all four warps have released unit j - kStages
        for (uint32_t j = kStages; j < nu; j++) {
            if (!mbar_wait(bar_empty + 8 * (j % kStages), ((j / kStages) - 1) & 1)) { timed_out = true; break; }
            issue(j);
        }
    }

    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[mt][i] = 0.f;

    for (uint32_t i = 0; i < (warp < 4 ? nu : 0u); i++) {
        const uint32_t s = i % kStages;
        if (!mbar_wait(bar_full + 8 * s, (i / kStages) & 1)) { timed_out = true; break; }
        const uint8_t* sb = base_p + s * STAGE;
        const uint8_t* wb = sb + kUnitBytes + warp * WBYTES;
        const uint8_t* xb = sb + (g * 4 + t) * 16;       // + bt * 512: limbs of block bt for column g, K quarter t
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            const uint8_t* r0 = wb + (mt * 16 + g) * 144;
            const uint8_t* r1 = r0 + 8 * 144;
            if (FMT == RUNIT_FMT_Q4K) {
                const uint4 h0 = *reinterpret_cast<const uint4*>(r0), h1 = *reinterpret_cast<const uint4*>(r1);
                const Q4KScales s0 = q4k_unpack_scales(h0.y, h0.z, h0.w), s1 = q4k_unpack_scales(h1.y, h1.z, h1.w);
                // sum over the unit's blocks of sc_j * (nibbles . activation limb), 16-fold: low-nibble tiles take 16 * sc_j,
                // high-nibble tiles are fed as (w & 0xF0F0F0F0) = 16 * nibble.  |ih| <= 16 * 8 * 63 * 32 * 15 * 128 < 2^29,
                // |il| <= 16 * 8 * 63 * 32 * 15 * 255 < 2^30
                int ih[4] = {0, 0, 0, 0}, il[4] = {0, 0, 0, 0};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const uint32_t w00 = lds32(r0 + 16 + 32 * j + 4 * t), w01 = lds32(r0 + 32 + 32 * j + 4 * t);
                    const uint32_t w10 = lds32(r1 + 16 + 32 * j + 4 * t), w11 = lds32(r1 + 32 + 32 * j + 4 * t);
                    const uint32_t alo[4] = {w00 & 0x0F0F0F0Fu, w10 & 0x0F0F0F0Fu, w01 & 0x0F0F0F0Fu, w11 & 0x0F0F0F0Fu};
                    const uint32_t ahi[4] = {w00 & 0xF0F0F0F0u, w10 & 0xF0F0F0F0u, w01 & 0xF0F0F0F0u, w11 & 0xF0F0F0F0u};
                    // low nibbles: sub-block j (elements 64j..64j+31); high nibbles: sub-block j+4 (64j+32..64j+63)
                    tile_mma_int(ih, il, alo, xb + (2 * j) * 512, (int)(__byte_perm(s0.sl, 0u, 0x4440u + j) << 4), (int)(__byte_perm(s1.sl, 0u, 0x4440u + j) << 4));
                    tile_mma_int(ih, il, ahi, xb + (2 * j + 1) * 512, (int)__byte_perm(s0.sh, 0u, 0x4440u + j), (int)__byte_perm(s1.sh, 0u, 0x4440u + j));
                }
                // sum over the blocks of m_j * (block sum of the activation integers): one MMA per limb of the sums, A = the
                // rows' minimums in K slots 0..7 (lanes t = 0, 1), zeros elsewhere
                const uint32_t am[4] = {t == 0 ? s0.ml : t == 1 ? s0.mh : 0u, t == 0 ? s1.ml : t == 1 ? s1.mh : 0u, 0u, 0u};
                const uint8_t* sl = sb + 4128 + g * 8 + (t & 1) * 4;
                const uint32_t b_h = t < 2 ? lds32(sl) : 0u, b_m = t < 2 ? lds32(sl + 64) : 0u, b_l = t < 2 ? lds32(sl + 128) : 0u;
                int mh[4], mm[4], ml[4];
                mma_u8s8(mh, am, b_h, 0u);
                mma_u8u8(mm, am, b_m, 0u);
                mma_u8u8(ml, am, b_l, 0u);
                const float2 xs = *reinterpret_cast<const float2*>(sb + 4096 + 8 * t);
                const float d0 = half_bits_to_float(h0.x) * 0.0625f, n0 = half_bits_to_float(h0.x >> 16);
                const float d1 = half_bits_to_float(h1.x) * 0.0625f, n1 = half_bits_to_float(h1.x >> 16);
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float vq = fmaf((float)ih[e], 256.f, (float)il[e]);
                    const float vm = (float)(mh[e] * 65536 + mm[e] * 256 + ml[e]);      // |.| <= 8 * 63 * 32 * 32767 < 2^29
                    const float dd = e < 2 ? d0 : d1, nn = e < 2 ? n0 : n1;
                    acc[mt][e] = fmaf((e & 1) ? xs.y : xs.x, fmaf(dd, vq, -nn * vm), acc[mt][e]);
                }
            } else {
                float au[4] = {0.f, 0.f, 0.f, 0.f};      // the unit's sums, before the activation scale
#pragma unroll
                for (int b = 0; b < 8; b++) {
                    // block b of the unit sits at byte 18b of the row: f16 scale, then 16 bytes of nibbles; for even b the
                    // nibble words straddle aligned words by two bytes
                    uint32_t w0, w1, sc0, sc1;
                    if ((b & 1) == 0) {
                        const uint8_t* p0 = r0 + 18 * b + 4 * t;
                        const uint8_t* p1 = r1 + 18 * b + 4 * t;
                        w0 = __funnelshift_r(lds32(p0), lds32(p0 + 4), 16);
                        w1 = __funnelshift_r(lds32(p1), lds32(p1 + 4), 16);
                        sc0 = lds32(r0 + 18 * b) & 0xFFFFu;
                        sc1 = lds32(r1 + 18 * b) & 0xFFFFu;
                    } else {
                        w0 = lds32(r0 + 18 * b + 2 + 4 * t);
                        w1 = lds32(r1 + 18 * b + 2 + 4 * t);
                        sc0 = lds32(r0 + 18 * b - 2) >> 16;
                        sc1 = lds32(r1 + 18 * b - 2) >> 16;
                    }
                    const uint32_t aa[4] = {w0 & 0x0F0F0F0Fu, w1 & 0x0F0F0F0Fu, (w0 >> 4) & 0x0F0F0F0Fu, (w1 >> 4) & 0x0F0F0F0Fu};
                    const float d0 = half_bits_to_float(sc0), d1 = half_bits_to_float(sc1);
                    const uint4 bf = *reinterpret_cast<const uint4*>(xb + b * 512);
                    const int2 sq = *reinterpret_cast<const int2*>(sb + 4128 + b * 32 + 8 * t);   // block sums of columns 2t, 2t+1
                    int ch[4], cl[4];
                    mma_u8s8(ch, aa, bf.x, bf.y);
                    mma_u8u8(cl, aa, bf.z, bf.w);
                    // sum (nibble - 8) * q over the block, exact: |.| <= 32 * 15 * 32767 + 8 * 32 * 32767 < 2^25
                    const int v0 = ch[0] * 256 + cl[0] - 8 * sq.x, v1 = ch[1] * 256 + cl[1] - 8 * sq.y;
                    const int v2 = ch[2] * 256 + cl[2] - 8 * sq.x, v3 = ch[3] * 256 + cl[3] - 8 * sq.y;
                    au[0] = fmaf((float)v0, d0, au[0]);
                    au[1] = fmaf((float)v1, d0, au[1]);
                    au[2] = fmaf((float)v2, d1, au[2]);
                    au[3] = fmaf((float)v3, d1, au[3]);
                }
                const float2 xs = *reinterpret_cast<const float2*>(sb + 4096 + 8 * t);
                acc[mt][0] = fmaf(xs.x, au[0], acc[mt][0]);
                acc[mt][1] = fmaf(xs.y, au[1], acc[mt][1]);
                acc[mt][2] = fmaf(xs.x, au[2], acc[mt][2]);
                acc[mt][3] = fmaf(xs.y, au[3], acc[mt][3]);
            }
        }
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_empty + 8 * s) : "memory");
    }

    // partial sums of this CTA: rows (warp * RW + mt * 16 + g, + 8), columns 2t, 2t+1
#pragma unroll
    for (int mt = 0; mt < (warp < 4 ? MT : 0); mt++) {
        red[warp * RW + mt * 16 + g][2 * t] = acc[mt][0];
        red[warp * RW + mt * 16 + g][2 * t + 1] = acc[mt][1];
        red[warp * RW + mt * 16 + g + 8][2 * t] = acc[mt][2];
        red[warp * RW + mt * 16 + g + 8][2 * t + 1] = acc[mt][3];
    }
    if (a.csplit > 1) cluster_sync();
    else __syncthreads();
    if (crank == 0 && tid < 128) {
        for (uint32_t e = tid; e < 4 * RW * 8; e += 128) {
            const uint32_t r = e % (4 * RW), c = e / (4 * RW);      // consecutive threads -> consecutive rows of one column
            float v = red[r][c];
            for (uint32_t p = 1; p < a.csplit; p++) v += ld_cluster_f32(&red[r][c], p);
            const uint32_t row = row_tile0 + r;
            if (row < seg_m && c < a.batch) {
                const size_t o = (size_t)c * seg_m + row;
                if (seg_res) v += seg_res[o];
                seg_y[o] = v;
            }
        }
    }
    if (a.csplit > 1) cluster_sync();   // keep every CTA's partial sums alive until rank 0 has read them
    if (a.ctl != nullptr && tid == 0) {
        __threadfence();
        if (atomicAdd(&a.ctl[1], 1u) == gridDim.x - 1) {   // every CTA has consumed its units: the next launch may number itself
            a.ctl[1] = 0;
            __threadfence();
            *reinterpret_cast<volatile uint32_t*>(a.ctl) = launch_no;
        }
    }
    if (timed_out && a.status) atomicExch(a.status, 1);
}

template <int FMT, int RW>
static int32_t launch(runit_ctx* ctx, const Maps& map, const Args& a, uint32_t tiles) {
    const int smem = (int)a.stages * (kUnitBytes + 4 * RW * 144) + 128;
    auto kern = gemv_imma_kernel<FMT, RW>;
    static bool configured[16] = {false};
    if (ctx->device < 16 && !configured[ctx->device]) {
        RUNIT_CUDA_TRY(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxStages * (kUnitBytes + 4 * RW * 144) + 128 > 227 * 1024 ? 227 * 1024 : kMaxStages * (kUnitBytes + 4 * RW * 144) + 128));
        configured[ctx->device] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles * a.csplit);
    cfg.blockDim = dim3(160);      // four consumer warps + the producer warp
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    na++;
    if (a.csplit > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = a.csplit;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        na++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, map, a);
    if (e != cudaSuccess) return runit_fail(ctx, RUNIT_ERR_LAUNCH, "launch of gemv_batched (integer MMA) failed: %s", cudaGetErrorString(e));
    return runit_after_launch(ctx, "gemv_batched_imma");
}

}  // namespace imma

// True if the integer tensor-core path serves this call (4-bit format, whole 256-K units, 16-byte aligned rows,
// the activations fit the context's staging area).
bool gemv_imma_applies(const runit_ctx* ctx, int fmt, uint32_t k, uint32_t batch) {
    if (fmt != RUNIT_FMT_Q4_0 && fmt != RUNIT_FMT_Q4K) return false;
    if (batch < 2 || batch > 8 || k % 256 != 0 || ctx->tune.gemv_math == 1 || !ctx->encode_tiled || !ctx->d_xq) return false;
    return (size_t)(k / 256) * imma::kUnitBytes <= ctx->xq_bytes;
}

// n_mats (1..3) matrices over the same activations in one launch; the activations are quantised once.
int32_t gemv_imma_multi(runit_ctx* ctx, int fmt, uint32_t n_mats, const void* const* w, const float* x, float* const* y,
                        const float* const* res, const uint32_t* m, uint32_t k, uint32_t batch) {
    using namespace imma;
    const uint32_t units = k / 256;
    int32_t st = RUNIT_OK;
    // rows per warp: 32 when that still gives every SM two CTAs, else 16
    const uint32_t sms = (uint32_t)ctx->sm_count;
    uint32_t tiles32 = 0, tiles16 = 0;
    for (uint32_t i = 0; i < n_mats; i++) {
        tiles32 += (m[i] + 127) / 128;
        tiles16 += (m[i] + 63) / 64;
    }
    const bool rw32 = ctx->tune.imma_rw ? ctx->tune.imma_rw == 32 : tiles32 >= 2 * sms;
    const uint32_t tiles = rw32 ? tiles32 : tiles16;
    uint32_t csplit = 1;
    // measured (rows per warp x cluster size x ring depth on six shapes): split K while the grid stays within two CTAs per SM
    while (csplit < 8 && tiles * csplit * 2 <= 2 * sms && units / (csplit * 2) >= 3) csplit *= 2;
    if (ctx->tune.imma_csplit > 0 && ctx->tune.imma_csplit <= 8 && units >= (uint32_t)ctx->tune.imma_csplit) csplit = (uint32_t)ctx->tune.imma_csplit;
    Args a{};
    Maps maps{};
    a.xq = (const uint8_t*)ctx->d_xq;
    a.nseg = n_mats;
    uint32_t t0 = 0;
    for (uint32_t i = 0; i < 3; i++) {
        const uint32_t s = i < n_mats ? i : 0;      // unused entries repeat segment 0 (never selected)
        a.y[i] = y[s];
        a.res[i] = res ? res[s] : nullptr;
        a.m[i] = m[s];
        a.tile0[i] = i < n_mats ? t0 : 0xFFFFFFFFu;
        if (i < n_mats) {
            st = runit_get_tmap(ctx, w[i], m[i], (uint64_t)units * 144, rw32 ? 128 : 64, 144, &maps.m[i]);
            if (st != RUNIT_OK) return st;
            t0 += rw32 ? (m[i] + 127) / 128 : (m[i] + 63) / 64;
        } else {
            maps.m[i] = maps.m[0];
        }
    }
    a.units = units;
    a.batch = batch;
    a.csplit = csplit;
    {   // ring depth: as deep as shared memory allows with every CTA of the grid resident (one wave), at most half the
        // CTA's units and 6, at least 3; a grid of several waves keeps 3 (more CTAs per SM pay more than a deeper ring)
        const uint32_t stage_bytes = imma::kUnitBytes + 4 * (rw32 ? 32 : 16) * 144, grid = tiles * csplit;
        const uint32_t want_per_sm = (grid + sms - 1) / sms, fit3 = (220u * 1024) / (3 * stage_bytes);
        uint32_t st3 = 3;
        if (want_per_sm <= fit3) st3 = (220u * 1024) / (want_per_sm * stage_bytes);
        const uint32_t nu = units / csplit;
        st3 = st3 < nu / 2 ? st3 : nu / 2;
        a.stages = st3 < 3 ? 3u : (st3 > 6 ? 6u : st3);
        if (ctx->tune.imma_stages >= 2 && ctx->tune.imma_stages <= (rw32 ? 6 : 8)) a.stages = (uint32_t)ctx->tune.imma_stages;
    }
    a.status = ctx->d_status;
    // Opt-in (tuning key imma_fold): the activation pre-pass rides inside the launch when the grid has a CTA per unit (all
    // of them resident in the first wave, so a CTA that waits for a unit never keeps its producer off the machine) and the
    // flag table covers the units.  Measured slower than the pre-pass as a small launch of its own (the quantisation and
    // the flag round trip then sit at the head of every CTA), so the default is the separate launch.
    const bool fold = ctx->d_xq_ctl && tiles * csplit >= units && units <= 960 && tiles * csplit >= 2 * units && ctx->tune.imma_fold != 0;
    if (fold) {
        a.x = x;
        a.k = k;
        a.ctl = ctx->d_xq_ctl;
    } else {
        if (fmt == RUNIT_FMT_Q4K) xq_prepare_kernel<RUNIT_FMT_Q4K><<<units, 256, 0, ctx->stream>>>(x, (uint8_t*)ctx->d_xq, k, batch);
        else xq_prepare_kernel<RUNIT_FMT_Q4_0><<<units, 256, 0, ctx->stream>>>(x, (uint8_t*)ctx->d_xq, k, batch);
        if ((st = runit_after_launch(ctx, "gemv_batched_quantise_x")) != RUNIT_OK) return st;
    }
    if (fmt == RUNIT_FMT_Q4K) return rw32 ? launch<RUNIT_FMT_Q4K, 32>(ctx, maps, a, tiles) : launch<RUNIT_FMT_Q4K, 16>(ctx, maps, a, tiles);
    return rw32 ? launch<RUNIT_FMT_Q4_0, 32>(ctx, maps, a, tiles) : launch<RUNIT_FMT_Q4_0, 16>(ctx, maps, a, tiles);
}

int32_t gemv_imma(runit_ctx* ctx, int fmt, const void* w, const float* x, float* y, const float* res, uint32_t m, uint32_t k,
                  uint32_t batch) {
    const void* ws[1] = {w};
    float* ys[1] = {y};
    const float* rs[1] = {res};
    return gemv_imma_multi(ctx, fmt, 1, ws, x, ys, rs, &m, k, batch);
}

}  // namespace runit
