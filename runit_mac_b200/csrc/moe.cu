// OLMoE-style mixture-of-experts block on the device, without the reference's per-layer host sync.
//
// Reference sequence (crates/engine/src/forward.rs:1644-1679): router GEMV -> flush -> CPU
// softmax/top-k (forward.rs:2420-2448) -> per selected expert: gate GEMV, up GEMV, silu*up, down
// GEMV, scale-accumulate -> residual add.  Here: router GEMV, device softmax/top-k, ONE grouped
// launch for gate+up+SiLU of all (token, expert) slots, ONE grouped launch for down, and a combine
// kernel that adds the weighted expert outputs in routing order (deterministic) plus the residual.
// All intermediates are f32.
#include "decode_ops.cuh"
#include "gemv_common.cuh"
#include "runit_internal.h"
#include "tma.cuh"

namespace runit {

// logits[t][e] = W[e][:] . x[t][:]   (f32 router weights).  One warp per expert; the weight row
// stays in registers while the warp walks the tokens.
template <int KPL>   // floats of the row per lane (K = 32*KPL)
__global__ void __launch_bounds__(256) router_f32_kernel(const float* __restrict__ w, const float* __restrict__ x,
                                                          float* __restrict__ logits, uint32_t E, uint32_t K, uint32_t T) {
    grid_dependency_wait();      // inputs come from the previous kernel of the chain
    grid_launch_dependents();
    const uint32_t e = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (e >= E) return;
    float wr[KPL];
    const float4* wrow = reinterpret_cast<const float4*>(w + (size_t)e * K);
#pragma unroll
    for (int i = 0; i < KPL / 4; i++) {
        const float4 v = wrow[lane + 32 * i];
        wr[4 * i] = v.x; wr[4 * i + 1] = v.y; wr[4 * i + 2] = v.z; wr[4 * i + 3] = v.w;
    }
    for (uint32_t t = blockIdx.y; t < T; t += gridDim.y) {
        const float4* xr = reinterpret_cast<const float4*>(x + (size_t)t * K);
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
        for (int i = 0; i < KPL / 4; i++) {
            const float4 v = xr[lane + 32 * i];
            a0 = fmaf(wr[4 * i], v.x, a0); a1 = fmaf(wr[4 * i + 1], v.y, a1);
            a2 = fmaf(wr[4 * i + 2], v.z, a2); a3 = fmaf(wr[4 * i + 3], v.w, a3);
        }
        float acc = (a0 + a1) + (a2 + a3);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) logits[(size_t)t * E + e] = acc;
    }
}

// The same product for many tokens: a tiled f32 GEMM (CTA: TM tokens x 64 experts, thread: TM/16 x 4, K in chunks of 32
// through shared memory; TM = 32 or 16 when larger token tiles would leave SMs idle).  Every logit is one fused multiply-add chain
// over k in ascending order, whatever the tile.
template <int TM>
__global__ void __launch_bounds__(256) router_f32_tiled_kernel(const float* __restrict__ w, const float* __restrict__ x,
                                                                float* __restrict__ logits, uint32_t E, uint32_t K, uint32_t T) {
    grid_dependency_wait();      // inputs come from the previous kernel of the chain
    grid_launch_dependents();
    constexpr int RT = TM / 16;                  // token rows per thread
    __shared__ __align__(16) float xs[32][TM + 4];   // [k][token]
    __shared__ __align__(16) float ws[32][68];       // [k][expert]
    const uint32_t tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const uint32_t e0 = blockIdx.x * 64, t0 = blockIdx.y * TM;
    float acc[RT][4];
#pragma unroll
    for (int i = 0; i < RT; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
    for (uint32_t kc = 0; kc < K; kc += 32) {
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const uint32_t i = tid + 256 * j, row = i >> 3, kq = i & 7;
            float4 wv = make_float4(0.f, 0.f, 0.f, 0.f);
            if (e0 + row < E) wv = *reinterpret_cast<const float4*>(w + (size_t)(e0 + row) * K + kc + kq * 4);
            ws[kq * 4][row] = wv.x; ws[kq * 4 + 1][row] = wv.y; ws[kq * 4 + 2][row] = wv.z; ws[kq * 4 + 3][row] = wv.w;
            if (row < TM) {
                float4 xv = make_float4(0.f, 0.f, 0.f, 0.f);
                if (t0 + row < T) xv = *reinterpret_cast<const float4*>(x + (size_t)(t0 + row) * K + kc + kq * 4);
                xs[kq * 4][row] = xv.x; xs[kq * 4 + 1][row] = xv.y; xs[kq * 4 + 2][row] = xv.z; xs[kq * 4 + 3][row] = xv.w;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 32; kk++) {
            float av[RT];
            if constexpr (RT == 4) {
                const float4 a = *reinterpret_cast<const float4*>(&xs[kk][ty * 4]);
                av[0] = a.x; av[1] = a.y; av[2] = a.z; av[3] = a.w;
            } else if constexpr (RT == 2) {
                const float2 a = *reinterpret_cast<const float2*>(&xs[kk][ty * 2]);
                av[0] = a.x; av[1] = a.y;
            } else {
                av[0] = xs[kk][ty];
            }
            const float4 b = *reinterpret_cast<const float4*>(&ws[kk][tx * 4]);
            const float bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < RT; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(bv[j], av[i], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < RT; i++) {
        const uint32_t t = t0 + ty * RT + i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t e = e0 + tx * 4 + j;
            if (e < E) logits[(size_t)t * E + e] = acc[i][j];
        }
    }
}

// Many tokens, few experts: the same product with K split over the eight warps of a CTA.  CTA = 16 tokens x 64 experts;
// warp w multiplies the whole tile over its eighth of K (chunks of 32 staged by cp.async in its own two shared-memory
// buffers, rows as in memory), a lane keeps 4 tokens x 8 experts (tokens ty + 4 i, experts tx + 8 j: consecutive rows per load, no bank
// conflicts) and reads 12 x 128 bits per 128 multiply-adds; the eight partial tiles are added in warp order.  Every logit is
// eight fused multiply-add chains over ascending k, added in order: the same bits whatever T is.  K must be a multiple of 256.
constexpr int kRsPitch = 36;                                    // floats per staged row (32 + 4)
constexpr int kRsWarpFloats = (16 + 64) * kRsPitch;             // one warp's slice
__global__ void __launch_bounds__(256) router_f32_splitk_kernel(const float* __restrict__ w, const float* __restrict__ x,
                                                                 float* __restrict__ logits, uint32_t E, uint32_t K, uint32_t T) {
    grid_dependency_wait();      // inputs come from the previous kernel of the chain
    grid_launch_dependents();
    extern __shared__ __align__(16) float rs_smem[];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, ty = lane >> 3, tx = lane & 7;
    const uint32_t e0 = blockIdx.x * 64, t0 = blockIdx.y * 16;
    float* xs = rs_smem + warp * (2 * kRsWarpFloats);            // two buffers of [16][36] + [64][36]
    float* ws = xs + 16 * kRsPitch;
    float acc[4][8];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = 0.f;
    const uint32_t kw = K / 8, k_begin = warp * kw, n_chunks = kw / 32;
    const uint32_t lrow = lane >> 3, lkq = lane & 7;             // a copy instruction covers 4 rows x 32 k
    // two buffers per warp: chunk c + 1 is copied (cp.async, 16 bytes per lane and row group) while chunk c is multiplied;
    // rows past T or E are copied from row 0 of the same matrix (never stored)
    auto stage = [&](uint32_t c) {
        if (c < n_chunks) {
            const uint32_t kc = k_begin + 32 * c;
            const uint32_t xb = smem_u32(xs + (c & 1) * kRsWarpFloats), wb = smem_u32(ws + (c & 1) * kRsWarpFloats);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint32_t row = lrow + 4 * j, tr = t0 + row < T ? t0 + row : 0u;
                cp_async16(xb + (row * kRsPitch + 4 * lkq) * 4, x + (size_t)tr * K + kc + 4 * lkq);
            }
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const uint32_t row = lrow + 4 * j, er = e0 + row < E ? e0 + row : 0u;
                cp_async16(wb + (row * kRsPitch + 4 * lkq) * 4, w + (size_t)er * K + kc + 4 * lkq);
            }
        }
        cp_async_commit();
    };
    stage(0);
    for (uint32_t c = 0; c < n_chunks; c++) {
        stage(c + 1);
        cp_async_wait<1>();
        __syncwarp();
        const float* xs_c = xs + (c & 1) * kRsWarpFloats;
        const float* ws_c = ws + (c & 1) * kRsWarpFloats;
#pragma unroll
        for (int k4 = 0; k4 < 8; k4++) {
            float4 xa[4], wb[8];
#pragma unroll
            for (int i = 0; i < 4; i++) xa[i] = *reinterpret_cast<const float4*>(xs_c + (ty + 4 * i) * kRsPitch + 4 * k4);
#pragma unroll
            for (int j = 0; j < 8; j++) wb[j] = *reinterpret_cast<const float4*>(ws_c + (tx + 8 * j) * kRsPitch + 4 * k4);
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    float a = acc[i][j];
                    a = fmaf(wb[j].x, xa[i].x, a);
                    a = fmaf(wb[j].y, xa[i].y, a);
                    a = fmaf(wb[j].z, xa[i].z, a);
                    a = fmaf(wb[j].w, xa[i].w, a);
                    acc[i][j] = a;
                }
        }
        __syncwarp();
    }
    // the eight partial tiles meet in shared memory ([warp][token][expert]) and are added in warp order
    __syncthreads();
    float* red = rs_smem;
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) red[(warp * 16 + ty + 4 * i) * 64 + tx + 8 * j] = acc[i][j];
    __syncthreads();
#pragma unroll
    for (int q = 0; q < 4; q++) {
        const uint32_t o = tid + 256 * q, tok = o >> 6, e = o & 63;
        float v = red[tok * 64 + e];
#pragma unroll
        for (int p = 1; p < 8; p++) v += red[(p * 16 + tok) * 64 + e];
        if (t0 + tok < T && e0 + e < E) logits[(size_t)(t0 + tok) * E + e0 + e] = v;
    }
}

// Generic fallback for any K (multiple of 4).
__global__ void __launch_bounds__(256) router_f32_generic_kernel(const float* __restrict__ w, const float* __restrict__ x,
                                                                  float* __restrict__ logits, uint32_t E, uint32_t K, uint32_t T) {
    grid_dependency_wait();      // inputs come from the previous kernel of the chain
    grid_launch_dependents();
    const uint32_t e = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (e >= E) return;
    for (uint32_t t = blockIdx.y; t < T; t += gridDim.y) {
        float acc = 0.f;
        for (uint32_t c = lane; c < K; c += 32) acc = fmaf(w[(size_t)e * K + c], x[(size_t)t * K + c], acc);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) logits[(size_t)t * E + e] = acc;
    }
}

// softmax over all experts, then the top-k probabilities in descending order (ties: lowest index),
// optionally renormalised to sum 1 (crates/engine/src/forward.rs:2420-2448).  One warp per token,
// E <= 256.  in_f16 != 0: the logits are f16 (the reference's router output dtype).
// Routing of one token by one warp; `logits` points at the token's E logits (global or shared memory),
// out_idx / out_w at its k outputs.
template <int NG>   // groups of 32 experts that can be non-empty (E <= 32 * NG); skipping the empty ones adds exact zeros less
__device__ __forceinline__ void route_topk_groups(const void* logits, int in_f16, uint32_t E, uint32_t k, int renorm, uint32_t lane,
                                                int32_t* out_idx, float* out_w) {
    float v[NG];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < NG; i++) {
        const uint32_t e = lane + 32 * i;
        float lv = -INFINITY;
        if (e < E) lv = in_f16 ? __half2float(reinterpret_cast<const __half*>(logits)[e])
                               : reinterpret_cast<const float*>(logits)[e];
        v[i] = lv;
        mx = fmaxf(mx, lv);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    // exp values; the sum runs over experts in index order so that it is reproducible
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NG; i++) v[i] = (lane + 32 * i < E) ? expf(v[i] - mx) : 0.f;
#pragma unroll
    for (int i = 0; i < NG; i++) {
        float part = v[i];   // 0 beyond E; a fixed shuffle tree per group of 32 experts: deterministic
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        sum += part;
    }
#pragma unroll
    for (int i = 0; i < NG; i++) v[i] = v[i] / sum;   // probabilities (0 beyond E)
    uint32_t taken = 0;
    float wsum = 0.f;
    float my_w = 0.f;   // lane s keeps the s-th selected weight (k <= 32)
    int my_i = 0;
    for (uint32_t s = 0; s < k; s++) {
        float bv = -1.f;
        uint32_t bi = 0xFFFFFFFFu;
#pragma unroll
        for (int i = 0; i < NG; i++) {
            const uint32_t e = lane + 32 * i;
            if (e < E && !((taken >> i) & 1u) && (v[i] > bv)) { bv = v[i]; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if ((bi & 31u) == lane && bi != 0xFFFFFFFFu) taken |= 1u << (bi >> 5);
        if (lane == s) { my_w = bv; my_i = (int)bi; }
        wsum += bv;
    }
    if (lane < k) {
        float wv = my_w;
        if (renorm && wsum > 0.f) wv = wv / wsum;
        out_idx[lane] = my_i;
        out_w[lane] = wv;
    }
}

__device__ __forceinline__ void route_topk_warp(const void* logits, int in_f16, uint32_t E, uint32_t k, int renorm, uint32_t lane,
                                                int32_t* out_idx, float* out_w) {
    if (E <= 32) route_topk_groups<1>(logits, in_f16, E, k, renorm, lane, out_idx, out_w);
    else if (E <= 64) route_topk_groups<2>(logits, in_f16, E, k, renorm, lane, out_idx, out_w);
    else if (E <= 128) route_topk_groups<4>(logits, in_f16, E, k, renorm, lane, out_idx, out_w);
    else route_topk_groups<8>(logits, in_f16, E, k, renorm, lane, out_idx, out_w);
}

__global__ void __launch_bounds__(128) route_topk_kernel(const void* __restrict__ logits, int in_f16, uint32_t E, uint32_t k,
                                                          int renorm, uint32_t T, int32_t* __restrict__ out_idx,
                                                          float* __restrict__ out_w) {
    grid_dependency_wait();      // inputs come from the previous kernel of the chain
    grid_launch_dependents();
    const uint32_t t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= T) return;
    const void* row = in_f16 ? (const void*)(reinterpret_cast<const __half*>(logits) + (size_t)t * E)
                             : (const void*)(reinterpret_cast<const float*>(logits) + (size_t)t * E);
    route_topk_warp(row, in_f16, E, k, renorm, lane, out_idx + (size_t)t * k, out_w + (size_t)t * k);
}

// Router and routing of ONE token in one launch (decode): CTAs of 8 warps compute 8 logits each with exactly the
// arithmetic of router_f32_kernel (same bits), publish them and take a ticket; the CTA that draws the last ticket
// routes from the complete logits and puts the ticket counter back to zero.  *counter must be zero before the
// first launch.
// gamma != nullptr: x is the un-normalised hidden state; every CTA first computes its RMSNorm (thread order, shuffle tree
// and rounding of rms_norm_kernel: the same bits in every CTA and as the separate launch), CTA 0 stores the normalised
// vector to xn_out for the expert GEMVs, and the router reads it from shared memory.
template <int KPL>
__global__ void __launch_bounds__(256) route_fused_kernel(const float* __restrict__ w, const float* __restrict__ x,
                                                           float* logits, uint32_t E, uint32_t K, uint32_t k, int renorm,
                                                           int32_t* __restrict__ out_idx, float* __restrict__ out_w, uint32_t* counter,
                                                           const float* __restrict__ gamma, float eps, float* __restrict__ xn_out) {
    __shared__ uint32_t s_last;
    __shared__ __align__(16) float xs[KPL * 32];
    __shared__ float part[8];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t e = blockIdx.x * 8 + warp;
    // the router row and gamma do not depend on the previous kernel of the chain: they are requested before the wait
    float4 wv[KPL / 4];
    float gv[KPL / 8];
    if (e < E) {
        const float4* wrow = reinterpret_cast<const float4*>(w + (size_t)e * K);
#pragma unroll
        for (int i = 0; i < KPL / 4; i++) wv[i] = wrow[lane + 32 * i];
    }
    if (gamma) {
#pragma unroll
        for (int j = 0; j < KPL / 8; j++) gv[j] = gamma[threadIdx.x + 256 * j];
    }
    grid_dependency_wait();
    grid_launch_dependents();
    if (gamma) {
        float xv[KPL / 8];
#pragma unroll
        for (int j = 0; j < KPL / 8; j++) xv[j] = x[threadIdx.x + 256 * j];
        float sq = 0.f;
#pragma unroll
        for (int j = 0; j < KPL / 8; j++) sq = fmaf(xv[j], xv[j], sq);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (lane == 0) part[warp] = sq;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) tot += part[i];
        const float r = rsqrtf(tot / (float)K + eps);
#pragma unroll
        for (int j = 0; j < KPL / 8; j++) {
            const float v = xv[j] * r * gv[j];
            xs[threadIdx.x + 256 * j] = v;
            if (blockIdx.x == 0) xn_out[threadIdx.x + 256 * j] = v;
        }
        __syncthreads();
    }
    if (e < E) {
        const float4* xr = gamma ? reinterpret_cast<const float4*>(xs) : reinterpret_cast<const float4*>(x);
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
        for (int i = 0; i < KPL / 4; i++) {
            const float4 v = xr[lane + 32 * i];
            a0 = fmaf(wv[i].x, v.x, a0); a1 = fmaf(wv[i].y, v.y, a1);
            a2 = fmaf(wv[i].z, v.z, a2); a3 = fmaf(wv[i].w, v.w, a3);
        }
        float acc = (a0 + a1) + (a2 + a3);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) logits[e] = acc;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();                                   // this CTA's logits are visible before its ticket
        s_last = atomicAdd(counter, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (s_last && warp == 0) {
        __threadfence();
        route_topk_warp(logits, 0, E, k, renorm, lane, out_idx, out_w);
        if (lane == 0) *counter = 0;
    }
}

// out[t][r] = (res ? res[t][r] : 0) + sum_i w[t][i] * y[t*k+i][r], i ascending (routing order).
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ y, const float* __restrict__ w,
                                                           const float* res, float* out, uint32_t T, uint32_t h, uint32_t k) {
    grid_dependency_wait();      // inputs come from the previous kernel of the chain
    grid_launch_dependents();
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
    if (r >= h) return;
    float acc = 0.f;
    for (uint32_t i = 0; i < k; i++) acc = fmaf(w[(size_t)t * k + i], y[((size_t)t * k + i) * h + r], acc);
    const size_t o = (size_t)t * h + r;
    out[o] = (res ? res[o] : 0.f) + acc;
}

struct MoeScratch {
    float* logits;   // [T][E]
    int32_t* idx;    // [T][k]
    float* w;        // [T][k]
    float* act;      // [T*k][ff]
    float* y;        // [T*k][h]
    size_t bytes;
};

// Expert-parallel decode block, replicated tokens.  This rank's weighted sum over the slots whose expert it owns
// (routing order), stored into slot `rank` of the partial buffer of every rank: plain stores into peer memory.
struct EpPeers {
    float* p[8];   // rank r's partial buffer [world][T][h], as mapped into this process
};
// The partial buffers have two halves that alternate by epoch parity.  The epoch is either given (call-by-call use)
// or read from a device word that the barrier kernel advances (recorded command lists: the same launch runs every token).
// (One launch that pushes the partial sums, lets its last CTA run the barrier and add everything was measured slower
// than these three: 37.6 vs 33.2 us per layer at one token, 172 vs 102 us at 16, two ranks.)
__global__ void __launch_bounds__(256) ep_partial_kernel(const float* __restrict__ y, const float* __restrict__ w,
                                                          const int32_t* __restrict__ idx, const EpPeers peers, uint32_t world,
                                                          uint32_t rank, int32_t lo, uint32_t cnt, uint32_t T, uint32_t h, uint32_t k,
                                                          uint32_t epoch, const uint32_t* __restrict__ epoch_ptr) {
    grid_dependency_wait();
    grid_launch_dependents();
    const uint32_t c = blockIdx.x * 256 + threadIdx.x, t = blockIdx.y;
    if (c >= h) return;
    const size_t half = (size_t)((epoch_ptr ? *epoch_ptr + 1u : epoch) & 1u) * world * T * h;
    float acc = 0.f;
    for (uint32_t i = 0; i < k; i++) {
        const int32_t e = idx[t * k + i] - lo;
        if (e >= 0 && (uint32_t)e < cnt) acc = fmaf(w[t * k + i], y[(size_t)(t * k + i) * h + c], acc);
    }
    const size_t o = half + ((size_t)rank * T + t) * h + c;
    for (uint32_t p = 0; p < world; p++) peers.p[p][o] = acc;
}
// out[t] = residual[t] + sum over ranks (rank order) of the partial sums that arrived in this rank's buffer.
// `out` may be the same buffer as `residual` (the decoder adds into its hidden state in place): neither is restrict.
__global__ void __launch_bounds__(256) ep_reduce_kernel(const float* __restrict__ partial, const float* residual,
                                                         float* out, uint32_t world, uint32_t T, uint32_t h,
                                                         uint32_t epoch, const uint32_t* __restrict__ epoch_ptr) {
    const uint32_t c = blockIdx.x * 256 + threadIdx.x, t = blockIdx.y;
    if (c >= h) return;
    partial += (size_t)((epoch_ptr ? *epoch_ptr : epoch) & 1u) * world * T * h;   // the barrier has advanced the word already
    float acc = residual ? residual[(size_t)t * h + c] : 0.f;
    for (uint32_t r = 0; r < world; r++) acc += partial[((size_t)r * T + t) * h + c];
    out[(size_t)t * h + c] = acc;
}

static MoeScratch moe_carve(void* base, uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k) {
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    uint8_t* p = reinterpret_cast<uint8_t*>(base);
    MoeScratch s;
    size_t o = 0;
    s.logits = reinterpret_cast<float*>(p + o); o += up((size_t)T * E * 4);
    s.idx = reinterpret_cast<int32_t*>(p + o); o += up((size_t)T * k * 4);
    s.w = reinterpret_cast<float*>(p + o); o += up((size_t)T * k * 4);
    s.act = reinterpret_cast<float*>(p + o); o += up((size_t)T * k * ff * 4);
    s.y = reinterpret_cast<float*>(p + o); o += up((size_t)T * k * h * 4);
    s.bytes = o;
    return s;
}

// Shared with the batched block (moe_grouped.cu).
int32_t moe_router(runit_ctx* ctx, const float* w, const float* x, float* logits, uint32_t E, uint32_t K, uint32_t T) {
    // (the tiled kernel, one CTA per 64 tokens walking all of K, has a floor of about 85 us: it serves K that is not a
    // multiple of 256 at large sizes and stays selectable, router_variant = 2)
    // measured (h = 2048, warm, us): one warp per expert / tiled / split over the warps of a CTA: 64 experts x 256 tokens
    // 10 / 87 / 22, x 1024: 32 / 87 / 22, x 2048: 60 / 87 / 22, x 4096: 117 / 122 / 42; 128 experts x 256: 19 / 86 / 22,
    // x 1024: 62 / 87 / 23, x 4096: 230 / 134 / 82 (the split kernel re-reads the router for every 16 tokens: about 4 TB/s from L2)
    if ((((uint64_t)T * E >= 49152ull && ctx->tune.router_variant == 0) || ctx->tune.router_variant == 3) && K % 256 == 0 && runit_aligned(w, 16) &&
        runit_aligned(x, 16)) {
        constexpr int smem = 8 * 2 * kRsWarpFloats * 4;
        static bool configured[64] = {false};
        if (ctx->device >= 0 && ctx->device < 64 && !configured[ctx->device]) {
            RUNIT_CUDA_TRY(ctx, cudaFuncSetAttribute(router_f32_splitk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            configured[ctx->device] = true;
        }
        runit_launch_chain_smem(ctx, router_f32_splitk_kernel, dim3((E + 63) / 64, (T + 15) / 16), dim3(256), smem, w, x, logits, E, K, T);
        return runit_after_launch(ctx, "moe_router_f32_splitk");
    }
    const bool big = (uint64_t)T * E >= 400000ull;
    if (ctx->tune.router_variant != 1 && (big || ctx->tune.router_variant == 2) && K % 32 == 0 && runit_aligned(w, 16) && runit_aligned(x, 16)) {
        const uint32_t ge = (E + 63) / 64;
        if (ge * ((T + 63) / 64) >= (uint32_t)ctx->sm_count)
            runit_launch_chain(ctx, router_f32_tiled_kernel<64>, dim3(ge, (T + 63) / 64), dim3(256), w, x, logits, E, K, T);
        else if (ge * ((T + 31) / 32) >= (uint32_t)ctx->sm_count)
            runit_launch_chain(ctx, router_f32_tiled_kernel<32>, dim3(ge, (T + 31) / 32), dim3(256), w, x, logits, E, K, T);
        else
            runit_launch_chain(ctx, router_f32_tiled_kernel<16>, dim3(ge, (T + 15) / 16), dim3(256), w, x, logits, E, K, T);
        return runit_after_launch(ctx, "moe_router_f32_tiled");
    }
    dim3 grid((E + 7) / 8, T < 64 ? T : 64);
    if (K == 2048) runit_launch_chain(ctx, router_f32_kernel<64>, dim3(grid), dim3(256), w, x, logits, E, K, T);
    else if (K == 1024) runit_launch_chain(ctx, router_f32_kernel<32>, dim3(grid), dim3(256), w, x, logits, E, K, T);
    else if (K == 4096) runit_launch_chain(ctx, router_f32_kernel<128>, dim3(grid), dim3(256), w, x, logits, E, K, T);
    else runit_launch_chain(ctx, router_f32_generic_kernel, dim3(grid), dim3(256), w, x, logits, E, K, T);
    return runit_after_launch(ctx, "moe_router_f32");
}

int32_t moe_topk(runit_ctx* ctx, const float* logits, uint32_t E, uint32_t k, int32_t renorm, uint32_t T, int32_t* idx, float* w) {
    runit_launch_chain(ctx, route_topk_kernel, dim3((T + 3) / 4), dim3(128), logits, 0, E, k, renorm, T, idx, w);
    return runit_after_launch(ctx, "moe_route_topk");
}

size_t moe_scratch_bytes_impl(uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k) {
    return moe_carve(nullptr, T, h, ff, E, k).bytes;
}

// The whole block; scratch carved from `scratch`.
int32_t moe_layer_q4k_impl(runit_ctx* ctx, const void* router_w, const void* gate, const void* up, const void* down,
                           const void* x, const void* residual, void* out, int32_t* idx_out, float* w_out, void* scratch,
                           size_t scratch_bytes, uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k, int32_t renorm,
                           const float* next_gamma, float* next_xn, float next_eps, uint32_t* route_counter,
                           const float* pre_x, const float* pre_gamma, float pre_eps) {
    RUNIT_REQUIRE(ctx, router_w && gate && up && down && x && out && scratch, "moe_layer_q4k: null pointer");
    RUNIT_REQUIRE(ctx, T > 0 && T <= 65536, "moe_layer_q4k: T=%u out of range", T);
    RUNIT_REQUIRE(ctx, h % 256 == 0 && ff % 256 == 0 && h > 0 && ff > 0, "moe_layer_q4k: h=%u, ff=%u must be multiples of 256", h, ff);
    RUNIT_REQUIRE(ctx, E > 0 && E <= 256 && k > 0 && k <= E && k <= 32, "moe_layer_q4k: E=%u, k=%u unsupported", E, k);
    RUNIT_REQUIRE(ctx, runit_aligned(scratch, 256), "moe_layer_q4k: scratch must be 256-byte aligned");
    const MoeScratch s = moe_carve(scratch, T, h, ff, E, k);
    if (s.bytes > scratch_bytes)
        return runit_fail(ctx, RUNIT_ERR_BUFFER_SIZE, "moe_layer_q4k: scratch has %zu bytes, needs %zu", scratch_bytes, s.bytes);
    int32_t* idx = idx_out ? idx_out : s.idx;
    float* wts = w_out ? w_out : s.w;
    int32_t st;
    // pre_gamma != nullptr: the block starts with the RMSNorm of pre_x (the un-normalised hidden state, another buffer than
    // x) into x, which the router and the experts then consume; one token takes it inside the routing launch, else it is a
    // launch of its own
    const bool fused_route = route_counter && T == 1 && (h == 1024 || h == 2048 || h == 4096) && runit_aligned(router_w, 16) && runit_aligned(x, 16) &&
                             (!pre_gamma || (pre_x && pre_x != x && runit_aligned(pre_x, 16)));
    float* pre_out = pre_gamma ? (float*)const_cast<void*>(x) : nullptr;
    const float* x_route = pre_gamma ? pre_x : (const float*)x;
    if (pre_gamma && !fused_route) {
        RUNIT_REQUIRE(ctx, pre_x, "moe_layer_q4k: null pre-norm input");
        if ((st = launch_rms_norm(ctx, pre_x, pre_out, pre_gamma, false, pre_eps, h, T)) != RUNIT_OK) return st;
        pre_gamma = nullptr;
        x_route = (const float*)x;
    }
    if (fused_route) {
        // one token: router GEMV and routing in one launch (same bits as the two launches below)
        const dim3 grid((E + 7) / 8);
        if (h == 2048) runit_launch_chain(ctx, route_fused_kernel<64>, grid, dim3(256), (const float*)router_w, x_route, s.logits, E, h, k, (int)renorm, idx, wts, route_counter, pre_gamma, pre_eps, pre_out);
        else if (h == 1024) runit_launch_chain(ctx, route_fused_kernel<32>, grid, dim3(256), (const float*)router_w, x_route, s.logits, E, h, k, (int)renorm, idx, wts, route_counter, pre_gamma, pre_eps, pre_out);
        else runit_launch_chain(ctx, route_fused_kernel<128>, grid, dim3(256), (const float*)router_w, x_route, s.logits, E, h, k, (int)renorm, idx, wts, route_counter, pre_gamma, pre_eps, pre_out);
        if ((st = runit_after_launch(ctx, "moe_route_fused")) != RUNIT_OK) return st;
    } else {
        st = moe_router(ctx, (const float*)router_w, (const float*)x, s.logits, E, h, T);
        if (st != RUNIT_OK) return st;
        runit_launch_chain(ctx, route_topk_kernel, dim3((T + 3) / 4), dim3(128), (const void*)s.logits, 0, E, k, (int)renorm, T, idx, wts);
        st = runit_after_launch(ctx, "moe_route_topk");
        if (st != RUNIT_OK) return st;
    }
    const uint32_t slots = T * k;
    // gate+up+SiLU for every (token, expert) slot: act[s][ff]
    const bool fused_sum = fused_route && h <= 32 * 960;
    st = gemv_grouped(ctx, "moe_gate_up", RUNIT_FMT_Q4K, gate, up, E, ff, h, x, k, s.act, idx, slots, 0, nullptr, nullptr, nullptr,
                      nullptr, fused_sum ? 1 : 0);
    if (st != RUNIT_OK) return st;
    // down: y[s][h] = Wd[e_s] . act[s]
    if (fused_sum) {
        // one token: the last down-projection tile of every 32 rows adds the experts' rows (same order as moe_combine_kernel)
        st = gemv_grouped(ctx, "moe_down", RUNIT_FMT_Q4K, down, nullptr, E, h, ff, s.act, 1, s.y, idx, slots, 0, wts,
                          (const float*)residual, (float*)out, route_counter + 32, 2);
        if (st != RUNIT_OK || !next_gamma) return st;
        return launch_rms_norm(ctx, (const float*)out, next_xn, next_gamma, false, next_eps, h, T);
    }
    st = gemv_grouped(ctx, "moe_down", RUNIT_FMT_Q4K, down, nullptr, E, h, ff, s.act, 1, s.y, idx, slots);
    if (st != RUNIT_OK) return st;
    runit_launch_chain(ctx, moe_combine_kernel, dim3((h + 255) / 256, T), dim3(256), (const float*)s.y, (const float*)wts, (const float*)residual, (float*)out, T, h, k);
    st = runit_after_launch(ctx, "moe_combine");
    if (st != RUNIT_OK || !next_gamma) return st;
    return launch_rms_norm(ctx, (const float*)out, next_xn, next_gamma, false, next_eps, h, T);
}

// ───────────────────────── built-in scratch (entry point that allocates nothing) ─────────────────────────
// A fixed region inside the library's own device image.  Every GPU that loads the library carries it
// until the process exits.  In host code `g_moe_static_scratch` is only a stand-in for the symbol, never a
// device address: the address a kernel may use comes from cudaGetSymbolAddress, asked once per device
// with that device current.
constexpr size_t kMoeStaticScratchBytes = 4u << 20;   // 4 MiB
static __device__ __align__(256) unsigned char g_moe_static_scratch[kMoeStaticScratchBytes];

static int32_t moe_static_scratch(runit_ctx* ctx, void** out) {
    static void* per_device[64] = {nullptr};
    *out = nullptr;
    if (ctx->device < 0 || ctx->device >= 64) return runit_fail(ctx, RUNIT_ERR_UNSUPPORTED, "device index %d out of range", ctx->device);
    if (!per_device[ctx->device]) {
        int cur = -1;
        RUNIT_CUDA_TRY(ctx, cudaGetDevice(&cur));
        if (cur != ctx->device) RUNIT_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_moe_static_scratch);
        if (cur != ctx->device) cudaSetDevice(cur);
        if (e != cudaSuccess || !p)
            return runit_fail(ctx, RUNIT_ERR_LAUNCH, "cudaGetSymbolAddress(built-in MoE scratch): %s", cudaGetErrorString(e));
        per_device[ctx->device] = p;
    }
    *out = per_device[ctx->device];
    return RUNIT_OK;
}

// The expert-parallel block behind runit_moe_layer_q4k_ep; epoch_ptr != nullptr: the epoch lives in that device word.
int32_t moe_layer_q4k_ep_impl(runit_ctx* ctx, const void* router_w, const void* gate_local, const void* up_local,
                              const void* down_local, const void* x, const void* residual, void* out, void* idx_out, void* w_out,
                              void* scratch, size_t scratch_bytes, void* const* partial_all, void* const* signal_pads,
                              uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k, int32_t renorm, uint32_t world,
                              uint32_t rank, uint32_t epoch, uint32_t* epoch_ptr, uint32_t* route_counter, const float* pre_x,
                              const float* pre_gamma, float pre_eps) {
    RUNIT_REQUIRE(ctx, router_w && gate_local && up_local && down_local && x && out && scratch && partial_all && signal_pads,
                  "moe_layer_q4k_ep: null pointer");
    RUNIT_REQUIRE(ctx, world >= 1 && world <= 8 && rank < world && E % world == 0 && (epoch > 0 || epoch_ptr),
                  "moe_layer_q4k_ep: world=%u rank=%u E=%u unsupported (1..8 ranks, experts divisible)", world, rank, E);
    RUNIT_REQUIRE(ctx, T > 0 && T <= 4096, "moe_layer_q4k_ep: T=%u out of range (replicated tokens, decode sizes)", T);
    RUNIT_REQUIRE(ctx, h % 256 == 0 && ff % 256 == 0 && h > 0 && ff > 0, "moe_layer_q4k_ep: h=%u, ff=%u must be multiples of 256", h, ff);
    RUNIT_REQUIRE(ctx, E > 0 && E <= 256 && k > 0 && k <= E && k <= 32, "moe_layer_q4k_ep: E=%u, k=%u unsupported", E, k);
    RUNIT_REQUIRE(ctx, runit_aligned(scratch, 256), "moe_layer_q4k_ep: scratch must be 256-byte aligned");
    const MoeScratch s = moe_carve(scratch, T, h, ff, E, k);
    if (s.bytes > scratch_bytes)
        return runit_fail(ctx, RUNIT_ERR_BUFFER_SIZE, "moe_layer_q4k_ep: scratch has %zu bytes, needs %zu", scratch_bytes, s.bytes);
    EpPeers peers{};
    for (uint32_t p = 0; p < world; p++) {
        RUNIT_REQUIRE(ctx, partial_all[p] && runit_aligned(partial_all[p], 4), "moe_layer_q4k_ep: null or misaligned partial buffer %u", p);
        // the two halves of a partial buffer alternate by epoch parity (in the kernels): a fast rank's next call cannot
        // overwrite what a slow rank is still adding (it would first have to pass the next barrier, which the slow rank
        // announces after its sum)
        peers.p[p] = (float*)partial_all[p];
    }
    int32_t* idx = idx_out ? (int32_t*)idx_out : s.idx;
    float* wts = w_out ? (float*)w_out : s.w;
    // every rank routes every token itself (the router is replicated): no dispatch exchange
    int32_t st;
    const bool fused_route = route_counter && T == 1 && (h == 1024 || h == 2048 || h == 4096) && runit_aligned(router_w, 16) && runit_aligned(x, 16) &&
                             (!pre_gamma || (pre_x && pre_x != x && runit_aligned(pre_x, 16)));
    float* pre_out = pre_gamma ? (float*)const_cast<void*>(x) : nullptr;
    const float* x_route = pre_gamma ? pre_x : (const float*)x;
    if (pre_gamma && !fused_route) {
        RUNIT_REQUIRE(ctx, pre_x, "moe_layer_q4k_ep: null pre-norm input");
        if ((st = launch_rms_norm(ctx, pre_x, pre_out, pre_gamma, false, pre_eps, h, T)) != RUNIT_OK) return st;
        pre_gamma = nullptr;
        x_route = (const float*)x;
    }
    if (fused_route) {
        // one token: (RMSNorm,) router GEMV and routing in one launch (same bits as the separate launches)
        const dim3 grid((E + 7) / 8);
        if (h == 2048) runit_launch_chain(ctx, route_fused_kernel<64>, grid, dim3(256), (const float*)router_w, x_route, s.logits, E, h, k, (int)renorm, idx, wts, route_counter, pre_gamma, pre_eps, pre_out);
        else if (h == 1024) runit_launch_chain(ctx, route_fused_kernel<32>, grid, dim3(256), (const float*)router_w, x_route, s.logits, E, h, k, (int)renorm, idx, wts, route_counter, pre_gamma, pre_eps, pre_out);
        else runit_launch_chain(ctx, route_fused_kernel<128>, grid, dim3(256), (const float*)router_w, x_route, s.logits, E, h, k, (int)renorm, idx, wts, route_counter, pre_gamma, pre_eps, pre_out);
        if ((st = runit_after_launch(ctx, "moe_route_fused")) != RUNIT_OK) return st;
    } else {
        if ((st = moe_router(ctx, (const float*)router_w, (const float*)x, s.logits, E, h, T)) != RUNIT_OK) return st;
        runit_launch_chain(ctx, route_topk_kernel, dim3((T + 3) / 4), dim3(128), (const void*)s.logits, 0, E, k, (int)renorm, T, idx, wts);
        if ((st = runit_after_launch(ctx, "moe_route_topk")) != RUNIT_OK) return st;
    }
    const uint32_t n_local = E / world, slots = T * k;
    const int32_t lo = (int32_t)(rank * n_local);
    // only the slots of this rank's experts are computed (the others are unused slots of the grouped launches)
    st = gemv_grouped(ctx, "moe_gate_up_ep", RUNIT_FMT_Q4K, gate_local, up_local, n_local, ff, h, x, k, s.act, idx, slots, lo);
    if (st != RUNIT_OK) return st;
    st = gemv_grouped(ctx, "moe_down_ep", RUNIT_FMT_Q4K, down_local, nullptr, n_local, h, ff, s.act, 1, s.y, idx, slots, lo);
    if (st != RUNIT_OK) return st;
    runit_launch_chain(ctx, ep_partial_kernel, dim3((h + 255) / 256, T), dim3(256), (const float*)s.y, (const float*)wts, (const int32_t*)idx,
                       peers, world, rank, lo, n_local, T, h, k, epoch, (const uint32_t*)epoch_ptr);
    if ((st = runit_after_launch(ctx, "moe_ep_partial")) != RUNIT_OK) return st;
    if ((st = peer_barrier_launch(ctx, signal_pads, world, rank, epoch, epoch_ptr)) != RUNIT_OK) return st;
    ep_reduce_kernel<<<dim3((h + 255) / 256, T), 256, 0, ctx->stream>>>(peers.p[rank], (const float*)residual, (float*)out, world, T, h,
                                                                         epoch, (const uint32_t*)epoch_ptr);
    return runit_after_launch(ctx, "moe_ep_reduce");
}

// Expert-parallel decode block of one token without launches of its own for the exchange: routing, grouped gate/up, and a
// grouped down projection whose epilogue pushes this rank's weighted partial sum to every rank and raises the flags
// (EpPush); the residual add and the sum over the ranks happen in the prologue of the next GEMV that reads the hidden
// state (EpWait).  Three launches, as on one GPU.
int32_t moe_layer_q4k_ep_push_impl(runit_ctx* ctx, const void* router_w, const void* gate_local, const void* up_local,
                                   const void* down_local, float* xn, const float* pre_x, const float* pre_gamma, float pre_eps,
                                   void* scratch, size_t scratch_bytes, uint32_t h, uint32_t ff, uint32_t E, uint32_t k, int32_t renorm,
                                   uint32_t* counters, const EpPush* push) {
    RUNIT_REQUIRE(ctx, router_w && gate_local && up_local && down_local && xn && pre_x && pre_gamma && scratch && counters && push,
                  "moe_layer_q4k_ep_push: null pointer");
    RUNIT_REQUIRE(ctx, (h == 1024 || h == 2048 || h == 4096) && ff % 256 == 0 && E % push->world == 0 && k <= 32 && k <= E,
                  "moe_layer_q4k_ep_push: hidden 1024 / 2048 / 4096, experts divisible by the ranks");
    const MoeScratch s = moe_carve(scratch, 1, h, ff, E, k);
    if (s.bytes > scratch_bytes)
        return runit_fail(ctx, RUNIT_ERR_BUFFER_SIZE, "moe_layer_q4k_ep_push: scratch has %zu bytes, needs %zu", scratch_bytes, s.bytes);
    int32_t st;
    const dim3 grid((E + 7) / 8);
    if (h == 2048) runit_launch_chain(ctx, route_fused_kernel<64>, grid, dim3(256), (const float*)router_w, pre_x, s.logits, E, h, k, (int)renorm, s.idx, s.w, counters, pre_gamma, pre_eps, xn);
    else if (h == 1024) runit_launch_chain(ctx, route_fused_kernel<32>, grid, dim3(256), (const float*)router_w, pre_x, s.logits, E, h, k, (int)renorm, s.idx, s.w, counters, pre_gamma, pre_eps, xn);
    else runit_launch_chain(ctx, route_fused_kernel<128>, grid, dim3(256), (const float*)router_w, pre_x, s.logits, E, h, k, (int)renorm, s.idx, s.w, counters, pre_gamma, pre_eps, xn);
    if ((st = runit_after_launch(ctx, "moe_route_fused")) != RUNIT_OK) return st;
    const uint32_t n_local = E / push->world;
    const int32_t lo = (int32_t)(push->rank * n_local);
    st = gemv_grouped(ctx, "moe_gate_up_ep", RUNIT_FMT_Q4K, gate_local, up_local, n_local, ff, h, xn, k, s.act, s.idx, k, lo, nullptr, nullptr,
                      nullptr, nullptr, 1);
    if (st != RUNIT_OK) return st;
    return gemv_grouped(ctx, "moe_down_ep_push", RUNIT_FMT_Q4K, down_local, nullptr, n_local, h, ff, s.act, 1, s.y, s.idx, k, lo, s.w, nullptr,
                        nullptr, counters + 32, 2, push);
}

}  // namespace runit

using namespace runit;

extern "C" {

size_t runit_moe_static_scratch_capacity(void) { return kMoeStaticScratchBytes; }

int32_t runit_moe_layer_q4k_static(runit_ctx_t* ctx, const void* router_w, const void* gate, const void* up,
                                   const void* down, const void* x, const void* residual, void* out, void* idx_out,
                                   void* w_out, uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k, int32_t renorm) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, T > 0 && h > 0 && ff > 0 && E > 0 && k > 0, "moe_layer_q4k_static: empty shape");
    const size_t need = moe_carve(nullptr, T, h, ff, E, k).bytes;
    if (need > kMoeStaticScratchBytes)
        return runit_fail(ctx, RUNIT_ERR_BUFFER_SIZE,
                          "moe_layer_q4k_static: T=%u k=%u h=%u ff=%u E=%u needs %zu bytes of scratch, the built-in region "
                          "holds %zu; use runit_moe_layer_q4k with caller-owned scratch",
                          T, k, h, ff, E, need, (size_t)kMoeStaticScratchBytes);
    void* scratch = nullptr;
    int32_t st = moe_static_scratch(ctx, &scratch);
    if (st != RUNIT_OK) return st;
    return moe_layer_q4k_impl(ctx, router_w, gate, up, down, x, residual, out, (int32_t*)idx_out, (float*)w_out, scratch,
                              kMoeStaticScratchBytes, T, h, ff, E, k, renorm, nullptr, nullptr, 0.f, nullptr, nullptr, nullptr, 0.f);
}

size_t runit_moe_scratch_bytes(uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k) {
    return moe_carve(nullptr, T, h, ff, E, k).bytes;
}

int32_t runit_moe_router_f32(runit_ctx_t* ctx, const void* router_w, const void* x, void* logits, uint32_t E, uint32_t h,
                             uint32_t T) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, router_w && x && logits && E > 0 && T > 0 && h > 0 && h % 4 == 0, "moe_router_f32: bad argument");
    return moe_router(ctx, (const float*)router_w, (const float*)x, (float*)logits, E, h, T);
}

int32_t runit_moe_route_topk(runit_ctx_t* ctx, const void* logits, int32_t logits_f16, uint32_t E, uint32_t k, int32_t renorm,
                             uint32_t T, void* out_idx, void* out_w) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, logits && out_idx && out_w, "moe_route_topk: null pointer");
    RUNIT_REQUIRE(ctx, E > 0 && E <= 256 && k > 0 && k <= E && k <= 32 && T > 0, "moe_route_topk: E=%u k=%u T=%u unsupported", E, k, T);
    runit_launch_chain(ctx, route_topk_kernel, dim3((T + 3) / 4), dim3(128), logits, logits_f16, E, k, renorm, T, (int32_t*)out_idx, (float*)out_w);
    return runit_after_launch(ctx, "moe_route_topk");
}

int32_t runit_moe_experts_q4k(runit_ctx_t* ctx, const void* gate, const void* up, const void* down, const void* x_slots,
                              const void* slot_expert, void* y_slots, void* act_scratch, uint32_t n_slots, uint32_t h,
                              uint32_t ff, uint32_t n_experts) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, gate && up && down && x_slots && slot_expert && y_slots && act_scratch, "moe_experts_q4k: null pointer");
    RUNIT_REQUIRE(ctx, n_slots > 0 && n_experts > 0 && h % 256 == 0 && ff % 256 == 0 && h > 0 && ff > 0, "moe_experts_q4k: bad shape");
    int32_t st = gemv_grouped(ctx, "moe_gate_up", RUNIT_FMT_Q4K, gate, up, n_experts, ff, h, x_slots, 1, act_scratch,
                              (const int32_t*)slot_expert, n_slots);
    if (st != RUNIT_OK) return st;
    return gemv_grouped(ctx, "moe_down", RUNIT_FMT_Q4K, down, nullptr, n_experts, h, ff, act_scratch, 1, y_slots,
                        (const int32_t*)slot_expert, n_slots);
}

int32_t runit_moe_layer_q4k_ep(runit_ctx_t* ctx, const void* router_w, const void* gate_local, const void* up_local,
                               const void* down_local, const void* x, const void* residual, void* out, void* idx_out, void* w_out,
                               void* scratch, size_t scratch_bytes, void* const* partial_all, void* const* signal_pads,
                               uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k, int32_t renorm, uint32_t world,
                               uint32_t rank, uint32_t epoch) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, epoch > 0, "moe_layer_q4k_ep: epoch must be positive");
    return moe_layer_q4k_ep_impl(ctx, router_w, gate_local, up_local, down_local, x, residual, out, idx_out, w_out, scratch,
                                 scratch_bytes, partial_all, signal_pads, T, h, ff, E, k, renorm, world, rank, epoch, nullptr, nullptr, nullptr, nullptr, 0.f);
}

int32_t runit_moe_layer_q4k(runit_ctx_t* ctx, const void* router_w, const void* gate, const void* up, const void* down,
                            const void* x, const void* residual, void* out, void* idx_out, void* w_out, void* scratch,
                            size_t scratch_bytes, uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k, int32_t renorm) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    return moe_layer_q4k_impl(ctx, router_w, gate, up, down, x, residual, out, (int32_t*)idx_out, (float*)w_out, scratch,
                              scratch_bytes, T, h, ff, E, k, renorm, nullptr, nullptr, 0.f, nullptr, nullptr, nullptr, 0.f);
}

}  // extern "C"
