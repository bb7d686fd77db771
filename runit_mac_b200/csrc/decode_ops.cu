// Decode-step operators besides the GEMVs: RMSNorm, RoPE, KV-cache scatter, q_len=1 attention, argmax.
//
// Twins of crates/kernels/shaders/{norm.metal:95-154, fused_rope.metal:17-56, activation.metal:13-110,
// attention.metal:172-308} of the reference.  The position / KV length can come from a device word
// (pos_ptr) so that a recorded command list can be replayed for successive tokens.
#include <type_traits>

#include "decode_ops.cuh"
#include "runit_internal.h"
#include "tma.cuh"

namespace runit {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// y = x * rsqrt(mean(x^2) + eps) * gamma, one CTA per row (norm.metal:95-154).
template <typename G>
__global__ void __launch_bounds__(256) rms_norm_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                        const G* __restrict__ gamma, float eps, uint32_t hidden) {
    grid_dependency_wait();      // inputs come from the previous kernel of the chain
    grid_launch_dependents();
    __shared__ float part[8];
    const float* row = x + (size_t)blockIdx.x * hidden;
    float* out = y + (size_t)blockIdx.x * hidden;
    float s = 0.f;
    for (uint32_t i = threadIdx.x; i < hidden; i += 256) {
        const float v = row[i];
        s = fmaf(v, v, s);
    }
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += part[i];
    const float r = rsqrtf(tot / (float)hidden + eps);
    for (uint32_t i = threadIdx.x; i < hidden; i += 256) {
        float g;
        if (sizeof(G) == 2) g = __half2float(reinterpret_cast<const __half*>(gamma)[i]);
        else g = reinterpret_cast<const float*>(gamma)[i];
        out[i] = row[i] * r * g;   // x and y may be the same buffer (QK-norm is applied in place)
    }
}

// Rotary embedding of Q and K in one launch: pairs (d, d+hd/2), freq = theta^(-2d/hd)
// (fused_rope.metal:17-56).  Optionally scatters the rotated K and the V vector into f16 caches.
__global__ void rope_qk_kernel(float* q, float* k, uint32_t head_dim, uint32_t q_heads, uint32_t kv_heads, uint32_t pos_val,
                               const int32_t* pos_ptr, float theta) {
    grid_dependency_wait();      // inputs come from the previous kernel of the chain
    grid_launch_dependents();
    const uint32_t d = threadIdx.x, hid = blockIdx.x, half = head_dim / 2;
    if (d >= half) return;
    const uint32_t pos = pos_ptr ? (uint32_t)*pos_ptr : pos_val;
    const float freq = 1.0f / powf(theta, (float)(2 * d) / (float)head_dim);
    const float angle = (float)pos * freq;
    const float c = cosf(angle), s = sinf(angle);
    if (hid < q_heads) {
        float* p = q + (size_t)hid * head_dim;
        const float a = p[d], b = p[d + half];
        p[d] = a * c - b * s;
        p[d + half] = a * s + b * c;
    }
    if (hid < kv_heads) {
        float* p = k + (size_t)hid * head_dim;
        const float a = p[d], b = p[d + half];
        p[d] = a * c - b * s;
        p[d + half] = a * s + b * c;
    }
}

// The same rotation, then K (rotated) and V of this position go into the f16 caches (activation.metal:13-44): one launch
// instead of three in the decode chain.  Same arithmetic per element as rope_qk_kernel + kv_copy_kernel<float, __half>.
__global__ void rope_kv_kernel(float* q, float* k, const float* __restrict__ v, __half* __restrict__ kc, __half* __restrict__ vc,
                               uint32_t head_dim, uint32_t q_heads, uint32_t kv_heads, const int32_t* pos_ptr, float theta,
                               uint32_t max_seq) {
    grid_dependency_wait();
    grid_launch_dependents();
    const uint32_t d = threadIdx.x, hid = blockIdx.x, half = head_dim / 2;
    if (d >= half) return;
    const uint32_t pos = (uint32_t)*pos_ptr;
    const float freq = 1.0f / powf(theta, (float)(2 * d) / (float)head_dim);
    const float angle = (float)pos * freq;
    const float c = cosf(angle), s = sinf(angle);
    if (hid < q_heads) {
        float* p = q + (size_t)hid * head_dim;
        const float a = p[d], b = p[d + half];
        p[d] = a * c - b * s;
        p[d + half] = a * s + b * c;
    }
    if (hid < kv_heads) {
        float* p = k + (size_t)hid * head_dim;
        const float a = p[d], b = p[d + half];
        const float r0 = a * c - b * s, r1 = a * s + b * c;
        p[d] = r0;
        p[d + half] = r1;
        if (pos < max_seq) {
            const size_t o = ((size_t)hid * max_seq + pos) * head_dim;
            kc[o + d] = __float2half_rn(r0);
            kc[o + d + half] = __float2half_rn(r1);
            const float* vp = v + (size_t)hid * head_dim;
            vc[o + d] = __float2half_rn(vp[d]);
            vc[o + d + half] = __float2half_rn(vp[d + half]);
        }
    }
}

// dst[(h*max_seq + pos)*hd + d] = src[h*hd + d]   (activation.metal:13-44)
template <typename S, typename D>
__global__ void kv_copy_kernel(const S* __restrict__ src, D* __restrict__ dst, uint32_t pos_val, const int32_t* pos_ptr,
                               uint32_t max_seq, uint32_t head_dim) {
    grid_dependency_wait();      // inputs come from the previous kernel of the chain
    grid_launch_dependents();
    const uint32_t d = blockIdx.x * blockDim.x + threadIdx.x, h = blockIdx.y;
    if (d >= head_dim) return;
    const uint32_t pos = pos_ptr ? (uint32_t)*pos_ptr : pos_val;
    if (pos >= max_seq) return;
    const float v = (float)src[(size_t)h * head_dim + d];
    dst[((size_t)h * max_seq + pos) * head_dim + d] = (D)v;
}

template <typename T>
__device__ __forceinline__ float ldf(const T* p, size_t i) { return (float)p[i]; }

// q_len = 1 attention with online softmax (attention.metal:172-308), split over the KV positions.
//   grid (heads, nsplit, batch), 128 threads.  Score phase: lane <-> KV position (32 positions per warp
//   step, full dot product per lane); value phase: lane <-> output dims, probabilities broadcast by
//   shuffle.  nsplit == 1: writes the normalised output; else partial (m, l, o[hd]) per split.
// Eight consecutive cache elements (16-byte aligned: rows are 256 or 512 bytes) as floats.
__device__ __forceinline__ void load8(const __half* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 f = __half22float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// Optional fusion of the rotary embedding and the cache update of the current position into the attention launch
// (decode, f32 q and f16 caches, batch 1): q is rotated while it is loaded, and the CTA whose split holds the current
// position rotates that position's k, rounds k and v to f16 and stores both cache rows before it reads them back.
// Same arithmetic per element as rope_kv_kernel.  k_raw == nullptr: off (q and the caches are used as they are).
struct RopeFuse {
    const float* k_raw;   // [kv_heads][head_dim], not yet rotated
    const float* v_raw;
    float theta;
};

template <typename TQ, typename TKV, typename TO, int DPL>
__global__ void __launch_bounds__(128) decode_attn_kernel(const TQ* __restrict__ Q, const TKV* K,
                                                           const TKV* V, TO* __restrict__ O, float* part,
                                                           uint32_t kv_len_val, const int32_t* pos_ptr, uint32_t heads,
                                                           uint32_t kv_heads, uint32_t kv_head_stride, float scale,
                                                           uint32_t* counters, const RopeFuse rope) {
    grid_dependency_wait();      // inputs come from the previous kernel of the chain
    grid_launch_dependents();
    constexpr int HD = 32 * DPL;
    __shared__ float qs[HD];
    __shared__ float sm_m[4], sm_l[4];
    __shared__ float sm_o[4][HD];
    const uint32_t head = blockIdx.x, split = blockIdx.y, nsplit = gridDim.y, batch = blockIdx.z;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t kv_len = pos_ptr ? (uint32_t)*pos_ptr + 1u : kv_len_val;
    const uint32_t kvh = head / (heads / kv_heads);
    const size_t qbase = ((size_t)batch * heads + head) * HD;
    const size_t kvbase = ((size_t)batch * kv_heads + kvh) * kv_head_stride * HD;
    // a split covers at least 128 positions (one group of 32 per warp): short contexts use few splits, and with a ticket
    // counter the splits beyond the context leave at once (without it they file an empty partial for the combine launch)
    const uint32_t chunk = max(128u, ((kv_len + nsplit - 1) / nsplit + 31) / 32 * 32);
    const uint32_t live = max(1u, (kv_len + chunk - 1) / chunk);
    if (counters && split >= live && split > 0) return;
    const uint32_t beg = split * chunk, end = min(kv_len, beg + chunk);
    bool roped = false;
    if constexpr (std::is_same<TQ, float>::value && std::is_same<TKV, __half>::value) {
        if (rope.k_raw) {
            roped = true;
            const uint32_t d = threadIdx.x, half = HD / 2, pos = kv_len - 1;
            if (d < half) {
                // every load is requested before the trigonometry needs the position
                const float* kp = rope.k_raw + (size_t)kvh * HD;
                const float* vp = rope.v_raw + (size_t)kvh * HD;
                const float a = Q[qbase + d], b = Q[qbase + d + half];
                const float ka = kp[d], kb = kp[d + half], va = vp[d], vb = vp[d + half];
                const float freq = 1.0f / powf(rope.theta, (float)(2 * d) / (float)HD);
                const float angle = (float)pos * freq;
                const float c = cosf(angle), sn = sinf(angle);
                qs[d] = a * c - b * sn;
                qs[d + half] = a * sn + b * c;
                if (pos >= beg && pos < end && pos < kv_head_stride) {
                    // several query heads may share this kv head: they store the same bits
                    __half* kc = const_cast<__half*>(K) + kvbase + (size_t)pos * HD;
                    __half* vc = const_cast<__half*>(V) + kvbase + (size_t)pos * HD;
                    kc[d] = __float2half_rn(ka * c - kb * sn);
                    kc[d + half] = __float2half_rn(ka * sn + kb * c);
                    vc[d] = __float2half_rn(va);
                    vc[d + half] = __float2half_rn(vb);
                }
            }
        }
    }
    if (!roped)
        for (uint32_t d = threadIdx.x; d < HD; d += 128) qs[d] = ldf(Q, qbase + d);
    __syncthreads();   // also orders this CTA's cache stores before its own loads of that row
    // value phase: lane <-> (row parity, 16-byte chunk of the row) where the chunks of a row divide the warp: the rows of a
    // group are fetched by coalesced 16-byte loads that are all in flight together; else lane <-> DPL output dims
    constexpr int CH = HD / 8;                    // 8-element chunks per row
    constexpr bool WIDE = (32 % CH) == 0;
    constexpr int RPI = WIDE ? 32 / CH : 1;       // rows per warp-wide load
    const uint32_t vr_row = lane / CH, vr_col = lane % CH;
    float m = -INFINITY, l = 0.f, o[DPL], o8[8];
#pragma unroll
    for (int i = 0; i < DPL; i++) o[i] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) o8[i] = 0.f;
    for (uint32_t g = beg + 32 * warp; g < end; g += 128) {
        const uint32_t p = g + lane;
        float score = -INFINITY;
        if (p < end) {
            // 16-byte loads of the key row; the two accumulators take even and odd dims in ascending order
            const TKV* kr = K + kvbase + (size_t)p * HD;
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int d = 0; d < HD; d += 8) {   // fully unrolled: all loads of the row are in flight together
                float kv8[8];
                load8(kr + d, kv8);
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                    a0 = fmaf(qs[d + i], kv8[i], a0);
                    a1 = fmaf(qs[d + i + 1], kv8[i + 1], a1);
                }
            }
            score = (a0 + a1) * scale;
        }
        const float m_new = fmaxf(m, warp_max(score));
        const float resc = expf(m - m_new);      // exp(-inf) = 0 on the first group
        const float pe = (p < end) ? expf(score - m_new) : 0.f;
        l = l * resc + warp_sum(pe);
        const uint32_t cnt = min(32u, end - g);
        if constexpr (WIDE) {
#pragma unroll
            for (int i = 0; i < 8; i++) o8[i] *= resc;
            float vv[32 / RPI][8];
#pragma unroll
            for (int t = 0; t < 32 / RPI; t++) {
                const uint32_t j = t * RPI + vr_row;      // rows past the end read row g and get weight 0 (pe is 0 there)
                load8(V + kvbase + (size_t)(g + (j < cnt ? j : 0)) * HD + vr_col * 8, vv[t]);
            }
#pragma unroll
            for (int t = 0; t < 32 / RPI; t++) {
                const float pj = __shfl_sync(0xffffffffu, pe, t * RPI + vr_row);
#pragma unroll
                for (int i = 0; i < 8; i++) o8[i] = fmaf(pj, vv[t][i], o8[i]);
            }
            m = m_new;
            continue;
        }
#pragma unroll
        for (int i = 0; i < DPL; i++) o[i] *= resc;
        // eight value rows are loaded before they are used (positions past the end read row g and get weight 0:
        // pe is 0 there), the accumulation order stays j ascending
        for (uint32_t j0 = 0; j0 < cnt; j0 += 8) {
            float vv[8][DPL];
#pragma unroll
            for (int jj = 0; jj < 8; jj++) {
                const uint32_t j = (j0 + jj < cnt) ? j0 + jj : 0;
                const TKV* vr = V + kvbase + (size_t)(g + j) * HD + lane * DPL;
#pragma unroll
                for (int i = 0; i < DPL; i++) vv[jj][i] = (float)vr[i];
            }
#pragma unroll
            for (int jj = 0; jj < 8; jj++) {
                if (j0 + jj < cnt) {
                    const float pj = __shfl_sync(0xffffffffu, pe, j0 + jj);
#pragma unroll
                    for (int i = 0; i < DPL; i++) o[i] = fmaf(pj, vv[jj][i], o[i]);
                }
            }
        }
        m = m_new;
    }
    // merge the four warps in warp order
    if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
    if constexpr (WIDE) {
        // add the row parities (ascending), then the lanes of parity 0 file their chunk
#pragma unroll
        for (int off = CH; off < 32; off <<= 1)
#pragma unroll
            for (int i = 0; i < 8; i++) o8[i] += __shfl_down_sync(0xffffffffu, o8[i], off);
        if (vr_row == 0) {
#pragma unroll
            for (int i = 0; i < 8; i++) sm_o[warp][vr_col * 8 + i] = o8[i];
        }
    } else {
#pragma unroll
        for (int i = 0; i < DPL; i++) sm_o[warp][lane * DPL + i] = o[i];
    }
    __syncthreads();
    if (warp == 0) {
        float M = fmaxf(fmaxf(sm_m[0], sm_m[1]), fmaxf(sm_m[2], sm_m[3]));
        float Lt = 0.f, acc[DPL];
#pragma unroll
        for (int i = 0; i < DPL; i++) acc[i] = 0.f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const float f = (sm_m[w] == -INFINITY) ? 0.f : expf(sm_m[w] - M);
            Lt += sm_l[w] * f;
#pragma unroll
            for (int i = 0; i < DPL; i++) acc[i] += sm_o[w][lane * DPL + i] * f;
        }
        if (nsplit == 1 || (counters && live == 1)) {
            const float inv = Lt > 0.f ? 1.0f / Lt : 0.f;
#pragma unroll
            for (int i = 0; i < DPL; i++) O[qbase + lane * DPL + i] = (TO)(acc[i] * inv);
        } else {
            float* pp = part + (((size_t)batch * heads + head) * nsplit + split) * (HD + 2);
            if (lane == 0) { pp[0] = M; pp[1] = Lt; }
#pragma unroll
            for (int i = 0; i < DPL; i++) pp[2 + lane * DPL + i] = acc[i];
        }
    }
    // With a ticket counter per (batch, head) the CTA that finishes last merges the partials itself (same order and
    // arithmetic as decode_attn_combine_kernel) and puts the counter back to zero: no second launch.
    if (nsplit > 1 && counters && live > 1) {
        __shared__ uint32_t s_last;
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            s_last = atomicAdd(&counters[batch * heads + head], 1u) == live - 1;
        }
        __syncthreads();
        if (s_last) {
            __threadfence();
            const uint32_t d = threadIdx.x;
            if (d < HD) {
                const float* pp = part + ((size_t)batch * heads + head) * nsplit * (HD + 2);
                float Mx = -INFINITY, L = 0.f, a = 0.f;
                if (live <= 8) {
                    // all partials requested together
                    float ms[8], ls[8], as[8];
#pragma unroll
                    for (uint32_t sp = 0; sp < 8; sp++) {
                        const bool on = sp < live;
                        ms[sp] = on ? __ldcg(pp + sp * (HD + 2)) : -INFINITY;
                        ls[sp] = on ? __ldcg(pp + sp * (HD + 2) + 1) : 0.f;
                        as[sp] = on ? __ldcg(pp + sp * (HD + 2) + 2 + d) : 0.f;
                    }
#pragma unroll
                    for (uint32_t sp = 0; sp < 8; sp++) Mx = fmaxf(Mx, ms[sp]);
#pragma unroll
                    for (uint32_t sp = 0; sp < 8; sp++) {
                        const float f = (ms[sp] == -INFINITY) ? 0.f : expf(ms[sp] - Mx);
                        L += ls[sp] * f;
                        a += as[sp] * f;
                    }
                } else {
                    for (uint32_t sp = 0; sp < live; sp++) Mx = fmaxf(Mx, pp[sp * (HD + 2)]);
                    for (uint32_t sp = 0; sp < live; sp++) {
                        const float ms = pp[sp * (HD + 2)];
                        const float f = (ms == -INFINITY) ? 0.f : expf(ms - Mx);
                        L += pp[sp * (HD + 2) + 1] * f;
                        a += pp[sp * (HD + 2) + 2 + d] * f;
                    }
                }
                O[qbase + d] = (TO)(L > 0.f ? a / L : 0.f);
            }
            if (threadIdx.x == 0) counters[batch * heads + head] = 0;
        }
    }
}

// Merge the per-split partials of one head in split order.
template <typename TO>
__global__ void decode_attn_combine_kernel(const float* __restrict__ part, TO* __restrict__ O, uint32_t nsplit, uint32_t hd) {
    grid_dependency_wait();      // inputs come from the previous kernel of the chain
    grid_launch_dependents();
    const uint32_t bh = blockIdx.x, d = threadIdx.x;
    if (d >= hd) return;
    const float* pp = part + (size_t)bh * nsplit * (hd + 2);
    float M = -INFINITY;
    for (uint32_t s = 0; s < nsplit; s++) M = fmaxf(M, pp[s * (hd + 2)]);
    float L = 0.f, acc = 0.f;
    for (uint32_t s = 0; s < nsplit; s++) {
        const float ms = pp[s * (hd + 2)];
        const float f = (ms == -INFINITY) ? 0.f : expf(ms - M);
        L += pp[s * (hd + 2) + 1] * f;
        acc += pp[s * (hd + 2) + 2 + d] * f;
    }
    O[(size_t)bh * hd + d] = (TO)(L > 0.f ? acc / L : 0.f);
}

// Index of the maximum, lowest index among equal maxima; one CTA of 1024 threads (activation.metal:56-110
// scans the same way but leaves ties unspecified).
template <typename T>
__global__ void __launch_bounds__(1024) argmax_kernel(const T* __restrict__ in, int32_t* __restrict__ result, uint32_t n) {
    grid_dependency_wait();      // inputs come from the previous kernel of the chain
    grid_launch_dependents();
    __shared__ float sv[32];
    __shared__ uint32_t sidx[32];
    float bv = -INFINITY;
    uint32_t bi = 0xFFFFFFFFu;
    for (uint32_t i = threadIdx.x; i < n; i += 1024) {
        const float v = (float)in[i];
        if (v > bv || bi == 0xFFFFFFFFu) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; sidx[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        bv = sv[threadIdx.x];
        bi = sidx[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (threadIdx.x == 0) result[0] = (int32_t)bi;
    }
}

// ───────────────────────── host launchers (shared with decode_model.cu) ─────────────────────────

int32_t launch_rms_norm(runit_ctx* ctx, const float* x, float* y, const void* gamma, bool gamma_f16, float eps,
                        uint32_t hidden, uint32_t rows) {
    if (gamma_f16) runit_launch_chain(ctx, rms_norm_kernel<__half>, dim3(rows), dim3(256), x, y, (const __half*)gamma, eps, hidden);
    else runit_launch_chain(ctx, rms_norm_kernel<float>, dim3(rows), dim3(256), x, y, (const float*)gamma, eps, hidden);
    return runit_after_launch(ctx, "rms_norm");
}

int32_t launch_rope(runit_ctx* ctx, float* q, float* k, uint32_t hd, uint32_t qh, uint32_t kvh, uint32_t pos,
                    const int32_t* pos_ptr, float theta) {
    const uint32_t hmax = qh > kvh ? qh : kvh;
    runit_launch_chain(ctx, rope_qk_kernel, dim3(hmax), dim3(hd / 2), q, k, hd, qh, kvh, pos, pos_ptr, theta);
    return runit_after_launch(ctx, "fused_rope_qk_f32");
}

int32_t launch_rope_kv(runit_ctx* ctx, float* q, float* k, const float* v, void* kcache, void* vcache, uint32_t hd, uint32_t qh,
                       uint32_t kvh, const int32_t* pos_ptr, float theta, uint32_t max_seq) {
    const uint32_t hmax = qh > kvh ? qh : kvh;
    runit_launch_chain(ctx, rope_kv_kernel, dim3(hmax), dim3(hd / 2), q, k, v, (__half*)kcache, (__half*)vcache, hd, qh, kvh, pos_ptr,
                       theta, max_seq);
    return runit_after_launch(ctx, "rope_kv");
}

int32_t launch_kv_copy(runit_ctx* ctx, const void* src, bool src_f16, void* dst, bool dst_f16, uint32_t pos,
                       const int32_t* pos_ptr, uint32_t max_seq, uint32_t hd, uint32_t kvh) {
    dim3 grid((hd + 127) / 128, kvh);
    if (src_f16 && dst_f16) runit_launch_chain(ctx, kv_copy_kernel<__half, __half>, dim3(grid), dim3(128), (const __half*)src, (__half*)dst, pos, pos_ptr, max_seq, hd);
    else if (!src_f16 && !dst_f16) runit_launch_chain(ctx, kv_copy_kernel<float, float>, dim3(grid), dim3(128), (const float*)src, (float*)dst, pos, pos_ptr, max_seq, hd);
    else if (!src_f16 && dst_f16) runit_launch_chain(ctx, kv_copy_kernel<float, __half>, dim3(grid), dim3(128), (const float*)src, (__half*)dst, pos, pos_ptr, max_seq, hd);
    else return runit_fail(ctx, RUNIT_ERR_UNSUPPORTED, "kv_copy: f16 source into an f32 cache");
    return runit_after_launch(ctx, "kv_copy_to_cache");
}

template <typename TQ, typename TKV, typename TO>
static int32_t attn_typed(runit_ctx* ctx, const void* q, const void* k, const void* v, void* out, float* part, uint32_t nsplit,
                          uint32_t batch, uint32_t kv_len, const int32_t* pos_ptr, uint32_t heads, uint32_t kv_heads,
                          uint32_t hd, uint32_t stride, uint32_t* counters, const RopeFuse rope = RopeFuse{nullptr, nullptr, 0.f}) {
    const float scale = 1.0f / sqrtf((float)hd);   // dispatch.rs:1588
    dim3 grid(heads, nsplit, batch);
#define ATTN_CASE(D)                                                                                                   \
    runit_launch_chain(ctx, decode_attn_kernel<TQ, TKV, TO, D>, dim3(grid), dim3(128), (const TQ*)q, (const TKV*)k, (const TKV*)v, (TO*)out, \
                                                                      part, kv_len, pos_ptr, heads, kv_heads, stride, scale, counters, rope)
    switch (hd) {
        case 32: ATTN_CASE(1); break;
        case 64: ATTN_CASE(2); break;
        case 96: ATTN_CASE(3); break;
        case 128: ATTN_CASE(4); break;
        default: return runit_fail(ctx, RUNIT_ERR_UNSUPPORTED, "decode_attention: head_dim %u not in {32,64,96,128}", hd);
    }
#undef ATTN_CASE
    int32_t st = runit_after_launch(ctx, "decode_attention");
    if (st != RUNIT_OK || nsplit == 1 || counters) return st;
    runit_launch_chain(ctx, decode_attn_combine_kernel<TO>, dim3(batch * heads), dim3(hd), part, (TO*)out, nsplit, hd);
    return runit_after_launch(ctx, "decode_attention_combine");
}

int32_t launch_decode_attention(runit_ctx* ctx, int q_kind, int kv_kind, const void* q, const void* k, const void* v, void* out,
                                float* part, uint32_t nsplit, uint32_t batch, uint32_t kv_len, const int32_t* pos_ptr,
                                uint32_t heads, uint32_t kv_heads, uint32_t hd, uint32_t stride, uint32_t* counters) {
    RUNIT_REQUIRE(ctx, runit_aligned(k, 16) && runit_aligned(v, 16), "decode_attention: key/value cache must be 16-byte aligned");
    if (q_kind == 0 && kv_kind == 0)
        return attn_typed<float, float, float>(ctx, q, k, v, out, part, nsplit, batch, kv_len, pos_ptr, heads, kv_heads, hd, stride, counters);
    if (q_kind == 1 && kv_kind == 1)
        return attn_typed<__half, __half, __half>(ctx, q, k, v, out, part, nsplit, batch, kv_len, pos_ptr, heads, kv_heads, hd, stride, counters);
    if (q_kind == 0 && kv_kind == 1)
        return attn_typed<float, __half, float>(ctx, q, k, v, out, part, nsplit, batch, kv_len, pos_ptr, heads, kv_heads, hd, stride, counters);
    return runit_fail(ctx, RUNIT_ERR_UNSUPPORTED, "decode_attention: f16 query with f32 cache");
}

// Decode step of the greedy model: rotary embedding of q and k, cache update and attention in one launch (batch 1, f32 q,
// f16 caches; the position comes from the device word pos_ptr).
int32_t launch_decode_attention_rope(runit_ctx* ctx, const float* q, const float* k_raw, const float* v_raw, void* kcache, void* vcache,
                                     float* out, float* part, uint32_t nsplit, const int32_t* pos_ptr, uint32_t heads, uint32_t kv_heads,
                                     uint32_t hd, uint32_t max_seq, float theta, uint32_t* counters) {
    RUNIT_REQUIRE(ctx, q && k_raw && v_raw && kcache && vcache && out && pos_ptr, "decode_attention_rope: null pointer");
    RUNIT_REQUIRE(ctx, runit_aligned(kcache, 16) && runit_aligned(vcache, 16), "decode_attention_rope: caches must be 16-byte aligned");
    RUNIT_REQUIRE(ctx, hd == 128 || hd == 64, "decode_attention_rope: head_dim %u unsupported (threads cover half a head)", hd);
    return attn_typed<float, __half, float>(ctx, q, kcache, vcache, out, part, nsplit, 1, 0, pos_ptr, heads, kv_heads, hd, max_seq, counters,
                                            RopeFuse{k_raw, v_raw, theta});
}

int32_t launch_argmax(runit_ctx* ctx, const void* in, bool in_f16, int32_t* result, uint32_t n) {
    if (in_f16) runit_launch_chain(ctx, argmax_kernel<__half>, dim3(1), dim3(1024), (const __half*)in, result, n);
    else runit_launch_chain(ctx, argmax_kernel<float>, dim3(1), dim3(1024), (const float*)in, result, n);
    return runit_after_launch(ctx, "argmax");
}

}  // namespace runit

using namespace runit;

extern "C" {

int32_t runit_rms_norm_f32_f32(runit_ctx_t* ctx, const void* x, void* y, const void* gamma, float eps, uint32_t hidden,
                               uint32_t num_rows) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, x && y && gamma && hidden > 0 && num_rows > 0, "rms_norm_f32_f32: bad argument");
    return launch_rms_norm(ctx, (const float*)x, (float*)y, gamma, true, eps, hidden, num_rows);
}

int32_t runit_rms_norm_f32_f32_f32g(runit_ctx_t* ctx, const void* x, void* y, const void* gamma, float eps, uint32_t hidden,
                                    uint32_t num_rows) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, x && y && gamma && hidden > 0 && num_rows > 0, "rms_norm_f32_f32_f32g: bad argument");
    return launch_rms_norm(ctx, (const float*)x, (float*)y, gamma, false, eps, hidden, num_rows);
}

int32_t runit_fused_rope_qk_f32(runit_ctx_t* ctx, void* q, void* k, uint32_t head_dim, uint32_t q_heads, uint32_t kv_heads,
                                uint32_t pos, float theta) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, q && k && head_dim >= 2 && head_dim % 2 == 0 && head_dim <= 2048 && (q_heads > 0 || kv_heads > 0),
                  "fused_rope_qk_f32: bad argument");
    return launch_rope(ctx, (float*)q, (float*)k, head_dim, q_heads, kv_heads, pos, nullptr, theta);
}

int32_t runit_kv_copy_to_cache_f16(runit_ctx_t* ctx, const void* src, void* dst, uint32_t pos, uint32_t max_seq,
                                   uint32_t head_dim, uint32_t num_kv_heads) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, src && dst && head_dim > 0 && num_kv_heads > 0, "kv_copy_to_cache_f16: bad argument");
    RUNIT_REQUIRE(ctx, pos < max_seq, "kv_copy_to_cache_f16: pos %u >= max_seq %u", pos, max_seq);   // kv_cache.rs:63
    return launch_kv_copy(ctx, src, true, dst, true, pos, nullptr, max_seq, head_dim, num_kv_heads);
}

int32_t runit_kv_copy_to_cache_f32(runit_ctx_t* ctx, const void* src, void* dst, uint32_t pos, uint32_t max_seq,
                                   uint32_t head_dim, uint32_t num_kv_heads) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, src && dst && head_dim > 0 && num_kv_heads > 0, "kv_copy_to_cache_f32: bad argument");
    RUNIT_REQUIRE(ctx, pos < max_seq, "kv_copy_to_cache_f32: pos %u >= max_seq %u", pos, max_seq);
    return launch_kv_copy(ctx, src, false, dst, false, pos, nullptr, max_seq, head_dim, num_kv_heads);
}

int32_t runit_kv_copy_to_cache_f32_f16(runit_ctx_t* ctx, const void* src, void* dst, uint32_t pos, uint32_t max_seq,
                                       uint32_t head_dim, uint32_t num_kv_heads) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, src && dst && head_dim > 0 && num_kv_heads > 0, "kv_copy_to_cache_f32_f16: bad argument");
    RUNIT_REQUIRE(ctx, pos < max_seq, "kv_copy_to_cache_f32_f16: pos %u >= max_seq %u", pos, max_seq);
    return launch_kv_copy(ctx, src, false, dst, true, pos, nullptr, max_seq, head_dim, num_kv_heads);
}

#define ATTN_ENTRY(NAME, QK, KVK)                                                                                        \
    int32_t runit_##NAME(runit_ctx_t* ctx, const void* q, const void* k, const void* v, void* out, uint32_t batch,       \
                         uint32_t kv_len, uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_dim,                   \
                         uint32_t kv_head_stride) {                                                                      \
        if (!ctx) return RUNIT_ERR_BAD_ARG;                                                                              \
        RUNIT_REQUIRE(ctx, q && k && v && out, #NAME ": null pointer");                                                  \
        RUNIT_REQUIRE(ctx, batch > 0 && kv_len > 0 && num_heads > 0 && num_kv_heads > 0 && num_heads % num_kv_heads == 0, \
                      #NAME ": bad shape");                                                                              \
        RUNIT_REQUIRE(ctx, kv_len <= kv_head_stride, #NAME ": kv_len %u exceeds the cache stride %u", kv_len, kv_head_stride); \
        return launch_decode_attention(ctx, QK, KVK, q, k, v, out, nullptr, 1, batch, kv_len, nullptr, num_heads,        \
                                       num_kv_heads, head_dim, kv_head_stride, nullptr);                                 \
    }
ATTN_ENTRY(decode_attention_f32, 0, 0)
ATTN_ENTRY(decode_attention_f16, 1, 1)
ATTN_ENTRY(decode_attention_f32q_f16kv, 0, 1)

int32_t runit_argmax_f16(runit_ctx_t* ctx, const void* input, void* result, uint32_t n) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, input && result && n > 0, "argmax_f16: bad argument");
    return launch_argmax(ctx, input, true, (int32_t*)result, n);
}

int32_t runit_argmax_f32(runit_ctx_t* ctx, const void* input, void* result, uint32_t n) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, input && result && n > 0, "argmax_f32: bad argument");
    return launch_argmax(ctx, input, false, (int32_t*)result, n);
}

}  // extern "C"
