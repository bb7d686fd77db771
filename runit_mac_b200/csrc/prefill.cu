// Batched prefill: the whole prompt in one pass, GEMMs instead of one GEMV per token (crates/engine/src/prefill.rs:29-255).
//
// The reference's pass runs in f16 with dequantised f16 weights: per layer RMSNorm, three projection GEMMs
// (gemm.metal:39,149: 16x16 scalar tiles), batched RoPE, a host loop that copies K and V into the cache, causal
// FlashAttention with q_len = seq (attention.metal:36-158), the output GEMM, the residual add, the second RMSNorm, and for
// a mixture-of-experts model the decode block once per token (prefill.rs:156-215).  Here:
//   * the hidden state stays f32 between operators (as in this library's decode path); GEMM operands are bf16: the
//     activations are rounded once, the weights are dequantised from Q4_K to bf16 tiles inside the tcgen05 GEMM of
//     moe_grouped.cu, used with one "expert" that owns the whole matrix and the tokens in their own order;
//   * RoPE of q and k, the f16 rounding of k and v and their scatter into the cache are one launch over all positions;
//   * causal attention over the f16 cache is a tensor-core kernel (below); its output is written as bf16, the operand of
//     the output GEMM;
//   * the mixture-of-experts block is runit_moe_layer_q4k_bf16 on all tokens at once;
//   * the last position's hidden state then goes through the decode path's lm_head launch (RMSNorm prologue, argmax
//     epilogue), and the decoder's state is left at position n with that token, so decoding continues from the cache.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "decode_ops.cuh"
#include "gemv_common.cuh"
#include "runit_internal.h"

namespace runit {
namespace pf {

// x[t][:] = emb[token[t]][:]
__global__ void __launch_bounds__(256) embed_rows_kernel(const float* __restrict__ emb, const int32_t* __restrict__ tokens,
                                                          float* __restrict__ x, uint32_t h) {
    const uint32_t t = blockIdx.x;
    const float4* src = reinterpret_cast<const float4*>(emb + (size_t)tokens[t] * h);
    float4* dst = reinterpret_cast<float4*>(x + (size_t)t * h);
    for (uint32_t i = threadIdx.x; i < h / 4; i += 256) dst[i] = src[i];
}

// y[t][:] = bf16(x[t][:] * rsqrt(mean(x[t]^2) + eps) * gamma)   (norm.metal:95-154, same sum order as rms_norm_kernel)
__global__ void __launch_bounds__(256) rms_norm_bf16_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                             __nv_bfloat16* __restrict__ y, float eps, uint32_t h) {
    __shared__ float part[8];
    const float* row = x + (size_t)blockIdx.x * h;
    __nv_bfloat16* out = y + (size_t)blockIdx.x * h;
    float s = 0.f;
    for (uint32_t i = threadIdx.x; i < h; i += 256) {
        const float v = row[i];
        s = fmaf(v, v, s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += part[i];
    const float r = rsqrtf(tot / (float)h + eps);
    for (uint32_t i = threadIdx.x; i < h; i += 256) out[i] = __float2bfloat16_rn(row[i] * r * gamma[i]);
}

// Rotary embedding of q (in place) and k for every position, then k (rotated) and v into the f16 caches: the arithmetic
// per element of rope_kv_kernel (fused_rope.metal:17-56, activation.metal:13-44).  grid (T, max(heads, kv_heads)).
// q_in / k / v: rows of `ld` floats (one matrix [T][q | k | v] when the three projections were one GEMM, ld = its width;
// or three matrices with ld = 0: rows as wide as their own heads); q_out: [T][heads * hd], may be q_in when ld = 0.
__global__ void rope_cache_rows_kernel(const float* q_in, float* q_out, const float* __restrict__ k, const float* __restrict__ v,
                                       __half* __restrict__ kc, __half* __restrict__ vc, uint32_t hd, uint32_t heads, uint32_t kv_heads,
                                       uint32_t start_pos, float theta, uint32_t max_seq, uint32_t ld) {
    const uint32_t t = blockIdx.x, hid = blockIdx.y, d = threadIdx.x, half = hd / 2;
    if (d >= half) return;
    const uint32_t pos = start_pos + t;
    const float freq = 1.0f / powf(theta, (float)(2 * d) / (float)hd);
    const float angle = (float)pos * freq;
    const float c = cosf(angle), s = sinf(angle);
    if (hid < heads) {
        const float* pi = q_in + (size_t)t * (ld ? ld : heads * hd) + (size_t)hid * hd;
        float* p = q_out + ((size_t)t * heads + hid) * hd;
        const float a = pi[d], b = pi[d + half];
        p[d] = a * c - b * s;
        p[d + half] = a * s + b * c;
    }
    if (hid < kv_heads && pos < max_seq) {
        const float* p = k + (size_t)t * (ld ? ld : kv_heads * hd) + (size_t)hid * hd;
        const float a = p[d], b = p[d + half];
        const size_t o = ((size_t)hid * max_seq + pos) * hd;
        kc[o + d] = __float2half_rn(a * c - b * s);
        kc[o + d + half] = __float2half_rn(a * s + b * c);
        const float* vp = v + (size_t)t * (ld ? ld : kv_heads * hd) + (size_t)hid * hd;
        vc[o + d] = __float2half_rn(vp[d]);
        vc[o + d + half] = __float2half_rn(vp[d + half]);
    }
}

// y[t][:] = bf16(x[t][:])
__global__ void __launch_bounds__(256) to_bf16_rows_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, size_t n4) {
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n4) return;
    const float4 a = reinterpret_cast<const float4*>(x)[i];
    __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(y) + 2 * i;
    o[0] = __floats2bfloat162_rn(a.x, a.y);
    o[1] = __floats2bfloat162_rn(a.z, a.w);
}

// x[t][:] += y[t][:]
__global__ void __launch_bounds__(256) add_rows_kernel(float* __restrict__ x, const float* __restrict__ y, size_t n4) {
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n4) return;
    float4 a = reinterpret_cast<float4*>(x)[i];
    const float4 b = reinterpret_cast<const float4*>(y)[i];
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    reinterpret_cast<float4*>(x)[i] = a;
}

// x[t][:] += y[t][:], then out[t][:] = x[t][:] * rsqrt(mean(x[t]^2) + eps) * gamma: the residual add after the o-projection
// and the RMSNorm in front of the feed-forward block as one launch, one CTA per token; the norm's arithmetic is
// rms_norm_kernel's (thread order, shuffle tree, part[0..7] in order), so the bits are those of the two launches.
__global__ void __launch_bounds__(256) add_rms_norm_rows_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ gamma,
                                                                 float* __restrict__ out, float eps, uint32_t hidden) {
    __shared__ float part[8];
    float* row = x + (size_t)blockIdx.x * hidden;
    const float* add = y + (size_t)blockIdx.x * hidden;
    float* o = out + (size_t)blockIdx.x * hidden;
    float s = 0.f;
    for (uint32_t i = threadIdx.x; i < hidden; i += 256) {
        const float v = row[i] + add[i];
        row[i] = v;
        s = fmaf(v, v, s);
    }
#pragma unroll
    for (int k = 16; k > 0; k >>= 1) s += __shfl_xor_sync(0xffffffffu, s, k);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += part[i];
    const float r = rsqrtf(tot / (float)hidden + eps);
    for (uint32_t i = threadIdx.x; i < hidden; i += 256) o[i] = row[i] * r * gamma[i];     // each thread re-reads what it stored
}

// ───────────────────────── causal attention over the f16 cache, tensor cores ─────────────────────────
// softmax(q.K^T / sqrt(hd)) . V with the causal mask key <= start_pos + query (attention.metal:36-158), online softmax.
//   grid (heads, ceil(T / 64)), 4 warps; a warp owns 16 queries, the CTA walks the keys in blocks of 64.
//   q (f32) is rounded to f16 and kept as MMA A fragments; K and V blocks are staged in shared memory by cp.async, two
//   stages deep (rows padded to HD + 8 halves: ldmatrix reads without bank conflicts); S = q.K^T and O += P.V are mma.sync m16n8k16 (f16 operands,
//   f32 accumulators); P is rounded to f16 for the second product, the usual flash-attention arrangement.
//   Output bf16 [T][heads * HD]: the B operand of the output projection GEMM.
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

template <int HD>
__global__ void __launch_bounds__(128, 3) prefill_attn_kernel(const float* __restrict__ q, const __half* __restrict__ kc,
                                                            const __half* __restrict__ vc, __nv_bfloat16* __restrict__ out, uint32_t T,
                                                            uint32_t heads, uint32_t kv_heads, uint32_t max_seq, uint32_t start_pos,
                                                            float scale) {
    constexpr int LDS = HD + 8;                  // row pitch in halves
    constexpr int KS = HD / 16;                  // k16 steps of q.K^T
    constexpr int ND = HD / 8;                   // n8 tiles of the output
    // two stages of (K block, V block): the next block is copied (cp.async) while the current one is multiplied
    extern __shared__ __align__(16) uint8_t attn_smem[];
    __half* const Ks = reinterpret_cast<__half*>(attn_smem);                    // [2][64 * LDS]
    __half* const Vs = Ks + 2 * 64 * LDS;                                      // [2][64 * LDS]
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const uint32_t head = blockIdx.x, kvh = head / (heads / kv_heads);
    // the last query blocks see the most keys: they are scheduled first (longest first), so that the short ones fill the tail
    const uint32_t q0 = (gridDim.y - 1 - blockIdx.y) * 64, ld = heads * HD;
    const uint32_t row_a = q0 + warp * 16 + g, row_b = row_a + 8;     // this thread's two query rows
    const __half* kbase = kc + (size_t)kvh * max_seq * HD;
    const __half* vbase = vc + (size_t)kvh * max_seq * HD;

    uint32_t qa[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
        const uint32_t c0 = head * HD + ks * 16 + 2 * t;
        const float2 z = make_float2(0.f, 0.f);
        const float2 a0 = row_a < T ? *reinterpret_cast<const float2*>(q + (size_t)row_a * ld + c0) : z;
        const float2 a1 = row_b < T ? *reinterpret_cast<const float2*>(q + (size_t)row_b * ld + c0) : z;
        const float2 a2 = row_a < T ? *reinterpret_cast<const float2*>(q + (size_t)row_a * ld + c0 + 8) : z;
        const float2 a3 = row_b < T ? *reinterpret_cast<const float2*>(q + (size_t)row_b * ld + c0 + 8) : z;
        qa[ks][0] = pack_h2(a0.x, a0.y);
        qa[ks][1] = pack_h2(a1.x, a1.y);
        qa[ks][2] = pack_h2(a2.x, a2.y);
        qa[ks][3] = pack_h2(a3.x, a3.y);
    }
    float o[ND][4];
#pragma unroll
    for (int nd = 0; nd < ND; nd++) { o[nd][0] = 0.f; o[nd][1] = 0.f; o[nd][2] = 0.f; o[nd][3] = 0.f; }
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

    const uint32_t kv_total = start_pos + T;                                   // cache rows that hold data
    const uint32_t last_q = min(T, q0 + 64) - 1;
    const uint32_t n_blocks = (start_pos + last_q) / 64 + 1;                   // key blocks any query of this CTA may see
    // stage K and V rows kb*64 .. +63 into buffer `buf` (rows past the data are zeros)
    auto stage = [&](uint32_t kb, uint32_t buf) {
        constexpr int CPR = HD / 8;                                            // 16-byte chunks per row
        __half* kd = Ks + buf * 64 * LDS;
        __half* vd = Vs + buf * 64 * LDS;
        for (uint32_t c = tid; c < 64 * CPR; c += 128) {
            const uint32_t r = c / CPR, cc = c % CPR, key = kb * 64 + r;
            if (key < kv_total && key < max_seq) {
                cp_async16(smem_u32(kd + r * LDS + cc * 8), kbase + (size_t)key * HD + cc * 8);
                cp_async16(smem_u32(vd + r * LDS + cc * 8), vbase + (size_t)key * HD + cc * 8);
            } else {
                *reinterpret_cast<uint4*>(kd + r * LDS + cc * 8) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(vd + r * LDS + cc * 8) = make_uint4(0, 0, 0, 0);
            }
        }
        cp_async_commit();
    };
    stage(0, 0);
    for (uint32_t kb = 0; kb < n_blocks; kb++) {
        if (kb + 1 < n_blocks) {
            stage(kb + 1, (kb + 1) & 1);       // its buffer was released by the barrier that ended block kb - 1
            cp_async_wait<1>();                // block kb has landed (for this thread's copies)
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();                       // ... and for everyone's
        const uint32_t ks_u32 = smem_u32(Ks + (kb & 1) * 64 * LDS), vs_u32 = smem_u32(Vs + (kb & 1) * 64 * LDS);
        // S = q.K^T for 64 keys: 8 n-tiles of 8 keys
        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
            s[nt][0] = 0.f; s[nt][1] = 0.f; s[nt][2] = 0.f; s[nt][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KS; ks += 2) {
                // four 8x8 matrices: keys nt*8.., columns ks*16 + {0, 8, 16, 24}: the B fragments of two k16 steps
                uint32_t b[4];
                ldsm_x4(b, ks_u32 + ((nt * 8 + (lane & 7)) * LDS + ks * 16 + (lane >> 3) * 8) * 2);
                mma_f16(s[nt], qa[ks], b[0], b[1]);
                mma_f16(s[nt], qa[ks + 1], b[2], b[3]);
            }
        }
        // scale, causal mask, running maximum
        float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
            const uint32_t key0 = kb * 64 + nt * 8 + 2 * t;
            s[nt][0] = key0 <= start_pos + row_a ? s[nt][0] * scale : -INFINITY;
            s[nt][1] = key0 + 1 <= start_pos + row_a ? s[nt][1] * scale : -INFINITY;
            s[nt][2] = key0 <= start_pos + row_b ? s[nt][2] * scale : -INFINITY;
            s[nt][3] = key0 + 1 <= start_pos + row_b ? s[nt][3] * scale : -INFINITY;
            mx_a = fmaxf(mx_a, fmaxf(s[nt][0], s[nt][1]));
            mx_b = fmaxf(mx_b, fmaxf(s[nt][2], s[nt][3]));
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
        // a row that has seen no key yet keeps m = -inf: its factors are taken as 0 (exp(-inf - -inf) would be NaN)
        const float ca = mn_a == -INFINITY ? 0.f : expf(m_a - mn_a), cb = mn_b == -INFINITY ? 0.f : expf(m_b - mn_b);
        float sum_a = 0.f, sum_b = 0.f;
        uint32_t pa[4][4];                                                     // P as A fragments of four k16 steps
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
            const float p0 = mn_a == -INFINITY ? 0.f : expf(s[nt][0] - mn_a), p1 = mn_a == -INFINITY ? 0.f : expf(s[nt][1] - mn_a);
            const float p2 = mn_b == -INFINITY ? 0.f : expf(s[nt][2] - mn_b), p3 = mn_b == -INFINITY ? 0.f : expf(s[nt][3] - mn_b);
            sum_a += p0 + p1;
            sum_b += p2 + p3;
            pa[nt >> 1][(nt & 1) * 2] = pack_h2(p0, p1);
            pa[nt >> 1][(nt & 1) * 2 + 1] = pack_h2(p2, p3);
        }
        l_a = l_a * ca + sum_a;
        l_b = l_b * cb + sum_b;
        m_a = mn_a;
        m_b = mn_b;
#pragma unroll
        for (int nd = 0; nd < ND; nd++) { o[nd][0] *= ca; o[nd][1] *= ca; o[nd][2] *= cb; o[nd][3] *= cb; }
        // O += P.V: per k16 step (16 keys) and pair of n-tiles one transposed load of V
#pragma unroll
        for (int kt = 0; kt < 4; kt++) {
#pragma unroll
            for (int nd = 0; nd < ND; nd += 2) {
                uint32_t b[4];
                ldsm_x4_trans(b, vs_u32 + ((kt * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LDS + nd * 8 + (lane >> 4) * 8) * 2);
                mma_f16(o[nd], pa[kt], b[0], b[1]);
                mma_f16(o[nd + 1], pa[kt], b[2], b[3]);
            }
        }
        __syncthreads();                       // every warp is done with buffer kb & 1: block kb + 2 may overwrite it
    }
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    const float ia = l_a > 0.f ? 1.0f / l_a : 0.f, ib = l_b > 0.f ? 1.0f / l_b : 0.f;
#pragma unroll
    for (int nd = 0; nd < ND; nd++) {
        const uint32_t col = head * HD + nd * 8 + 2 * t;
        if (row_a < T) *reinterpret_cast<__nv_bfloat162*>(out + (size_t)row_a * ld + col) = __floats2bfloat162_rn(o[nd][0] * ia, o[nd][1] * ia);
        if (row_b < T) *reinterpret_cast<__nv_bfloat162*>(out + (size_t)row_b * ld + col) = __floats2bfloat162_rn(o[nd][2] * ib, o[nd][3] * ib);
    }
}

}  // namespace pf
}  // namespace runit

// ───────────────────────── launchers (used by the decoder's prefill) ─────────────────────────
namespace runit {

int32_t prefill_embed(runit_ctx* ctx, const float* emb, const int32_t* tokens, float* x, uint32_t T, uint32_t h) {
    pf::embed_rows_kernel<<<T, 256, 0, ctx->stream>>>(emb, tokens, x, h);
    return runit_after_launch(ctx, "prefill_embed");
}

int32_t prefill_norm_bf16(runit_ctx* ctx, const float* x, const float* gamma, void* y_bf16, float eps, uint32_t T, uint32_t h) {
    pf::rms_norm_bf16_kernel<<<T, 256, 0, ctx->stream>>>(x, gamma, (__nv_bfloat16*)y_bf16, eps, h);
    return runit_after_launch(ctx, "prefill_rms_norm_bf16");
}

int32_t prefill_rope_cache(runit_ctx* ctx, const float* q_in, float* q_out, const float* k, const float* v, void* kcache, void* vcache,
                           uint32_t hd, uint32_t heads, uint32_t kv_heads, uint32_t start_pos, float theta, uint32_t max_seq, uint32_t T,
                           uint32_t ld) {
    const uint32_t hmax = heads > kv_heads ? heads : kv_heads;
    pf::rope_cache_rows_kernel<<<dim3(T, hmax), hd / 2, 0, ctx->stream>>>(q_in, q_out, k, v, (__half*)kcache, (__half*)vcache, hd, heads,
                                                                           kv_heads, start_pos, theta, max_seq, ld);
    return runit_after_launch(ctx, "prefill_rope_cache");
}

int32_t prefill_attention(runit_ctx* ctx, const float* q, const void* kcache, const void* vcache, void* out_bf16, uint32_t T, uint32_t heads,
                          uint32_t kv_heads, uint32_t hd, uint32_t max_seq, uint32_t start_pos) {
    RUNIT_REQUIRE(ctx, hd == 128 || hd == 64, "prefill_attention: head_dim %u unsupported (64 or 128)", hd);
    RUNIT_REQUIRE(ctx, T > 0 && heads % kv_heads == 0 && (uint64_t)start_pos + T <= max_seq, "prefill_attention: bad shape");
    const float scale = 1.0f / sqrtf((float)hd);
    const dim3 grid(heads, (T + 63) / 64);      // heads fastest: the launch order walks the query blocks from the last (most keys) to the first
    const size_t smem = (size_t)4 * 64 * (hd + 8) * 2;      // two stages of a K and a V block
    static bool configured[64] = {false};
    if (ctx->device >= 0 && ctx->device < 64 && !configured[ctx->device]) {
        RUNIT_CUDA_TRY(ctx, cudaFuncSetAttribute(pf::prefill_attn_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 64 * 136 * 2));
        RUNIT_CUDA_TRY(ctx, cudaFuncSetAttribute(pf::prefill_attn_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 64 * 72 * 2));
        configured[ctx->device] = true;
    }
    if (hd == 128)
        pf::prefill_attn_kernel<128><<<grid, 128, smem, ctx->stream>>>(q, (const __half*)kcache, (const __half*)vcache, (__nv_bfloat16*)out_bf16, T,
                                                                    heads, kv_heads, max_seq, start_pos, scale);
    else
        pf::prefill_attn_kernel<64><<<grid, 128, smem, ctx->stream>>>(q, (const __half*)kcache, (const __half*)vcache, (__nv_bfloat16*)out_bf16, T,
                                                                   heads, kv_heads, max_seq, start_pos, scale);
    return runit_after_launch(ctx, "prefill_attention");
}

int32_t prefill_add_rms_norm(runit_ctx* ctx, float* x, const float* y, const float* gamma, float* out, float eps, uint32_t T, uint32_t h) {
    pf::add_rms_norm_rows_kernel<<<T, 256, 0, ctx->stream>>>(x, y, gamma, out, eps, h);
    return runit_after_launch(ctx, "prefill_add_rms_norm");
}

int32_t prefill_add_rows(runit_ctx* ctx, float* x, const float* y, size_t n) {
    const size_t n4 = n / 4;
    pf::add_rows_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, ctx->stream>>>(x, y, n4);
    return runit_after_launch(ctx, "prefill_add_rows");
}

}  // namespace runit

using namespace runit;

extern "C" {

// Dense feed-forward block of a prefill pass (prefill.rs:217-227: gate GEMM, up GEMM, silu_mul, down GEMM, residual add) on
// the tensor cores: out[t] = residual[t] + Wd . bf16(silu(Wg . xb[t]) * (Wu . xb[t])), xb = bf16(x) or, with gamma,
// bf16(RMSNorm(x) * gamma).  The two GEMM launches of moe_grouped.cu with one "expert" that owns the whole matrices.
size_t runit_ffn_q4k_bf16_scratch_bytes(uint32_t T, uint32_t h, uint32_t ff) {
    const size_t rows = ((size_t)T + 255) / 256 * 256 + 256, tiles = ((size_t)T + 255) / 256;
    auto up = [](size_t v) { return (v + 1023) & ~(size_t)1023; };
    return up(4 * (3 * tiles + 4)) + up(rows * h * 2) + up(rows * ff * 2) + up((size_t)T * h * 4);
}

int32_t runit_ffn_q4k_bf16(runit_ctx_t* ctx, const void* w_gate, const void* w_up, const void* w_down, const void* x, const void* gamma,
                           float eps, const void* residual, void* out, void* scratch, size_t scratch_bytes, uint32_t T, uint32_t h,
                           uint32_t ff) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, w_gate && w_up && w_down && x && out && scratch && T > 0, "ffn_q4k_bf16: null pointer or no tokens");
    RUNIT_REQUIRE(ctx, h % 256 == 0 && ff % 256 == 0 && h > 0 && ff > 0, "ffn_q4k_bf16: hidden %u and intermediate %u must be multiples of 256", h, ff);
    RUNIT_REQUIRE(ctx, runit_aligned(scratch, 1024) && runit_aligned(x, 16) && runit_aligned(out, 16) && (!residual || runit_aligned(residual, 16)) &&
                           runit_aligned(w_gate, 16) && runit_aligned(w_up, 16) && runit_aligned(w_down, 16),
                  "ffn_q4k_bf16: scratch must be 1024-byte aligned, tensors 16-byte aligned");
    if (runit_ffn_q4k_bf16_scratch_bytes(T, h, ff) > scratch_bytes)
        return runit_fail(ctx, RUNIT_ERR_BUFFER_SIZE, "ffn_q4k_bf16: scratch has %zu bytes, needs %zu", scratch_bytes,
                          runit_ffn_q4k_bf16_scratch_bytes(T, h, ff));
    const size_t rows = ((size_t)T + 255) / 256 * 256 + 256, tiles = ((size_t)T + 255) / 256;
    auto up = [](size_t v) { return (v + 1023) & ~(size_t)1023; };
    uint8_t* p = (uint8_t*)scratch;
    int32_t* tables = (int32_t*)p;              p += up(4 * (3 * tiles + 4));
    void* xb = p;                               p += up(rows * h * 2);
    void* act = p;                              p += up(rows * ff * 2);
    float* y = (float*)p;
    int32_t st;
    if ((st = dense_tiles_prepare(ctx, tables, T))) return st;
    if (gamma) {
        if ((st = prefill_norm_bf16(ctx, (const float*)x, (const float*)gamma, xb, eps, T, h))) return st;
    } else {
        const size_t n4 = (size_t)T * h / 4;
        pf::to_bf16_rows_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, ctx->stream>>>((const float*)x, (__nv_bfloat16*)xb, n4);
        if ((st = runit_after_launch(ctx, "ffn_to_bf16"))) return st;
    }
    if ((st = dense_gemm_q4k_bf16(ctx, "ffn_gate_up", w_gate, w_up, ff, h, xb, (uint32_t)rows, act, ff, T, tables))) return st;
    float* dst = residual ? y : (float*)out;
    if ((st = dense_gemm_q4k_bf16(ctx, "ffn_down", w_down, nullptr, h, ff, act, (uint32_t)rows, dst, h, T, tables))) return st;
    if (!residual) return RUNIT_OK;
    if (residual != out) RUNIT_CUDA_TRY(ctx, cudaMemcpyAsync(out, residual, (size_t)T * h * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    return prefill_add_rows(ctx, (float*)out, y, (size_t)T * h);
}

// Stand-alone entry of the attention kernel (tests, other callers): q f32 [T][heads*hd] already rotated, caches f16
// [kv_heads][max_seq][hd] holding positions 0 .. start_pos + T - 1, out bf16 [T][heads*hd].
int32_t runit_prefill_attention_f16kv(runit_ctx_t* ctx, const void* q, const void* kcache, const void* vcache, void* out_bf16, uint32_t T,
                                      uint32_t heads, uint32_t kv_heads, uint32_t head_dim, uint32_t max_seq, uint32_t start_pos) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, q && kcache && vcache && out_bf16 && kv_heads > 0, "prefill_attention_f16kv: null pointer");
    RUNIT_REQUIRE(ctx, runit_aligned(q, 16) && runit_aligned(kcache, 16) && runit_aligned(vcache, 16) && runit_aligned(out_bf16, 16),
                  "prefill_attention_f16kv: tensors must be 16-byte aligned");
    return prefill_attention(ctx, (const float*)q, kcache, vcache, out_bf16, T, heads, kv_heads, head_dim, max_seq, start_pos);
}

}  // extern "C"
