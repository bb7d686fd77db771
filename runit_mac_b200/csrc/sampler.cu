// Token sampling on the device: repetition penalty, temperature, softmax, top-k, top-p and the draw, in one launch of one
// CTA, so that a decode step needs no host round trip for its logits.  Follows the reference's host sampler
// (crates/engine/src/sampler.rs:61-111 and its helpers :114-168) step by step:
//   0a  context shorter than min_tokens: the end-of-sequence ids get -inf                      (sampler.rs:64-71)
//   0b  repetition penalty, once per OCCURRENCE of a token in the context: positive scores are divided by the penalty,
//       the others multiplied                                                                   (sampler.rs:74-76, 124-135)
//       temperature == 0: argmax of the scores, the LAST index among equal maxima (Iterator::max_by) (sampler.rs:79, 114-119)
//   1   scores /= temperature                                                                   (sampler.rs:82)
//   2   softmax: exp(s - max) / sum                                                             (sampler.rs:137-142)
//   3   top-k: threshold = k-th largest probability; the first k entries IN INDEX ORDER with p >= threshold stay (sampler.rs:144-152)
//   4   top-p: in descending order of probability entries stay until the running sum has reached p (sampler.rs:154-162)
//   5   total = sum of what is left; r = rng * total; the first index whose running sum reaches r (sampler.rs:98-110)
// Generator: xorshift64 with the reference's seeding and its u64 -> [0, 1] float conversion (sampler.rs:12-27).
//
// What differs from the host code: the softmax sum over the vocabulary is a tree sum (the reference adds sequentially), and
// expf is the device's; probabilities agree to rounding, so a draw can differ where r falls within rounding of a boundary.
// Steps 3-5 then run on at most 1024 surviving entries: their sorts, running sums and the draw are sequential in the
// reference's order.  Entries with equal probability are ordered by index in step 4 (the reference's unstable sort leaves
// that open).  Limits: top_k <= 1024; with top-k off and top_p < 1 the nucleus must lie within the 1024 most probable
// tokens, else the launch reports status 4 and returns the most probable token.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>

#include "runit_internal.h"
#include "tma.cuh"

namespace runit {

constexpr int kST = 1024;          // threads of the sampling CTA
constexpr uint32_t kCand = 1024;   // most entries that survive into steps 4 and 5
constexpr int kTile = 4096;        // probabilities staged per step of the sequential sum (draw without a filter)
constexpr int kMaxTiles = 512;     // 2,097,152 entries

struct SampleArgs {
    const float* logits;
    float* scores;               // scratch, n floats
    uint32_t n;
    float temperature, top_p, penalty;
    uint32_t top_k, min_tokens;
    const int32_t* context;      // generated tokens so far
    const int32_t* ctx_range;    // device words {begin, end} into context, or null: ctx_begin / ctx_end below
    uint32_t ctx_begin, ctx_end;
    const int32_t* eos;
    uint32_t n_eos;
    unsigned long long* rng;     // generator state, advanced by one draw
    int32_t* result;
    int32_t* status;
};

__device__ __forceinline__ float block_reduce_max(float v, float* sm) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if (lane == 0) sm[warp] = v;
    __syncthreads();
    v = sm[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float block_reduce_sum(float v, float* sm) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) sm[warp] = v;
    __syncthreads();
    v = sm[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// Exclusive prefix sum of one count per thread over the CTA (thread order); *total = sum of all.
__device__ __forceinline__ uint32_t block_scan_excl(uint32_t v, uint32_t* sm, uint32_t* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    __syncthreads();
    if (lane == 31) sm[warp] = inc;
    __syncthreads();
    uint32_t w = sm[lane];
    uint32_t winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, winc, o);
        if (lane >= o) winc += t;
    }
    *total = __shfl_sync(0xffffffffu, winc, 31);
    const uint32_t wbase = __shfl_sync(0xffffffffu, winc - w, warp);
    return wbase + inc - v;
}

// Index of the largest score, the last one among equal maxima (Iterator::max_by keeps the later of two equal elements).
__device__ __forceinline__ uint32_t block_argmax_last(const float* s, uint32_t n, float* smv, uint32_t* smi) {
    float bv = -INFINITY;
    uint32_t bi = 0;
    bool have = false;
    for (uint32_t i = threadIdx.x; i < n; i += kST) {
        const float v = s[i];
        if (!have || v >= bv) { bv = v; bi = i; have = true; }
    }
    if (!have) bi = 0;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    auto merge = [&](float ov, uint32_t oi, bool oh) {
        if (oh && (!have || ov > bv || (ov == bv && oi > bi))) { bv = ov; bi = oi; have = true; }
    };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
        const bool oh = __shfl_xor_sync(0xffffffffu, (int)have, o) != 0;
        merge(ov, oi, oh);
    }
    __syncthreads();
    if (lane == 0) { smv[warp] = have ? bv : -INFINITY; smi[warp] = have ? bi : 0xFFFFFFFFu; }
    __syncthreads();
    bv = smv[lane];
    bi = smi[lane];
    have = bi != 0xFFFFFFFFu;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
        const bool oh = __shfl_xor_sync(0xffffffffu, (int)have, o) != 0;
        merge(ov, oi, oh);
    }
    return have ? bi : 0u;
}

// Bits of the k-th largest of n non-negative floats (their bit patterns order like the values): four passes of an 8-bit
// radix histogram, most significant byte first.  k in 1..n.
__device__ __forceinline__ uint32_t block_kth_largest(const float* s, uint32_t n, uint32_t k, uint32_t* hist, uint32_t* sm_pick) {
    uint32_t prefix = 0, mask = 0, want = k;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (uint32_t b = threadIdx.x; b < 256; b += kST) hist[b] = 0;
        __syncthreads();
        for (uint32_t i = threadIdx.x; i < n; i += kST) {
            const uint32_t u = __float_as_uint(s[i]);
            if ((u & mask) == prefix) atomicAdd(&hist[(u >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t acc = 0;
            int b = 255;
            for (; b > 0; b--) {
                if (acc + hist[b] >= want) break;
                acc += hist[b];
            }
            sm_pick[0] = (uint32_t)b;
            sm_pick[1] = want - acc;
        }
        __syncthreads();
        prefix |= sm_pick[0] << shift;
        mask |= 255u << shift;
        want = sm_pick[1];
        __syncthreads();
    }
    return prefix;
}

// xorshift64 step and the reference's conversion to a float in [0, 1] (sampler.rs:18-27): the 53 high bits, rounded to f32.
__device__ __forceinline__ float rng_next_f32(unsigned long long* state) {
    unsigned long long x = *state;
    x ^= x << 13;
    x ^= x >> 7;
    x ^= x << 17;
    *state = x;
    return __ull2float_rn(x >> 11) / 9007199254740992.0f;
}

__global__ void __launch_bounds__(kST) sample_kernel(const SampleArgs a) {
    grid_dependency_wait();      // the logits come from the previous kernel of the chain
    grid_launch_dependents();
    __shared__ float smf[32];
    __shared__ uint32_t smu[32];
    __shared__ uint32_t hist[256];
    __shared__ uint32_t pick[2];
    __shared__ float cval[kCand], sval[kCand];
    __shared__ uint32_t cidx[kCand], spos[kCand];
    __shared__ uint8_t ckeep[kCand];
    __shared__ uint32_t s_claim;
    __shared__ float s_r;
    const uint32_t n = a.n, tid = threadIdx.x;
    float* s = a.scores;
    uint32_t cb = a.ctx_begin, ce = a.ctx_end;
    if (a.ctx_range) {
        cb = (uint32_t)max(0, a.ctx_range[0]);
        ce = (uint32_t)max(0, a.ctx_range[1]);
    }
    const uint32_t clen = ce > cb ? ce - cb : 0u;
    const int32_t* ctxp = a.context + cb;

    for (uint32_t i = tid; i < n; i += kST) s[i] = a.logits[i];
    __syncthreads();
    // 0a: no end of sequence before min_tokens
    if (clen < a.min_tokens) {
        for (uint32_t e = tid; e < a.n_eos; e += kST) {
            const int32_t id = a.eos[e];
            if (id >= 0 && (uint32_t)id < n) s[id] = -INFINITY;
        }
        __syncthreads();
    }
    // 0b: repetition penalty, once per occurrence; the thread of a token's first occurrence applies all of them
    if (a.penalty != 1.0f && clen > 0) {
        for (uint32_t i = tid; i < clen; i += kST) {
            const int32_t tok = ctxp[i];
            if (tok < 0 || (uint32_t)tok >= n) continue;
            bool first = true;
            for (uint32_t j = 0; j < i; j++)
                if (ctxp[j] == tok) { first = false; break; }
            if (!first) continue;
            uint32_t cnt = 0;
            for (uint32_t j = i; j < clen; j++) cnt += ctxp[j] == tok;
            float v = s[tok];
            for (uint32_t c = 0; c < cnt; c++) v = v > 0.0f ? v / a.penalty : v * a.penalty;
            s[tok] = v;
        }
        __syncthreads();
    }
    if (a.temperature == 0.0f) {
        const uint32_t best = block_argmax_last(s, n, smf, smu);
        if (tid == 0) a.result[0] = (int32_t)best;
        return;
    }
    // 1, 2: temperature and softmax
    float m = -INFINITY;
    for (uint32_t i = tid; i < n; i += kST) {
        const float v = s[i] / a.temperature;
        s[i] = v;
        m = fmaxf(m, v);
    }
    m = block_reduce_max(m, smf);
    float acc = 0.f;
    for (uint32_t i = tid; i < n; i += kST) {
        const float e = expf(s[i] - m);
        s[i] = e;
        acc += e;
    }
    const float denom = block_reduce_sum(acc, smf);
    for (uint32_t i = tid; i < n; i += kST) s[i] = s[i] / denom;
    __syncthreads();

    const bool do_k = a.top_k > 0 && a.top_k < n, do_p = a.top_p < 1.0f;
    const uint32_t chunk = (n + kST - 1) / kST, c_beg = min(n, tid * chunk), c_end = min(n, c_beg + chunk);
    if (do_k || do_p) {
        // 3: the candidates are the first kk entries in index order with p >= the kk-th largest probability
        const uint32_t kk = do_k ? min(a.top_k, kCand) : min(kCand, n);
        const float thr = __uint_as_float(block_kth_largest(s, n, kk, hist, pick));
        uint32_t ge = 0;
        for (uint32_t i = c_beg; i < c_end; i++) ge += s[i] >= thr;
        uint32_t total_ge = 0;
        uint32_t run = block_scan_excl(ge, smu, &total_ge);
        const uint32_t nc = min(total_ge, kk);
        for (uint32_t i = c_beg; i < c_end; i++) {
            const float p = s[i];
            if (p >= thr && run < kk) {
                cval[run] = p;
                cidx[run] = i;
                run++;
            } else if (do_k) {
                s[i] = 0.f;
            }
        }
        for (uint32_t c = tid; c < kCand; c += kST) {
            ckeep[c] = c < nc;
        }
        __syncthreads();
        if (do_p) {
            // 4: descending by probability (equal ones by index), a sequential running sum
            for (uint32_t c = tid; c < kCand; c += kST) {
                sval[c] = c < nc ? cval[c] : -1.f;
                spos[c] = c;
            }
            __syncthreads();
            for (uint32_t k2 = 2; k2 <= kCand; k2 <<= 1) {
                for (uint32_t j = k2 >> 1; j > 0; j >>= 1) {
                    for (uint32_t t = tid; t < kCand; t += kST) {
                        const uint32_t o = t ^ j;
                        if (o > t) {
                            const float va = sval[t], vb = sval[o];
                            const uint32_t pa = spos[t], pb = spos[o];
                            const bool a_first = va > vb || (va == vb && pa < pb);   // a belongs before b in the final order
                            const bool up = (t & k2) == 0;
                            if (up ? !a_first : a_first) {
                                sval[t] = vb; sval[o] = va;
                                spos[t] = pb; spos[o] = pa;
                            }
                        }
                    }
                    __syncthreads();
                }
            }
            if (tid == 0) {
                float cum = 0.f;
                for (uint32_t r = 0; r < nc; r++) {
                    const uint32_t pos = spos[r];
                    if (cum >= a.top_p) ckeep[pos] = 0;
                    else cum += sval[r];
                }
                // with top-k off the entries beyond the candidates come later in the order: they go only if the sum was reached
                s_claim = (!do_k && nc < n && !(cum >= a.top_p)) ? 1u : 0u;
            }
            __syncthreads();
            if (s_claim) {
                if (tid == 0) {
                    if (a.status) atomicCAS(a.status, 0, 4);
                    a.result[0] = (int32_t)cidx[spos[0]];
                }
                return;
            }
            if (!do_k) {
                for (uint32_t i = tid; i < n; i += kST) s[i] = 0.f;
                __syncthreads();
            }
            for (uint32_t c = tid; c < nc; c += kST) s[cidx[c]] = ckeep[c] ? cval[c] : 0.f;
        }
        // 5: sequential over the survivors in index order, as the reference's loops over the whole vector are
        if (tid == 0) {
            float total = 0.f;
            for (uint32_t c = 0; c < nc; c++)
                if (ckeep[c]) total += cval[c];
            int32_t tok = (int32_t)(n - 1);      // nothing left: the argmax of an all-zero vector is its last index
            if (total > 0.f) {
                const float r = rng_next_f32(a.rng) * total;
                float cum = 0.f, bestv = -1.f;
                bool hit = false;
                for (uint32_t c = 0; c < nc && !hit; c++) {
                    if (!ckeep[c]) continue;
                    cum += cval[c];
                    if (cval[c] >= bestv) { bestv = cval[c]; tok = (int32_t)cidx[c]; }
                    if (r <= cum) { tok = (int32_t)cidx[c]; hit = true; }
                }
            }
            a.result[0] = tok;
        }
        return;
    }
    // no filter: the draw over the whole vocabulary.  The boundaries of the running sum lie about one probability apart, so
    // the sum is taken in the reference's order, one term after the other by one thread, over tiles the CTA stages in
    // shared memory; the running sum at every tile boundary is kept, and the walk then revisits only the tile r falls in.
    {
        __shared__ float tile[kTile];
        __shared__ float tprefix[kMaxTiles + 1];
        __shared__ int32_t s_pick;
        const uint32_t n_tiles = (n + kTile - 1) / kTile;
        float cum = 0.f;
        if (tid == 0) tprefix[0] = 0.f;
        for (uint32_t t = 0; t < n_tiles; t++) {
            const uint32_t base = t * kTile, cnt = min((uint32_t)kTile, n - base);
            for (uint32_t i = tid; i < cnt; i += kST) tile[i] = s[base + i];
            __syncthreads();
            if (tid == 0) {
                for (uint32_t i = 0; i < cnt; i++) cum += tile[i];
                tprefix[t + 1] = cum;
            }
            __syncthreads();
        }
        if (tid == 0) {
            s_pick = -1;                              // -1: nothing to draw from; -2: r beyond the last running sum
            if (cum > 0.f) {
                const float r = rng_next_f32(a.rng) * cum;
                s_r = r;
                s_pick = -2;
                for (uint32_t t = 0; t < n_tiles; t++)
                    if (r <= tprefix[t + 1]) { s_pick = (int32_t)t; break; }
            }
        }
        __syncthreads();
        const int32_t pickt = s_pick;
        if (pickt < 0) {                              // sampler.rs:100 and :110: the argmax of what is left
            const uint32_t best = block_argmax_last(s, n, smf, smu);
            if (tid == 0) a.result[0] = (int32_t)best;
            return;
        }
        const uint32_t base = (uint32_t)pickt * kTile, cnt = min((uint32_t)kTile, n - base);
        for (uint32_t i = tid; i < cnt; i += kST) tile[i] = s[base + i];
        __syncthreads();
        if (tid == 0) {
            const float r = s_r;
            float c2 = tprefix[pickt];
            uint32_t tok = base + cnt - 1;
            for (uint32_t i = 0; i < cnt; i++) {
                c2 += tile[i];
                if (r <= c2) { tok = base + i; break; }
            }
            a.result[0] = (int32_t)tok;
        }
    }
}

}  // namespace runit

using namespace runit;

extern "C" {

int32_t runit_sample_f32(runit_ctx_t* ctx, const void* logits, void* scores_scratch, uint32_t n, const runit_sampler_cfg* cfg,
                         const void* context, const void* ctx_range, uint32_t ctx_begin, uint32_t ctx_end, const void* eos_ids,
                         uint32_t n_eos, void* rng_state, void* result) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, logits && scores_scratch && cfg && rng_state && result && n > 0, "sample_f32: null pointer or n == 0");
    RUNIT_REQUIRE(ctx, runit_aligned(rng_state, 8) && runit_aligned(result, 4), "sample_f32: misaligned state or result");
    RUNIT_REQUIRE(ctx, cfg->temperature >= 0.f && cfg->top_k >= 0 && cfg->top_k <= (int32_t)kCand,
                  "sample_f32: temperature %g or top_k %d unsupported (top_k in 0..1024)", (double)cfg->temperature, cfg->top_k);
    RUNIT_REQUIRE(ctx, n <= (uint32_t)kTile * kMaxTiles, "sample_f32: n=%u exceeds 2,097,152", n);
    RUNIT_REQUIRE(ctx, (context || (ctx_begin == ctx_end && !ctx_range)) && (eos_ids || n_eos == 0), "sample_f32: null context or eos list");
    SampleArgs a{};
    a.logits = (const float*)logits;
    a.scores = (float*)scores_scratch;
    a.n = n;
    a.temperature = cfg->temperature;
    a.top_p = cfg->top_p;
    a.penalty = cfg->repetition_penalty;
    a.top_k = (uint32_t)cfg->top_k;
    a.min_tokens = (uint32_t)cfg->min_tokens;
    a.context = (const int32_t*)context;
    a.ctx_range = (const int32_t*)ctx_range;
    a.ctx_begin = ctx_begin;
    a.ctx_end = ctx_end;
    a.eos = (const int32_t*)eos_ids;
    a.n_eos = n_eos;
    a.rng = (unsigned long long*)rng_state;
    a.result = (int32_t*)result;
    a.status = ctx->d_status;
    runit_launch_chain(ctx, sample_kernel, dim3(1), dim3(kST), a);
    return runit_after_launch(ctx, "sample_f32");
}

// SimpleRng::new (sampler.rs:15-17): the state a generator with this seed starts from.
uint64_t runit_sampler_seed_state(uint64_t seed) { return seed == 0 ? 0x9e3779b97f4a7c15ull : seed ^ 0x9e3779b97f4a7c15ull; }

}  // extern "C"
