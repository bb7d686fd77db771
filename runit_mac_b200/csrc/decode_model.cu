// Greedy decoder for an OLMoE-shaped model with Q4_K matrices: the op sequence of
// Executor::forward_greedy (crates/engine/src/forward.rs:1795-1975) as one recorded command list per
// token, with the token id, the position and the argmax result kept on the device so that successive
// tokens need no host round trip (the reference synchronises once per MoE layer and once per token).
//
// Differences from the reference that the benchmark configuration asks for: f32 router weights, f32
// expert intermediates and combine, top-k weights not renormalised unless cfg.renorm, f16 KV cache
// fed from f32 K/V, f32 logits with a lowest-index argmax.
#include "decode_ops.cuh"
#include "gemv_stream_host.h"
#include "runit_internal.h"
#include "tma.cuh"

#include <cstring>
#include <new>
#include <vector>

struct runit_model {
    runit_ctx* ctx = nullptr;
    runit_model_cfg cfg;
    runit_model_weights w;
    // device state
    __half* kc = nullptr;       // [L][kv_heads][max_seq][head_dim]
    __half* vc = nullptr;
    bool ep_fused = false;      // exchange inside the GEMVs (tuning key ep_fused_exchange at creation)
    float* ep_copies = nullptr; // per-CTA copies of the summed hidden state (expert parallelism), ep_copies_rows rows
    uint32_t ep_copies_rows = 0;
    float* x2 = nullptr;        // second hidden-state buffer (expert parallelism: the summed state is formed next to the old one)
    float *x = nullptr, *xn = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *ao = nullptr, *logits = nullptr;
    float* attn_part = nullptr;
    uint32_t* attn_counters = nullptr;   // one ticket counter per head, zero at rest
    uint32_t* moe_counters = nullptr;    // 1024 ticket counters of the MoE block (routing; weighted sum per row tile), zero at rest
    void* moe_scratch = nullptr;
    size_t moe_scratch_bytes = 0;
    int32_t* state = nullptr;   // [0] = token, [1] = pos, [2] = step counter
    int32_t* forced = nullptr;  // forced input tokens (prompt), n_forced entries
    int32_t* out_tokens = nullptr;
    uint32_t forced_cap = 0, out_cap = 0;
    uint32_t nsplit = 8;
    // expert parallelism (ep_world > 1): gate/up/down hold this rank's experts only, tokens are replicated
    uint32_t ep_world = 1, ep_rank = 0;
    void* ep_partial[8] = {nullptr};    // every rank's partial buffer f32 [2][world][1][hidden], as mapped here
    void* ep_pads[8] = {nullptr};       // every rank's signal pad
    uint32_t* ep_epoch = nullptr;       // device word: barrier epoch, advanced by the barrier kernel, never reset
    cudaGraphExec_t graph_full = nullptr;    // step with lm_head + argmax
    cudaGraphExec_t graph_prompt = nullptr;  // step without them (prompt positions whose logits nobody reads)
    // sampled decoding: the step with lm_head + sampler, recorded on first use and when the configuration changes
    cudaGraphExec_t graph_sampled = nullptr;
    runit_sampler_cfg sampler_cfg{};
    uint32_t sampler_n_eos = 0;
    float* scores = nullptr;                 // [vocab]
    int32_t* eos = nullptr;                  // [16]
    unsigned long long* rng = nullptr;
    // batched prefill (allocated on first use, for prompts up to max_seq)
    struct {
        float *x = nullptr, *q = nullptr, *qkv = nullptr, *proj = nullptr, *xn2 = nullptr;
        uint8_t* wqkv = nullptr;            // per layer the rows of wq, wk, wv in one matrix: the three projections are one GEMM
        void *xn_bf16 = nullptr, *ao_bf16 = nullptr, *moe_scratch = nullptr;
        int32_t *tokens = nullptr, *tables = nullptr;
        size_t moe_bytes = 0;
        uint32_t rows_alloc = 0;
    } pf;
    std::vector<void*> owned;
};

namespace runit {

// x = tok_emb[token]; token comes from the forced list while step < n_forced, else from state[0].
__global__ void embed_kernel(const float* __restrict__ emb, float* __restrict__ x, int32_t* state,
                             const int32_t* __restrict__ forced, uint32_t n_forced, uint32_t hidden, uint32_t vocab) {
    grid_dependency_wait();      // inputs come from the previous kernel of the chain
    grid_launch_dependents();
    const uint32_t step = (uint32_t)state[2];
    int32_t tok = state[0];
    if (step < n_forced) {
        const int32_t f = forced[step];   // negative = this step is not forced
        if (f >= 0) tok = f;
    }
    if (tok < 0 || (uint32_t)tok >= vocab) tok = 0;   // ids are validated on the host; never index out of range
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < hidden; i += gridDim.x * blockDim.x)
        x[i] = emb[(size_t)tok * hidden + i];
}

// After the step: record the produced token, advance position and step.
__global__ void advance_kernel(int32_t* state, const int32_t* argmax_result, int32_t* out_tokens, uint32_t out_cap,
                               int has_logits) {
    grid_dependency_wait();      // inputs come from the previous kernel of the chain
    grid_launch_dependents();
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        const uint32_t step = (uint32_t)state[2];
        if (has_logits) {
            state[0] = argmax_result[0];
            if (step < out_cap) out_tokens[step] = argmax_result[0];
        } else if (step < out_cap) {
            out_tokens[step] = -1;
        }
        state[1] += 1;
        state[2] += 1;
        state[5] = state[2];   // end of the sampler's context range {state[4], state[5]} inside out_tokens
    }
}

static int32_t dev_alloc(runit_model* m, void** p, size_t bytes) {
    cudaError_t e = cudaMalloc(p, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return runit_fail(m->ctx, RUNIT_ERR_ALLOC, "model: allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    }
    m->owned.push_back(*p);
    return RUNIT_OK;
}

// Issue the launches of one decode step on the context's stream.
static int32_t issue_step(runit_model* m, bool with_logits, uint32_t n_forced, bool sampled = false) {
    runit_ctx* ctx = m->ctx;
    const runit_model_cfg& c = m->cfg;
    const uint32_t h = c.hidden, hd = c.head_dim, q_dim = c.n_heads * hd, kv_dim = c.n_kv_heads * hd;
    const size_t rb_h = runit_row_bytes(RUNIT_FMT_Q4K, h), rb_q = runit_row_bytes(RUNIT_FMT_Q4K, q_dim);
    const size_t rb_ff = runit_row_bytes(RUNIT_FMT_Q4K, c.ff);
    const size_t kv_layer = (size_t)c.n_kv_heads * c.max_seq * hd;
    const int32_t* pos_ptr = m->state + 1;
    int32_t st;
    runit_launch_chain(ctx, embed_kernel, dim3(8), dim3(256), (const float*)m->w.tok_emb, m->x, m->state, m->forced, n_forced, h, c.vocab);
    if ((st = runit_after_launch(ctx, "embed")) != RUNIT_OK) return st;
    // Expert parallelism with the exchange inside the GEMVs (hidden 1024 / 2048 / 4096): a block leaves its result as
    // partial sums in every rank's buffer; the next reader of the hidden state forms residual + sum in its prologue, into
    // the other of two buffers.
    // Opt-in (tuning key ep_fused_exchange, read when the model is created): it brings the launch count down to the single
    // GPU's, but measured 1077 tok/s against 1380 with the exchange as three small launches (OLMoE shape, 2 GPUs): the flag
    // round trip and the sum then sit in the prologue of every CTA of the consuming GEMV.
    const bool ep_fused = m->ep_fused && m->ep_world > 1 && (h == 1024 || h == 2048 || h == 4096);
    float* xc = m->x;            // the hidden state
    float* xo = m->x2;
    bool pending = false;
    EpWait wait{};
    wait.partial = (const float*)m->ep_partial[m->ep_rank];
    wait.pad = (const uint32_t*)m->ep_pads[m->ep_rank];
    wait.world = m->ep_world;
    wait.epoch = m->ep_epoch;
    wait.copies = m->ep_copies;
    wait.copies_rows = m->ep_copies_rows;
    EpPush push{};
    push.partial_all = m->ep_partial;
    push.pads = m->ep_pads;
    push.world = m->ep_world;
    push.rank = m->ep_rank;
    push.epoch = m->ep_epoch;
    push.done = m->moe_counters + 1;
    for (int l = 0; l < c.n_layers; l++) {
        const uint8_t* wq = (const uint8_t*)m->w.wq + (size_t)l * q_dim * rb_h;
        const uint8_t* wk = (const uint8_t*)m->w.wk + (size_t)l * kv_dim * rb_h;
        const uint8_t* wv = (const uint8_t*)m->w.wv + (size_t)l * kv_dim * rb_h;
        const uint8_t* wo = (const uint8_t*)m->w.wo + (size_t)l * h * rb_q;
        // attention block (forward.rs:1833-1896)
        // the attention RMSNorm runs inside the q|k|v launch (every CTA computes the scale of the hidden state itself)
        const void* ws[3] = {wq, wk, wv};
        void* ys[3] = {m->q, m->k, m->v};
        const uint32_t rows[3] = {q_dim, kv_dim, kv_dim};
        const EpWait* w_now = nullptr;
        if (pending) {
            wait.residual = xc;
            w_now = &wait;
            float* t = xc; xc = xo; xo = t;
            pending = false;
        }
        if ((st = gemv_segments(ctx, "qkv_q4k", RUNIT_FMT_Q4K, 3, ws, ys, rows, xc, h, (const float*)m->w.attn_norm + (size_t)l * h, c.eps, w_now)))
            return st;
        __half* kcl = m->kc + (size_t)l * kv_layer;
        __half* vcl = m->vc + (size_t)l * kv_layer;
        if (hd == 128 || hd == 64) {
            // rotary embedding, cache update and attention in one launch
            if ((st = launch_decode_attention_rope(ctx, m->q, m->k, m->v, kcl, vcl, m->ao, m->attn_part, m->nsplit, pos_ptr, c.n_heads,
                                                   c.n_kv_heads, hd, c.max_seq, c.theta, m->attn_counters)))
                return st;
        } else {
            if ((st = launch_rope_kv(ctx, m->q, m->k, m->v, kcl, vcl, hd, c.n_heads, c.n_kv_heads, pos_ptr, c.theta, c.max_seq))) return st;
            if ((st = launch_decode_attention(ctx, 0, 1, m->q, kcl, vcl, m->ao, m->attn_part, m->nsplit, 1, 0, pos_ptr, c.n_heads,
                                              c.n_kv_heads, hd, c.max_seq, m->attn_counters)))
                return st;
        }
        if ((st = gemv_plain(ctx, "attn_out_q4k", RUNIT_FMT_Q4K, wo, m->ao, xc, xc, h, q_dim))) return st;
        // MoE block (forward.rs:1898-1931)
        // (the block's RMSNorm runs inside its routing launch)
        const float* ffn_gamma = (const float*)m->w.ffn_norm + (size_t)l * h;
        const uint32_t e_local = c.n_experts / m->ep_world;
        const size_t eg = (size_t)e_local * c.ff * rb_h, ed = (size_t)e_local * h * rb_ff;
        if (ep_fused) {
            if ((st = moe_layer_q4k_ep_push_impl(ctx, (const float*)m->w.router + (size_t)l * c.n_experts * h,
                                                 (const uint8_t*)m->w.gate + (size_t)l * eg, (const uint8_t*)m->w.up + (size_t)l * eg,
                                                 (const uint8_t*)m->w.down + (size_t)l * ed, m->xn, xc, ffn_gamma, c.eps, m->moe_scratch,
                                                 m->moe_scratch_bytes, h, c.ff, c.n_experts, c.top_k, c.renorm, m->moe_counters, &push)))
                return st;
            pending = true;
            continue;
        }
        if (m->ep_world > 1) {
            // experts split over the ranks, combine over peer memory as launches of its own (other hidden sizes)
            if ((st = moe_layer_q4k_ep_impl(ctx, (const float*)m->w.router + (size_t)l * c.n_experts * h,
                                            (const uint8_t*)m->w.gate + (size_t)l * eg, (const uint8_t*)m->w.up + (size_t)l * eg,
                                            (const uint8_t*)m->w.down + (size_t)l * ed, m->xn, xc, xc, nullptr, nullptr, m->moe_scratch,
                                            m->moe_scratch_bytes, m->ep_partial, m->ep_pads, 1, h, c.ff, c.n_experts, c.top_k, c.renorm,
                                            m->ep_world, m->ep_rank, 0, m->ep_epoch, m->moe_counters, xc, ffn_gamma,
                                            c.eps)))
                return st;
            continue;
        }
        if ((st = moe_layer_q4k_impl(ctx, (const float*)m->w.router + (size_t)l * c.n_experts * h,
                                     (const uint8_t*)m->w.gate + (size_t)l * eg, (const uint8_t*)m->w.up + (size_t)l * eg,
                                     (const uint8_t*)m->w.down + (size_t)l * ed, m->xn, xc, xc, nullptr, nullptr,
                                     m->moe_scratch, m->moe_scratch_bytes, 1, h, c.ff, c.n_experts, c.top_k, c.renorm,
                                     // (the next operator's RMSNorm runs inside that operator's own launch)
                                     nullptr, nullptr, c.eps, m->moe_counters,
                                     xc, ffn_gamma, c.eps)))
            return st;
    }
    const EpWait* w_last = nullptr;
    if (pending && with_logits) {
        wait.residual = xc;
        w_last = &wait;
        float* t = xc; xc = xo; xo = t;
    }
    int32_t* argmax_out = m->state + 3;
    if (with_logits && sampled) {
        if ((st = gemv_plain(ctx, "lm_head_q4k", RUNIT_FMT_Q4K, m->w.lm_head, xc, m->logits, nullptr, c.vocab, h,
                             (const float*)m->w.out_norm, c.eps, nullptr, w_last))) return st;
        // the context of the draw: what has been generated so far, out_tokens[state[4] .. state[5])
        if ((st = runit_sample_f32(ctx, m->logits, m->scores, (uint32_t)c.vocab, &m->sampler_cfg, m->out_tokens, m->state + 4, 0, 0,
                                   m->eos, m->sampler_n_eos, m->rng, argmax_out))) return st;
    } else if (with_logits) {
        if ((st = gemv_plain(ctx, "lm_head_q4k", RUNIT_FMT_Q4K, m->w.lm_head, xc, m->logits, nullptr, c.vocab, h,
                             (const float*)m->w.out_norm, c.eps, argmax_out, w_last))) return st;   // argmax inside the launch
    }
    runit_launch_chain(ctx, advance_kernel, dim3(1), dim3(32), m->state, argmax_out, m->out_tokens, m->out_cap, with_logits ? 1 : 0);
    return runit_after_launch(ctx, "advance");
}

static int32_t record_graph(runit_model* m, bool with_logits, cudaGraphExec_t* out, bool sampled = false) {
    runit_ctx* ctx = m->ctx;
    RUNIT_CUDA_TRY(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    ctx->capturing = true;
    stream_rec_begin(ctx);
    int32_t st = issue_step(m, with_logits, m->forced_cap, sampled);
    ctx->capturing = false;
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &g);
    if (st != RUNIT_OK) {
        stream_rec_discard(ctx);
        if (g) cudaGraphDestroy(g);
        return st;
    }
    if (e != cudaSuccess || !g) {
        cudaGetLastError();
        stream_rec_discard(ctx);
        return runit_fail(ctx, RUNIT_ERR_LAUNCH, "model: stream capture failed: %s", cudaGetErrorString(e));
    }
    // adjacent GEMVs of the step (none today: every GEMV of this model is followed by another kind of operator) would share
    // one persistent launch, as in any recorded command list
    st = stream_rec_fuse(ctx, g, &m->owned, nullptr);
    stream_rec_discard(ctx);
    if (st != RUNIT_OK) {
        cudaGraphDestroy(g);
        return st;
    }
    e = cudaGraphInstantiate(out, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return runit_fail(ctx, RUNIT_ERR_LAUNCH, "model: graph instantiate failed: %s", cudaGetErrorString(e));
    return RUNIT_OK;
}

}  // namespace runit

using namespace runit;

extern "C" {

static int32_t model_create_impl(runit_ctx_t* ctx, const runit_model_cfg* cfg, const runit_model_weights* weights, uint32_t world,
                                 uint32_t rank, void* const* partial_all, void* const* signal_pads, runit_model_t** out) {
    if (!ctx || !out) return RUNIT_ERR_BAD_ARG;
    *out = nullptr;
    RUNIT_REQUIRE(ctx, world >= 1 && world <= 8 && rank < world, "model_create: world=%u rank=%u unsupported", world, rank);
    RUNIT_REQUIRE(ctx, world == 1 || (partial_all && signal_pads && cfg && cfg->n_experts % (int32_t)world == 0),
                  "model_create: expert parallelism needs peer buffers and an expert count divisible by the ranks");
    RUNIT_REQUIRE(ctx, cfg && weights, "model_create: null config or weights");
    const runit_model_cfg& c = *cfg;
    RUNIT_REQUIRE(ctx, c.n_layers > 0 && c.n_layers <= 256 && c.hidden > 0 && c.hidden % 256 == 0, "model_create: bad hidden/layers");
    RUNIT_REQUIRE(ctx, c.n_heads > 0 && c.n_kv_heads > 0 && c.n_heads % c.n_kv_heads == 0, "model_create: bad head counts");
    RUNIT_REQUIRE(ctx, c.head_dim == 32 || c.head_dim == 64 || c.head_dim == 96 || c.head_dim == 128, "model_create: head_dim must be 32/64/96/128");
    RUNIT_REQUIRE(ctx, (c.n_heads * c.head_dim) % 256 == 0, "model_create: n_heads*head_dim must be a multiple of 256");
    RUNIT_REQUIRE(ctx, c.ff > 0 && c.ff % 256 == 0 && c.n_experts > 0 && c.n_experts <= 256 && c.top_k > 0 && c.top_k <= c.n_experts && c.top_k <= 32,
                  "model_create: bad MoE shape");
    RUNIT_REQUIRE(ctx, c.vocab > 0 && c.max_seq > 0, "model_create: bad vocab/max_seq");
    const void* ptrs[] = {weights->tok_emb, weights->attn_norm, weights->ffn_norm, weights->out_norm, weights->wq, weights->wk,
                          weights->wv, weights->wo, weights->router, weights->gate, weights->up, weights->down, weights->lm_head};
    for (const void* p : ptrs) RUNIT_REQUIRE(ctx, p != nullptr, "model_create: null weight pointer");
    runit_model* m = new (std::nothrow) runit_model();
    if (!m) return RUNIT_ERR_ALLOC;
    m->ctx = ctx;
    m->cfg = c;
    m->w = *weights;
    m->ep_world = world;
    m->ep_rank = rank;
    m->ep_fused = ctx->tune.ep_fused_exchange != 0;
    for (uint32_t p = 0; world > 1 && p < world; p++) {
        m->ep_partial[p] = partial_all[p];
        m->ep_pads[p] = signal_pads[p];
    }
    const uint32_t h = c.hidden, q_dim = c.n_heads * c.head_dim, kv_dim = c.n_kv_heads * c.head_dim;
    const size_t kv_elems = (size_t)c.n_layers * c.n_kv_heads * c.max_seq * c.head_dim;
    m->moe_scratch_bytes = moe_scratch_bytes_impl(1, h, c.ff, c.n_experts, c.top_k);
    m->forced_cap = (uint32_t)c.max_seq;
    m->out_cap = (uint32_t)c.max_seq;
    int32_t st = RUNIT_OK;
    auto A = [&](void** p, size_t b) { if (st == RUNIT_OK) st = dev_alloc(m, p, b); };
    A((void**)&m->kc, kv_elems * 2); A((void**)&m->vc, kv_elems * 2);
    A((void**)&m->x, h * 4); A((void**)&m->x2, h * 4); A((void**)&m->xn, h * 4); A((void**)&m->q, q_dim * 4); A((void**)&m->k, kv_dim * 4);
    A((void**)&m->v, kv_dim * 4); A((void**)&m->ao, q_dim * 4); A((void**)&m->logits, (size_t)c.vocab * 4);
    A((void**)&m->attn_part, (size_t)c.n_heads * m->nsplit * (c.head_dim + 2) * 4);
    A(&m->moe_scratch, m->moe_scratch_bytes);
    A((void**)&m->attn_counters, (size_t)c.n_heads * 4);
    A((void**)&m->ep_epoch, 64);
    A((void**)&m->moe_counters, 4096);
    if (world > 1) {
        // one row per 32-row tile of the widest launch that may consume an exchange (q|k|v or lm_head)
        const uint32_t widest = (uint32_t)c.vocab > q_dim + 2 * kv_dim ? (uint32_t)c.vocab : q_dim + 2 * kv_dim;
        m->ep_copies_rows = 4 * ((widest + 31) / 32 + 3);      // a cluster split along K has up to 4 CTAs per tile
        A((void**)&m->ep_copies, (size_t)m->ep_copies_rows * h * 4);
    }
    A((void**)&m->scores, (size_t)c.vocab * 4); A((void**)&m->eos, 64); A((void**)&m->rng, 8);
    A((void**)&m->state, 64); A((void**)&m->forced, (size_t)m->forced_cap * 4); A((void**)&m->out_tokens, (size_t)m->out_cap * 4);
    if (st == RUNIT_OK) {
        cudaMemsetAsync(m->kc, 0, kv_elems * 2, ctx->stream);
        cudaMemsetAsync(m->vc, 0, kv_elems * 2, ctx->stream);
        cudaMemsetAsync(m->state, 0, 64, ctx->stream);
        cudaMemsetAsync(m->ep_epoch, 0, 64, ctx->stream);   // once: the epoch only ever grows afterwards
        cudaMemsetAsync(m->attn_counters, 0, (size_t)c.n_heads * 4, ctx->stream);
        cudaMemsetAsync(m->moe_counters, 0, 4096, ctx->stream);
        cudaMemsetAsync(m->forced, 0xFF, (size_t)m->forced_cap * 4, ctx->stream);   // nothing forced
        // one eager step configures every kernel (shared-memory attributes, tensor maps) before capture
        st = issue_step(m, true, 0);
        if (st == RUNIT_OK) st = runit_flush(ctx);
        cudaMemsetAsync(m->state, 0, 64, ctx->stream);
        cudaMemsetAsync(m->kc, 0, kv_elems * 2, ctx->stream);
        cudaMemsetAsync(m->vc, 0, kv_elems * 2, ctx->stream);
    }
    if (st == RUNIT_OK) st = record_graph(m, true, &m->graph_full);
    if (st == RUNIT_OK) st = record_graph(m, false, &m->graph_prompt);
    if (st != RUNIT_OK) {
        runit_model_destroy(m);
        return st;
    }
    *out = m;
    return RUNIT_OK;
}

int32_t runit_model_create(runit_ctx_t* ctx, const runit_model_cfg* cfg, const runit_model_weights* weights, runit_model_t** out) {
    return model_create_impl(ctx, cfg, weights, 1, 0, nullptr, nullptr, out);
}

int32_t runit_model_create_ep(runit_ctx_t* ctx, const runit_model_cfg* cfg, const runit_model_weights* weights, uint32_t world,
                              uint32_t rank, void* const* partial_all, void* const* signal_pads, runit_model_t** out) {
    return model_create_impl(ctx, cfg, weights, world, rank, partial_all, signal_pads, out);
}

int32_t runit_model_destroy(runit_model_t* m) {
    if (!m) return RUNIT_ERR_BAD_ARG;
    cudaStreamSynchronize(m->ctx->stream);
    if (m->graph_full) cudaGraphExecDestroy(m->graph_full);
    if (m->graph_prompt) cudaGraphExecDestroy(m->graph_prompt);
    if (m->graph_sampled) cudaGraphExecDestroy(m->graph_sampled);
    for (void* p : m->owned) cudaFree(p);
    delete m;
    return RUNIT_OK;
}

// After a batched prefill: the decoder stands at position n with the token the last position produced.
__global__ void prefill_finish_kernel(int32_t* state, int32_t n) {
    if (threadIdx.x == 0) {
        state[0] = state[3];
        state[1] = n;
        state[2] = 0;
        state[5] = 0;
    }
}

// Executor::prefill (crates/engine/src/prefill.rs:29-255): the whole prompt in one batched pass from an empty cache; the
// cache then holds positions 0 .. n-1 and *next_token is the argmax of the last position's logits (they stay readable
// through runit_model_logits).  Decoding continues with runit_model_generate_greedy(&next, 1, n_gen, n, ...).
int32_t runit_model_prefill(runit_model_t* m, const int32_t* tokens, uint32_t n, int32_t* next_token) {
    if (!m) return RUNIT_ERR_BAD_ARG;
    runit_ctx* ctx = m->ctx;
    const runit_model_cfg& c = m->cfg;
    RUNIT_REQUIRE(ctx, tokens && n > 0 && next_token, "model_prefill: null or empty prompt");     // prefill.rs:35-37
    RUNIT_REQUIRE(ctx, n <= (uint32_t)c.max_seq, "model_prefill: %u tokens exceed max_seq %d", n, c.max_seq);
    RUNIT_REQUIRE(ctx, m->ep_world == 1, "model_prefill: not available on the expert-parallel decoder");
    const uint32_t h = c.hidden, hd = c.head_dim, q_dim = c.n_heads * hd, kv_dim = c.n_kv_heads * hd;
    RUNIT_REQUIRE(ctx, (hd == 64 || hd == 128) && q_dim % 256 == 0 && kv_dim % 256 == 0 && c.ff % 256 == 0,
                  "model_prefill: head_dim 64/128 and projection widths that are multiples of 256 only");
    for (uint32_t i = 0; i < n; i++)
        RUNIT_REQUIRE(ctx, tokens[i] >= 0 && tokens[i] < c.vocab, "model_prefill: token id %d out of range", tokens[i]);   // prefill.rs:55-57
    int32_t st = RUNIT_OK;
    if (!m->pf.x) {
        const uint32_t cap = (uint32_t)c.max_seq;
        m->pf.rows_alloc = (cap + 255) / 256 * 256 + 256;
        m->pf.moe_bytes = runit_moe_grouped_scratch_bytes(cap, h, c.ff, c.n_experts, c.top_k);
        auto A = [&](void** p, size_t b) { if (st == RUNIT_OK) st = dev_alloc(m, p, b); };
        A((void**)&m->pf.x, (size_t)cap * h * 4); A((void**)&m->pf.q, (size_t)cap * q_dim * 4);
        A((void**)&m->pf.qkv, (size_t)cap * (q_dim + 2 * kv_dim) * 4);
        A((void**)&m->pf.wqkv, (size_t)c.n_layers * (q_dim + 2 * kv_dim) * runit_row_bytes(RUNIT_FMT_Q4K, h));
        A((void**)&m->pf.proj, (size_t)cap * h * 4); A((void**)&m->pf.xn2, (size_t)cap * h * 4);
        A(&m->pf.xn_bf16, (size_t)m->pf.rows_alloc * h * 2); A(&m->pf.ao_bf16, (size_t)m->pf.rows_alloc * q_dim * 2);
        A(&m->pf.moe_scratch, m->pf.moe_bytes);
        A((void**)&m->pf.tokens, (size_t)cap * 4); A((void**)&m->pf.tables, (size_t)(3 * ((cap + 255) / 256) + 4) * 4);
        if (st != RUNIT_OK) return st;
        // rows past the prompt are read by the GEMMs' tile loads (never stored): keep them finite
        cudaMemsetAsync(m->pf.xn_bf16, 0, (size_t)m->pf.rows_alloc * h * 2, ctx->stream);
        cudaMemsetAsync(m->pf.ao_bf16, 0, (size_t)m->pf.rows_alloc * q_dim * 2, ctx->stream);
        // q | k | v of a layer as one matrix (a copy of 0.56 bytes per weight of the three projections): 192 tiles of one
        // GEMM launch keep the CTA pairs busy where three launches of 64 tiles each ran one tile per pair
        const size_t rbh = runit_row_bytes(RUNIT_FMT_Q4K, h), qb = (size_t)q_dim * rbh, kb = (size_t)kv_dim * rbh;
        for (int l = 0; l < c.n_layers; l++) {
            uint8_t* dst = m->pf.wqkv + (size_t)l * (qb + 2 * kb);
            cudaMemcpyAsync(dst, (const uint8_t*)m->w.wq + (size_t)l * qb, qb, cudaMemcpyDeviceToDevice, ctx->stream);
            cudaMemcpyAsync(dst + qb, (const uint8_t*)m->w.wk + (size_t)l * kb, kb, cudaMemcpyDeviceToDevice, ctx->stream);
            cudaMemcpyAsync(dst + qb + kb, (const uint8_t*)m->w.wv + (size_t)l * kb, kb, cudaMemcpyDeviceToDevice, ctx->stream);
        }
    }
    RUNIT_CUDA_TRY(ctx, cudaMemcpyAsync(m->pf.tokens, tokens, (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream));
    if ((st = dense_tiles_prepare(ctx, m->pf.tables, n))) return st;
    if ((st = prefill_embed(ctx, (const float*)m->w.tok_emb, m->pf.tokens, m->pf.x, n, h))) return st;
    const size_t rb_h = runit_row_bytes(RUNIT_FMT_Q4K, h), rb_q = runit_row_bytes(RUNIT_FMT_Q4K, q_dim), rb_ff = runit_row_bytes(RUNIT_FMT_Q4K, c.ff);
    const size_t kv_layer = (size_t)c.n_kv_heads * c.max_seq * hd;
    for (int l = 0; l < c.n_layers; l++) {
        const uint32_t qkv_dim = q_dim + 2 * kv_dim;
        const uint8_t* wqkv = m->pf.wqkv + (size_t)l * qkv_dim * rb_h;
        const uint8_t* wo = (const uint8_t*)m->w.wo + (size_t)l * h * rb_q;
        // attention block (prefill.rs:84-150)
        if ((st = prefill_norm_bf16(ctx, m->pf.x, (const float*)m->w.attn_norm + (size_t)l * h, m->pf.xn_bf16, c.eps, n, h))) return st;
        if ((st = dense_gemm_q4k_bf16(ctx, "prefill_qkv", wqkv, nullptr, qkv_dim, h, m->pf.xn_bf16, m->pf.rows_alloc, m->pf.qkv, qkv_dim, n, m->pf.tables))) return st;
        __half* kcl = m->kc + (size_t)l * kv_layer;
        __half* vcl = m->vc + (size_t)l * kv_layer;
        if ((st = prefill_rope_cache(ctx, m->pf.qkv, m->pf.q, m->pf.qkv + q_dim, m->pf.qkv + q_dim + kv_dim, kcl, vcl, hd, c.n_heads, c.n_kv_heads, 0,
                                     c.theta, c.max_seq, n, qkv_dim)))
            return st;
        if ((st = prefill_attention(ctx, m->pf.q, kcl, vcl, m->pf.ao_bf16, n, c.n_heads, c.n_kv_heads, hd, c.max_seq, 0))) return st;
        if ((st = dense_gemm_q4k_bf16(ctx, "prefill_o", wo, nullptr, h, q_dim, m->pf.ao_bf16, m->pf.rows_alloc, m->pf.proj, h, n, m->pf.tables))) return st;
        // residual add and the block's RMSNorm in one launch; then the mixture-of-experts block on all tokens at once
        // (prefill.rs:153-215 runs it token by token)
        if ((st = prefill_add_rms_norm(ctx, m->pf.x, m->pf.proj, (const float*)m->w.ffn_norm + (size_t)l * h, m->pf.xn2, c.eps, n, h))) return st;
        const size_t eg = (size_t)c.n_experts * c.ff * rb_h, ed = (size_t)c.n_experts * h * rb_ff;
        if ((st = runit_moe_layer_q4k_bf16(ctx, (const float*)m->w.router + (size_t)l * c.n_experts * h, (const uint8_t*)m->w.gate + (size_t)l * eg,
                                           (const uint8_t*)m->w.up + (size_t)l * eg, (const uint8_t*)m->w.down + (size_t)l * ed, m->pf.xn2, m->pf.x,
                                           m->pf.x, nullptr, nullptr, m->pf.moe_scratch, m->pf.moe_bytes, n, h, c.ff, c.n_experts, c.top_k, c.renorm)))
            return st;
    }
    // final norm + lm_head on the last position only (prefill.rs:229-250), through the decode path's launch
    RUNIT_CUDA_TRY(ctx, cudaMemcpyAsync(m->x, m->pf.x + (size_t)(n - 1) * h, (size_t)h * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    if ((st = gemv_plain(ctx, "lm_head_q4k", RUNIT_FMT_Q4K, m->w.lm_head, m->x, m->logits, nullptr, c.vocab, h, (const float*)m->w.out_norm, c.eps,
                         m->state + 3)))
        return st;
    prefill_finish_kernel<<<1, 32, 0, ctx->stream>>>(m->state, (int32_t)n);
    if ((st = runit_after_launch(ctx, "prefill_finish"))) return st;
    RUNIT_CUDA_TRY(ctx, cudaMemcpyAsync(next_token, m->state, 4, cudaMemcpyDeviceToHost, ctx->stream));
    return runit_flush(ctx);
}

// Clear the KV position: the next step runs at `pos` with input token `token`.
int32_t runit_model_reset(runit_model_t* m, int32_t token, int32_t pos) {
    if (!m) return RUNIT_ERR_BAD_ARG;
    runit_ctx* ctx = m->ctx;
    RUNIT_REQUIRE(ctx, token >= 0 && token < m->cfg.vocab, "model_reset: token id %d out of range", token);   // forward.rs:1804-1806
    RUNIT_REQUIRE(ctx, pos >= 0 && pos < m->cfg.max_seq, "model_reset: position %d out of range", pos);
    const int32_t init[4] = {token, pos, 0, 0};
    RUNIT_CUDA_TRY(ctx, cudaMemcpyAsync(m->state, init, sizeof(init), cudaMemcpyHostToDevice, ctx->stream));
    RUNIT_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));   // `init` lives on this stack frame
    return RUNIT_OK;
}

// Executor::forward_greedy(token_id, pos, kv) -> next token (forward.rs:1795-1975): one step, synchronous.
int32_t runit_model_forward_greedy(runit_model_t* m, int32_t token_id, int32_t pos, int32_t* next_token) {
    if (!m) return RUNIT_ERR_BAD_ARG;
    runit_ctx* ctx = m->ctx;
    int32_t st = runit_model_reset(m, token_id, pos);
    if (st != RUNIT_OK) return st;
    // step 0 must not be forced by a prompt left over from runit_model_generate_greedy
    RUNIT_CUDA_TRY(ctx, cudaMemsetAsync(m->forced, 0xFF, 4, ctx->stream));
    RUNIT_CUDA_TRY(ctx, cudaGraphLaunch(m->graph_full, ctx->stream));
    int32_t tok = -1;
    RUNIT_CUDA_TRY(ctx, cudaMemcpyAsync(&tok, m->state, 4, cudaMemcpyDeviceToHost, ctx->stream));
    st = runit_flush(ctx);
    if (st != RUNIT_OK) return st;
    if (next_token) *next_token = tok;
    return RUNIT_OK;
}

// Run a prompt of n_prompt known tokens followed by n_gen greedy steps, starting at position start_pos,
// entirely on the device.  out_tokens (host, n_prompt + n_gen entries): out_tokens[i] is the arg-max token
// after step i; prompt steps before the last give -1 when skip_prompt_logits is set (their logits are not
// computed).  The generated continuation is out_tokens[n_prompt-1 ...].  One synchronisation at the end.
static int32_t generate_impl(runit_model_t* m, const int32_t* prompt, uint32_t n_prompt, uint32_t n_gen, int32_t start_pos,
                             int32_t skip_prompt_logits, int32_t* out_tokens, cudaGraphExec_t graph_step);

int32_t runit_model_generate_greedy(runit_model_t* m, const int32_t* prompt, uint32_t n_prompt, uint32_t n_gen,
                                    int32_t start_pos, int32_t skip_prompt_logits, int32_t* out_tokens) {
    if (!m) return RUNIT_ERR_BAD_ARG;
    return generate_impl(m, prompt, n_prompt, n_gen, start_pos, skip_prompt_logits, out_tokens, m->graph_full);
}

int32_t runit_model_generate_sampled(runit_model_t* m, const int32_t* prompt, uint32_t n_prompt, uint32_t n_gen, int32_t start_pos,
                                     const runit_sampler_cfg* cfg, uint64_t seed, const int32_t* eos_ids, uint32_t n_eos,
                                     int32_t* out_tokens) {
    if (!m) return RUNIT_ERR_BAD_ARG;
    runit_ctx* ctx = m->ctx;
    RUNIT_REQUIRE(ctx, cfg && n_eos <= 16 && (eos_ids || n_eos == 0) && n_prompt > 0, "model_generate_sampled: null configuration or more than 16 eos ids");
    RUNIT_REQUIRE(ctx, m->ep_world == 1, "model_generate_sampled: the expert-parallel decoder is greedy only");
    const bool same = m->graph_sampled && memcmp(&m->sampler_cfg, cfg, sizeof(*cfg)) == 0 && m->sampler_n_eos == n_eos;
    if (!same) {
        RUNIT_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
        if (m->graph_sampled) cudaGraphExecDestroy(m->graph_sampled);
        m->graph_sampled = nullptr;
        m->sampler_cfg = *cfg;
        m->sampler_n_eos = n_eos;
        // an eager launch of the sampler checks the configuration before it is recorded (its result is discarded)
        int32_t st = runit_sample_f32(ctx, m->logits, m->scores, (uint32_t)m->cfg.vocab, &m->sampler_cfg, m->out_tokens, nullptr, 0, 0,
                                      m->eos, 0, m->rng, m->state + 3);
        if (st == RUNIT_OK) st = runit_flush(ctx);
        if (st == RUNIT_OK) st = record_graph(m, true, &m->graph_sampled, true);
        if (st != RUNIT_OK) return st;
    }
    const unsigned long long state0 = runit_sampler_seed_state(seed);
    int32_t eos_host[16] = {0};
    for (uint32_t i = 0; i < n_eos; i++) eos_host[i] = eos_ids[i];
    RUNIT_CUDA_TRY(ctx, cudaMemcpyAsync(m->rng, &state0, 8, cudaMemcpyHostToDevice, ctx->stream));
    RUNIT_CUDA_TRY(ctx, cudaMemcpyAsync(m->eos, eos_host, 64, cudaMemcpyHostToDevice, ctx->stream));
    RUNIT_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));   // the sources live on this stack frame
    return generate_impl(m, prompt, n_prompt, n_gen, start_pos, 1, out_tokens, m->graph_sampled);
}

static int32_t generate_impl(runit_model_t* m, const int32_t* prompt, uint32_t n_prompt, uint32_t n_gen, int32_t start_pos,
                             int32_t skip_prompt_logits, int32_t* out_tokens, cudaGraphExec_t graph_step) {
    runit_ctx* ctx = m->ctx;
    RUNIT_REQUIRE(ctx, prompt && n_prompt > 0 && out_tokens, "model_generate_greedy: null or empty prompt");
    const uint32_t n_steps = n_prompt + n_gen;
    RUNIT_REQUIRE(ctx, start_pos >= 0 && (uint64_t)start_pos + n_steps <= (uint64_t)m->cfg.max_seq,
                  "model_generate_greedy: %u steps from position %d exceed max_seq %d", n_steps, start_pos, m->cfg.max_seq);   // kv_cache.rs:63
    RUNIT_REQUIRE(ctx, n_prompt <= m->forced_cap && n_steps <= m->out_cap, "model_generate_greedy: too many steps");
    for (uint32_t i = 0; i < n_prompt; i++)
        RUNIT_REQUIRE(ctx, prompt[i] >= 0 && prompt[i] < m->cfg.vocab, "model_generate_greedy: token id %d out of range", prompt[i]);
    RUNIT_CUDA_TRY(ctx, cudaMemcpyAsync(m->forced, prompt, (size_t)n_prompt * 4, cudaMemcpyHostToDevice, ctx->stream));
    // the sampler's context range inside out_tokens: from the step that produces the first generated token to the current step
    const int32_t range[2] = {(int32_t)n_prompt - 1, 0};
    RUNIT_CUDA_TRY(ctx, cudaMemcpyAsync(m->state + 4, range, sizeof(range), cudaMemcpyHostToDevice, ctx->stream));
    int32_t st = runit_model_reset(m, prompt[0], start_pos);   // synchronises: `range` lives on this stack frame
    if (st != RUNIT_OK) return st;
    // Steps past the prompt are not forced: their entries are negative and the step takes the previous argmax.
    RUNIT_CUDA_TRY(ctx, cudaMemsetAsync(m->forced + n_prompt, 0xFF, (size_t)(m->forced_cap - n_prompt) * 4, ctx->stream));
    for (uint32_t i = 0; i < n_steps; i++) {
        const bool prompt_step = i + 1 < n_prompt;
        cudaGraphExec_t g = (prompt_step && skip_prompt_logits) ? m->graph_prompt : graph_step;
        RUNIT_CUDA_TRY(ctx, cudaGraphLaunch(g, ctx->stream));
        // a bounded wait already gave up (e.g. a rank of the expert-parallel group is missing): stop feeding the stream,
        // the flush below reports it
        if (ctx->h_status && *reinterpret_cast<volatile int32_t*>(ctx->h_status) != 0) break;
    }
    RUNIT_CUDA_TRY(ctx, cudaMemcpyAsync(out_tokens, m->out_tokens, (size_t)n_steps * 4, cudaMemcpyDeviceToHost, ctx->stream));
    return runit_flush(ctx);
}

void* runit_model_logits(runit_model_t* m) { return m ? (void*)m->logits : nullptr; }
uint64_t runit_model_launches_per_token(runit_model_t* m) {
    if (!m) return 0;
    // embed + per layer (q|k|v with its RMSNorm, [rope +] attention, o-proj, [norm,] MoE block) + lm_head with its RMSNorm and the argmax,
    // advance.  MoE block at hidden 1024 / 2048 / 4096: norm + router + routing, gate/up, down + weighted sum (3); else
    // norm, router, routing, gate/up, down, weighted sum.  Expert-parallel: router + routing, gate/up, down, partial sums,
    // barrier, sum (6; 7 with router and routing apart; 3 with the opt-in exchange inside the GEMVs).
    const bool fused = m->cfg.hidden == 1024 || m->cfg.hidden == 2048 || m->cfg.hidden == 4096;
    const uint64_t moe = m->ep_world > 1 ? (fused ? (m->ep_fused ? 3 : 6) : 7) : (fused ? 3 : 5);
    const uint64_t attn = (m->cfg.head_dim == 128 || m->cfg.head_dim == 64) ? 1 : 2;   // rope + cache update fused into the attention launch
    const uint64_t norm2 = fused ? 0 : 1;
    return 1 + (uint64_t)m->cfg.n_layers * (1 + attn + 1 + norm2 + moe) + 2;
}

}  // extern "C"
