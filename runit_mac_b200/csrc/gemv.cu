// Host side of the fused-dequant GEMV family: argument validation, kernel selection and
// the extern "C" twins of the reference's dispatch functions (crates/kernels/src/dispatch.rs).
//
// Kernel selection mirrors WeightBuf's role in the reference (crates/engine/src/forward.rs:84-248):
// one operator per (weight format, input dtype, output dtype, residual) combination.  Here
// every combination is an epilogue/prologue flag of one streaming kernel per format.
#include "gemv_launch.cuh"

namespace runit {

struct GemvCall {
    int fmt = 0;
    const void* w[3] = {nullptr, nullptr, nullptr};
    const void* w2 = nullptr;          // fused gate/up: second matrix
    void* y[3] = {nullptr, nullptr, nullptr};
    const void* res[3] = {nullptr, nullptr, nullptr};
    const void* bias[3] = {nullptr, nullptr, nullptr};
    uint32_t rows[3] = {0, 0, 0};
    int nseg = 1;
    const void* x = nullptr;
    uint32_t k = 0, batch = 1;
    bool x_f16 = false, out_f16 = false;
    int res_kind = RES_NONE, bias_kind = BIAS_NONE;
    bool dual = false;
    const char* name = "gemv";
    // grouped (mixture-of-experts) launch: see GemvArgs
    const int32_t* grp_expert = nullptr;
    uint32_t grp_slots = 0, grp_experts = 0, grp_xdiv = 1;
    int32_t grp_lo = 0;
    // fused all-gather: the same output slice in the memory of the other GPUs
    float* peer_y[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    uint32_t n_peer = 0;
    // grouped, one token: weighted sum of the slots (+ residual) by the last tile of every row tile
    const float* cmb_w = nullptr;
    const float* cmb_res = nullptr;
    float* cmb_out = nullptr;
    uint32_t* cmb_cnt = nullptr;
    bool late_trigger = false, grp_early = false;   // see GemvArgs
    const EpPush* ep_push = nullptr;
    const EpWait* ep_wait = nullptr;
    // greedy epilogue: (largest result, row index + am_base) into am_dst[0..am_ndst) and the index into am_token
    bool am = false;
    uint32_t am_base = 0, am_ndst = 0;
    uint2* am_dst[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    int32_t* am_token = nullptr;
    // RMSNorm prologue: x is the un-normalised vector, gamma f32 [k]
    const float* norm_gamma = nullptr;
    float norm_eps = 0.f;
};

static int32_t gemv_dispatch(runit_ctx* ctx, const GemvCall& c) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    const char* nm = c.name;
    RUNIT_REQUIRE(ctx, c.fmt >= 0 && c.fmt <= 2, "%s: unknown weight format %d", nm, c.fmt);
    const uint32_t be = (uint32_t)runit_block_elems(c.fmt);
    RUNIT_REQUIRE(ctx, c.k > 0 && c.k % be == 0, "%s: k=%u is not a positive multiple of %u", nm, c.k, be);
    RUNIT_REQUIRE(ctx, c.k <= (1u << 24), "%s: k=%u exceeds 2^24", nm, c.k);
    RUNIT_REQUIRE(ctx, c.batch >= 1 && c.batch <= 8, "%s: batch=%u not in 1..8", nm, c.batch);
    RUNIT_REQUIRE(ctx, c.x && runit_aligned(c.x, 16), "%s: input null or not 16-byte aligned", nm);
    RUNIT_REQUIRE(ctx, !c.dual || c.nseg == 1, "%s: fused gate/up takes one segment", nm);
    RUNIT_REQUIRE(ctx, c.nseg == 1 || c.batch == 1, "%s: multi-segment launch is batch 1", nm);

    GemvArgs a;
    memset(&a, 0, sizeof(a));
    a.nseg = c.nseg;
    a.x = c.x;
    a.k = c.k;
    a.nb = c.k / be;
    a.row_bytes = (uint32_t)runit_row_bytes(c.fmt, c.k);
    a.out_f16 = c.out_f16;
    a.res_kind = c.res_kind;
    a.bias_kind = c.bias_kind;
    a.dual = c.dual;

    uint32_t tiles = 0, total_rows = 0;
    const uint32_t rpt = c.dual ? kRT / 2 : kRT;
    bool w_align4 = (a.row_bytes % 4) == 0, w_align8 = (a.row_bytes % 8) == 0, w_align16 = (a.row_bytes % 16) == 0;
    for (int i = 0; i < c.nseg; i++) {
        RUNIT_REQUIRE(ctx, c.rows[i] > 0, "%s: segment %d has zero rows", nm, i);
        RUNIT_REQUIRE(ctx, c.rows[i] <= (1u << 28), "%s: segment %d has too many rows", nm, i);
        RUNIT_REQUIRE(ctx, c.w[i] && c.y[i], "%s: null weight or output pointer", nm);
        RUNIT_REQUIRE(ctx, runit_aligned(c.w[i], 16), "%s: weight pointer not 16-byte aligned", nm);
        RUNIT_REQUIRE(ctx, runit_aligned(c.y[i], 4), "%s: output pointer misaligned", nm);
        RUNIT_REQUIRE(ctx, c.res_kind == RES_NONE || c.res[i], "%s: null residual", nm);
        RUNIT_REQUIRE(ctx, c.bias_kind == BIAS_NONE || c.bias[i], "%s: null bias", nm);
        a.seg[i].w = (const uint8_t*)c.w[i];
        a.seg[i].w2 = (const uint8_t*)c.w2;
        a.seg[i].y = c.y[i];
        a.seg[i].res = c.res[i];
        a.seg[i].bias = c.bias[i];
        a.seg[i].rows = c.rows[i];
        a.seg[i].tile_begin = tiles;
        tiles += (c.rows[i] + rpt - 1) / rpt;
        total_rows += c.rows[i];
    }
    if (c.dual) RUNIT_REQUIRE(ctx, c.w2 && runit_aligned(c.w2, 16), "%s: null or misaligned second weight", nm);
    a.ldy = c.rows[0];
    if (c.grp_expert) {
        RUNIT_REQUIRE(ctx, c.nseg == 1 && c.batch == 1 && c.grp_slots > 0 && c.grp_experts > 0 && c.grp_xdiv > 0,
                      "%s: bad grouped launch", nm);
        a.grp_expert = c.grp_expert;
        a.grp_rows = c.rows[0];
        a.grp_tiles = tiles;           // tiles per slot
        a.grp_xdiv = c.grp_xdiv;
        a.grp_lo = c.grp_lo;
        a.grp_cnt = c.grp_experts;
        RUNIT_REQUIRE(ctx, (uint64_t)tiles * c.grp_slots < (1ull << 31), "%s: too many grouped tiles", nm);
        if (c.ep_push) {
            const EpPush& e = *c.ep_push;
            RUNIT_REQUIRE(ctx, c.cmb_w && c.cmb_cnt && e.partial_all && e.pads && e.epoch && e.done && e.world >= 1 && e.world <= 8 && e.rank < e.world,
                          "%s: bad expert-parallel push", nm);
            for (uint32_t p = 0; p < e.world; p++) {
                RUNIT_REQUIRE(ctx, e.partial_all[p] && e.pads[p], "%s: null peer buffer %u", nm, p);
                a.ep_peer[p] = (float*)e.partial_all[p];
                a.ep_pad[p] = (uint32_t*)e.pads[p];
            }
            a.ep_npeer = e.world;
            a.ep_rank = e.rank;
            a.ep_epoch = e.epoch;
            a.ep_done = e.done;
        }
        if (c.cmb_out || c.ep_push) {
            RUNIT_REQUIRE(ctx, c.cmb_w && c.cmb_cnt && !c.dual && !c.out_f16 && !c.x_f16 && c.grp_slots <= 32,
                          "%s: the fused weighted sum takes f32 slots of one token", nm);
            a.cmb_w = c.cmb_w;
            a.cmb_res = c.cmb_res;
            a.cmb_out = c.cmb_out;
            a.cmb_cnt = c.cmb_cnt;
            a.cmb_slots = c.grp_slots;
        }
        a.late_trigger = c.late_trigger ? 1 : 0;
        a.grp_early = c.grp_early ? 1 : 0;
        tiles *= c.grp_slots;
        total_rows *= c.grp_slots;
    }

    const bool staged_ok = (c.fmt == RUNIT_FMT_Q8_0) ? w_align4 : w_align16;
    const bool simple = (ctx->tune.gemv_variant == 1 || !staged_ok) && !c.grp_expert;
    RUNIT_REQUIRE(ctx, staged_ok || !c.grp_expert, "%s: grouped launch needs aligned rows", nm);
    const int cpb = w_align16 ? 16 : (w_align8 ? 8 : 4);
    const uint32_t bpu = c.fmt == RUNIT_FMT_Q8_0 ? Traits<RUNIT_FMT_Q8_0>::BPU
                         : c.fmt == RUNIT_FMT_Q4_0 ? Traits<RUNIT_FMT_Q4_0>::BPU : Traits<RUNIT_FMT_Q4K>::BPU;
    a.n_units = (a.nb + bpu - 1) / bpu;
    if (c.n_peer) {
        RUNIT_REQUIRE(ctx, c.nseg == 1 && c.batch == 1 && !c.out_f16 && !c.dual && !c.grp_expert && c.n_peer <= 7,
                      "%s: the fused all-gather takes one f32 segment, batch 1", nm);
        for (uint32_t p = 0; p < c.n_peer; p++) {
            RUNIT_REQUIRE(ctx, c.peer_y[p] && runit_aligned(c.peer_y[p], 4), "%s: null or misaligned peer output", nm);
            a.peer_y[p] = c.peer_y[p];
        }
        a.n_peer = c.n_peer;
    }
    if (c.am) {
        RUNIT_REQUIRE(ctx, c.batch == 1 && c.nseg == 1 && !c.dual && !c.out_f16 && !c.x_f16 && !c.grp_expert && !simple && ctx->d_am &&
                      tiles <= 65536 && c.am_ndst <= 8,
                      "%s: the greedy epilogue takes one f32 segment of at most 2,097,152 rows with 16-byte aligned weight rows", nm);
        a.am_part = reinterpret_cast<uint2*>((uint8_t*)ctx->d_am + 256);
        a.am_cnt = reinterpret_cast<uint32_t*>(ctx->d_am);
        a.am_base = c.am_base;
        a.am_ndst = c.am_ndst;
        for (uint32_t d = 0; d < c.am_ndst; d++) {
            RUNIT_REQUIRE(ctx, c.am_dst[d] && runit_aligned(c.am_dst[d], 8), "%s: null or misaligned pair destination", nm);
            a.am_dst[d] = c.am_dst[d];
        }
        a.am_token = c.am_token;
    }
    if (c.ep_wait) {
        const EpWait& e = *c.ep_wait;
        RUNIT_REQUIRE(ctx, c.batch == 1 && !c.x_f16 && !c.dual && !c.grp_expert && !simple && e.partial && e.pad && e.residual && e.epoch &&
                          e.world >= 1 && e.world <= 8 && e.residual != c.x,
                      "%s: bad expert-parallel wait (the summed hidden state needs a buffer of its own)", nm);
        a.epw_partial = e.partial;
        a.epw_pad = e.pad;
        a.epw_res = e.residual;
        a.epw_out = (float*)const_cast<void*>(c.x);
        a.epw_copies = e.copies;
        a.epw_epoch = e.epoch;
        // (the grid is at most one CTA per 32-row tile; checked against the scratch below, once the tiles are known)
        a.epw_abort = ctx->d_abort;
        a.epw_world = e.world;
    }
    if (c.norm_gamma) {
        RUNIT_REQUIRE(ctx, c.batch == 1 && !c.x_f16 && !c.grp_expert && runit_aligned(c.norm_gamma, 4),
                      "%s: the RMSNorm prologue takes one f32 input vector", nm);
        a.norm_gamma = c.norm_gamma;
        a.norm_eps = c.norm_eps;
    }
    a.status = ctx->d_status;
    a.n_tiles = tiles;
    // Tiled bulk loads (TMA) for the 4-bit formats: one tensor map per weight matrix.
    GemvMaps maps;
    const bool tma = !simple && c.fmt != RUNIT_FMT_Q8_0 && ctx->tune.gemv_load == 0 && ctx->encode_tiled != nullptr;
    if (tma) {
        const uint32_t box_rows = c.dual ? kRT / 2 : kRT;
        for (int i = 0; i < c.nseg; i++) {
            const uint64_t map_rows = c.grp_expert ? (uint64_t)c.rows[i] * c.grp_experts : c.rows[i];
            int32_t st = runit_get_tmap(ctx, c.w[i], map_rows, a.row_bytes, box_rows, 144, &maps.m[i]);
            if (st != RUNIT_OK) return st;
        }
        if (c.dual) {
            const uint64_t map_rows = c.grp_expert ? (uint64_t)c.rows[0] * c.grp_experts : c.rows[0];
            int32_t st = runit_get_tmap(ctx, c.w2, map_rows, a.row_bytes, box_rows, 144, &maps.m[3]);
            if (st != RUNIT_OK) return st;
        }
    }
    if (c.ep_wait && (!c.ep_wait->copies || 4 * tiles > c.ep_wait->copies_rows))    // a cluster split along K has up to 4 CTAs per tile
        return runit_fail(ctx, RUNIT_ERR_BUFFER_SIZE, "%s: the expert-parallel prologue needs %u copies of the hidden state, has %u", nm, 4 * tiles,
                          c.ep_wait->copies ? c.ep_wait->copies_rows : 0u);
    if (c.ep_wait && !tma)
        return runit_fail(ctx, RUNIT_ERR_UNSUPPORTED, "%s: the expert-parallel prologue needs the tiled bulk-load path (4-bit formats)", nm);
    switch (c.fmt) {
        case RUNIT_FMT_Q8_0:
            return gemv_launch_q8_0(ctx, a, maps, tiles, total_rows, cpb, tma, c.batch, c.x_f16, simple, nm);
        case RUNIT_FMT_Q4_0:
            return gemv_launch_q4_0(ctx, a, maps, tiles, total_rows, cpb, tma, c.batch, c.x_f16, simple, nm);
        default:
            return gemv_launch_q4k(ctx, a, maps, tiles, total_rows, cpb, tma, c.batch, c.x_f16, simple, nm);
    }
}

// Plain single-matrix call shared by the twins below.
static int32_t gemv1(runit_ctx* ctx, const char* name, int fmt, const void* w, const void* x, void* y, const void* res,
                     uint32_t m, uint32_t k, bool x_f16, bool out_f16, int res_kind, const float* norm_gamma = nullptr,
                     float norm_eps = 0.f, int32_t* argmax_token = nullptr, const EpWait* ep_wait = nullptr) {
    GemvCall c;
    c.ep_wait = ep_wait;
    if (argmax_token) {
        c.am = true;
        c.am_token = argmax_token;
    }
    c.norm_gamma = norm_gamma;
    c.norm_eps = norm_eps;
    c.name = name;
    c.fmt = fmt;
    c.w[0] = w;
    c.x = x;
    c.y[0] = y;
    c.res[0] = res;
    c.rows[0] = m;
    c.k = k;
    c.x_f16 = x_f16;
    c.out_f16 = out_f16;
    c.res_kind = res_kind;
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, m > 0, "%s: m == 0", name);
    return gemv_dispatch(ctx, c);
}

static int32_t fused_qkv(runit_ctx* ctx, const char* name, int fmt, const void* wq, const void* wk, const void* wv,
                         const void* x, void* oq, void* ok, void* ov, const void* bq, const void* bk, const void* bv,
                         int bias_kind, uint32_t q_dim, uint32_t kv_dim, uint32_t k) {
    GemvCall c;
    c.name = name;
    c.fmt = fmt;
    c.nseg = 3;
    c.w[0] = wq; c.w[1] = wk; c.w[2] = wv;
    c.y[0] = oq; c.y[1] = ok; c.y[2] = ov;
    c.bias[0] = bq; c.bias[1] = bk; c.bias[2] = bv;
    c.rows[0] = q_dim; c.rows[1] = kv_dim; c.rows[2] = kv_dim;
    c.x = x;
    c.k = k;
    c.bias_kind = bias_kind;
    return gemv_dispatch(ctx, c);
}

static int32_t fused_ffn(runit_ctx* ctx, const char* name, int fmt, const void* wg, const void* wu, const void* x,
                         void* act, uint32_t ff, uint32_t k) {
    GemvCall c;
    c.name = name;
    c.fmt = fmt;
    c.w[0] = wg;
    c.w2 = wu;
    c.y[0] = act;
    c.rows[0] = ff;
    c.x = x;
    c.k = k;
    c.dual = true;
    return gemv_dispatch(ctx, c);
}

// Grouped fused-dequant GEMVs for the MoE block: slot s multiplies the rows of expert slot_expert[s]
// (inside the stacked matrix w: [n_experts][rows][k]) with input row s / xdiv and writes output row s.
// With w2 != nullptr the launch computes silu(w.x) * (w2.x) (gate/up fusion).
int32_t gemv_grouped(runit_ctx* ctx, const char* name, int fmt, const void* w, const void* w2, uint32_t n_experts,
                     uint32_t rows, uint32_t k, const void* x, uint32_t xdiv, void* y, const int32_t* slot_expert,
                     uint32_t n_slots, int32_t expert_lo, const float* cmb_w, const float* cmb_res, float* cmb_out,
                     uint32_t* cmb_cnt, int order, const EpPush* ep) {
    GemvCall c;
    c.ep_push = ep;
    c.late_trigger = order == 1;
    c.grp_early = order == 2;
    c.cmb_w = cmb_w;
    c.cmb_res = cmb_res;
    c.cmb_out = cmb_out;
    c.cmb_cnt = cmb_cnt;
    c.name = name;
    c.fmt = fmt;
    c.w[0] = w;
    c.w2 = w2;
    c.dual = w2 != nullptr;
    c.x = x;
    c.y[0] = y;
    c.rows[0] = rows;
    c.k = k;
    c.grp_expert = slot_expert;
    c.grp_slots = n_slots;
    c.grp_experts = n_experts;
    c.grp_xdiv = xdiv;
    c.grp_lo = expert_lo;
    return gemv_dispatch(ctx, c);
}

int32_t gemv_segments(runit_ctx* ctx, const char* name, int fmt, int nseg, const void* const* w, void* const* y,
                      const uint32_t* rows, const void* x, uint32_t k, const float* norm_gamma, float norm_eps, const EpWait* ep_wait) {
    GemvCall c;
    c.ep_wait = ep_wait;
    c.norm_gamma = norm_gamma;
    c.norm_eps = norm_eps;
    c.name = name;
    c.fmt = fmt;
    c.nseg = nseg;
    for (int i = 0; i < nseg && i < 3; i++) {
        c.w[i] = w[i];
        c.y[i] = y[i];
        c.rows[i] = rows[i];
    }
    c.x = x;
    c.k = k;
    return gemv_dispatch(ctx, c);
}

int32_t gemv_plain(runit_ctx* ctx, const char* name, int fmt, const void* w, const void* x, void* y, const void* res_f32,
                   uint32_t m, uint32_t k, const float* norm_gamma, float norm_eps, int32_t* argmax_token, const EpWait* ep_wait) {
    return gemv1(ctx, name, fmt, w, x, y, res_f32, m, k, false, false, res_f32 ? RES_F32 : RES_NONE, norm_gamma, norm_eps,
                 argmax_token, ep_wait);
}

}  // namespace runit

using namespace runit;

extern "C" {

#define GEMV_TWIN(NAME, FMT, XF16, OF16)                                                                     \
    int32_t runit_##NAME(runit_ctx_t* ctx, const void* w, const void* x, void* y, uint32_t m, uint32_t k) { \
        return gemv1(ctx, #NAME, FMT, w, x, y, nullptr, m, k, XF16, OF16, RES_NONE);                         \
    }
#define GEMV_TWIN_RES(NAME, FMT, XF16, OF16, RES)                                                            \
    int32_t runit_##NAME(runit_ctx_t* ctx, const void* w, const void* x, void* y, const void* r, uint32_t m, \
                         uint32_t k) {                                                                       \
        return gemv1(ctx, #NAME, FMT, w, x, y, r, m, k, XF16, OF16, RES);                                    \
    }

// Q8_0: crates/kernels/shaders/gemv_q8_0.metal:56-240
GEMV_TWIN(gemv_q8_0_f32in_f32out, RUNIT_FMT_Q8_0, false, false)
GEMV_TWIN_RES(gemv_q8_0_add_f32_f32in, RUNIT_FMT_Q8_0, false, false, RES_F32)
GEMV_TWIN(gemv_q8_0_f32in, RUNIT_FMT_Q8_0, false, true)
GEMV_TWIN(gemv_q8_0_f16, RUNIT_FMT_Q8_0, true, true)
GEMV_TWIN_RES(gemv_q8_0_add_f16, RUNIT_FMT_Q8_0, true, true, RES_F16)
GEMV_TWIN_RES(gemv_q8_0_add_f32res_f16, RUNIT_FMT_Q8_0, true, false, RES_F32)
// launch-shape variants: gemv_multirow.metal:163-243, gemv_q8_0_wide.metal:28-163
GEMV_TWIN(gemv_q8_0_f32in_f32out_mr, RUNIT_FMT_Q8_0, false, false)
GEMV_TWIN_RES(gemv_q8_0_add_f32_f32in_mr, RUNIT_FMT_Q8_0, false, false, RES_F32)
GEMV_TWIN(gemv_q8_0_f32in_f32out_wide, RUNIT_FMT_Q8_0, false, false)
GEMV_TWIN_RES(gemv_q8_0_add_f32_f32in_wide, RUNIT_FMT_Q8_0, false, false, RES_F32)
GEMV_TWIN(gemv_q8_0_f32in_wide, RUNIT_FMT_Q8_0, false, true)
// Q4_0: crates/kernels/shaders/gemv_q4_0.metal:75-246
GEMV_TWIN(gemv_q4_0_f32in_f32out, RUNIT_FMT_Q4_0, false, false)
GEMV_TWIN_RES(gemv_q4_0_add_f32_f32in, RUNIT_FMT_Q4_0, false, false, RES_F32)
GEMV_TWIN(gemv_q4_0_f32in, RUNIT_FMT_Q4_0, false, true)
GEMV_TWIN(gemv_q4_0_f16, RUNIT_FMT_Q4_0, true, true)
GEMV_TWIN_RES(gemv_q4_0_add_f16, RUNIT_FMT_Q4_0, true, true, RES_F16)
// Q4_K: crates/kernels/shaders/gemv_q4k.metal:126-271
GEMV_TWIN(gemv_q4k_f32in_f32out, RUNIT_FMT_Q4K, false, false)
GEMV_TWIN_RES(gemv_q4k_add_f32_f32in, RUNIT_FMT_Q4K, false, false, RES_F32)
GEMV_TWIN(gemv_q4k_f16, RUNIT_FMT_Q4K, true, true)
GEMV_TWIN_RES(gemv_q4k_add_f16, RUNIT_FMT_Q4K, true, true, RES_F16)
GEMV_TWIN_RES(gemv_q4k_add_f32res_f16, RUNIT_FMT_Q4K, true, false, RES_F32)

// crates/kernels/shaders/fused_qkv.metal:13-119
int32_t runit_fused_qkv_q8_0_f32(runit_ctx_t* ctx, const void* w_q, const void* w_k, const void* w_v, const void* x,
                                 void* out_q, void* out_k, void* out_v, uint32_t q_dim, uint32_t kv_dim, uint32_t k) {
    return fused_qkv(ctx, "fused_qkv_q8_0_f32", RUNIT_FMT_Q8_0, w_q, w_k, w_v, x, out_q, out_k, out_v, nullptr, nullptr,
                     nullptr, BIAS_NONE, q_dim, kv_dim, k);
}
int32_t runit_fused_qkv_bias_q8_0_f32(runit_ctx_t* ctx, const void* w_q, const void* w_k, const void* w_v, const void* x,
                                      void* out_q, void* out_k, void* out_v, const void* bias_q, const void* bias_k,
                                      const void* bias_v, uint32_t q_dim, uint32_t kv_dim, uint32_t k) {
    return fused_qkv(ctx, "fused_qkv_bias_q8_0_f32", RUNIT_FMT_Q8_0, w_q, w_k, w_v, x, out_q, out_k, out_v, bias_q, bias_k,
                     bias_v, BIAS_F16, q_dim, kv_dim, k);
}
int32_t runit_fused_qkv_f32bias_q8_0_f32(runit_ctx_t* ctx, const void* w_q, const void* w_k, const void* w_v,
                                         const void* x, void* out_q, void* out_k, void* out_v, const void* bias_q,
                                         const void* bias_k, const void* bias_v, uint32_t q_dim, uint32_t kv_dim,
                                         uint32_t k) {
    const bool has_bias = bias_q || bias_k || bias_v;
    return fused_qkv(ctx, "fused_qkv_f32bias_q8_0_f32", RUNIT_FMT_Q8_0, w_q, w_k, w_v, x, out_q, out_k, out_v, bias_q,
                     bias_k, bias_v, has_bias ? BIAS_F32 : BIAS_NONE, q_dim, kv_dim, k);
}
// crates/kernels/shaders/fused_ffn.metal:36-93 and gemv_q4_0.metal:254-311
int32_t runit_fused_ffn_q8_0_f32(runit_ctx_t* ctx, const void* w_gate, const void* w_up, const void* x, void* act_out,
                                 uint32_t ff_dim, uint32_t k) {
    return fused_ffn(ctx, "fused_ffn_q8_0_f32", RUNIT_FMT_Q8_0, w_gate, w_up, x, act_out, ff_dim, k);
}
int32_t runit_fused_ffn_q4_0_f32(runit_ctx_t* ctx, const void* w_gate, const void* w_up, const void* x, void* act_out,
                                 uint32_t ff_dim, uint32_t k) {
    return fused_ffn(ctx, "fused_ffn_q4_0_f32", RUNIT_FMT_Q4_0, w_gate, w_up, x, act_out, ff_dim, k);
}

// No twins: the reference fuses Q|K|V and gate/up only for Q8_0 (and gate/up for Q4_0); the same launches
// for the other formats save two (one) kernel launches per layer.
int32_t runit_fused_qkv_q4_0_f32(runit_ctx_t* ctx, const void* w_q, const void* w_k, const void* w_v, const void* x,
                                 void* out_q, void* out_k, void* out_v, uint32_t q_dim, uint32_t kv_dim, uint32_t k) {
    return fused_qkv(ctx, "fused_qkv_q4_0_f32", RUNIT_FMT_Q4_0, w_q, w_k, w_v, x, out_q, out_k, out_v, nullptr, nullptr,
                     nullptr, BIAS_NONE, q_dim, kv_dim, k);
}
int32_t runit_fused_qkv_q4k_f32(runit_ctx_t* ctx, const void* w_q, const void* w_k, const void* w_v, const void* x,
                                void* out_q, void* out_k, void* out_v, uint32_t q_dim, uint32_t kv_dim, uint32_t k) {
    return fused_qkv(ctx, "fused_qkv_q4k_f32", RUNIT_FMT_Q4K, w_q, w_k, w_v, x, out_q, out_k, out_v, nullptr, nullptr,
                     nullptr, BIAS_NONE, q_dim, kv_dim, k);
}
int32_t runit_fused_ffn_q4k_f32(runit_ctx_t* ctx, const void* w_gate, const void* w_up, const void* x, void* act_out,
                                uint32_t ff_dim, uint32_t k) {
    return fused_ffn(ctx, "fused_ffn_q4k_f32", RUNIT_FMT_Q4K, w_gate, w_up, x, act_out, ff_dim, k);
}

int32_t runit_rms_norm_gemv_f32(runit_ctx_t* ctx, int32_t fmt, const void* weight, const void* x, const void* gamma, float eps,
                                void* output, const void* residual, uint32_t m, uint32_t k) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, gamma && m > 0, "rms_norm_gemv_f32: null gamma or m == 0");
    return gemv_plain(ctx, "rms_norm_gemv_f32", fmt, weight, x, output, residual, m, k, (const float*)gamma, eps, nullptr, nullptr);
}
int32_t runit_rms_norm_fused_qkv_f32(runit_ctx_t* ctx, int32_t fmt, const void* w_q, const void* w_k, const void* w_v, const void* x,
                                     const void* gamma, float eps, void* out_q, void* out_k, void* out_v, uint32_t q_dim,
                                     uint32_t kv_dim, uint32_t k) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, gamma, "rms_norm_fused_qkv_f32: null gamma");
    const void* ws[3] = {w_q, w_k, w_v};
    void* ys[3] = {out_q, out_k, out_v};
    const uint32_t rows[3] = {q_dim, kv_dim, kv_dim};
    return gemv_segments(ctx, "rms_norm_fused_qkv_f32", fmt, 3, ws, ys, rows, x, k, (const float*)gamma, eps, nullptr);
}

// (largest value, index) pairs pushed by the ranks -> index of the overall maximum (lowest index among equal values).
__global__ void argmax_pairs_kernel(const uint2* __restrict__ pairs, uint32_t n, int32_t* __restrict__ result) {
    grid_dependency_wait();
    grid_launch_dependents();
    float bv = -INFINITY;
    uint32_t bi = 0xFFFFFFFFu;
    for (uint32_t i = threadIdx.x; i < n; i += 32) {
        const uint2 pr = __ldcg(&pairs[i]);
        am_better(bv, bi, __uint_as_float(pr.x), pr.y);
    }
    am_warp_reduce(bv, bi);
    if (threadIdx.x == 0) result[0] = (int32_t)bi;
}

int32_t runit_gemv_argmax_f32(runit_ctx_t* ctx, int32_t fmt, const void* weight, const void* x, const void* gamma, float eps,
                              void* logits, void* result, uint32_t m, uint32_t k) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, result && runit_aligned(result, 4) && m > 0, "gemv_argmax_f32: null or misaligned result, or m == 0");
    return gemv_plain(ctx, "gemv_argmax_f32", fmt, weight, x, logits, nullptr, m, k, (const float*)gamma, eps, (int32_t*)result, nullptr);
}

int32_t runit_gemv_argmax_allgather(runit_ctx_t* ctx, int32_t fmt, const void* w_local, const void* x, void* logits_local,
                                    void* const* pairs_all, uint32_t world, uint32_t rank, uint32_t rows_total, uint32_t k) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, pairs_all && world >= 1 && world <= 8 && rank < world && rows_total > 0 && rows_total % world == 0,
                  "gemv_argmax_allgather: world=%u rank=%u rows=%u unsupported (1..8 ranks, rows divisible)", world, rank, rows_total);
    const uint32_t n = rows_total / world;
    GemvCall c;
    c.name = "gemv_argmax_allgather";
    c.fmt = fmt;
    c.w[0] = w_local;
    c.x = x;
    c.y[0] = logits_local;
    c.rows[0] = n;
    c.k = k;
    c.am = true;
    c.am_base = rank * n;
    for (uint32_t p = 0; p < world; p++) {
        RUNIT_REQUIRE(ctx, pairs_all[p], "gemv_argmax_allgather: null pair table for rank %u", p);
        c.am_dst[c.am_ndst++] = reinterpret_cast<uint2*>(pairs_all[p]) + rank;
    }
    return gemv_dispatch(ctx, c);
}

int32_t runit_argmax_pairs(runit_ctx_t* ctx, const void* pairs, uint32_t n, void* result) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, pairs && result && n > 0 && runit_aligned(pairs, 8) && runit_aligned(result, 4), "argmax_pairs: bad argument");
    runit_launch_chain(ctx, argmax_pairs_kernel, dim3(1), dim3(32), (const uint2*)pairs, n, (int32_t*)result);
    return runit_after_launch(ctx, "argmax_pairs");
}

int32_t runit_gemv_batched_multi_f32(runit_ctx_t* ctx, int32_t fmt, uint32_t n_mats, const void* const* weights, const void* input,
                                     void* const* outputs, const uint32_t* rows, uint32_t k, uint32_t batch) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, n_mats >= 1 && n_mats <= 3 && weights && outputs && rows && input, "gemv_batched_multi_f32: 1..3 matrices, no null table");
    RUNIT_REQUIRE(ctx, batch >= 1 && batch <= 8, "gemv_batched_multi_f32: batch=%u not in 1..8", batch);
    bool ok = gemv_imma_applies(ctx, fmt, k, batch) && runit_aligned(input, 16) && (k / 256 * 144) % 16 == 0 && ctx->tune.gemv_variant != 1;
    for (uint32_t i = 0; i < n_mats; i++) {
        RUNIT_REQUIRE(ctx, weights[i] && outputs[i] && rows[i] > 0, "gemv_batched_multi_f32: null matrix or output %u", i);
        ok = ok && runit_aligned(weights[i], 16) && runit_aligned(outputs[i], 4);
    }
    if (ok) return gemv_imma_multi(ctx, fmt, n_mats, weights, (const float*)input, (float* const*)outputs, nullptr, rows, k, batch);
    for (uint32_t i = 0; i < n_mats; i++) {      // other formats and batch 1: one launch per matrix
        const int32_t st = runit_gemv_batched_f32(ctx, fmt, weights[i], input, outputs[i], nullptr, rows[i], k, batch);
        if (st != RUNIT_OK) return st;
    }
    return RUNIT_OK;
}

int32_t runit_gemv_batched_f32(runit_ctx_t* ctx, int32_t fmt, const void* weight, const void* input, void* output,
                               const void* residual, uint32_t m, uint32_t k, uint32_t batch) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, batch >= 1 && batch <= 8, "gemv_batched_f32: batch=%u not in 1..8", batch);
    RUNIT_REQUIRE(ctx, m > 0, "gemv_batched_f32: m == 0");
    // 4-bit formats, batch 2..8: integer tensor-core path (activations quantised once, weights streamed once).
    if (gemv_imma_applies(ctx, fmt, k, batch) && weight && input && output && runit_aligned(weight, 16) && runit_aligned(input, 16) &&
        runit_aligned(output, 4) && (k / 256 * 144) % 16 == 0 && ctx->tune.gemv_variant != 1)
        return gemv_imma(ctx, fmt, weight, (const float*)input, (float*)output, (const float*)residual, m, k, batch);
    // Kernels exist for batch 1, 2, 4, 8; other sizes run as a sum of those.
    uint32_t done = 0;
    while (done < batch) {
        const uint32_t left = batch - done;
        const uint32_t b = left >= 8 ? 8 : left >= 4 ? 4 : left >= 2 ? 2 : 1;
        GemvCall c;
        c.name = "gemv_batched_f32";
        c.fmt = fmt;
        c.w[0] = weight;
        c.x = (const float*)input + (size_t)done * k;
        c.y[0] = (float*)output + (size_t)done * m;
        c.res[0] = residual ? (const float*)residual + (size_t)done * m : nullptr;
        c.res_kind = residual ? RES_F32 : RES_NONE;
        c.rows[0] = m;
        c.k = k;
        c.batch = b;
        int32_t st = gemv_dispatch(ctx, c);
        if (st != RUNIT_OK) return st;
        done += b;
    }
    return RUNIT_OK;
}


// ───────────────────────── row-sharded GEMV with the all-gather in the epilogue ─────────────────────────
// Waits for the flags of all ranks with a time bound; the flags only ever grow (epoch numbers), so nothing is reset.
struct PeerPads {
    uint32_t* p[8];   // signal words of every rank: pad[r][q] = latest epoch rank q has announced to rank r
};
// epoch_ptr != nullptr: the epoch is that device word + 1, and the word is advanced once the barrier has been passed
// (recorded command lists replay the same launch for every call).
// abort: device word of the context.  The first barrier that gives up sets it; while it is set every later barrier still
// announces its epoch and advances the epoch word but does not wait, so a queue of recorded barriers behind a missing
// rank costs one time limit in total instead of one each.  runit_flush clears it when it reports the time-out.
// pairs != nullptr: after the barrier, lane p reads the (value, index) pair that rank p pushed into slot p of this rank's
// table (runit_gemv_argmax_allgather) and the warp reduces them to the greedy token in *pair_result.
__global__ void peer_barrier_kernel(const PeerPads pp, uint32_t world, uint32_t rank, uint32_t epoch, int32_t* status,
                                    uint32_t* epoch_ptr, uint32_t* abort, const uint2* pairs, int32_t* pair_result) {
    uint32_t* const* pads = pp.p;
    const uint32_t p = threadIdx.x;
    if (epoch_ptr) epoch = *epoch_ptr + 1u;
    const bool aborted = abort && *reinterpret_cast<volatile uint32_t*>(abort) != 0u;
    __syncwarp();
    if (p == 0 && epoch_ptr) *epoch_ptr = epoch;   // read by every lane above; the following kernels see the new value
    if (p < world) {
        // The stores of the preceding kernels (results pushed into the peers' memory) are ordered before the flag.
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pads[p] + rank), "r"(epoch) : "memory");
        if (!aborted) {
            const uint32_t* mine = pads[rank] + p;
            const long long t0 = clock64();
            while (true) {
                uint32_t v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
                if ((int32_t)(v - epoch) >= 0) break;
                if (clock64() - t0 > (1ll << 30)) {   // about half a second: the peer never signalled
                    if (status) atomicExch(status, 3);
                    if (abort) atomicExch(abort, 1u);
                    break;
                }
                __nanosleep(200);
            }
        }
    }
    if (pairs == nullptr) return;
    __syncwarp();
    float bv = -INFINITY;
    uint32_t bi = 0xFFFFFFFFu;
    if (p < world) {
        const uint2 pr = __ldcg(&pairs[p]);    // written by rank p before the flag this lane has just acquired
        bv = __uint_as_float(pr.x);
        bi = pr.y;
    }
    am_warp_reduce(bv, bi);
    if (p == 0) pair_result[0] = (int32_t)bi;
}

int32_t runit_gemv_allgather_f32(runit_ctx_t* ctx, int32_t fmt, const void* w_local, const void* x, void* const* y_all,
                                 uint32_t world, uint32_t rank, uint32_t rows_total, uint32_t k) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, y_all && world >= 1 && world <= 8 && rank < world && rows_total > 0 && rows_total % world == 0,
                  "gemv_allgather_f32: world=%u rank=%u rows=%u unsupported (1..8 ranks, rows divisible)", world, rank, rows_total);
    const uint32_t n = rows_total / world;
    GemvCall c;
    c.name = "gemv_allgather_f32";
    c.fmt = fmt;
    c.w[0] = w_local;
    c.x = x;
    c.rows[0] = n;
    c.k = k;
    for (uint32_t p = 0; p < world; p++) {
        RUNIT_REQUIRE(ctx, y_all[p], "gemv_allgather_f32: null output pointer for rank %u", p);
        float* slice = (float*)y_all[p] + (size_t)rank * n;
        if (p == rank) c.y[0] = slice;
        else c.peer_y[c.n_peer++] = slice;
    }
    return gemv_dispatch(ctx, c);
}

int32_t runit_peer_barrier_argmax(runit_ctx_t* ctx, void* const* signal_pads, uint32_t world, uint32_t rank, uint32_t epoch,
                                  const void* pairs, void* result) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, epoch > 0 && pairs && result && runit_aligned(pairs, 8) && runit_aligned(result, 4), "peer_barrier_argmax: bad argument");
    return runit::peer_barrier_launch(ctx, signal_pads, world, rank, epoch, nullptr, pairs, (int32_t*)result);
}

int32_t runit_peer_barrier(runit_ctx_t* ctx, void* const* signal_pads, uint32_t world, uint32_t rank, uint32_t epoch) {
    if (!ctx) return RUNIT_ERR_BAD_ARG;
    RUNIT_REQUIRE(ctx, epoch > 0, "peer_barrier: epoch must be positive");
    return runit::peer_barrier_launch(ctx, signal_pads, world, rank, epoch, nullptr);
}

}  // extern "C"

namespace runit {
int32_t peer_barrier_launch(runit_ctx* ctx, void* const* signal_pads, uint32_t world, uint32_t rank, uint32_t epoch, uint32_t* epoch_ptr,
                            const void* pairs, int32_t* pair_result) {
    RUNIT_REQUIRE(ctx, signal_pads && world >= 1 && world <= 8 && rank < world && (epoch > 0 || epoch_ptr), "peer_barrier: bad argument");
    PeerPads h{};
    for (uint32_t p = 0; p < world; p++) {
        RUNIT_REQUIRE(ctx, signal_pads[p] && runit_aligned(signal_pads[p], 4), "peer_barrier: null or misaligned pad %u", p);
        h.p[p] = (uint32_t*)signal_pads[p];
    }
    peer_barrier_kernel<<<1, 32, 0, ctx->stream>>>(h, world, rank, epoch, ctx->d_status, epoch_ptr, ctx->d_abort, (const uint2*)pairs,
                                                   pair_result);
    return runit_after_launch(ctx, "peer_barrier");
}
}  // namespace runit
