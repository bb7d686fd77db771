// Host side of the fused GEMV stream: collects the fusable GEMV launches of a recording, and rewrites the captured
// graph so that every run of consecutive ones becomes one launch of gemv_stream_kernel.
//
// The reference commits all the dispatches of a token in one command buffer (crates/kernels/src/context.rs:248-296)
// and its GPU runs them back to back; the ops of a recorded command list here keep exactly that meaning — in-order
// execution, results identical to the separate launches up to the summation order over K-slices — while the
// dependent GEMVs of a token share one persistent kernel.  Ordering between two fused GEMVs is kept wherever it can
// be observed: a GEMV waits for every earlier one whose outputs it reads or overwrites, or whose inputs it overwrites
// (byte-range overlap of the recorded pointers).
#include "gemv_stream.cuh"
#include "gemv_stream_host.h"
#include "runit_internal.h"

#include <algorithm>
#include <bitset>
#include <vector>

namespace runit {

using RecVec = std::vector<StreamRec>;

void stream_rec_begin(runit_ctx* ctx) {
    if (!ctx->stream_rec) ctx->stream_rec = new RecVec();
    static_cast<RecVec*>(ctx->stream_rec)->clear();
}
void stream_rec_push(runit_ctx* ctx, const StreamRec& r) {
    if (ctx->capturing && ctx->stream_rec && ctx->tune.stream_fuse) static_cast<RecVec*>(ctx->stream_rec)->push_back(r);
}
void stream_rec_discard(runit_ctx* ctx) {
    if (ctx->stream_rec) static_cast<RecVec*>(ctx->stream_rec)->clear();
}

namespace gs {

struct Range {
    uintptr_t lo, hi;
};
static bool overlaps(const std::vector<Range>& a, const std::vector<Range>& b) {
    for (const Range& p : a)
        for (const Range& q : b)
            if (p.lo < q.hi && q.lo < p.hi) return true;
    return false;
}
static void add_range(std::vector<Range>& v, const void* p, size_t bytes) {
    if (p && bytes) v.push_back({reinterpret_cast<uintptr_t>(p), reinterpret_cast<uintptr_t>(p) + bytes});
}

struct KernelChoice {
    const void* func;
    int nw, stages;
    size_t smem;
};
template <int FMT, int NW, int S>
static KernelChoice choice() {
    return {reinterpret_cast<const void*>(&gemv_stream_kernel<FMT, NW, S>), NW, S, (size_t)NW * (S * kStageBytes + kXqBytes) + 128};
}
static KernelChoice pick_kernel(int fmt, int cfg) {
    const bool q4k = fmt == RUNIT_FMT_Q4K;
    switch (cfg) {
        case 1: return q4k ? choice<RUNIT_FMT_Q4K, 20, 2>() : choice<RUNIT_FMT_Q4_0, 20, 2>();
        case 2: return q4k ? choice<RUNIT_FMT_Q4K, 14, 3>() : choice<RUNIT_FMT_Q4_0, 14, 3>();
        case 3: return q4k ? choice<RUNIT_FMT_Q4K, 12, 3>() : choice<RUNIT_FMT_Q4_0, 12, 3>();
        default: return q4k ? choice<RUNIT_FMT_Q4K, 16, 2>() : choice<RUNIT_FMT_Q4_0, 16, 2>();
    }
}

struct Program {
    std::vector<OpFull> full;
    std::vector<OpLite> lite;
    std::vector<std::vector<Range>> reads, writes;
    std::vector<std::bitset<kMaxOps>> anc;   // every earlier GEMV this one is ordered after (transitively)
    uint32_t total_items = 0;
};

// Warps per tile (K-slices) and tiles per CTA-item for a GEMV of `tiles` tiles and `units` K-units on `sms` CTAs of `nw`
// warps: the split with the lowest estimated time in units of one warp-stage.  One wave of items (items <= CTAs) costs
// the units a warp streams; more waves cost their number plus half an item for the tail that dynamic hand-out leaves;
// every item and every team reduction adds a little.
static void pick_split(uint32_t tiles, uint32_t units, uint32_t nw, uint32_t sms, uint32_t* ksl_out, uint32_t* tpc_out) {
    double best = 1e30;
    uint32_t bk = 1;
    for (uint32_t ksl = 1; ksl <= nw && ksl <= units; ksl++) {
        const uint32_t tpc = nw / ksl;
        const uint32_t items = (tiles + tpc - 1) / tpc;
        const double pwu = (double)((units + ksl - 1) / ksl);
        const double waves = (double)items / sms;
        double cost = items <= sms ? pwu : (waves + 0.5) * pwu;
        cost += 0.35 * std::max(1.0, waves) + (ksl > 1 ? 0.3 : 0.0);
        if (cost < best - 1e-9) { best = cost; bk = ksl; }
    }
    *ksl_out = bk;
    *tpc_out = nw / bk;
}

// Appends the GEMV to the program.  Returns false (and leaves the program unchanged) if it does not fit: the table is
// full, or it would need more dependency slots than an entry has.
static bool program_add(Program& P, const StreamRec& r, uint32_t nw, uint32_t sms, uint32_t force_ksl) {
    const uint32_t n = (uint32_t)P.lite.size();
    if (n >= kMaxOps) return false;
    OpFull f;
    memset(&f, 0, sizeof(f));
    OpLite l;
    memset(&l, 0, sizeof(l));
    const uint32_t rpt = r.dual ? kRT / 2 : kRT;
    std::vector<Range> rd, wr;
    uint32_t tiles = 0;
    l.tile_begin1 = l.tile_begin2 = kNoSeg;
    for (int i = 0; i < r.nseg; i++) {
        f.map[i] = r.map[i];
        l.y[i] = r.y[i];
        l.res[i] = r.res[i];
        l.bias[i] = r.bias[i];
        l.rows[i] = r.rows[i];
        if (i == 1) l.tile_begin1 = tiles;
        if (i == 2) l.tile_begin2 = tiles;
        tiles += (r.rows[i] + rpt - 1) / rpt;
        add_range(wr, r.y[i], (size_t)r.rows[i] * (r.out_f16 ? 2 : 4));
        if (r.res_kind != RES_NONE) add_range(rd, r.res[i], (size_t)r.rows[i] * 4);
        if (r.bias_kind != BIAS_NONE) add_range(rd, r.bias[i], (size_t)r.rows[i] * (r.bias_kind == BIAS_F16 ? 2 : 4));
    }
    if (r.dual) f.map[3] = r.map[3];
    l.out_f16 = (uint8_t)r.out_f16;
    l.res_kind = (uint8_t)r.res_kind;
    l.bias_kind = (uint8_t)r.bias_kind;
    add_range(rd, r.x, (size_t)r.k * 4);

    uint32_t ksl = 1, tpc = nw;
    pick_split(tiles, r.n_units, nw, sms, &ksl, &tpc);
    if (force_ksl >= 1 && force_ksl <= nw && force_ksl <= r.n_units) { ksl = force_ksl; tpc = nw / ksl; }
    l.item_begin = P.total_items;
    l.n_items = (tiles + tpc - 1) / tpc;
    l.ksl = ksl;
    l.tpc = tpc;
    l.n_units = r.n_units;
    l.n_tiles = tiles;
    l.dual = (uint32_t)r.dual;
    l.k = r.k;
    l.nb = r.nb;
    l.x = static_cast<const float*>(r.x);
    if ((uint64_t)P.total_items + l.n_items >= (1ull << 31)) return false;

    // dependencies: the latest earlier GEMVs with a read-after-write, write-after-write or write-after-read overlap
    // that are not already ordered before one of the chosen ones
    std::bitset<kMaxOps> anc;
    uint32_t nd = 0;
    for (uint32_t d = 0; d < kMaxDeps; d++) l.dep[d] = (uint16_t)kNoDep;
    for (int m = (int)n - 1; m >= 0; m--) {
        if (anc.test((size_t)m)) continue;
        const bool hazard = overlaps(P.writes[m], rd) || overlaps(P.writes[m], wr) || overlaps(P.reads[m], wr);
        if (!hazard) continue;
        if (nd == kMaxDeps) return false;
        l.dep[nd++] = (uint16_t)m;
        anc |= P.anc[m];
        anc.set((size_t)m);
    }
    P.full.push_back(f);
    P.lite.push_back(l);
    P.reads.push_back(rd);
    P.writes.push_back(wr);
    P.anc.push_back(anc);
    P.total_items += l.n_items;
    return true;
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Uploads the program and adds its kernel node to `graph` after `pred` (nullptr: a root).  The node is returned.
static int32_t program_emit(runit_ctx* ctx, const Program& P, int fmt, const KernelChoice& kc, cudaGraph_t graph, cudaGraphNode_t pred,
                            std::vector<void*>* allocs, cudaGraphNode_t* out_node) {
    const size_t n = P.lite.size();
    const size_t off_full = 0;
    const size_t off_lite = align_up(off_full + n * sizeof(OpFull), 256);
    const size_t off_done = align_up(off_lite + n * sizeof(OpLite), 256);
    const size_t off_ctl = align_up(off_done + n * 4, 256);
    const size_t bytes = off_ctl + 256;
    uint8_t* d = nullptr;
    cudaError_t e = cudaMalloc((void**)&d, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return runit_fail(ctx, RUNIT_ERR_ALLOC, "fused GEMV stream: allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    }
    allocs->push_back(d);
    RUNIT_CUDA_TRY(ctx, cudaMemset(d, 0, bytes));   // counters at rest
    RUNIT_CUDA_TRY(ctx, cudaMemcpy(d + off_full, P.full.data(), n * sizeof(OpFull), cudaMemcpyHostToDevice));
    RUNIT_CUDA_TRY(ctx, cudaMemcpy(d + off_lite, P.lite.data(), n * sizeof(OpLite), cudaMemcpyHostToDevice));
    Params prm;
    memset(&prm, 0, sizeof(prm));
    prm.full = reinterpret_cast<const OpFull*>(d + off_full);
    prm.lite = reinterpret_cast<const OpLite*>(d + off_lite);
    prm.n_ops = (uint32_t)n;
    prm.total_items = P.total_items;
    prm.done = reinterpret_cast<uint32_t*>(d + off_done);
    prm.ctl = reinterpret_cast<uint32_t*>(d + off_ctl);
    prm.status = ctx->d_status;
    prm.dynamic = ctx->tune.stream_dynamic ? 1 : 0;
    (void)fmt;
    void* kargs[1] = {&prm};
    cudaKernelNodeParams kp;
    memset(&kp, 0, sizeof(kp));
    kp.func = const_cast<void*>(kc.func);
    kp.gridDim = dim3((unsigned)ctx->sm_count);
    kp.blockDim = dim3((unsigned)(kc.nw * 32));
    kp.sharedMemBytes = (unsigned)kc.smem;
    kp.kernelParams = kargs;
    kp.extra = nullptr;
    RUNIT_CUDA_TRY(ctx, cudaGraphAddKernelNode(out_node, graph, pred ? &pred : nullptr, pred ? 1 : 0, &kp));
    return RUNIT_OK;
}

}  // namespace gs

int32_t stream_rec_fuse(runit_ctx* ctx, cudaGraph_t graph, std::vector<void*>* allocs, uint32_t* n_fused_launches) {
    using namespace gs;
    if (n_fused_launches) *n_fused_launches = 0;
    RecVec* recs = static_cast<RecVec*>(ctx->stream_rec);
    if (!recs || recs->size() < 2 || !ctx->tune.stream_fuse) return RUNIT_OK;

    // ── the captured graph as a chain (one stream was recorded: every node has one successor) ──
    size_t n_nodes = 0;
    RUNIT_CUDA_TRY(ctx, cudaGraphGetNodes(graph, nullptr, &n_nodes));
    size_t n_roots = 0;
    RUNIT_CUDA_TRY(ctx, cudaGraphGetRootNodes(graph, nullptr, &n_roots));
    if (n_nodes < 2 || n_roots != 1) return RUNIT_OK;
    cudaGraphNode_t node = nullptr;
    n_roots = 1;
    RUNIT_CUDA_TRY(ctx, cudaGraphGetRootNodes(graph, &node, &n_roots));
    std::vector<cudaGraphNode_t> chain;
    while (node) {
        chain.push_back(node);
        if (chain.size() > n_nodes) return RUNIT_OK;   // not a chain
        size_t nd = 0;
        RUNIT_CUDA_TRY(ctx, cudaGraphNodeGetDependentNodes_v2(node, nullptr, nullptr, &nd));
        if (nd == 0) break;
        if (nd != 1) return RUNIT_OK;
        cudaGraphNode_t next = nullptr;
        cudaGraphEdgeData ed;
        RUNIT_CUDA_TRY(ctx, cudaGraphNodeGetDependentNodes_v2(node, &next, &ed, &nd));
        node = next;
    }
    if (chain.size() != n_nodes) return RUNIT_OK;

    // ── which nodes are the recorded launches (same kernel, same first weight pointer, same input) ──
    std::vector<int> rec_of(chain.size(), -1);
    size_t ri = 0;
    for (size_t i = 0; i < chain.size() && ri < recs->size(); i++) {
        cudaGraphNodeType ty;
        RUNIT_CUDA_TRY(ctx, cudaGraphNodeGetType(chain[i], &ty));
        if (ty != cudaGraphNodeTypeKernel) continue;
        cudaKernelNodeParams kp;
        RUNIT_CUDA_TRY(ctx, cudaGraphKernelNodeGetParams(chain[i], &kp));
        const StreamRec& r = (*recs)[ri];
        if (kp.func != r.func || !kp.kernelParams || !kp.kernelParams[0]) continue;
        const GemvArgs* a = static_cast<const GemvArgs*>(kp.kernelParams[0]);
        if (a->seg[0].w != r.w0 || a->x != r.x || a->grp_expert != nullptr || a->n_peer != 0) continue;
        rec_of[i] = (int)ri++;
    }
    if (ri != recs->size()) return RUNIT_OK;   // a record without its node: leave the graph as recorded

    const uint32_t force_ksl = ctx->tune.stream_ksl > 0 ? (uint32_t)ctx->tune.stream_ksl : 0u;
    uint32_t fused = 0;
    size_t i = 0;
    while (i < chain.size()) {
        if (rec_of[i] < 0) { i++; continue; }
        const int fmt = (*recs)[rec_of[i]].fmt;
        const KernelChoice kc = pick_kernel(fmt, ctx->tune.stream_cfg);
        static bool configured[16][8] = {{false}};
        const int slot = (fmt == RUNIT_FMT_Q4K ? 0 : 4) + (ctx->tune.stream_cfg & 3);
        if (ctx->device < 16 && !configured[ctx->device][slot]) {
            RUNIT_CUDA_TRY(ctx, cudaFuncSetAttribute(kc.func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kc.smem));
            configured[ctx->device][slot] = true;
        }
        int resident = 0;
        RUNIT_CUDA_TRY(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kc.func, kc.nw * 32, kc.smem));
        if (resident < 1) return RUNIT_OK;   // the persistent grid would not be co-resident: keep the separate launches
        Program P;
        size_t j = i;
        while (j < chain.size() && rec_of[j] >= 0 && (*recs)[rec_of[j]].fmt == fmt &&
               program_add(P, (*recs)[rec_of[j]], (uint32_t)kc.nw, (uint32_t)ctx->sm_count, force_ksl))
            j++;
        if (j - i < 2) { i = std::max(j, i + 1); continue; }
        cudaGraphNode_t pred = i > 0 ? chain[i - 1] : nullptr, fresh = nullptr;
        int32_t st = program_emit(ctx, P, fmt, kc, graph, pred, allocs, &fresh);
        if (st != RUNIT_OK) return st;
        if (j < chain.size()) RUNIT_CUDA_TRY(ctx, cudaGraphAddDependencies(graph, &fresh, &chain[j], 1));
        for (size_t q = i; q < j; q++) RUNIT_CUDA_TRY(ctx, cudaGraphDestroyNode(chain[q]));
        chain[j - 1] = fresh;   // predecessor of whatever follows
        fused += (uint32_t)(j - i);
        i = j;
    }
    if (n_fused_launches) *n_fused_launches = fused;
    ctx->fused_launches += fused;
    return RUNIT_OK;
}

}  // namespace runit
