// Host-side interface of the fused GEMV stream (gemv_stream.cu): while a command list is being recorded, every
// fusable GEMV launch leaves a record here; when the recording ends, each run of consecutive recorded launches in the
// captured graph is replaced by one launch of the persistent kernel (gemv_stream.cuh).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <vector>

struct runit_ctx;

namespace runit {

// One fusable launch: batch 1, 4-bit format, f32 activations, tiled bulk loads, integer tensor-core arithmetic,
// no expert grouping, no peer stores.
struct StreamRec {
    const void* func;        // kernel the launch used (to find its node in the captured graph)
    const void* w0;          // first weight pointer and input pointer: checked against the node's own arguments
    const void* x;
    int32_t fmt, dual, nseg;
    CUtensorMap map[4];      // per segment; [3] = second matrix of a fused gate/up launch
    void* y[3];
    const void* res[3];
    const void* bias[3];
    uint32_t rows[3];
    uint32_t k, nb, n_units;
    int32_t out_f16, res_kind, bias_kind;
};

void stream_rec_begin(runit_ctx* ctx);                       // start collecting (clears earlier records)
void stream_rec_push(runit_ctx* ctx, const StreamRec& r);    // no-op unless a recording is open
void stream_rec_discard(runit_ctx* ctx);
// Rewrites `graph` in place; device memory the new nodes use is appended to `allocs` (the owner of the instantiated
// graph frees it).  Returns a status; on any doubt about the graph's shape the graph is left as recorded.
int32_t stream_rec_fuse(runit_ctx* ctx, cudaGraph_t graph, std::vector<void*>* allocs, uint32_t* n_fused_launches);

}  // namespace runit
