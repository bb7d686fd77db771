/*
 * runit_cuda.h — C ABI of the B200 (sm_100a) implementation of RunIT's quantized decode path.
 *
 * Every "twin" entry point replaces one free function of the reference's dispatch layer
 * (crates/kernels/src/dispatch.rs, cited per function as dispatch.rs:LINE; paths are relative
 * to the reference project root).  Names are the reference's, prefixed `runit_`; the argument
 * order is the reference's with `&MetalContext` -> `runit_ctx_t*`, `&metal::Buffer` -> device
 * pointer, `u32` -> uint32_t, `Result<()>` -> int32_t status.
 *
 * Execution model (replaces MetalContext::encode / flush, crates/kernels/src/context.rs:248-296):
 * every op is an in-order launch on the context's CUDA stream and returns at once;
 * runit_flush() waits for the stream and returns the first error since the last flush.
 * Ops never allocate, never synchronise and never retain pointers; the caller keeps buffers
 * alive until the next flush.  `output == residual` aliasing is allowed (the engine relies on
 * it, crates/engine/src/forward.rs:1619).  Arguments are validated on the host: a bad call
 * returns a status and launches nothing.
 *
 * There is no CPU fallback: without a CUDA device runit_ctx_create fails with
 * RUNIT_ERR_NO_DEVICE.  A context is used by one host thread at a time (the reference's
 * MetalContext is !Sync, context.rs:158).
 *
 * Weight layouts (row-major rows of blocks, as the reference lays them out):
 *   Q8_0: 34-byte blocks {f16 d; i8 qs[32]}, value = d*qs            gemv_q8_0.metal:11-14
 *   Q4_0: 18-byte blocks {f16 d; u8 qs[16]}, low nibble = element 2i, high = 2i+1,
 *         value = d*(nibble-8)                                        gemv_q4_0.metal:10-15
 *   Q4_K: 144-byte superblocks {f16 d; f16 dmin; u8 scales[12]; u8 qs[128]} of 256 elements;
 *         pair j: low nibbles of qs[32j..] -> elements 64j.., scale index j; high nibbles ->
 *         elements 64j+32.., scale index j+4                          dequant.metal:74-82
 * Alignment contract: weight base pointers 16-byte aligned (cudaMalloc gives 256); vectors
 * 16-byte aligned; k a multiple of 32 (Q8_0, Q4_0) or 256 (Q4_K).
 */
#ifndef RUNIT_CUDA_H
#define RUNIT_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct runit_ctx runit_ctx_t;

/* Status codes; the Rust shim maps them onto KernelError (crates/kernels/src/error.rs:4-22). */
enum {
    RUNIT_OK = 0,
    RUNIT_ERR_NO_DEVICE = 1,   /* KernelError::NoDevice */
    RUNIT_ERR_BAD_ARG = 2,     /* null pointer, k not a block multiple, zero rows, ... */
    RUNIT_ERR_BUFFER_SIZE = 3, /* KernelError::BufferSize */
    RUNIT_ERR_LAUNCH = 4,      /* a CUDA call failed; text in runit_last_error_string */
    RUNIT_ERR_NCCL = 5,
    RUNIT_ERR_TIMEOUT = 6,     /* a bounded device- or host-side wait ran out */
    RUNIT_ERR_UNSUPPORTED = 7,
    RUNIT_ERR_ALLOC = 8
};

enum { RUNIT_BUF_DEVICE = 0, RUNIT_BUF_HOST_VISIBLE = 1 };
enum { RUNIT_FMT_Q8_0 = 0, RUNIT_FMT_Q4_0 = 1, RUNIT_FMT_Q4K = 2, RUNIT_FMT_Q5_0 = 3, RUNIT_FMT_Q5K = 4, RUNIT_FMT_Q6K = 5 };

/* ── context, buffers, flush: MetalContext::{new,new_buffer,flush}, context.rs:163-296 ── */
int32_t runit_ctx_create(int32_t device, runit_ctx_t** out);
/* Adopt a stream the caller owns (e.g. the stream a collective library runs on). */
int32_t runit_ctx_create_on_stream(int32_t device, void* cuda_stream, runit_ctx_t** out);
int32_t runit_ctx_destroy(runit_ctx_t* ctx);
void*   runit_ctx_stream(runit_ctx_t* ctx);
int32_t runit_flush(runit_ctx_t* ctx);
const char* runit_last_error_string(runit_ctx_t* ctx);
const char* runit_status_string(int32_t status);
int32_t runit_buf_alloc(runit_ctx_t* ctx, size_t bytes, int32_t flags, void** dptr);
int32_t runit_buf_free(runit_ctx_t* ctx, void* dptr);
int32_t runit_memcpy_h2d(runit_ctx_t* ctx, void* dst_dev, const void* src_host, size_t bytes);
int32_t runit_memcpy_d2h(runit_ctx_t* ctx, void* dst_host, const void* src_dev, size_t bytes);
int32_t runit_memset(runit_ctx_t* ctx, void* dst_dev, int32_t byte, size_t bytes);
/* Per-op launch counter (kernels launched by this context since creation). */
uint64_t runit_launch_count(runit_ctx_t* ctx);
/* Test-only: selects kernel variants so that the parity tests can exercise every code path of the GEMV family
 * (0 = the default choice for every key).  Not part of the reference's interface; an engine never calls it. */
int32_t runit_set_tuning(runit_ctx_t* ctx, const char* key, int32_t value);

/* ── recorded command lists (no twin as a function; the role of the reference's command buffer,
 *    context.rs:248-296: ops are encoded once and committed together) ──
 * Between begin and end every op call on the context is recorded instead of executed; the
 * recorded list replays with one launch.  Pointers and sizes are baked in at record time.  */
typedef struct runit_graph runit_graph_t;
int32_t runit_graph_begin(runit_ctx_t* ctx);
int32_t runit_graph_end(runit_ctx_t* ctx, runit_graph_t** out);
int32_t runit_graph_launch(runit_ctx_t* ctx, runit_graph_t* graph);
int32_t runit_graph_destroy(runit_ctx_t* ctx, runit_graph_t* graph);
/* Opt-in (runit_set_tuning(ctx, "stream_fuse", 1) before runit_graph_begin): runs of consecutive batch-1 fused-dequant
 * GEMVs (4-bit formats, f32 activations) of a recording are executed by ONE persistent launch whose warps stream the
 * weights of the whole run without stopping at the boundaries between the GEMVs; the ops keep their recorded order
 * wherever one reads or overwrites what another wrote or read, and the results equal those of the separate launches up
 * to the summation order over K-slices.  Off by default: on B200 the separate launches (with dependent launch) are still
 * faster for decode-size matrices.  Returns how many of the recorded GEMV launches the list folded this way. */
uint32_t runit_graph_fused_launches(runit_graph_t* graph);
/* Kernel launches one replay of the list performs (after that folding). */
uint32_t runit_graph_kernel_launches(runit_graph_t* graph);

/* ── Q8_0 fused-dequant GEMV family ── */
/* dispatch.rs:1280  y_f32[m] = W_q8_0[m,k] . x_f32[k] */
int32_t runit_gemv_q8_0_f32in_f32out(runit_ctx_t*, const void* weight, const void* input, void* output, uint32_t m, uint32_t k);
/* dispatch.rs:1298  y_f32 = W.x_f32 + residual_f32 (output may alias residual) */
int32_t runit_gemv_q8_0_add_f32_f32in(runit_ctx_t*, const void* weight, const void* input, void* output, const void* residual, uint32_t m, uint32_t k);
/* dispatch.rs:1317  y_f16 = W.x_f32 */
int32_t runit_gemv_q8_0_f32in(runit_ctx_t*, const void* weight, const void* input, void* output, uint32_t m, uint32_t k);
/* dispatch.rs:1335  y_f16 = W.x_f16 */
int32_t runit_gemv_q8_0_f16(runit_ctx_t*, const void* weight, const void* input, void* output, uint32_t m, uint32_t k);
/* dispatch.rs:1353  y_f16 = W.x_f16 + residual_f16 */
int32_t runit_gemv_q8_0_add_f16(runit_ctx_t*, const void* weight, const void* input, void* output, const void* residual, uint32_t m, uint32_t k);
/* dispatch.rs:1372  y_f32 = W.x_f16 + residual_f32 */
int32_t runit_gemv_q8_0_add_f32res_f16(runit_ctx_t*, const void* weight, const void* input, void* output, const void* residual, uint32_t m, uint32_t k);
/* dispatch.rs:1083,1101 (4 rows per threadgroup) and dispatch.rs:1397,1414,1432 (256-wide):
 * launch-shape variants of the same operators; here they are the same kernel. */
int32_t runit_gemv_q8_0_f32in_f32out_mr(runit_ctx_t*, const void* weight, const void* input, void* output, uint32_t m, uint32_t k);
int32_t runit_gemv_q8_0_add_f32_f32in_mr(runit_ctx_t*, const void* weight, const void* input, void* output, const void* residual, uint32_t m, uint32_t k);
int32_t runit_gemv_q8_0_f32in_f32out_wide(runit_ctx_t*, const void* weight, const void* input, void* output, uint32_t m, uint32_t k);
int32_t runit_gemv_q8_0_add_f32_f32in_wide(runit_ctx_t*, const void* weight, const void* input, void* output, const void* residual, uint32_t m, uint32_t k);
int32_t runit_gemv_q8_0_f32in_wide(runit_ctx_t*, const void* weight, const void* input, void* output, uint32_t m, uint32_t k);
/* dispatch.rs:813  Q|K|V rows in one launch, f32 in/out */
int32_t runit_fused_qkv_q8_0_f32(runit_ctx_t*, const void* w_q, const void* w_k, const void* w_v, const void* x_vec,
                                 void* out_q, void* out_k, void* out_v, uint32_t q_dim, uint32_t kv_dim, uint32_t k);
/* dispatch.rs:842  same + f16 bias per row (the reference uploads biases as f16) */
int32_t runit_fused_qkv_bias_q8_0_f32(runit_ctx_t*, const void* w_q, const void* w_k, const void* w_v, const void* x_vec,
                                      void* out_q, void* out_k, void* out_v, const void* bias_q, const void* bias_k,
                                      const void* bias_v, uint32_t q_dim, uint32_t kv_dim, uint32_t k);
/* dispatch.rs:903  act_f32[ff] = silu(Wg.x) * (Wu.x) */
int32_t runit_fused_ffn_q8_0_f32(runit_ctx_t*, const void* w_gate, const void* w_up, const void* x_vec, void* act_out, uint32_t ff_dim, uint32_t k);

/* ── Q4_0 ── */
/* dispatch.rs:1456 */
int32_t runit_gemv_q4_0_f32in_f32out(runit_ctx_t*, const void* weight, const void* input, void* output, uint32_t m, uint32_t k);
/* dispatch.rs:1471 */
int32_t runit_gemv_q4_0_add_f32_f32in(runit_ctx_t*, const void* weight, const void* input, void* output, const void* residual, uint32_t m, uint32_t k);
/* dispatch.rs:1486  f32 in, f16 out */
int32_t runit_gemv_q4_0_f32in(runit_ctx_t*, const void* weight, const void* input, void* output, uint32_t m, uint32_t k);
/* dispatch.rs:1501  f16 in, f16 out */
int32_t runit_gemv_q4_0_f16(runit_ctx_t*, const void* weight, const void* input, void* output, uint32_t m, uint32_t k);
/* dispatch.rs:1516  f16 in, f16 out + f16 residual */
int32_t runit_gemv_q4_0_add_f16(runit_ctx_t*, const void* weight, const void* input, void* output, const void* residual, uint32_t m, uint32_t k);
/* dispatch.rs:1531 */
int32_t runit_fused_ffn_q4_0_f32(runit_ctx_t*, const void* w_gate, const void* w_up, const void* x_vec, void* act_out, uint32_t ff_dim, uint32_t k);

/* ── Q4_K ── */
/* dispatch.rs:1229 */
int32_t runit_gemv_q4k_f32in_f32out(runit_ctx_t*, const void* weight_q4k, const void* input, void* output, uint32_t m, uint32_t k);
/* dispatch.rs:1251 */
int32_t runit_gemv_q4k_add_f32_f32in(runit_ctx_t*, const void* weight_q4k, const void* input, void* output, const void* residual, uint32_t m, uint32_t k);
/* dispatch.rs:621  f16 in, f16 out */
int32_t runit_gemv_q4k_f16(runit_ctx_t*, const void* weight_q4k, const void* input, void* output, uint32_t m, uint32_t k);
/* dispatch.rs:585  f16 in, f16 out + f16 residual */
int32_t runit_gemv_q4k_add_f16(runit_ctx_t*, const void* weight_q4k, const void* input, void* output, const void* residual, uint32_t m, uint32_t k);
/* dispatch.rs:358  f16 in, f32 out + f32 residual */
int32_t runit_gemv_q4k_add_f32res_f16(runit_ctx_t*, const void* weight_q4k, const void* input, void* output, const void* residual, uint32_t m, uint32_t k);
/* dispatch.rs:756  Q4_K blocks -> f16 elements */
int32_t runit_dequant_q4k_f16(runit_ctx_t*, const void* input, void* output, uint32_t n_blocks);

/* ── Q5_0, Q5_K, Q6_K: fused-dequant GEMVs for formats the reference only expands on the CPU at load time
 *    (crates/engine/src/forward.rs:900-919 Q5_0, 920-949 Q6_K, 979-1012 Q5_K) and then multiplies as f16.  No twin in
 *    dispatch.rs; names follow the Q4_K twins.  Layouts as the reference decodes them:
 *      Q5_0: 22-byte blocks {f16 d; u8 qh[4]; u8 qs[16]}, byte j = elements j (low nibble) and j+16 (high), fifth bits in
 *            bit j of qh (little-endian u32) and bit j+16, value = d*(q-16); k a multiple of 32
 *      Q5_K: 176-byte superblocks {f16 d; f16 dmin; u8 scales[12]; u8 qh[32]; u8 qs[128]}: Q4_K plus the fifth bit of
 *            element e in bit e%8 of qh[e/8]; k a multiple of 256
 *      Q6_K: 210-byte superblocks {u8 ql[128]; u8 qh[64]; i8 scales[16]; f16 d}, value = d*scale*(q-32), scale index
 *            8*(e/128) + 2*((e%128)/32); k a multiple of 256
 *    y_f32[m] = W[m,k] . x_f32[k] (+ residual_f32; output may alias residual). ── */
int32_t runit_gemv_q5_0_f32in_f32out(runit_ctx_t*, const void* weight, const void* input, void* output, uint32_t m, uint32_t k);
int32_t runit_gemv_q5_0_add_f32_f32in(runit_ctx_t*, const void* weight, const void* input, void* output, const void* residual, uint32_t m, uint32_t k);
int32_t runit_gemv_q5k_f32in_f32out(runit_ctx_t*, const void* weight, const void* input, void* output, uint32_t m, uint32_t k);
int32_t runit_gemv_q5k_add_f32_f32in(runit_ctx_t*, const void* weight, const void* input, void* output, const void* residual, uint32_t m, uint32_t k);
int32_t runit_gemv_q6k_f32in_f32out(runit_ctx_t*, const void* weight, const void* input, void* output, uint32_t m, uint32_t k);
int32_t runit_gemv_q6k_add_f32_f32in(runit_ctx_t*, const void* weight, const void* input, void* output, const void* residual, uint32_t m, uint32_t k);

/* ── MoE glue and router ── */
/* dispatch.rs:270  y_f16[m] = W_f16[m,k] . x_f32[k]  (router logits) */
int32_t runit_gemv_f16w_f32in(runit_ctx_t*, const void* weight, const void* input, void* output, uint32_t m, uint32_t k);
/* dispatch.rs:15 / dispatch.rs:35 */
int32_t runit_silu_mul_f16(runit_ctx_t*, const void* gate, const void* up, void* out, uint32_t n);
int32_t runit_silu_mul_f32(runit_ctx_t*, const void* gate, const void* up, void* out, uint32_t n);
/* dispatch.rs:1639  acc_f16 += half(float(src_f16) * weight) */
int32_t runit_scale_accumulate_f16(runit_ctx_t*, const void* src, void* acc, float weight, uint32_t n);
/* dispatch.rs:316  acc_f32 += float(src_f16) */
int32_t runit_add_f16_into_f32(runit_ctx_t*, const void* src, void* acc, uint32_t n);

/* ── entry points with no twin in the reference ── */
/* Q|K|V in one launch for the 4-bit formats and gate/up+SiLU for Q4_K (the reference has these fusions only
 * for Q8_0 / Q4_0: dispatch.rs:813, 903, 1531). */
int32_t runit_fused_qkv_q4_0_f32(runit_ctx_t*, const void* w_q, const void* w_k, const void* w_v, const void* x_vec,
                                 void* out_q, void* out_k, void* out_v, uint32_t q_dim, uint32_t kv_dim, uint32_t k);
int32_t runit_fused_qkv_q4k_f32(runit_ctx_t*, const void* w_q, const void* w_k, const void* w_v, const void* x_vec,
                                void* out_q, void* out_k, void* out_v, uint32_t q_dim, uint32_t kv_dim, uint32_t k);
int32_t runit_fused_ffn_q4k_f32(runit_ctx_t*, const void* w_gate, const void* w_up, const void* x_vec, void* act_out,
                                uint32_t ff_dim, uint32_t k);
/* Batched fused-dequant GEMV: x [batch][k] f32, y [batch][m] f32 (+ residual [batch][m], may be
 * NULL); weights streamed once for the whole batch; batch in 1..8. */
int32_t runit_gemv_batched_f32(runit_ctx_t*, int32_t fmt, const void* weight, const void* input, void* output,
                               const void* residual, uint32_t m, uint32_t k, uint32_t batch);
/* The same for up to three matrices that share the input (q | k | v, gate | up): one launch, the activations are
 * prepared once; outputs[i] f32 [batch][rows[i]].  (Host pointer tables of n_mats device pointers.) */
int32_t runit_gemv_batched_multi_f32(runit_ctx_t*, int32_t fmt, uint32_t n_mats, const void* const* weights, const void* input,
                                     void* const* outputs, const uint32_t* rows, uint32_t k, uint32_t batch);
/* RMSNorm fused into the GEMV that consumes it: x is the un-normalised f32 vector [k], gamma f32 [k]; the matrices multiply
 * x * rsqrt(mean(x^2) + eps) * gamma (the reference runs rms_norm_f32_f32_f32g, forward.rs:1528-1569 / dispatch.rs:177, then the
 * GEMV, as two encoders).  Every CTA computes the scale itself, so the scale agrees with the stand-alone operator to
 * rounding, not to the bit.  fmt: RUNIT_FMT_Q8_0 / Q4_0 / Q4K.  residual f32 [m], may be NULL. */
int32_t runit_rms_norm_gemv_f32(runit_ctx_t*, int32_t fmt, const void* weight, const void* x, const void* gamma, float eps,
                                void* output, const void* residual, uint32_t m, uint32_t k);
int32_t runit_rms_norm_fused_qkv_f32(runit_ctx_t*, int32_t fmt, const void* w_q, const void* w_k, const void* w_v, const void* x,
                                     const void* gamma, float eps, void* out_q, void* out_k, void* out_v, uint32_t q_dim,
                                     uint32_t kv_dim, uint32_t k);
/* Greedy lm_head: the GEMV of runit_rms_norm_gemv_f32 (gamma may be NULL: then x is used as it is) whose epilogue also
 * finds the index of the largest logit, lowest index among equal values (argmax after lm_head, forward.rs:1967-1973):
 * logits f32 [m] and result int32 [1] come out of one launch.  Needs 16-byte aligned weight rows and m <= 2,097,152. */
int32_t runit_gemv_argmax_f32(runit_ctx_t*, int32_t fmt, const void* weight, const void* x, const void* gamma, float eps,
                              void* logits, void* result, uint32_t m, uint32_t k);
/* Row-sharded greedy lm_head: rank `rank` multiplies its rows_total / world rows (logits_local f32, this rank's slice) and
 * stores its (largest logit, global row index) pair, 8 bytes, into slot `rank` of every rank's pair table pairs_all[p]
 * (uint2 [world], peer-mapped memory, plain stores).  After runit_peer_barrier, runit_argmax_pairs over the own table gives
 * the same token on every rank: an 8-byte all-gather instead of the logits. */
int32_t runit_gemv_argmax_allgather(runit_ctx_t*, int32_t fmt, const void* w_local, const void* x, void* logits_local,
                                    void* const* pairs_all, uint32_t world, uint32_t rank, uint32_t rows_total, uint32_t k);
int32_t runit_argmax_pairs(runit_ctx_t*, const void* pairs, uint32_t n, void* result);
/* runit_peer_barrier followed by runit_argmax_pairs over this rank's own table (uint2 [world]) in one launch */
int32_t runit_peer_barrier_argmax(runit_ctx_t*, void* const* signal_pads, uint32_t world, uint32_t rank, uint32_t epoch,
                                  const void* pairs, void* result);
/* Fused Q|K|V with an f32 bias (the benchmark configuration states an f32 bias); bias may be NULL. */
int32_t runit_fused_qkv_f32bias_q8_0_f32(runit_ctx_t*, const void* w_q, const void* w_k, const void* w_v, const void* x_vec,
                                         void* out_q, void* out_k, void* out_v, const void* bias_q, const void* bias_k,
                                         const void* bias_v, uint32_t q_dim, uint32_t kv_dim, uint32_t k);
/* ── row-sharded GEMV with the all-gather fused into the epilogue (no twin: the reference is single-device,
 *    crates/engine/src/server/mod.rs:20-30).  Rank `rank` of `world` (<= 8) owns rows [rank*n, (rank+1)*n), n =
 *    rows_total/world, of the weight matrix (w_local: those n rows).  y_all: HOST array of `world` DEVICE pointers, entry p
 *    = rank p's full-length f32 output vector as mapped into this process (peer memory for p != rank, e.g. from CUDA
 *    virtual-memory or IPC mappings / torch symmetric memory).  Every result is stored into all of them by plain peer
 *    stores.  The vectors are complete on every rank once all ranks have passed runit_peer_barrier.
 *    Reuse: passing the barrier of call n means every rank has ANNOUNCED epoch n, not that it has finished reading
 *    the result of call n.  A rank that runs ahead would overwrite a vector a slower rank still reads, so alternate
 *    between two sets of output vectors from call to call (call n+2 can only start after barrier n+1, which each rank
 *    announces in stream order after its own reads of result n), or put a second barrier after the consumer. ── */
int32_t runit_gemv_allgather_f32(runit_ctx_t*, int32_t fmt, const void* w_local, const void* x, void* const* y_all,
                                 uint32_t world, uint32_t rank, uint32_t rows_total, uint32_t k);
/* ── expert-parallel MoE block for prefill-sized batches (no twin: the reference is single-device) ──
 * Tokens are data-parallel (the same T on every rank), experts are split over the ranks (E / world each; placement 0:
 * expert e on rank e / (E/world), 1: on rank e % world); token rows are stored into the owners' receive buffers and the
 * expert outputs back into the senders' return buffers with plain peer stores, two bounded barriers per call, no host
 * read and no collective library on the data path.  The result equals runit_moe_layer_q4k_bf16 on one GPU bit for bit.
 * Peer-mapped buffers, one per rank, given as pointer tables of `world` entries (this rank's own included):
 *   recv_rows   bf16  [world * T * k][h]     recv_meta  int32 [world * T * k][2]     recv_counts  int32 [world]
 *   return_rows f32   [T * k][h]             signal_pads uint32 [>= world], zeroed before the first call
 * epoch counts the calls on these buffers from 1 (it uses barrier epochs 2*epoch-1 and 2*epoch).  scratch: local memory,
 * runit_moe_ep_prefill_scratch_bytes, 1024-byte aligned.  x / residual / out: f32 [T][h]; idx_out / w_out may be NULL. */
size_t  runit_moe_ep_prefill_scratch_bytes(uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k, uint32_t world);
int32_t runit_moe_layer_q4k_bf16_ep(runit_ctx_t*, const void* router_w, const void* gate_local, const void* up_local,
                                    const void* down_local, const void* x, const void* residual, void* out, void* idx_out, void* w_out,
                                    void* scratch, size_t scratch_bytes, void* const* recv_rows_all, void* const* recv_meta_all,
                                    void* const* recv_counts_all, void* const* return_rows_all, void* const* signal_pads, uint32_t T,
                                    uint32_t h, uint32_t ff, uint32_t E, uint32_t k, int32_t renorm, uint32_t world, uint32_t rank,
                                    uint32_t epoch, int32_t placement);
/* One-kernel barrier over peer memory.  signal_pads: HOST array of `world` DEVICE pointers, entry p = rank p's pad of at
 * least `world` uint32 words (zero before the first use), as mapped into this process.  Announces `epoch` (> 0,
 * strictly increasing from call to call) to every rank and waits until every rank has announced it; a rank that does
 * not show up within about half a second makes the next runit_flush return RUNIT_ERR_TIMEOUT (the context stays
 * usable). */
int32_t runit_peer_barrier(runit_ctx_t*, void* const* signal_pads, uint32_t world, uint32_t rank, uint32_t epoch);

/* ── MoE block (no twin as one function; replaces the sequence crates/engine/src/forward.rs:1644-1679
 *    and the CPU routing forward.rs:2420-2448, without the per-layer host synchronisation) ── */
/* logits_f32[T][E] = router_f32[E][h] . x_f32[T][h] */
int32_t runit_moe_router_f32(runit_ctx_t*, const void* router_w, const void* x, void* logits, uint32_t E, uint32_t h, uint32_t T);
/* softmax over all E experts, top-k by probability (descending; ties: lowest index), weights optionally
 * renormalised to sum 1.  logits: [T][E] f32, or f16 when logits_f16 != 0 (the reference's router dtype);
 * out_idx: int32 [T][k]; out_w: f32 [T][k].  E <= 256, k <= 32. */
int32_t runit_moe_route_topk(runit_ctx_t*, const void* logits, int32_t logits_f16, uint32_t E, uint32_t k, int32_t renorm,
                             uint32_t T, void* out_idx, void* out_w);
/* Scratch bytes runit_moe_layer_q4k needs for these shapes. */
size_t runit_moe_scratch_bytes(uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k);
/* One MoE block over T tokens, all on the device:
 *   out[t] = (residual ? residual[t] : 0) + sum_i w_i * Wdown[e_i] . (silu(Wgate[e_i].x[t]) * (Wup[e_i].x[t]))
 * router_w: f32 [E][h]; gate, up: Q4_K [E][ff][h]; down: Q4_K [E][h][ff] (experts stacked contiguously, as
 * the reference slices merged expert tensors, forward.rs:1339-1408); x, residual, out: f32 [T][h] (out may
 * alias residual); idx_out (int32 [T][k]) and w_out (f32 [T][k]) may be NULL; scratch: caller-owned device
 * memory of at least runit_moe_scratch_bytes(), 256-byte aligned.  h, ff multiples of 256. */
int32_t runit_moe_layer_q4k(runit_ctx_t*, const void* router_w, const void* gate, const void* up, const void* down,
                            const void* x, const void* residual, void* out, void* idx_out, void* w_out, void* scratch,
                            size_t scratch_bytes, uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k, int32_t renorm);

/* The expert part alone, for expert-parallel execution: slot s holds one token row x_slots[s] (f32 [h]) routed to
 * local expert slot_expert[s] (int32; a negative id marks an unused slot: nothing is computed or written for it);
 * y_slots[s] = Wdown[e] . (silu(Wgate[e].x) * (Wup[e].x)).  gate/up: Q4_K [n_experts][ff][h]; down: Q4_K
 * [n_experts][h][ff]; act_scratch: f32 [n_slots][ff], caller-owned. */
int32_t runit_moe_experts_q4k(runit_ctx_t*, const void* gate, const void* up, const void* down, const void* x_slots,
                              const void* slot_expert, void* y_slots, void* act_scratch, uint32_t n_slots, uint32_t h,
                              uint32_t ff, uint32_t n_experts);

/* Expert-parallel form of runit_moe_layer_q4k for decode sizes, tokens replicated on every rank (no counterpart in
 * the reference, which runs on one device).  Rank r holds the replicated router and the experts
 * [r * E/world, (r+1) * E/world) (gate_local, up_local: Q4_K [E/world][ff][h]; down_local: Q4_K [E/world][h][ff]).  Every
 * rank routes all T tokens itself, computes only the (token, expert) slots it owns, and stores its weighted partial sum
 * into slot r of the partial buffer of EVERY rank with plain peer stores (the combine exchange fused into the kernel: no
 * collective library call, no TMA, no multicast); after the one-kernel barrier each rank adds the `world` partial sums in
 * rank order plus the residual, so all ranks end with identical bits in `out`.
 * partial_all: HOST array of `world` DEVICE pointers, entry p = rank p's partial buffer, f32 [2][world][T][h], as mapped
 * into this process (the two halves alternate by epoch parity, so a fast rank's next call never overwrites what a slow
 * rank is still adding); signal_pads / epoch: as for runit_peer_barrier (a missing rank makes the next runit_flush return
 * RUNIT_ERR_TIMEOUT).  scratch: runit_moe_scratch_bytes(T, h, ff, E, k). */
int32_t runit_moe_layer_q4k_ep(runit_ctx_t*, const void* router_w, const void* gate_local, const void* up_local,
                               const void* down_local, const void* x, const void* residual, void* out, void* idx_out, void* w_out,
                               void* scratch, size_t scratch_bytes, void* const* partial_all, void* const* signal_pads,
                               uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k, int32_t renorm, uint32_t world,
                               uint32_t rank, uint32_t epoch);

/* No counterpart in the reference.  The same MoE block as runit_moe_layer_q4k for callers that cannot hand
 * over scratch memory: a host engine that gives every free byte of device memory to its own weight and
 * KV-cache pools at start-up, or a serving loop that must not call cudaMalloc because that call stalls the
 * whole device.  This entry point allocates nothing (no cudaMalloc/cudaFree, no allocating library call);
 * its intermediates live in a fixed 4 MiB region (runit_moe_static_scratch_capacity()) built into the
 * library image, which every GPU that loads the library holds until the process exits.
 *   - Shapes whose intermediates do not fit (runit_moe_scratch_bytes(T,h,ff,E,k) > capacity; e.g. OLMoE
 *     shapes beyond 32 tokens) are rejected with RUNIT_ERR_BUFFER_SIZE and nothing is launched.
 *   - The first call on a device looks up the region's device address (once per device, with that device
 *     made current for the lookup) and keeps it for the life of the process; make that first call before any
 *     stream capture is started.  The kept address does not survive cudaDeviceReset: a process that resets a
 *     device must not use this entry point on it afterwards.
 *   - All calls share the one region and it keeps the previous call's contents; every part the block reads
 *     is rewritten first, so nothing needs clearing, but two calls that overlap on the GPU (different
 *     streams or contexts of one process on the same device) race on it: keep them ordered. */
size_t  runit_moe_static_scratch_capacity(void);
int32_t runit_moe_layer_q4k_static(runit_ctx_t*, const void* router_w, const void* gate, const void* up, const void* down,
                                   const void* x, const void* residual, void* out, void* idx_out, void* w_out,
                                   uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k, int32_t renorm);

/* ── batched (prefill-sized) MoE block on the tensor cores.  No twin: the reference's prefill runs the decode
 *    block once per token (crates/engine/src/prefill.rs:156-215).  Same block as runit_moe_layer_q4k with bf16
 *    operands: slots are sorted by expert on the device, every Q4_K weight d*sc*q - dmin*m
 *    (crates/engine/src/forward.rs:1026-1057) is rounded to bf16 in shared-memory tiles, activations are rounded to
 *    bf16, products accumulate in f32 (tcgen05.mma, accumulators in tensor memory):
 *      act[s] = bf16(silu(Wg[e].bf16(x[t])) * (Wu[e].bf16(x[t]))), y[s] = Wd[e].act[s],
 *      out[t] = (residual ? residual[t] : 0) + sum_i w_i * y[s_i]        (routing order)
 *    Shapes: h, ff multiples of 256; E <= 256; k <= min(E, 32).  scratch: caller-owned, 1024-byte aligned,
 *    at least runit_moe_grouped_scratch_bytes(); tensors 16-byte aligned; out may alias residual. ── */
size_t  runit_moe_grouped_scratch_bytes(uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k);
/* router (f32 [E][h]) -> softmax/top-k -> experts; idx_out (int32 [T][k]) and w_out (f32 [T][k]) may be NULL. */
int32_t runit_moe_layer_q4k_bf16(runit_ctx_t*, const void* router_w, const void* gate, const void* up, const void* down,
                                 const void* x, const void* residual, void* out, void* idx_out, void* w_out, void* scratch,
                                 size_t scratch_bytes, uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k, int32_t renorm);
/* The expert part for given routing: idx int32 [T][k] (ids outside [0, E) are skipped), w f32 [T][k]. */
int32_t runit_moe_experts_grouped_q4k_bf16(runit_ctx_t*, const void* gate, const void* up, const void* down, const void* x,
                                           const void* idx, const void* w, const void* residual, void* out, void* scratch,
                                           size_t scratch_bytes, uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k);

/* ── decode-step operators besides the GEMVs ── */
/* dispatch.rs:152  y = x * rsqrt(mean(x^2)+eps) * gamma_f16, num_rows rows of `hidden` (x may equal y) */
int32_t runit_rms_norm_f32_f32(runit_ctx_t*, const void* x, void* y, const void* gamma, float eps, uint32_t hidden, uint32_t num_rows);
/* dispatch.rs:177  same with f32 gamma */
int32_t runit_rms_norm_f32_f32_f32g(runit_ctx_t*, const void* x, void* y, const void* gamma, float eps, uint32_t hidden, uint32_t num_rows);
/* dispatch.rs:945  rotary embedding of Q [q_heads][hd] and K [kv_heads][hd] in place, pairs (d, d+hd/2) */
int32_t runit_fused_rope_qk_f32(runit_ctx_t*, void* q, void* k, uint32_t head_dim, uint32_t q_heads, uint32_t kv_heads, uint32_t pos, float theta);
/* dispatch.rs:1159 / 1183  scatter [kv_heads][hd] into the cache [kv_heads][max_seq][hd] at pos */
int32_t runit_kv_copy_to_cache_f16(runit_ctx_t*, const void* src, void* dst, uint32_t pos, uint32_t max_seq, uint32_t head_dim, uint32_t num_kv_heads);
int32_t runit_kv_copy_to_cache_f32(runit_ctx_t*, const void* src, void* dst, uint32_t pos, uint32_t max_seq, uint32_t head_dim, uint32_t num_kv_heads);
/* no twin: f32 source rounded into an f16 cache */
int32_t runit_kv_copy_to_cache_f32_f16(runit_ctx_t*, const void* src, void* dst, uint32_t pos, uint32_t max_seq, uint32_t head_dim, uint32_t num_kv_heads);
/* dispatch.rs:1575 (f32) / dispatch.rs:697 (f16)  q_len = 1 attention over kv_len cached positions,
 * scale 1/sqrt(head_dim), GQA kv_head = q_head / (heads/kv_heads); head_dim in {32,64,96,128} */
int32_t runit_decode_attention_f32(runit_ctx_t*, const void* q, const void* k, const void* v, void* out, uint32_t batch, uint32_t kv_len,
                                   uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_dim, uint32_t kv_head_stride);
int32_t runit_decode_attention_f16(runit_ctx_t*, const void* q, const void* k, const void* v, void* out, uint32_t batch, uint32_t kv_len,
                                   uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_dim, uint32_t kv_head_stride);
/* no twin: f32 query and output over an f16 cache */
int32_t runit_decode_attention_f32q_f16kv(runit_ctx_t*, const void* q, const void* k, const void* v, void* out, uint32_t batch, uint32_t kv_len,
                                          uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_dim, uint32_t kv_head_stride);
/* dispatch.rs:1615  index of the maximum of n f16 values -> result[0] (int32); ties: lowest index */
int32_t runit_argmax_f16(runit_ctx_t*, const void* input, void* result, uint32_t n);
/* no twin: f32 input (sampler.rs:111-116 on the device) */
int32_t runit_argmax_f32(runit_ctx_t*, const void* input, void* result, uint32_t n);

/* ── token sampling on the device: the reference's host sampler (crates/engine/src/sampler.rs:61-111) as one launch ──
 * Steps, in the reference's order: end-of-sequence ids suppressed while the context is shorter than min_tokens;
 * repetition penalty once per occurrence of a token in the context; temperature 0 -> argmax (last index among equal
 * maxima, as Iterator::max_by); else scores / temperature, softmax, top-k (the first k entries in index order with
 * p >= the k-th largest), top-p (descending order until the running sum has reached p), and the draw r = rng * total over
 * the survivors in index order.  The generator is the reference's xorshift64 (sampler.rs:12-27); its state lives in
 * device memory and advances by one draw.  top_k in 0..1024 (0 = off); with top-k off and top_p < 1 the nucleus must lie
 * within the 1024 most probable tokens (else status: RUNIT_ERR_UNSUPPORTED at the next flush, most probable token returned). */
typedef struct {
    float   temperature;          /* 0 = greedy */
    int32_t top_k;                /* 0 = off */
    float   top_p;                /* >= 1 = off */
    float   repetition_penalty;   /* 1 = off */
    int32_t min_tokens;
} runit_sampler_cfg;
/* logits f32 [n]; scores_scratch f32 [n] (holds the final distribution afterwards, unless greedy); context int32 tokens,
 * the range [ctx_begin, ctx_end) of it is the context, or, when ctx_range is not NULL, the two device words it points to
 * give that range; eos_ids int32 [n_eos]; rng_state uint64 [1]; result int32 [1].  All pointers are device pointers. */
int32_t runit_sample_f32(runit_ctx_t*, const void* logits, void* scores_scratch, uint32_t n, const runit_sampler_cfg* cfg,
                         const void* context, const void* ctx_range, uint32_t ctx_begin, uint32_t ctx_end, const void* eos_ids,
                         uint32_t n_eos, void* rng_state, void* result);
/* SimpleRng::new (sampler.rs:15-17): the state to store in rng_state for a seed */
uint64_t runit_sampler_seed_state(uint64_t seed);

/* ── greedy decoder for an OLMoE-shaped model with Q4_K matrices: the role of Executor::forward_greedy,
 *    crates/engine/src/forward.rs:1795-1975, with token id, position and arg-max kept on the device ── */
typedef struct {
    int32_t n_layers, hidden, n_heads, n_kv_heads, head_dim, vocab;
    int32_t n_experts, top_k, ff, max_seq, renorm;
    float   eps, theta;
} runit_model_cfg;
typedef struct {          /* device pointers; the model keeps them, the caller keeps the memory alive */
    const void* tok_emb;   /* f32 [vocab][hidden] */
    const void* attn_norm; /* f32 [L][hidden] */
    const void* ffn_norm;  /* f32 [L][hidden] */
    const void* out_norm;  /* f32 [hidden] */
    const void* wq;        /* Q4_K [L][n_heads*head_dim][hidden] */
    const void* wk;        /* Q4_K [L][n_kv_heads*head_dim][hidden] */
    const void* wv;        /* Q4_K [L][n_kv_heads*head_dim][hidden] */
    const void* wo;        /* Q4_K [L][hidden][n_heads*head_dim] */
    const void* router;    /* f32 [L][E][hidden] */
    const void* gate;      /* Q4_K [L][E][ff][hidden] */
    const void* up;        /* Q4_K [L][E][ff][hidden] */
    const void* down;      /* Q4_K [L][E][hidden][ff] */
    const void* lm_head;   /* Q4_K [vocab][hidden] */
} runit_model_weights;
typedef struct runit_model runit_model_t;
/* Allocates the f16 KV cache and all scratch, runs one warm-up step and records the per-token command lists. */
int32_t runit_model_create(runit_ctx_t* ctx, const runit_model_cfg* cfg, const runit_model_weights* weights, runit_model_t** out);
/* The same decoder with the experts split over `world` ranks (one process and context per GPU): weights->gate / up / down
 * hold this rank's experts [rank * E/world, (rank+1) * E/world) only ([L][E/world][...]), everything else is replicated and
 * every rank decodes the same token stream (runit_moe_layer_q4k_ep per layer, barrier epochs kept on the device so the
 * recorded command list can be replayed).  partial_all / signal_pads: as for runit_moe_layer_q4k_ep with T = 1.  All ranks
 * must call this (and every generate call) together: the warm-up step already runs the barriers. */
int32_t runit_model_create_ep(runit_ctx_t* ctx, const runit_model_cfg* cfg, const runit_model_weights* weights, uint32_t world,
                              uint32_t rank, void* const* partial_all, void* const* signal_pads, runit_model_t** out);
int32_t runit_model_destroy(runit_model_t* model);
int32_t runit_model_reset(runit_model_t* model, int32_t token, int32_t pos);
/* forward.rs:1795  one token at position pos -> arg-max next token (synchronous, like the reference) */
int32_t runit_model_forward_greedy(runit_model_t* model, int32_t token_id, int32_t pos, int32_t* next_token);
/* prompt (forced tokens) + n_gen greedy steps without host round trips; out_tokens: n_prompt+n_gen int32 on the host */
int32_t runit_model_generate_greedy(runit_model_t* model, const int32_t* prompt, uint32_t n_prompt, uint32_t n_gen,
                                    int32_t start_pos, int32_t skip_prompt_logits, int32_t* out_tokens);
/* The same loop with the sampler in place of the argmax (generate.rs:299, 346: the context of a draw is what has been
 * generated so far, empty for the first one).  eos_ids: host array, at most 16.  The command list of the sampled step is
 * recorded on first use and again whenever cfg changes. */
int32_t runit_model_generate_sampled(runit_model_t* model, const int32_t* prompt, uint32_t n_prompt, uint32_t n_gen,
                                     int32_t start_pos, const runit_sampler_cfg* cfg, uint64_t seed, const int32_t* eos_ids,
                                     uint32_t n_eos, int32_t* out_tokens);
/* Executor::prefill (crates/engine/src/prefill.rs:29-255): the whole prompt in one batched pass from an empty cache
 * (tensor-core GEMMs with bf16 operands over the Q4_K matrices, causal attention over the f16 cache, the batched MoE
 * block).  Afterwards the cache holds positions 0 .. n-1, *next_token is the argmax of the last position's logits, and
 * runit_model_generate_greedy(&next, 1, n_gen, n, ...) continues.  head_dim 64 or 128; tokens: host array. */
int32_t runit_model_prefill(runit_model_t* model, const int32_t* tokens, uint32_t n, int32_t* next_token);
/* The causal attention kernel of the prefill by itself: q f32 [T][heads*head_dim] (already rotated), caches f16
 * [kv_heads][max_seq][head_dim] holding positions 0 .. start_pos+T-1, out bf16 [T][heads*head_dim]; query t sees keys
 * 0 .. start_pos+t (attention.metal:36-158). */
int32_t runit_prefill_attention_f16kv(runit_ctx_t*, const void* q, const void* kcache, const void* vcache, void* out_bf16, uint32_t T,
                                      uint32_t heads, uint32_t kv_heads, uint32_t head_dim, uint32_t max_seq, uint32_t start_pos);
/* Dense feed-forward block of a prefill pass (prefill.rs:217-227: gemm_f16 gate, gemm_f16 up, silu_mul_f16, gemm_f16 down,
 * add_f16) on the tensor cores with bf16 operands: out[t] = residual[t] + Wd . bf16(silu(Wg . xb[t]) * (Wu . xb[t])), where
 * xb = bf16(x) or, when gamma is not NULL, bf16(RMSNorm(x) * gamma) (the rms_norm_f16 of prefill.rs:150-151).  x / residual /
 * out f32 [T][h] (residual may be NULL or equal to out); Q4_K matrices; scratch 1024-byte aligned. */
size_t  runit_ffn_q4k_bf16_scratch_bytes(uint32_t T, uint32_t h, uint32_t ff);
int32_t runit_ffn_q4k_bf16(runit_ctx_t*, const void* w_gate, const void* w_up, const void* w_down, const void* x, const void* gamma,
                           float eps, const void* residual, void* out, void* scratch, size_t scratch_bytes, uint32_t T, uint32_t h,
                           uint32_t ff);
void*   runit_model_logits(runit_model_t* model);           /* device pointer, f32 [vocab], of the last step */
uint64_t runit_model_launches_per_token(runit_model_t* model);

/* Synthetic weights written on the device (benchmark / test data, distributions of the
 * benchmark configurations): n_blocks blocks of the format from a counter-based generator. */
int32_t runit_fill_weights(runit_ctx_t*, int32_t fmt, void* dst, uint64_t n_blocks, uint64_t seed, float sigma);
/* Q4_K blocks whose weights have zero mean: dmin = f16(7.5 d) and min index = scale index in every sub-block, so that
 * d*sc*q - dmin*m = d*sc*(q - 7.5).  With the benchmark's distributions every weight has a positive mean and a
 * random-init decoder repeats one token; the parity tests of the full decoder use this variant so that the greedy
 * token stream depends on its input. */
int32_t runit_fill_weights_q4k_zero_mean(runit_ctx_t*, void* dst, uint64_t n_blocks, uint64_t seed, float sigma);
/* N(0, sigma) f32 values from the same generator. */
int32_t runit_fill_normal_f32(runit_ctx_t*, void* dst, uint64_t n, uint64_t seed, float sigma);

#ifdef __cplusplus
}
#endif
#endif
