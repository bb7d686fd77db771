/*
 * runit_oracle.h — CPU oracle for the quantized decode path (TEST INFRASTRUCTURE ONLY).
 *
 * A plain-C restatement of the arithmetic of RunIT's fused-dequant GEMV family and
 * MoE block.  It exists to check the CUDA library and to be timed as the CPU baseline.
 * It is never linked into, imported by or called from the product library: only the
 * test-suite, the smoke check and the benchmark's cpu_baseline/reference legs use it.
 *
 * PARITY UNPINNED for the quantized operators: the reference project holds no golden
 * vector, known-answer test or fixture for any Q8_0/Q4_0/Q4_K GEMV, the fused QKV/FFN
 * kernels, scale_accumulate, top-k routing or the MoE block, and its own
 * implementation (Rust + Apple Metal) can be neither compiled nor run outside macOS.
 * What the reference does pin is used: the f16-weight GEMV known answers of
 * crates/engine/src/bin/test_gemv.rs:10-136 (router GEMV), the all-zero Q4_K blocks of
 * crates/engine/tests/qwen2_load_test.rs:104-118, and single-block cases derived by
 * hand from the block layouts documented in the shaders.
 *
 * Every function cites the reference file:line (paths relative to the reference
 * project root) whose arithmetic it follows.
 */
#ifndef RUNIT_ORACLE_H
#define RUNIT_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Weight formats (block sizes: crates/kernels/src/dispatch.rs:735-747). */
enum { RO_Q8_0 = 0, RO_Q4_0 = 1, RO_Q4K = 2, RO_Q5_0 = 3, RO_Q5K = 4, RO_Q6K = 5 };

/* Accumulation tiers.
 *   SHADER : per-lane block partition and f32 accumulation order of the Metal kernels,
 *            lanes summed 0..31 (the hardware simd_sum order is unspecified).
 *   DEQUANT: dequantise the row with the engine's CPU formulas, then a sequential f32
 *            dot product (cpu_gemv, crates/kernels/src/dispatch.rs:1705-1709).
 *   F64    : same dequantised values, f64 accumulation ("truth" for tolerances). */
enum { RO_TIER_SHADER = 0, RO_TIER_DEQUANT = 1, RO_TIER_F64 = 2 };

/* MoE numeric modes.
 *   F32    : f32 router, f32 intermediates, f32 combine (the graded mode).
 *   REF_F16: rounding points of the reference engine (f16 router logits, f16 gate/up/
 *            act/down, f16 accumulator; crates/engine/src/forward.rs:1644-1679). */
enum { RO_MOE_F32 = 0, RO_MOE_REF_F16 = 1 };

int      ro_num_threads(void);
void     ro_set_num_threads(int n);

uint16_t ro_f32_to_f16(float f);
float    ro_f16_to_f32(uint16_t h);
void     ro_f32_to_f16_array(const float* in, uint16_t* out, size_t n);
void     ro_f16_to_f32_array(const uint16_t* in, float* out, size_t n);

size_t   ro_block_elems(int fmt);
size_t   ro_block_bytes(int fmt);
size_t   ro_row_bytes(int fmt, int k);

void     ro_q4k_get_scale_min(int j, const uint8_t* scales, uint8_t* sc, uint8_t* m);
void     ro_dequant_row(int fmt, const uint8_t* row, int k, float* out);
void     ro_dequant_q4k_f16(const uint8_t* in, uint16_t* out, size_t n_blocks);

/* y[b][r] = dequant(W)[r][:] . x[b][:]   W: m rows of ro_row_bytes(fmt,k); x: [batch][k] f32;
 * y: [batch][m] f32; y64 (optional, may be NULL): [batch][m] f64 accumulators (tier F64). */
int      ro_gemv(int fmt, int tier, const uint8_t* w, const float* x, float* y, double* y64,
                 int m, int k, int batch);

/* Router GEMV with f16 weights: crates/kernels/shaders/gemv.metal:82-106 (f32 result;
 * the caller rounds to f16 where the reference does). */
void     ro_gemv_f16w_f32in(const uint16_t* w, const float* x, float* y, int m, int k);
void     ro_gemv_f32w(const float* w, const float* x, float* y, int m, int k);

float    ro_silu(float v);
void     ro_silu_mul_f32(const float* gate, const float* up, float* out, size_t n);
void     ro_silu_mul_f16(const uint16_t* gate, const uint16_t* up, uint16_t* out, size_t n);
void     ro_scale_accumulate_f16(const uint16_t* src, uint16_t* acc, float weight, size_t n);
void     ro_add_f16_into_f32(const uint16_t* src, float* acc, size_t n);

/* softmax over all experts, then top-k by probability (descending; ties: lowest index
 * first), optional renormalisation: crates/engine/src/forward.rs:2420-2448. */
int      ro_topk_softmax(const float* logits, int n_experts, int top_k, int renorm,
                         int32_t* idx, float* weights, float* probs_out /* nullable [E] */);

/* One MoE block over T tokens.  router: f32 [E][h]; gate/up: Q4_K [E][ff][h]; down: Q4_K
 * [E][h][ff]; x: [T][h]; out: [T][h] = (residual ? residual : 0) + sum_i w_i * expert_i(x).
 * idx_out/w_out (nullable): [T][top_k]. */
float    ro_bf16_round(float f);
int      ro_moe_grouped_q4k_bf16(const float* router, int renorm, const uint8_t* gate, const uint8_t* up,
                                 const uint8_t* down, const float* x, const float* residual, float* out,
                                 int32_t* idx_io, float* w_io, int T, int h, int ff, int E, int top_k);
int      ro_moe_layer_q4k(int mode, int renorm, const float* router,
                          const uint8_t* gate, const uint8_t* up, const uint8_t* down,
                          const float* x, const float* residual, float* out,
                          int32_t* idx_out, float* w_out,
                          int T, int h, int ff, int E, int top_k);

void     ro_rms_norm_f32(const float* x, const float* gamma, float* y, float eps, int hidden,
                         int rows);
void     ro_rope_qk_f32(float* q, float* k, int head_dim, int q_heads, int kv_heads, int pos,
                        float theta);
void     ro_kv_copy_to_cache_f16(const float* src, uint16_t* dst, int pos, int max_seq,
                                 int head_dim, int kv_heads);
void     ro_decode_attention_f32q_f16kv(const float* q, const uint16_t* kc, const uint16_t* vc,
                                        float* out, int kv_len, int heads, int kv_heads,
                                        int head_dim, int kv_head_stride);
int32_t  ro_argmax_f32(const float* v, size_t n);

/* Host sampler of the reference, crates/engine/src/sampler.rs:12-168, restated line for line (sequential sums, the
 * reference's order of operations).  probs_out (may be NULL): the vector the draw was made from (n floats; for the
 * greedy path the penalised scores).  rng_state: xorshift64 state, advanced by one draw when a draw is made. */
typedef struct {
    float   temperature;
    int32_t top_k;
    float   top_p;
    float   repetition_penalty;
    int32_t min_tokens;
} ro_sampler_cfg;
uint64_t ro_sampler_seed_state(uint64_t seed);                      /* sampler.rs:15-17 */
float    ro_sampler_next_f32(uint64_t* state);                      /* sampler.rs:18-27 */
int32_t  ro_sampler_argmax_last(const float* v, size_t n);          /* sampler.rs:114-119: Iterator::max_by keeps the LAST maximum */
int32_t  ro_sample(const float* logits, size_t n, const ro_sampler_cfg* cfg, const int32_t* context, size_t n_context,
                   const int32_t* eos_ids, size_t n_eos, uint64_t* rng_state, float* probs_out);

/* Full OLMoE-shaped decoder with Q4_K matrices (op order of Executor::forward_greedy,
 * crates/engine/src/forward.rs:1795-1975). */
typedef struct {
    int32_t n_layers, hidden, n_heads, n_kv_heads, head_dim, vocab;
    int32_t n_experts, top_k, ff, max_seq, renorm;
    float   eps, theta;
} ro_model_cfg;

typedef struct {
    const float*   tok_emb;     /* [vocab][hidden] f32 */
    const float*   attn_norm;   /* [L][hidden] */
    const float*   ffn_norm;    /* [L][hidden] */
    const float*   out_norm;    /* [hidden] */
    const uint8_t* wq;          /* [L] Q4_K [q_dim][hidden] */
    const uint8_t* wk;          /* [L] Q4_K [kv_dim][hidden] */
    const uint8_t* wv;          /* [L] Q4_K [kv_dim][hidden] */
    const uint8_t* wo;          /* [L] Q4_K [hidden][q_dim] */
    const float*   router;      /* [L][E][hidden] f32 */
    const uint8_t* gate;        /* [L][E] Q4_K [ff][hidden] */
    const uint8_t* up;          /* [L][E] Q4_K [ff][hidden] */
    const uint8_t* down;        /* [L][E] Q4_K [hidden][ff] */
    const uint8_t* lm_head;     /* Q4_K [vocab][hidden] */
} ro_model_weights;

/* One greedy step: token at position pos -> next token.  kc/vc: [L][kv_heads][max_seq][head_dim]
 * f16.  logits_out (nullable): [vocab]. */
int32_t  ro_decode_step(const ro_model_cfg* cfg, const ro_model_weights* w, uint16_t* kc,
                        uint16_t* vc, int32_t token, int32_t pos, float* logits_out);

/* Comparator: semantics of validate_layer_output / diff_stats
 * (crates/reference/src/lib.rs:28-96) plus a relative metric
 * |a-b| <= rel_tol * max(|ref|, rms(ref)).  Returns the number of mismatches. */
typedef struct {
    double max_abs, mean_abs, rms, ref_rms, max_rel;
    int64_t n, n_mismatch_abs, n_mismatch_rel;
} ro_diff_stats;
int64_t  ro_compare(const float* ref, const float* got, size_t n, float abs_tol, float rel_tol,
                    ro_diff_stats* st);

#ifdef __cplusplus
}
#endif
#endif
