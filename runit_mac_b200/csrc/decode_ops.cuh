// Launchers of the decode-step operators, shared by the C-ABI twins and the decoder (decode_model.cu).
// pos_ptr != nullptr: the position (and kv_len = pos + 1) is read from that device word at run time.
#pragma once

#include "runit_internal.h"

namespace runit {

int32_t launch_rms_norm(runit_ctx* ctx, const float* x, float* y, const void* gamma, bool gamma_f16, float eps,
                        uint32_t hidden, uint32_t rows);
int32_t launch_rope(runit_ctx* ctx, float* q, float* k, uint32_t hd, uint32_t qh, uint32_t kvh, uint32_t pos,
                    const int32_t* pos_ptr, float theta);
// rotary embedding of q and k, then k and v of this position into the f16 caches, in one launch (decode)
int32_t launch_rope_kv(runit_ctx* ctx, float* q, float* k, const float* v, void* kcache, void* vcache, uint32_t hd, uint32_t qh,
                       uint32_t kvh, const int32_t* pos_ptr, float theta, uint32_t max_seq);
int32_t launch_kv_copy(runit_ctx* ctx, const void* src, bool src_f16, void* dst, bool dst_f16, uint32_t pos,
                       const int32_t* pos_ptr, uint32_t max_seq, uint32_t hd, uint32_t kvh);
// q_kind / kv_kind: 0 = f32, 1 = f16.  part: scratch of batch*heads*nsplit*(hd+2) floats when nsplit > 1.
int32_t launch_decode_attention(runit_ctx* ctx, int q_kind, int kv_kind, const void* q, const void* k, const void* v, void* out,
                                float* part, uint32_t nsplit, uint32_t batch, uint32_t kv_len, const int32_t* pos_ptr,
                                uint32_t heads, uint32_t kv_heads, uint32_t hd, uint32_t stride,
                                uint32_t* counters = nullptr);   // batch*heads zeroed words: the last split merges, no combine launch
// rotary embedding of q and k, cache update of this position and attention in one launch (decode, batch 1, head_dim 64 / 128)
int32_t launch_decode_attention_rope(runit_ctx* ctx, const float* q, const float* k_raw, const float* v_raw, void* kcache, void* vcache,
                                     float* out, float* part, uint32_t nsplit, const int32_t* pos_ptr, uint32_t heads, uint32_t kv_heads,
                                     uint32_t hd, uint32_t max_seq, float theta, uint32_t* counters);
int32_t launch_argmax(runit_ctx* ctx, const void* in, bool in_f16, int32_t* result, uint32_t n);

// gemv.cu: one fused-dequant GEMV with up to three row segments sharing the input (Q|K|V) — any format.
int32_t gemv_segments(runit_ctx* ctx, const char* name, int fmt, int nseg, const void* const* w, void* const* y,
                      const uint32_t* rows, const void* x, uint32_t k,
                      // norm_gamma != nullptr: x is the un-normalised vector; RMSNorm(x) * gamma is what the matrices multiply
                      const float* norm_gamma = nullptr, float norm_eps = 0.f,
                      // expert parallelism: x is first formed as residual + the ranks' partial sums (see EpWait)
                      const EpWait* ep_wait = nullptr);
int32_t gemv_plain(runit_ctx* ctx, const char* name, int fmt, const void* w, const void* x, void* y, const void* res_f32,
                   uint32_t m, uint32_t k, const float* norm_gamma = nullptr, float norm_eps = 0.f,
                   // argmax_token != nullptr: the index of the largest result is written there by the launch itself
                   int32_t* argmax_token = nullptr, const EpWait* ep_wait = nullptr);
// prefill.cu: launchers of the batched prefill's own kernels
int32_t prefill_embed(runit_ctx* ctx, const float* emb, const int32_t* tokens, float* x, uint32_t T, uint32_t h);
int32_t prefill_norm_bf16(runit_ctx* ctx, const float* x, const float* gamma, void* y_bf16, float eps, uint32_t T, uint32_t h);
// q_in / k / v have rows of `ld` floats (0: as wide as their own heads); q_out [T][heads * hd] receives the rotated queries
int32_t prefill_rope_cache(runit_ctx* ctx, const float* q_in, float* q_out, const float* k, const float* v, void* kcache, void* vcache,
                           uint32_t hd, uint32_t heads, uint32_t kv_heads, uint32_t start_pos, float theta, uint32_t max_seq, uint32_t T,
                           uint32_t ld);
int32_t prefill_attention(runit_ctx* ctx, const float* q, const void* kcache, const void* vcache, void* out_bf16, uint32_t T, uint32_t heads,
                          uint32_t kv_heads, uint32_t hd, uint32_t max_seq, uint32_t start_pos);
int32_t prefill_add_rows(runit_ctx* ctx, float* x, const float* y, size_t n);
// x += y, then out = RMSNorm(x) * gamma, T rows of h (one launch; the bits of prefill_add_rows + launch_rms_norm)
int32_t prefill_add_rms_norm(runit_ctx* ctx, float* x, const float* y, const float* gamma, float* out, float eps, uint32_t T, uint32_t h);
// moe_grouped.cu: the tensor-core GEMM of the batched MoE block used on a dense matrix (see there)
int32_t dense_tiles_prepare(runit_ctx* ctx, int32_t* tables, uint32_t T);
int32_t dense_gemm_q4k_bf16(runit_ctx* ctx, const char* name, const void* w, const void* w_up, uint32_t rows, uint32_t K,
                            const void* x_bf16, uint32_t x_rows, void* out, uint32_t ld, uint32_t T, const int32_t* tables);
// moe.cu
int32_t moe_layer_q4k_impl(runit_ctx* ctx, const void* router_w, const void* gate, const void* up, const void* down,
                           const void* x, const void* residual, void* out, int32_t* idx_out, float* w_out, void* scratch,
                           size_t scratch_bytes, uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k, int32_t renorm,
                           const float* next_gamma, float* next_xn, float next_eps,    // next_*: also RMSNorm the result
                           // 1024 zeroed words (zero again after every launch): with T == 1, router and routing run in one
                           // launch and the weighted sum of the experts runs inside the down-projection launch
                           uint32_t* route_counter,
                           // pre_gamma != nullptr: the block first writes RMSNorm(pre_x) into x (inside the routing launch when T == 1)
                           const float* pre_x, const float* pre_gamma, float pre_eps);
size_t moe_scratch_bytes_impl(uint32_t T, uint32_t h, uint32_t ff, uint32_t E, uint32_t k);

}  // namespace runit
