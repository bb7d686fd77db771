"""CPU restatement of the batched prefill (test infrastructure: only tests may import it).

The operator sequence is the reference's Executor::prefill (crates/engine/src/prefill.rs:29-255): embedding rows, per
layer RMSNorm -> q/k/v projections -> batched RoPE -> cache fill -> causal attention with q_len = seq -> output projection ->
residual -> RMSNorm -> feed-forward block -> residual, then the final norm and lm_head on the last position.  The
reference computes in f16 with dequantised f16 weights; the device path keeps the hidden state in f32 and rounds GEMM
operands to bf16 (weights: the bf16 rounding of the Q4_K value of crates/engine/src/forward.rs:1026-1057), attention
operands to f16.  This restatement applies exactly those operand roundings, in numpy, and accumulates in f64:
  * GEMM:       y = bf16(x) . bf16(W)^T
  * attention:  per 64-key block, S = f16(q) . f16(K)^T / sqrt(hd) with the causal mask key <= query, the running maximum
                and sum of an online softmax, P = exp(S - max) rounded to f16 for the product with V
                (crates/kernels/shaders/attention.metal:36-158 is the same online softmax in f16)
  * the mixture-of-experts block: oracle.moe_grouped_q4k_bf16 on all tokens
  * lm_head:    the f32 fused-dequant GEMV of the decode path on the last position
"""
from __future__ import annotations

import numpy as np

from . import binding as B


def causal_attention_f16(q, kc, vc, heads, kv_heads, hd, start_pos=0, block=64):
    """q f32 [T][heads*hd] (rotated); kc, vc f16 [kv_heads][max_seq][hd].  Returns f32 [T][heads*hd] (before the bf16
    rounding of the device output)."""
    T = q.shape[0]
    out = np.zeros((T, heads * hd), np.float32)
    scale = np.float32(1.0 / np.sqrt(np.float32(hd)))
    qpos = start_pos + np.arange(T)
    n_keys = start_pos + T
    for h in range(heads):
        kvh = h // (heads // kv_heads)
        q16 = q[:, h * hd:(h + 1) * hd].astype(np.float16).astype(np.float64)
        K = kc[kvh, :n_keys].astype(np.float64)
        V = vc[kvh, :n_keys].astype(np.float64)
        m = np.full(T, -np.inf)
        l = np.zeros(T)
        o = np.zeros((T, hd))
        for k0 in range(0, n_keys, block):
            k1 = min(n_keys, k0 + block)
            s = ((q16 @ K[k0:k1].T).astype(np.float32) * scale).astype(np.float64)
            keys = np.arange(k0, k1)
            s = np.where(keys[None, :] <= qpos[:, None], s, -np.inf)
            m_new = np.maximum(m, s.max(axis=1))
            live = np.isfinite(m_new)
            corr = np.where(live, np.exp(np.where(live, m - m_new, 0.0)), 0.0)
            corr = np.where(np.isfinite(m), corr, 0.0)
            p = np.where(live[:, None], np.exp(np.where(live[:, None], s - np.where(live, m_new, 0.0)[:, None], -np.inf)), 0.0)
            p = p.astype(np.float32)
            l = l * corr + p.sum(axis=1, dtype=np.float64)
            o = o * corr[:, None] + p.astype(np.float16).astype(np.float64) @ V[k0:k1]
            m = m_new
        out[:, h * hd:(h + 1) * hd] = (o / np.where(l > 0, l, 1.0)[:, None]).astype(np.float32)
    return out


def _gemm_bf16(x, w_rows, m, k):
    """y[t][r] = sum_k bf16(x[t][k]) * bf16(W[r][k]); w_rows: Q4_K bytes of m rows."""
    W = B.bf16_round(B.dequant_rows(B.Q4K, w_rows, m, k)).astype(np.float64)
    return (B.bf16_round(x).astype(np.float64) @ W.T).astype(np.float32)


def prefill(cfg: dict, host: dict, tokens, want_hidden: bool = False):
    """cfg: the decoder's configuration as a dict; host: its tensors as numpy arrays (Q4_K matrices as bytes, f32 norms,
    router, embedding).  Returns (next_token, logits of the last position, kc, vc)."""
    L, h, hd = cfg["n_layers"], cfg["hidden"], cfg["head_dim"]
    heads, kvh, E, ff, V = cfg["n_heads"], cfg["n_kv_heads"], cfg["n_experts"], cfg["ff"], cfg["vocab"]
    q_dim, kv_dim, S = heads * hd, kvh * hd, cfg["max_seq"]
    rb = lambda k: k // 256 * 144
    T = len(tokens)
    x = host["tok_emb"].reshape(V, h)[np.asarray(tokens)].astype(np.float32).copy()
    kc = np.zeros((L, kvh, S, hd), np.float16)
    vc = np.zeros((L, kvh, S, hd), np.float16)
    sl = lambda name, l, rows, k: host[name].reshape(-1)[l * rows * rb(k):(l + 1) * rows * rb(k)]
    for l in range(L):
        xn = B.rms_norm_f32(x, host["attn_norm"].reshape(L, h)[l], cfg["eps"])
        q = _gemm_bf16(xn, sl("wq", l, q_dim, h), q_dim, h)
        k = _gemm_bf16(xn, sl("wk", l, kv_dim, h), kv_dim, h)
        v = _gemm_bf16(xn, sl("wv", l, kv_dim, h), kv_dim, h)
        for t in range(T):       # the decode oracle's rotation, position by position
            q[t], k[t] = B.rope_qk_f32(q[t], k[t], hd, heads, kvh, t, cfg["theta"])
        kc[l, :, :T] = k.reshape(T, kvh, hd).transpose(1, 0, 2).astype(np.float16)
        vc[l, :, :T] = v.reshape(T, kvh, hd).transpose(1, 0, 2).astype(np.float16)
        ao = B.bf16_round(causal_attention_f16(q, kc[l], vc[l], heads, kvh, hd))
        x = x + _gemm_bf16(ao, sl("wo", l, h, q_dim), h, q_dim)
        xn2 = B.rms_norm_f32(x, host["ffn_norm"].reshape(L, h)[l], cfg["eps"])
        x, _, _ = B.moe_grouped_q4k_bf16(host["router"].reshape(L, E, h)[l], sl("gate", l, E * ff, h), sl("up", l, E * ff, h),
                                         sl("down", l, E * h, ff), xn2, h=h, ff=ff, E=E, top_k=cfg["top_k"], renorm=bool(cfg["renorm"]),
                                         residual=x)
    last = B.rms_norm_f32(x[T - 1], host["out_norm"], cfg["eps"])
    logits = B.gemv(B.Q4K, host["lm_head"], last, V, h)
    tok = B.argmax_f32(logits)
    if want_hidden:
        return tok, logits, kc, vc, x
    return tok, logits, kc, vc
