"""ctypes binding of ``librunit_oracle.so`` (the plain-C CPU oracle; test infrastructure).

numpy arrays in, numpy arrays out.  The C functions cite the reference file:line they follow.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

__all__ = [
    "Q8_0", "Q4_0", "Q4K", "Q5_0", "Q5K", "Q6K", "TIER_SHADER", "TIER_DEQUANT", "TIER_F64", "MOE_F32", "MOE_REF_F16",
    "build_oracle", "lib", "num_threads", "set_num_threads", "row_bytes", "block_elems",
    "block_bytes", "dequant_rows", "dequant_q4k_f16", "gemv", "gemv_f64", "gemv_f16w_f32in",
    "gemv_f32w", "silu_mul_f32", "silu_mul_f16", "scale_accumulate_f16", "add_f16_into_f32",
    "topk_softmax", "moe_layer_q4k", "moe_grouped_q4k_bf16", "bf16_round", "rms_norm_f32", "rope_qk_f32", "kv_copy_to_cache_f16",
    "decode_attention_f32q_f16kv", "argmax_f32", "ModelCfg", "ModelWeights", "decode_step",
    "compare", "DiffStats", "f32_to_f16_bits", "f16_bits_to_f32", "SamplerCfg", "SamplerRng", "sample", "sampler_argmax_last",
]

Q8_0, Q4_0, Q4K, Q5_0, Q5K, Q6K = 0, 1, 2, 3, 4, 5
TIER_SHADER, TIER_DEQUANT, TIER_F64 = 0, 1, 2
MOE_F32, MOE_REF_F16 = 0, 1

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "librunit_oracle.so"
_lib = None


def build_oracle(force: bool = False) -> Path:
    """Compile the C oracle with the Makefile beside it (gcc only; no GPU involved)."""
    src_m = max((_HERE / n).stat().st_mtime for n in ("runit_oracle.c", "runit_oracle.h", "Makefile"))
    if force or not _SO.exists() or _SO.stat().st_mtime < src_m:
        subprocess.run(["make", "-C", str(_HERE), "-B", "librunit_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _SO


class DiffStats(C.Structure):
    _fields_ = [("max_abs", C.c_double), ("mean_abs", C.c_double), ("rms", C.c_double),
                ("ref_rms", C.c_double), ("max_rel", C.c_double), ("n", C.c_int64),
                ("n_mismatch_abs", C.c_int64), ("n_mismatch_rel", C.c_int64)]

    def __repr__(self):
        return ("DiffStats(max_abs=%.3e mean_abs=%.3e rms=%.3e ref_rms=%.3e max_rel=%.3e n=%d "
                "mis_abs=%d mis_rel=%d)" % (self.max_abs, self.mean_abs, self.rms, self.ref_rms,
                                            self.max_rel, self.n, self.n_mismatch_abs,
                                            self.n_mismatch_rel))


class ModelCfg(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim",
                                         "vocab", "n_experts", "top_k", "ff", "max_seq", "renorm")]
    _fields_ += [("eps", C.c_float), ("theta", C.c_float)]


class ModelWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("tok_emb", "attn_norm", "ffn_norm", "out_norm", "wq", "wk",
                                          "wv", "wo", "router", "gate", "up", "down", "lm_head")]


class SamplerCfg(C.Structure):
    """SamplerConfig without the seed (crates/engine/src/sampler.rs:31-45)."""
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_int32), ("top_p", C.c_float), ("repetition_penalty", C.c_float),
                ("min_tokens", C.c_int32)]


def lib():
    global _lib
    if _lib is None:
        if not _SO.exists():
            build_oracle()
        _lib = C.CDLL(str(_SO))
        L = _lib
        L.ro_num_threads.restype = C.c_int
        L.ro_f32_to_f16.restype = C.c_uint16
        L.ro_f32_to_f16.argtypes = [C.c_float]
        L.ro_f16_to_f32.restype = C.c_float
        L.ro_f16_to_f32.argtypes = [C.c_uint16]
        for n in ("ro_block_elems", "ro_block_bytes"):
            getattr(L, n).restype = C.c_size_t
            getattr(L, n).argtypes = [C.c_int]
        L.ro_row_bytes.restype = C.c_size_t
        L.ro_row_bytes.argtypes = [C.c_int, C.c_int]
        L.ro_gemv.restype = C.c_int
        L.ro_gemv.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                              C.c_int, C.c_int, C.c_int]
        L.ro_dequant_row.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_void_p]
        L.ro_dequant_q4k_f16.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        L.ro_gemv_f16w_f32in.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        L.ro_gemv_f32w.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        L.ro_silu_mul_f32.argtypes = [C.c_void_p] * 3 + [C.c_size_t]
        L.ro_silu_mul_f16.argtypes = [C.c_void_p] * 3 + [C.c_size_t]
        L.ro_scale_accumulate_f16.argtypes = [C.c_void_p, C.c_void_p, C.c_float, C.c_size_t]
        L.ro_add_f16_into_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        L.ro_topk_softmax.restype = C.c_int
        L.ro_topk_softmax.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                      C.c_void_p]
        L.ro_moe_grouped_q4k_bf16.restype = C.c_int
        L.ro_moe_grouped_q4k_bf16.argtypes = [C.c_void_p, C.c_int] + [C.c_void_p] * 8 + [C.c_int] * 5
        L.ro_bf16_round.restype = C.c_float
        L.ro_bf16_round.argtypes = [C.c_float]
        L.ro_moe_layer_q4k.restype = C.c_int
        L.ro_moe_layer_q4k.argtypes = [C.c_int, C.c_int] + [C.c_void_p] * 9 + [C.c_int] * 5
        L.ro_rms_norm_f32.argtypes = [C.c_void_p] * 3 + [C.c_float, C.c_int, C.c_int]
        L.ro_rope_qk_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                     C.c_float]
        L.ro_kv_copy_to_cache_f16.argtypes = [C.c_void_p, C.c_void_p] + [C.c_int] * 4
        L.ro_decode_attention_f32q_f16kv.argtypes = [C.c_void_p] * 4 + [C.c_int] * 5
        L.ro_argmax_f32.restype = C.c_int32
        L.ro_argmax_f32.argtypes = [C.c_void_p, C.c_size_t]
        L.ro_sampler_seed_state.restype = C.c_uint64
        L.ro_sampler_seed_state.argtypes = [C.c_uint64]
        L.ro_sampler_next_f32.restype = C.c_float
        L.ro_sampler_next_f32.argtypes = [C.POINTER(C.c_uint64)]
        L.ro_sampler_argmax_last.restype = C.c_int32
        L.ro_sampler_argmax_last.argtypes = [C.c_void_p, C.c_size_t]
        L.ro_sample.restype = C.c_int32
        L.ro_sample.argtypes = [C.c_void_p, C.c_size_t, C.POINTER(SamplerCfg), C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t,
                                C.POINTER(C.c_uint64), C.c_void_p]
        L.ro_decode_step.restype = C.c_int32
        L.ro_decode_step.argtypes = [C.POINTER(ModelCfg), C.POINTER(ModelWeights), C.c_void_p,
                                     C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]
        L.ro_compare.restype = C.c_int64
        L.ro_compare.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_float, C.c_float,
                                 C.POINTER(DiffStats)]
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def num_threads() -> int:
    return lib().ro_num_threads()


def set_num_threads(n: int) -> None:
    lib().ro_set_num_threads(int(n))


def block_elems(fmt: int) -> int:
    return lib().ro_block_elems(fmt)


def block_bytes(fmt: int) -> int:
    return lib().ro_block_bytes(fmt)


def row_bytes(fmt: int, k: int) -> int:
    return lib().ro_row_bytes(fmt, k)


def f32_to_f16_bits(x) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().ro_f32_to_f16_array(_p(x), _p(out), C.c_size_t(x.size))
    return out


def f16_bits_to_f32(h) -> np.ndarray:
    h = _c(h, np.uint16)
    out = np.empty(h.shape, np.float32)
    lib().ro_f16_to_f32_array(_p(h), _p(out), C.c_size_t(h.size))
    return out


def dequant_rows(fmt: int, w: np.ndarray, m: int, k: int) -> np.ndarray:
    w = _c(w, np.uint8).reshape(-1)
    rb = row_bytes(fmt, k)
    assert w.size >= m * rb
    out = np.empty((m, k), np.float32)
    for r in range(m):
        lib().ro_dequant_row(fmt, C.c_void_p(w.ctypes.data + r * rb), k,
                             C.c_void_p(out.ctypes.data + r * k * 4))
    return out


def dequant_q4k_f16(w: np.ndarray, n_blocks: int) -> np.ndarray:
    w = _c(w, np.uint8).reshape(-1)
    out = np.empty(n_blocks * 256, np.float16)
    lib().ro_dequant_q4k_f16(_p(w), _p(out), C.c_size_t(n_blocks))
    return out


def gemv(fmt: int, w: np.ndarray, x: np.ndarray, m: int, k: int, tier: int = TIER_F64) -> np.ndarray:
    """y[b, r] for x of shape [k] or [batch, k]; returns the same leading shape."""
    w = _c(w, np.uint8).reshape(-1)
    x = _c(x, np.float32)
    batch = 1 if x.ndim == 1 else x.shape[0]
    assert x.shape[-1] == k and w.size >= m * row_bytes(fmt, k)
    y = np.empty((batch, m), np.float32)
    rc = lib().ro_gemv(fmt, tier, _p(w), _p(x), _p(y), None, m, k, batch)
    if rc:
        raise ValueError("ro_gemv rejected fmt=%d m=%d k=%d" % (fmt, m, k))
    return y[0] if x.ndim == 1 else y


def gemv_f64(fmt: int, w: np.ndarray, x: np.ndarray, m: int, k: int) -> np.ndarray:
    w = _c(w, np.uint8).reshape(-1)
    x = _c(x, np.float32)
    batch = 1 if x.ndim == 1 else x.shape[0]
    y = np.empty((batch, m), np.float32)
    y64 = np.empty((batch, m), np.float64)
    rc = lib().ro_gemv(fmt, TIER_F64, _p(w), _p(x), _p(y), _p(y64), m, k, batch)
    if rc:
        raise ValueError("ro_gemv rejected")
    return y64[0] if x.ndim == 1 else y64


def gemv_f16w_f32in(w_f16: np.ndarray, x: np.ndarray, m: int, k: int) -> np.ndarray:
    w = _c(w_f16, np.float16).view(np.uint16)
    x = _c(x, np.float32)
    y = np.empty(m, np.float32)
    lib().ro_gemv_f16w_f32in(_p(w), _p(x), _p(y), m, k)
    return y


def gemv_f32w(w: np.ndarray, x: np.ndarray, m: int, k: int) -> np.ndarray:
    w = _c(w, np.float32)
    x = _c(x, np.float32)
    y = np.empty(m, np.float32)
    lib().ro_gemv_f32w(_p(w), _p(x), _p(y), m, k)
    return y


def silu_mul_f32(g, u) -> np.ndarray:
    g, u = _c(g, np.float32), _c(u, np.float32)
    out = np.empty_like(g)
    lib().ro_silu_mul_f32(_p(g), _p(u), _p(out), C.c_size_t(g.size))
    return out


def silu_mul_f16(g, u) -> np.ndarray:
    g, u = _c(g, np.float16), _c(u, np.float16)
    out = np.empty_like(g)
    lib().ro_silu_mul_f16(_p(g), _p(u), _p(out), C.c_size_t(g.size))
    return out


def scale_accumulate_f16(src, acc, weight: float) -> np.ndarray:
    src = _c(src, np.float16)
    acc = np.array(acc, dtype=np.float16, copy=True)
    lib().ro_scale_accumulate_f16(_p(src), _p(acc), C.c_float(weight), C.c_size_t(src.size))
    return acc


def add_f16_into_f32(src, acc) -> np.ndarray:
    src = _c(src, np.float16)
    acc = np.array(acc, dtype=np.float32, copy=True)
    lib().ro_add_f16_into_f32(_p(src), _p(acc), C.c_size_t(src.size))
    return acc


def topk_softmax(logits, top_k: int, renorm: bool):
    logits = _c(logits, np.float32)
    E = logits.size
    idx = np.empty(top_k, np.int32)
    w = np.empty(top_k, np.float32)
    probs = np.empty(E, np.float32)
    rc = lib().ro_topk_softmax(_p(logits), E, top_k, int(renorm), _p(idx), _p(w), _p(probs))
    if rc:
        raise ValueError("ro_topk_softmax rejected E=%d k=%d" % (E, top_k))
    return idx, w, probs


def moe_layer_q4k(router, gate, up, down, x, *, h, ff, E, top_k, renorm=False, mode=MOE_F32,
                  residual=None):
    router = _c(router, np.float32)
    gate, up, down = (_c(a, np.uint8).reshape(-1) for a in (gate, up, down))
    x = _c(x, np.float32).reshape(-1, h)
    T = x.shape[0]
    res = None if residual is None else _c(residual, np.float32).reshape(T, h)
    out = np.empty((T, h), np.float32)
    idx = np.empty((T, top_k), np.int32)
    w = np.empty((T, top_k), np.float32)
    rc = lib().ro_moe_layer_q4k(mode, int(renorm), _p(router), _p(gate), _p(up), _p(down), _p(x),
                                None if res is None else _p(res), _p(out), _p(idx), _p(w), T, h, ff,
                                E, top_k)
    if rc:
        raise ValueError("ro_moe_layer_q4k rejected the shapes")
    return out, idx, w


def moe_grouped_q4k_bf16(router, gate, up, down, x, *, h, ff, E, top_k, renorm=False, residual=None, routing=None):
    """Batched block with bf16 operands.  routing=(idx, w): use it (router ignored); else route with the f32 router."""
    gate, up, down = (_c(a, np.uint8).reshape(-1) for a in (gate, up, down))
    x = _c(x, np.float32).reshape(-1, h)
    T = x.shape[0]
    res = None if residual is None else _c(residual, np.float32).reshape(T, h)
    out = np.empty((T, h), np.float32)
    if routing is None:
        router = _c(router, np.float32)
        idx = np.empty((T, top_k), np.int32)
        w = np.empty((T, top_k), np.float32)
        rp = _p(router)
    else:
        idx = np.array(routing[0], dtype=np.int32, copy=True).reshape(T, top_k)
        w = np.array(routing[1], dtype=np.float32, copy=True).reshape(T, top_k)
        rp = None
    rc = lib().ro_moe_grouped_q4k_bf16(rp, int(renorm), _p(gate), _p(up), _p(down), _p(x),
                                       None if res is None else _p(res), _p(out), _p(idx), _p(w), T, h, ff, E, top_k)
    if rc:
        raise ValueError("ro_moe_grouped_q4k_bf16 rejected the shapes")
    return out, idx, w


def bf16_round(a) -> np.ndarray:
    """Round-to-nearest-even to bf16, returned as f32."""
    u = _c(a, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


def rms_norm_f32(x, gamma, eps: float) -> np.ndarray:
    x = _c(x, np.float32)
    gamma = _c(gamma, np.float32)
    hidden = x.shape[-1]
    rows = x.size // hidden
    y = np.empty_like(x)
    lib().ro_rms_norm_f32(_p(x), _p(gamma), _p(y), C.c_float(eps), hidden, rows)
    return y


def rope_qk_f32(q, k, head_dim, q_heads, kv_heads, pos, theta):
    q = np.array(q, dtype=np.float32, copy=True)
    k = np.array(k, dtype=np.float32, copy=True)
    lib().ro_rope_qk_f32(_p(q), _p(k), head_dim, q_heads, kv_heads, pos, C.c_float(theta))
    return q, k


def kv_copy_to_cache_f16(src, cache, pos, max_seq, head_dim, kv_heads) -> None:
    src = _c(src, np.float32)
    assert cache.dtype == np.float16 and cache.flags.c_contiguous
    lib().ro_kv_copy_to_cache_f16(_p(src), _p(cache), pos, max_seq, head_dim, kv_heads)


def decode_attention_f32q_f16kv(q, kc, vc, kv_len, heads, kv_heads, head_dim, kv_head_stride):
    q = _c(q, np.float32)
    kc, vc = _c(kc, np.float16), _c(vc, np.float16)
    out = np.empty(heads * head_dim, np.float32)
    lib().ro_decode_attention_f32q_f16kv(_p(q), _p(kc), _p(vc), _p(out), kv_len, heads, kv_heads,
                                         head_dim, kv_head_stride)
    return out


def argmax_f32(v) -> int:
    v = _c(v, np.float32)
    return int(lib().ro_argmax_f32(_p(v), C.c_size_t(v.size)))


class SamplerRng:
    """SimpleRng (sampler.rs:12-27)."""

    def __init__(self, seed: int):
        self.state = C.c_uint64(lib().ro_sampler_seed_state(C.c_uint64(seed)))

    def next_f32(self) -> float:
        return float(lib().ro_sampler_next_f32(C.byref(self.state)))


def sampler_argmax_last(v) -> int:
    v = _c(v, np.float32)
    return int(lib().ro_sampler_argmax_last(_p(v), C.c_size_t(v.size)))


def sample(logits, cfg: SamplerCfg, context, eos_ids, rng: SamplerRng, want_probs: bool = False):
    """sample() of sampler.rs:61-111.  Returns the token, or (token, vector the draw was made from)."""
    logits = _c(logits, np.float32)
    context = _c(np.asarray(context, np.int32), np.int32)
    eos_ids = _c(np.asarray(eos_ids, np.int32), np.int32)
    probs = np.empty(logits.size, np.float32) if want_probs else None
    tok = int(lib().ro_sample(_p(logits), C.c_size_t(logits.size), C.byref(cfg), _p(context), C.c_size_t(context.size),
                              _p(eos_ids), C.c_size_t(eos_ids.size), C.byref(rng.state), _p(probs) if want_probs else None))
    return (tok, probs) if want_probs else tok


def decode_step(cfg: ModelCfg, weights: ModelWeights, kc: np.ndarray, vc: np.ndarray, token: int,
                pos: int, want_logits: bool = False):
    logits = np.empty(cfg.vocab, np.float32) if want_logits else None
    tok = lib().ro_decode_step(C.byref(cfg), C.byref(weights), _p(kc), _p(vc), token, pos,
                               None if logits is None else _p(logits))
    if tok < 0:
        raise ValueError("ro_decode_step rejected token=%d pos=%d" % (token, pos))
    return (tok, logits) if want_logits else tok


def compare(ref, got, abs_tol: float = 1e-2, rel_tol: float = 1e-3) -> DiffStats:
    ref, got = _c(ref, np.float32).reshape(-1), _c(got, np.float32).reshape(-1)
    assert ref.size == got.size, "reference and custom output lengths must match"
    st = DiffStats()
    lib().ro_compare(_p(ref), _p(got), C.c_size_t(ref.size), C.c_float(abs_tol), C.c_float(rel_tol),
                     C.byref(st))
    return st
