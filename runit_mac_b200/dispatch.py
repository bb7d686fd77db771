"""Host-side mirror of the reference's kernel dispatch layer over the C ABI.

The reference exposes free functions ``op(ctx: &MetalContext, buffers..., dims...) -> Result<()>``
(crates/kernels/src/dispatch.rs) and a ``MetalContext`` with ``new_buffer`` / ``flush``
(crates/kernels/src/context.rs:163-296).  This module keeps those names and argument orders:
``Context`` replaces ``MetalContext``, ``DeviceBuffer`` replaces ``metal::Buffer``, a failed call
raises ``KernelError`` (crates/kernels/src/error.rs:4-22) instead of returning ``Err``.

Every function here forwards to the ``extern "C"`` symbol of the same name prefixed ``runit_``;
nothing is computed in Python.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib

OK = 0
ERR_NO_DEVICE, ERR_BAD_ARG, ERR_BUFFER_SIZE, ERR_LAUNCH, ERR_NCCL, ERR_TIMEOUT, ERR_UNSUPPORTED, ERR_ALLOC = range(1, 9)
FMT_Q8_0, FMT_Q4_0, FMT_Q4K, FMT_Q5_0, FMT_Q5K, FMT_Q6K = 0, 1, 2, 3, 4, 5
BUF_DEVICE, BUF_HOST_VISIBLE = 0, 1

BLOCK_ELEMS = {FMT_Q8_0: 32, FMT_Q4_0: 32, FMT_Q4K: 256, FMT_Q5_0: 32, FMT_Q5K: 256, FMT_Q6K: 256}     # dispatch.rs:735-747
BLOCK_BYTES = {FMT_Q8_0: 34, FMT_Q4_0: 18, FMT_Q4K: 144, FMT_Q5_0: 22, FMT_Q5K: 176, FMT_Q6K: 210}


def row_bytes(fmt: int, k: int) -> int:
    return k // BLOCK_ELEMS[fmt] * BLOCK_BYTES[fmt]


class KernelError(RuntimeError):
    """Mirror of KernelError (crates/kernels/src/error.rs:4-22); ``status`` is the C status code."""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


class DeviceBuffer:
    """Device memory owned by a Context (replaces metal::Buffer; caller-owned, ops never allocate)."""

    def __init__(self, ctx: "Context", nbytes: int, flags: int = BUF_DEVICE):
        self.ctx, self.nbytes = ctx, int(nbytes)
        p = C.c_void_p()
        ctx._check(ctx.lib.runit_buf_alloc(ctx.handle, self.nbytes, flags, C.byref(p)))
        self.ptr = p.value

    def free(self):
        if self.ptr:
            self.ctx.lib.runit_buf_free(self.ctx.handle, self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            if self.ptr and self.ctx.handle:
                self.free()
        except Exception:
            pass

    def upload(self, arr: np.ndarray, offset: int = 0) -> "DeviceBuffer":
        arr = np.ascontiguousarray(arr)
        if offset + arr.nbytes > self.nbytes:
            raise KernelError(ERR_BUFFER_SIZE, "upload of %d bytes at %d into a %d-byte buffer"
                              % (arr.nbytes, offset, self.nbytes))
        self.ctx._check(self.ctx.lib.runit_memcpy_h2d(self.ctx.handle, self.ptr + offset, arr.ctypes.data, arr.nbytes))
        self.ctx.flush()   # the host array may go away after this call
        return self

    def download(self, dtype, count: int, offset: int = 0) -> np.ndarray:
        out = np.empty(count, dtype)
        if offset + out.nbytes > self.nbytes:
            raise KernelError(ERR_BUFFER_SIZE, "download of %d bytes at %d from a %d-byte buffer"
                              % (out.nbytes, offset, self.nbytes))
        self.ctx._check(self.ctx.lib.runit_memcpy_d2h(self.ctx.handle, out.ctypes.data, self.ptr + offset, out.nbytes))
        self.ctx.flush()
        return out


def _ptr(b) -> int:
    """Accept a DeviceBuffer, a raw integer address, or anything with ``data_ptr()`` (torch)."""
    if b is None:
        return None
    if isinstance(b, DeviceBuffer):
        return b.ptr
    if isinstance(b, int):
        return b
    if hasattr(b, "data_ptr"):
        return b.data_ptr()
    raise TypeError("not a device buffer: %r" % (b,))


class Context:
    """One CUDA stream on one GPU; replaces MetalContext.  Single-threaded, like the reference's."""

    def __init__(self, device: int = 0, stream: int | None = None):
        self.lib = _lib.load()
        h = C.c_void_p()
        if stream is None:
            st = self.lib.runit_ctx_create(device, C.byref(h))
        else:
            st = self.lib.runit_ctx_create_on_stream(device, C.c_void_p(stream), C.byref(h))
        if st != OK:
            raise KernelError(st, "runit_ctx_create(device=%d) failed: %s (no CPU fallback exists)"
                              % (device, self.lib.runit_status_string(st).decode()))
        self.handle = h
        self.device = device

    def close(self):
        if self.handle:
            self.lib.runit_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, status: int):
        if status != OK:
            raise KernelError(status, self.lib.runit_last_error_string(self.handle).decode())

    # MetalContext::new_buffer (context.rs:215-220)
    def new_buffer(self, nbytes: int, host_visible: bool = False) -> DeviceBuffer:
        return DeviceBuffer(self, nbytes, BUF_HOST_VISIBLE if host_visible else BUF_DEVICE)

    def buffer_from(self, arr: np.ndarray) -> DeviceBuffer:
        arr = np.ascontiguousarray(arr)
        return DeviceBuffer(self, max(arr.nbytes, 16)).upload(arr)

    # MetalContext::flush (context.rs:289-296)
    def flush(self):
        self._check(self.lib.runit_flush(self.handle))

    @property
    def stream(self) -> int:
        return self.lib.runit_ctx_stream(self.handle) or 0

    @property
    def launches(self) -> int:
        return self.lib.runit_launch_count(self.handle)

    def set_tuning(self, key: str, value: int):
        self._check(self.lib.runit_set_tuning(self.handle, key.encode(), value))

    # Recorded command lists (the role of the reference's command buffer, context.rs:248-296).
    def graph_begin(self):
        self._check(self.lib.runit_graph_begin(self.handle))

    def graph_end(self) -> "Graph":
        g = C.c_void_p()
        self._check(self.lib.runit_graph_end(self.handle, C.byref(g)))
        return Graph(self, g)

    def call(self, name: str, *args):
        """Call ``runit_<name>(ctx, *args)``; buffers may be DeviceBuffers, ints or torch tensors."""
        fn = getattr(self.lib, "runit_" + name)
        conv = [(_ptr(a) if (isinstance(a, DeviceBuffer) or hasattr(a, "data_ptr") or a is None) else a) for a in args]
        self._check(fn(self.handle, *conv))


class Graph:
    """A recorded list of ops that replays with one launch."""

    def __init__(self, ctx: Context, handle):
        self.ctx, self.handle = ctx, handle

    def launch(self):
        self.ctx._check(self.ctx.lib.runit_graph_launch(self.ctx.handle, self.handle))

    @property
    def fused_launches(self) -> int:
        """Recorded GEMV launches that were folded into persistent launches."""
        return self.ctx.lib.runit_graph_fused_launches(self.handle)

    @property
    def kernel_launches(self) -> int:
        """Kernel launches one replay performs."""
        return self.ctx.lib.runit_graph_kernel_launches(self.handle)

    def destroy(self):
        if self.handle:
            self.ctx.lib.runit_graph_destroy(self.ctx.handle, self.handle)
            self.handle = None


def _twin(name: str, doc: str):
    def f(ctx: Context, *args):
        ctx.call(name, *args)
    f.__name__ = name
    f.__doc__ = doc
    return f


# (name, reference citation) — signatures are those of include/runit_cuda.h
_TWINS = [
    ("gemv_q8_0_f32in_f32out", "dispatch.rs:1280 (weight, input, output, m, k)"),
    ("gemv_q8_0_add_f32_f32in", "dispatch.rs:1298 (weight, input, output, residual, m, k)"),
    ("gemv_q8_0_f32in", "dispatch.rs:1317"),
    ("gemv_q8_0_f16", "dispatch.rs:1335"),
    ("gemv_q8_0_add_f16", "dispatch.rs:1353"),
    ("gemv_q8_0_add_f32res_f16", "dispatch.rs:1372"),
    ("gemv_q8_0_f32in_f32out_mr", "dispatch.rs:1083"),
    ("gemv_q8_0_add_f32_f32in_mr", "dispatch.rs:1101"),
    ("gemv_q8_0_f32in_f32out_wide", "dispatch.rs:1397"),
    ("gemv_q8_0_add_f32_f32in_wide", "dispatch.rs:1414"),
    ("gemv_q8_0_f32in_wide", "dispatch.rs:1432"),
    ("fused_qkv_q8_0_f32", "dispatch.rs:813 (w_q, w_k, w_v, x, out_q, out_k, out_v, q_dim, kv_dim, k)"),
    ("fused_qkv_bias_q8_0_f32", "dispatch.rs:842 (+ bias_q, bias_k, bias_v as f16)"),
    ("fused_qkv_f32bias_q8_0_f32", "no twin: f32 bias"),
    ("fused_qkv_q4_0_f32", "no twin: Q|K|V for Q4_0"),
    ("fused_qkv_q4k_f32", "no twin: Q|K|V for Q4_K"),
    ("fused_ffn_q4k_f32", "no twin: gate/up + SiLU for Q4_K"),
    ("fused_ffn_q8_0_f32", "dispatch.rs:903 (w_gate, w_up, x, act_out, ff_dim, k)"),
    ("gemv_q4_0_f32in_f32out", "dispatch.rs:1456"),
    ("gemv_q4_0_add_f32_f32in", "dispatch.rs:1471"),
    ("gemv_q4_0_f32in", "dispatch.rs:1486"),
    ("gemv_q4_0_f16", "dispatch.rs:1501"),
    ("gemv_q4_0_add_f16", "dispatch.rs:1516"),
    ("fused_ffn_q4_0_f32", "dispatch.rs:1531"),
    ("gemv_q4k_f32in_f32out", "dispatch.rs:1229"),
    ("gemv_q4k_add_f32_f32in", "dispatch.rs:1251"),
    ("gemv_q4k_f16", "dispatch.rs:621"),
    ("gemv_q4k_add_f16", "dispatch.rs:585"),
    ("gemv_q4k_add_f32res_f16", "dispatch.rs:358"),
    ("dequant_q4k_f16", "dispatch.rs:756 (input, output, n_blocks)"),
    ("gemv_q5_0_f32in_f32out", "no twin (forward.rs:900-919 on the device): (weight, input, output, m, k)"),
    ("gemv_q5_0_add_f32_f32in", "no twin: (weight, input, output, residual, m, k)"),
    ("gemv_q5k_f32in_f32out", "no twin (forward.rs:979-1012 on the device)"),
    ("gemv_q5k_add_f32_f32in", "no twin"),
    ("gemv_q6k_f32in_f32out", "no twin (forward.rs:920-949 on the device)"),
    ("gemv_q6k_add_f32_f32in", "no twin"),
    ("gemv_f16w_f32in", "dispatch.rs:270 (weight, input, output, m, k)"),
    ("silu_mul_f16", "dispatch.rs:15 (gate, up, out, n)"),
    ("silu_mul_f32", "dispatch.rs:35"),
    ("scale_accumulate_f16", "dispatch.rs:1639 (src, acc, weight, n)"),
    ("add_f16_into_f32", "dispatch.rs:316 (src, acc, n)"),
    ("gemv_batched_f32", "no twin: (fmt, weight, input, output, residual, m, k, batch)"),
    ("rms_norm_gemv_f32", "no twin: RMSNorm inside the GEMV (fmt, weight, x, gamma_f32, eps, output, residual, m, k)"),
    ("rms_norm_fused_qkv_f32", "no twin: RMSNorm inside Q|K|V (fmt, w_q, w_k, w_v, x, gamma_f32, eps, out_q, out_k, out_v, "
                               "q_dim, kv_dim, k)"),
    ("gemv_argmax_f32", "no twin: lm_head GEMV with the argmax in its epilogue (fmt, weight, x, gamma_f32 or None, eps, logits, "
                        "result_i32, m, k)"),
    ("gemv_argmax_allgather", "no twin: row-sharded greedy lm_head (fmt, w_local, x, logits_local, pairs_all[world] pointer "
                              "table, world, rank, rows_total, k)"),
    ("argmax_pairs", "no twin: (pairs, n, result_i32)"),
    ("peer_barrier_argmax", "no twin: (signal_pads[world], world, rank, epoch, pairs, result_i32)"),
    ("prefill_attention_f16kv", "dispatch.rs flash_attention_f16 with q_len = seq (prefill.rs:134-145): (q_f32, kcache, vcache, out_bf16, T, "
                                "heads, kv_heads, head_dim, max_seq, start_pos)"),
    ("ffn_q4k_bf16", "prefill.rs:217-227 as one call: (w_gate, w_up, w_down, x, gamma_or_None, eps, residual_or_None, out, scratch, "
                     "scratch_bytes, T, h, ff)"),
    ("rms_norm_f32_f32", "dispatch.rs:152 (x, y, gamma_f16, eps, hidden, num_rows)"),
    ("rms_norm_f32_f32_f32g", "dispatch.rs:177 (x, y, gamma_f32, eps, hidden, num_rows)"),
    ("fused_rope_qk_f32", "dispatch.rs:945 (q, k, head_dim, q_heads, kv_heads, pos, theta)"),
    ("kv_copy_to_cache_f16", "dispatch.rs:1159 (src, dst, pos, max_seq, head_dim, num_kv_heads)"),
    ("kv_copy_to_cache_f32", "dispatch.rs:1183"),
    ("kv_copy_to_cache_f32_f16", "no twin: f32 source, f16 cache"),
    ("decode_attention_f32", "dispatch.rs:1575 (q, k, v, out, batch, kv_len, num_heads, num_kv_heads, head_dim, kv_head_stride)"),
    ("decode_attention_f16", "dispatch.rs:697"),
    ("decode_attention_f32q_f16kv", "no twin: f32 query over an f16 cache"),
    ("argmax_f16", "dispatch.rs:1615 (input, result, n)"),
    ("argmax_f32", "no twin: f32 logits"),
    ("moe_router_f32", "no twin: (router_w, x, logits, E, h, T)"),
    ("moe_route_topk", "forward.rs:2420-2448 on the device: (logits, logits_f16, E, k, renorm, T, out_idx, out_w)"),
    ("moe_layer_q4k", "forward.rs:1644-1679 as one call: (router_w, gate, up, down, x, residual, out, idx_out, w_out, "
                      "scratch, scratch_bytes, T, h, ff, E, k, renorm)"),
    ("moe_experts_q4k", "no twin: (gate, up, down, x_slots, slot_expert, y_slots, act_scratch, n_slots, h, ff, n_experts)"),
    ("moe_layer_q4k_static", "no twin: moe_layer_q4k without the scratch arguments (built-in 4 MiB region)"),
    ("moe_layer_q4k_bf16", "no twin (prefill.rs:156-215 batched): same arguments as moe_layer_q4k, scratch from "
                           "moe_grouped_scratch_bytes"),
    ("moe_experts_grouped_q4k_bf16", "no twin: (gate, up, down, x, idx, w, residual, out, scratch, scratch_bytes, T, h, ff, E, k)"),
    ("gemv_allgather_f32", "no twin: (fmt, w_local, x, y_all[world] pointer table, world, rank, rows_total, k)"),
    ("peer_barrier", "no twin: (signal_pads[world] pointer table, world, rank, epoch)"),
    ("moe_layer_q4k_ep", "no twin: expert-parallel decode block with replicated tokens, combine fused over peer memory"),
    ("moe_layer_q4k_bf16_ep", "no twin: expert-parallel batched block, token rows exchanged by peer stores"),
    ("fill_weights", "no twin: (fmt, dst, n_blocks, seed, sigma)"),
    ("fill_weights_q4k_zero_mean", "no twin: (dst, n_blocks, seed, sigma), Q4_K blocks with zero-mean weights"),
    ("fill_normal_f32", "no twin: (dst, n, seed, sigma)"),
]
for _n, _d in _TWINS:
    globals()[_n] = _twin(_n, _d)
del _n, _d

def gemv_batched_multi_f32(ctx: Context, fmt: int, weights, x, outputs, rows, k: int, batch: int):
    """Up to three matrices over the same activations in one launch (q | k | v, gate | up); no twin in the reference."""
    n = len(weights)
    wt = (C.c_void_p * n)(*[_ptr(w) for w in weights])
    ot = (C.c_void_p * n)(*[_ptr(o) for o in outputs])
    rt = (C.c_uint32 * n)(*[int(r) for r in rows])
    ctx._check(ctx.lib.runit_gemv_batched_multi_f32(ctx.handle, fmt, n, wt, _ptr(x), ot, rt, k, batch))


class ModelCfg(C.Structure):
    """runit_model_cfg; field names follow ModelConfig (crates/engine/src/config.rs:42-89)."""
    _fields_ = [(n, C.c_int32) for n in ("n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim", "vocab", "n_experts",
                                         "top_k", "ff", "max_seq", "renorm")] + [("eps", C.c_float), ("theta", C.c_float)]


class SamplerCfg(C.Structure):
    """runit_sampler_cfg; SamplerConfig without the seed (crates/engine/src/sampler.rs:31-45)."""
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_int32), ("top_p", C.c_float), ("repetition_penalty", C.c_float),
                ("min_tokens", C.c_int32)]


def sampler_seed_state(ctx: Context, seed: int) -> int:
    """State of a SimpleRng::new(seed) generator (sampler.rs:15-17), to be stored in the sampler's rng_state word."""
    return int(ctx.lib.runit_sampler_seed_state(seed))


def sample_f32(ctx: Context, logits, scores_scratch, n: int, cfg: SamplerCfg, context, ctx_begin: int, ctx_end: int, eos_ids,
               n_eos: int, rng_state, result, ctx_range=None):
    """sample() of sampler.rs:61-111 as one launch; all buffers on the device."""
    ctx._check(ctx.lib.runit_sample_f32(ctx.handle, _ptr(logits), _ptr(scores_scratch), n, C.byref(cfg), _ptr(context), _ptr(ctx_range),
                                        ctx_begin, ctx_end, _ptr(eos_ids), n_eos, _ptr(rng_state), _ptr(result)))


class ModelWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("tok_emb", "attn_norm", "ffn_norm", "out_norm", "wq", "wk", "wv", "wo", "router",
                                          "gate", "up", "down", "lm_head")]


class Model:
    """Greedy decoder over device-resident Q4_K weights; the role of Executor (forward.rs:1239, 1795-1975)."""

    def __init__(self, ctx: Context, cfg: ModelCfg, weights: dict, ep=None):
        """ep = (world, rank, partial_ptrs, pad_ptrs): experts split over the ranks (weights hold this rank's experts),
        pointer tables as for moe_layer_q4k_ep with one token; every rank creates and drives its model together."""
        self.ctx, self.cfg, self._keep = ctx, cfg, (weights, ep)
        w = ModelWeights(**{k: _ptr(v) for k, v in weights.items()})
        h = C.c_void_p()
        if ep is None:
            ctx._check(ctx.lib.runit_model_create(ctx.handle, C.byref(cfg), C.byref(w), C.byref(h)))
        else:
            world, rank, partial_ptrs, pad_ptrs = ep
            ctx._check(ctx.lib.runit_model_create_ep(ctx.handle, C.byref(cfg), C.byref(w), world, rank, partial_ptrs, pad_ptrs, C.byref(h)))
        self.handle = h

    def forward_greedy(self, token_id: int, pos: int) -> int:
        nxt = C.c_int32(-1)
        self.ctx._check(self.ctx.lib.runit_model_forward_greedy(self.handle, token_id, pos, C.byref(nxt)))
        return nxt.value

    def generate_greedy(self, prompt, n_gen: int, start_pos: int = 0, skip_prompt_logits: bool = True) -> np.ndarray:
        prompt = np.ascontiguousarray(prompt, np.int32)
        out = np.empty(len(prompt) + n_gen, np.int32)
        self.ctx._check(self.ctx.lib.runit_model_generate_greedy(
            self.handle, prompt.ctypes.data_as(C.POINTER(C.c_int32)), len(prompt), n_gen, start_pos,
            int(skip_prompt_logits), out.ctypes.data_as(C.POINTER(C.c_int32))))
        return out

    def generate_sampled(self, prompt, n_gen: int, cfg: SamplerCfg, seed: int, eos_ids=(), start_pos: int = 0) -> np.ndarray:
        """The generate loop of generate.rs:299-350 with the sampler on the device."""
        prompt = np.ascontiguousarray(prompt, np.int32)
        eos = np.ascontiguousarray(np.asarray(eos_ids, np.int32))
        out = np.empty(len(prompt) + n_gen, np.int32)
        self.ctx._check(self.ctx.lib.runit_model_generate_sampled(
            self.handle, prompt.ctypes.data_as(C.POINTER(C.c_int32)), len(prompt), n_gen, start_pos, C.byref(cfg), seed,
            eos.ctypes.data_as(C.POINTER(C.c_int32)), len(eos), out.ctypes.data_as(C.POINTER(C.c_int32))))
        return out

    def prefill(self, tokens) -> int:
        """Executor::prefill (prefill.rs:29-255): batched pass over the prompt from an empty cache; returns the next token."""
        tokens = np.ascontiguousarray(tokens, np.int32)
        nxt = C.c_int32(-1)
        self.ctx._check(self.ctx.lib.runit_model_prefill(self.handle, tokens.ctypes.data_as(C.POINTER(C.c_int32)), len(tokens), C.byref(nxt)))
        return nxt.value

    def logits(self) -> np.ndarray:
        out = np.empty(self.cfg.vocab, np.float32)
        p = self.ctx.lib.runit_model_logits(self.handle)
        self.ctx._check(self.ctx.lib.runit_memcpy_d2h(self.ctx.handle, out.ctypes.data, p, out.nbytes))
        self.ctx.flush()
        return out

    @property
    def launches_per_token(self) -> int:
        return self.ctx.lib.runit_model_launches_per_token(self.handle)

    def close(self):
        if self.handle:
            self.ctx.lib.runit_model_destroy(self.handle)
            self.handle = None


def moe_scratch_bytes(ctx: Context, T: int, h: int, ff: int, E: int, k: int) -> int:
    return ctx.lib.runit_moe_scratch_bytes(T, h, ff, E, k)


def moe_grouped_scratch_bytes(ctx: Context, T: int, h: int, ff: int, E: int, k: int) -> int:
    return ctx.lib.runit_moe_grouped_scratch_bytes(T, h, ff, E, k)


def moe_layer_q4k_bf16_host(ctx: Context, router, gate, up, down, x, *, h, ff, E, top_k, renorm=False, residual=None,
                            routing=None):
    """Convenience for tests: upload host arrays, run the batched tensor-core block once, download
    (out [T][h], idx [T][k], weights [T][k]).  routing=(idx, w) skips the router and uses the given routing."""
    x = np.ascontiguousarray(x, np.float32).reshape(-1, h)
    T = x.shape[0]
    gate, up, down, xb = (ctx.buffer_from(np.ascontiguousarray(a)) for a in (gate, up, down, x))
    res = None if residual is None else ctx.buffer_from(np.ascontiguousarray(residual, np.float32))
    out = ctx.new_buffer(T * h * 4)
    nbytes = moe_grouped_scratch_bytes(ctx, T, h, ff, E, top_k)
    scratch = ctx.new_buffer(nbytes)
    if routing is None:
        rb = ctx.buffer_from(np.ascontiguousarray(router, np.float32))
        idx, w = ctx.new_buffer(T * top_k * 4), ctx.new_buffer(T * top_k * 4)
        ctx.call("moe_layer_q4k_bf16", rb, gate, up, down, xb, res, out, idx, w, scratch, nbytes, T, h, ff, E, top_k, int(renorm))
    else:
        idx = ctx.buffer_from(np.ascontiguousarray(routing[0], np.int32))
        w = ctx.buffer_from(np.ascontiguousarray(routing[1], np.float32))
        ctx.call("moe_experts_grouped_q4k_bf16", gate, up, down, xb, idx, w, res, out, scratch, nbytes, T, h, ff, E, top_k)
    ctx.flush()
    return (out.download(np.float32, T * h).reshape(T, h), idx.download(np.int32, T * top_k).reshape(T, top_k),
            w.download(np.float32, T * top_k).reshape(T, top_k))


def moe_layer_q4k_host(ctx: Context, router, gate, up, down, x, *, h, ff, E, top_k, renorm=False, residual=None):
    """Convenience for tests: upload host arrays, run runit_moe_layer_q4k once, download
    (out [T][h], idx [T][k], weights [T][k])."""
    x = np.ascontiguousarray(x, np.float32).reshape(-1, h)
    T = x.shape[0]
    bufs = [ctx.buffer_from(np.ascontiguousarray(a)) for a in (np.asarray(router, np.float32), gate, up, down, x)]
    res = None if residual is None else ctx.buffer_from(np.ascontiguousarray(residual, np.float32))
    out, idx, w = ctx.new_buffer(T * h * 4), ctx.new_buffer(T * top_k * 4), ctx.new_buffer(T * top_k * 4)
    nbytes = moe_scratch_bytes(ctx, T, h, ff, E, top_k)
    scratch = ctx.new_buffer(nbytes)
    ctx.call("moe_layer_q4k", *bufs, res, out, idx, w, scratch, nbytes, T, h, ff, E, top_k, int(renorm))
    ctx.flush()
    return (out.download(np.float32, T * h).reshape(T, h), idx.download(np.int32, T * top_k).reshape(T, top_k),
            w.download(np.float32, T * top_k).reshape(T, top_k))


__all__ = ["Context", "DeviceBuffer", "Graph", "KernelError", "Model", "ModelCfg", "ModelWeights", "SamplerCfg", "sample_f32", "sampler_seed_state", "gemv_batched_multi_f32", "moe_scratch_bytes", "moe_layer_q4k_host", "moe_grouped_scratch_bytes", "moe_layer_q4k_bf16_host", "row_bytes", "BLOCK_ELEMS", "BLOCK_BYTES",
           "FMT_Q8_0", "FMT_Q4_0", "FMT_Q4K", "FMT_Q5_0", "FMT_Q5K", "FMT_Q6K"] + [n for n, _ in _TWINS]
