"""Single-node multi-GPU execution of the two parts of the path that shard: one process per GPU,
`torch.distributed` (NCCL over NVLink / NVSwitch on GPUs, gloo on CPU for the host-logic tests).

The reference is single-device (crates/engine/src/server/mod.rs:20-30 serialises everything behind one
Mutex<Executor>); both schemes below are new:

* row-sharded GEMV (lm_head): rank r owns rows [r*M/G, (r+1)*M/G) of the weight matrix, the input vector is
  replicated, the logits are all-gathered;
* expert-parallel MoE: rank r owns experts [r*E/G, (r+1)*E/G); tokens are data-parallel.  Every rank routes
  its own tokens, sends each (token, expert) slot to the expert's owner with ONE fixed-capacity all-to-all
  (no count exchange, hence no host synchronisation), the owner runs the expert FFN on the slots it received,
  a second all-to-all returns the results and the source adds them weighted in routing order.

All remote data lands in local memory through the collective before a kernel reads it.  The arithmetic is
supplied by a backend object so the same host logic runs on CPU in the tests (backend supplied by the test)
and on GPU (`CudaBackend`, C-ABI calls on torch tensors).
"""
from __future__ import annotations

import numpy as np


def shard_rows(m: int, world: int, rank: int):
    """(first row, row count) of `rank`; requires world | m (152064 and 50304 divide by 2, 4, 8)."""
    if m % world:
        raise ValueError("rows %d do not divide over %d ranks" % (m, world))
    n = m // world
    return rank * n, n


def expert_owner(expert_ids, n_experts: int, world: int):
    """Rank owning each expert id (contiguous blocks of n_experts/world)."""
    if n_experts % world:
        raise ValueError("experts %d do not divide over %d ranks" % (n_experts, world))
    return expert_ids // (n_experts // world)


def sharded_gemv(backend, dist, torch, x, rows_total: int, world: int, rank: int):
    """y = W.x with W row-sharded: local product + all-gather.  backend.local_gemv(x) -> [rows_total/world]."""
    _, n = shard_rows(rows_total, world, rank)
    y_local = backend.local_gemv(x)
    assert y_local.numel() == n
    y = torch.empty(rows_total, dtype=y_local.dtype, device=y_local.device)
    if world > 1:
        dist.all_gather_into_tensor(y, y_local.contiguous())
    else:
        y.copy_(y_local)
    return y


def ep_pack(torch, idx, n_experts: int, world: int):
    """Placement of the local (token, expert) slots in the fixed-capacity send buffer.

    idx: [T, k] expert ids.  Returns (dest [T*k], pos [T*k], cap) with slot s = t*k+i going to row
    dest[s]*cap + pos[s] of a [world*cap] buffer; pos counts the slots already sent to that destination in
    slot order (deterministic)."""
    T, k = idx.shape
    cap = T * k
    flat = idx.reshape(-1).to(torch.int64)
    dest = expert_owner(flat, n_experts, world)
    onehot = torch.nn.functional.one_hot(dest, world)                       # [S, world]
    pos = (torch.cumsum(onehot, 0) - onehot).gather(1, dest[:, None])[:, 0]  # exclusive running count per destination
    return dest, pos, cap


def ep_moe_forward(backend, dist, torch, x, n_experts: int, top_k: int, renorm: bool, world: int, rank: int, residual=None):
    """Expert-parallel MoE block for this rank's tokens x [T, h] (f32).  Returns (out [T, h], idx, w).

    backend.route(x) -> (idx int32 [T,k], w f32 [T,k]); backend.experts(x_slots [n,h], local_expert int32 [n])
    -> y [n,h] (rows with local_expert < 0 are ignored)."""
    T, h = x.shape
    idx, w = backend.route(x)
    dest, pos, cap = ep_pack(torch, idx, n_experts, world)
    per_rank = n_experts // world
    row = dest * cap + pos
    send_x = torch.zeros(world * cap, h, dtype=x.dtype, device=x.device)
    send_e = torch.full((world * cap,), -1, dtype=torch.int32, device=x.device)
    tok = torch.arange(T * top_k, device=x.device) // top_k
    send_x[row] = x[tok]
    send_e[row] = (idx.reshape(-1).to(torch.int64) - dest * per_rank).to(torch.int32)   # expert id local to its owner
    if world > 1:
        recv_x, recv_e = torch.empty_like(send_x), torch.empty_like(send_e)
        dist.all_to_all_single(recv_x, send_x)
        dist.all_to_all_single(recv_e, send_e)
    else:
        recv_x, recv_e = send_x, send_e
    y = backend.experts(recv_x, recv_e)
    if world > 1:
        back = torch.empty_like(y)
        dist.all_to_all_single(back, y.contiguous())
    else:
        back = y
    ys = back[row].reshape(T, top_k, h)
    out = torch.zeros(T, h, dtype=x.dtype, device=x.device) if residual is None else residual.clone()
    acc = torch.zeros(T, h, dtype=x.dtype, device=x.device)
    for i in range(top_k):            # routing order, like scale_accumulate in forward.rs:1667-1676
        acc = acc + w[:, i:i + 1] * ys[:, i, :]
    return out + acc, idx, w


def ep_moe_forward_counted(backend, dist, torch, x, n_experts: int, top_k: int, renorm: bool, world: int, rank: int,
                           residual=None):
    """The same block for prefill-sized batches: slots are sorted by destination rank and exchanged with their true
    counts (one small all-to-all of counts and one host read of them per call), so no padding crosses NVLink and the
    owner computes only real slots.  Returns (out [T, h], idx, w)."""
    T, h = x.shape
    idx, w = backend.route(x)
    per_rank = n_experts // world
    flat = idx.reshape(-1).to(torch.int64)
    dest = expert_owner(flat, n_experts, world)
    order = torch.argsort(dest, stable=True)                      # slots grouped by destination, slot order kept
    send_counts = torch.bincount(dest, minlength=world)
    recv_counts = torch.empty_like(send_counts)
    if world > 1:
        dist.all_to_all_single(recv_counts, send_counts)
    else:
        recv_counts.copy_(send_counts)
    sc, rc = send_counts.tolist(), recv_counts.tolist()            # the one host synchronisation
    tok = torch.arange(T * top_k, device=x.device) // top_k
    send_x = x[tok[order]].contiguous()
    send_e = (flat[order] - dest[order] * per_rank).to(torch.int32)
    n_recv = int(sum(rc))
    recv_x = torch.empty(n_recv, h, dtype=x.dtype, device=x.device)
    recv_e = torch.empty(n_recv, dtype=torch.int32, device=x.device)
    if world > 1:
        dist.all_to_all_single(recv_x, send_x, output_split_sizes=rc, input_split_sizes=sc)
        dist.all_to_all_single(recv_e, send_e, output_split_sizes=rc, input_split_sizes=sc)
    else:
        recv_x, recv_e = send_x, send_e
    y = backend.experts(recv_x, recv_e) if n_recv else recv_x
    back = torch.empty(T * top_k, h, dtype=x.dtype, device=x.device)
    if world > 1:
        dist.all_to_all_single(back, y.contiguous(), output_split_sizes=sc, input_split_sizes=rc)
    else:
        back = y
    ys = torch.empty_like(back)
    ys[order] = back                                               # back to slot order
    ys = ys.reshape(T, top_k, h)
    acc = torch.zeros(T, h, dtype=x.dtype, device=x.device)
    for i in range(top_k):                                         # routing order
        acc = acc + w[:, i:i + 1] * ys[:, i, :]
    base = torch.zeros(T, h, dtype=x.dtype, device=x.device) if residual is None else residual
    return base + acc, idx, w


# ───────────────────────── GPU backend (C-ABI calls on torch tensors) ─────────────────────────

class CudaBackend:
    """Arithmetic of the two schemes on the local GPU through librunit_cuda.so."""

    def __init__(self, R, ctx, torch, grouped_min_slots=1 << 30):
        self.R, self.ctx, self.torch = R, ctx, torch
        self.grouped_min_slots = grouped_min_slots   # slot count from which the tensor-core block serves the experts
        self._scratch = self._ones = None

    # row-sharded GEMV
    def set_lm_head(self, fmt, w_local, rows_local, k):
        self.fmt, self.w_local, self.rows_local, self.k = fmt, w_local, rows_local, k
        self.y_local = self.torch.empty(rows_local, dtype=self.torch.float32, device="cuda")

    def local_gemv(self, x):
        name = {0: "q8_0", 1: "q4_0", 2: "q4k"}[self.fmt]
        getattr(self.R, "gemv_%s_f32in_f32out" % name)(self.ctx, self.w_local, x, self.y_local, self.rows_local, self.k)
        return self.y_local

    # expert parallel
    def set_experts(self, router, gate, up, down, n_experts, n_local, h, ff, top_k, renorm):
        self.router, self.gate, self.up, self.down = router, gate, up, down
        self.E, self.n_local, self.h, self.ff, self.top_k, self.renorm = n_experts, n_local, h, ff, top_k, renorm

    def route(self, x):
        t, T = self.torch, x.shape[0]
        logits = t.empty(T, self.E, dtype=t.float32, device="cuda")
        idx = t.empty(T, self.top_k, dtype=t.int32, device="cuda")
        w = t.empty(T, self.top_k, dtype=t.float32, device="cuda")
        self.R.moe_router_f32(self.ctx, self.router, x, logits, self.E, self.h, T)
        self.R.moe_route_topk(self.ctx, logits, 0, self.E, self.top_k, int(self.renorm), T, idx, w)
        return idx, w

    def experts(self, x_slots, local_expert):
        """Slots received from all ranks -> expert outputs.  Few slots: grouped GEMV (f32).  grouped_min_slots or more:
        the tensor-core block (bf16 operands) with one slot per "token" (k = 1, weight 1)."""
        t, n = self.torch, x_slots.shape[0]
        y = t.zeros(n, self.h, dtype=t.float32, device="cuda")
        if n >= self.grouped_min_slots:
            nbytes = self.R.moe_grouped_scratch_bytes(self.ctx, n, self.h, self.ff, self.n_local, 1)
            if self._scratch is None or self._scratch.nbytes < nbytes:
                self._scratch = self.ctx.new_buffer(nbytes)
            if self._ones is None or self._ones.numel() < n:
                self._ones = t.ones(n, dtype=t.float32, device="cuda")
            self.R.moe_experts_grouped_q4k_bf16(self.ctx, self.gate, self.up, self.down, x_slots.contiguous(), local_expert.contiguous(),
                                                self._ones, None, y, self._scratch, self._scratch.nbytes, n, self.h, self.ff,
                                                self.n_local, 1)
            return y
        act = t.empty(n, self.ff, dtype=t.float32, device="cuda")
        self.R.moe_experts_q4k(self.ctx, self.gate, self.up, self.down, x_slots, local_expert, y, act, n, self.h, self.ff, self.n_local)
        return y


class FusedAllGatherGemv:
    """Row-sharded GEMV whose all-gather happens in the kernel's epilogue: every rank stores its slice of the output
    straight into the output vectors of all ranks (peer stores over NVLink into symmetric memory) and one small
    barrier kernel announces completion; no collective library call on the data path.  The NCCL variant is
    `sharded_gemv`."""

    def __init__(self, R, ctx, torch, dist, fmt, w_local, rows_total, k, world, rank):
        import ctypes as C
        import torch.distributed._symmetric_memory as symm
        self.R, self.ctx, self.torch, self.C = R, ctx, torch, C
        self.fmt, self.w, self.rows_total, self.k, self.world, self.rank = fmt, w_local, rows_total, k, world, rank
        self.y = symm.empty(rows_total, dtype=torch.float32, device="cuda")
        self.pad = symm.empty(64, dtype=torch.int32, device="cuda")
        self.pad.zero_()
        torch.cuda.synchronize()
        group = dist.group.WORLD
        self._hy = symm.rendezvous(self.y, group)
        self._hp = symm.rendezvous(self.pad, group)
        self.y_ptrs = (C.c_void_p * world)(*[int(p) for p in self._hy.buffer_ptrs])
        self.pad_ptrs = (C.c_void_p * world)(*[int(p) for p in self._hp.buffer_ptrs])
        self.epoch = 0
        dist.barrier()        # every pad is zero and mapped before the first flag is written
        torch.cuda.synchronize()

    def __call__(self, x):
        """Returns this rank's full-length output vector (valid once the stream has passed the barrier kernel)."""
        self.epoch += 1
        # ranks may be an epoch apart: the barrier at the end of call n also keeps call n+1 of a fast rank from
        # overwriting a vector that a slow rank is still reading, as long as the caller consumes y before the next call
        self.R.gemv_allgather_f32(self.ctx, self.fmt, self.w, x, self.y_ptrs, self.world, self.rank, self.rows_total, self.k)
        self.R.peer_barrier(self.ctx, self.pad_ptrs, self.world, self.rank, self.epoch)
        return self.y


class FusedEpDecodeMoe:
    """Expert-parallel MoE block for decode sizes with replicated tokens: every rank routes the tokens itself, runs the
    experts it owns and stores its weighted partial sums into every rank's buffer (peer stores into symmetric memory);
    one barrier kernel, then each rank adds the partials in rank order.  No collective library call on the data path;
    all ranks end with identical bits.  The NCCL variant (tokens data-parallel, three all-to-alls) is `ep_moe_forward`."""

    def __init__(self, R, ctx, torch, dist, router, gate_local, up_local, down_local, E, h, ff, k, renorm, world, rank, max_tokens=16):
        import ctypes as C
        import torch.distributed._symmetric_memory as symm
        self.R, self.ctx, self.torch = R, ctx, torch
        self.w = (router, gate_local, up_local, down_local)
        self.E, self.h, self.ff, self.k, self.renorm, self.world, self.rank, self.max_tokens = E, h, ff, k, renorm, world, rank, max_tokens
        self.partial = symm.empty(2 * world * max_tokens * h, dtype=torch.float32, device="cuda")
        self.pad = symm.empty(64, dtype=torch.int32, device="cuda")
        self.pad.zero_()
        torch.cuda.synchronize()
        group = dist.group.WORLD
        self._hq = symm.rendezvous(self.partial, group)
        self._hp = symm.rendezvous(self.pad, group)
        self.partial_ptrs = (C.c_void_p * world)(*[int(p) for p in self._hq.buffer_ptrs])
        self.pad_ptrs = (C.c_void_p * world)(*[int(p) for p in self._hp.buffer_ptrs])
        self.scratch_bytes = R.moe_scratch_bytes(ctx, max_tokens, h, ff, E, k)
        self.scratch = ctx.new_buffer(self.scratch_bytes)
        self.out = torch.empty(max_tokens, h, dtype=torch.float32, device="cuda")
        self.idx = torch.empty(max_tokens, k, dtype=torch.int32, device="cuda")
        self.wts = torch.empty(max_tokens, k, dtype=torch.float32, device="cuda")
        self.epoch = 0
        dist.barrier()
        torch.cuda.synchronize()

    def __call__(self, x, residual=None):
        """x: f32 [T][h], the same on every rank.  Returns (out [T][h], idx [T][k], weights [T][k]) views."""
        T = x.shape[0]
        assert T <= self.max_tokens
        self.epoch += 1
        router, gate, up, down = self.w
        self.R.moe_layer_q4k_ep(self.ctx, router, gate, up, down, x, residual, self.out, self.idx, self.wts, self.scratch,
                                self.scratch_bytes, self.partial_ptrs, self.pad_ptrs, T, self.h, self.ff, self.E, self.k,
                                int(self.renorm), self.world, self.rank, self.epoch)
        return self.out[:T], self.idx[:T], self.wts[:T]


def _time_steps(torch, dist, stream, ctx, fn, steps, world):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        fn()
    e1.record(stream)
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / steps], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def bench_sharded_lm_head(R, ctx, torch, dist, stream, rank, world, steps=20):
    """Qwen2.5-7B lm_head (152064 x 3584), Q4_K and Q4_0, rows split over the ranks, logits all-gathered."""
    out = {}
    M, K = 152064, 3584
    _, n = shard_rows(M, world, rank)
    x = torch.randn(K, dtype=torch.float32, device="cuda")
    for fmt, name in ((2, "q4k"), (1, "q4_0")):
        be = CudaBackend(R, ctx, torch)
        rb = R.row_bytes(fmt, K)
        w = ctx.new_buffer(n * rb)
        R.fill_weights(ctx, fmt, w, n * (K // R.BLOCK_ELEMS[fmt]), 1002 + rank, 0.01)
        be.set_lm_head(fmt, w, n, K)
        ms = _time_steps(torch, dist, stream, ctx, lambda: sharded_gemv(be, dist, torch, x, M, world, rank), steps, world)
        ms_local = _time_steps(torch, dist, stream, ctx, lambda: be.local_gemv(x), steps, world)
        alg = M * rb + 4 * (K + M)
        out[name] = {"us_per_call": ms * 1e3, "us_local_gemv": ms_local * 1e3, "aggregate_gbs": alg / (ms * 1e-3) / 1e9,
                     "rows_per_rank": n}
        if world > 1:
            try:
                fused = FusedAllGatherGemv(R, ctx, torch, dist, fmt, w, M, K, world, rank)
                ms_f = _time_steps(torch, dist, stream, ctx, lambda: fused(x), steps, world)
                out[name].update({"us_per_call_fused_peer_stores": ms_f * 1e3, "aggregate_gbs_fused": alg / (ms_f * 1e-3) / 1e9})
            except Exception as exc:   # symmetric memory unavailable on this host: keep the NCCL figures
                out[name]["fused_unavailable"] = repr(exc)[:200]
        w.free()
    return out


def bench_expert_parallel(R, ctx, torch, dist, stream, rank, world, steps=10):
    """One OLMoE-shaped MoE layer (hidden 2048, 64 experts, top-8, intermediate 1024, Q4_K), experts split 64/G per
    rank, T tokens per rank."""
    E, h, ff, k = 64, 2048, 1024, 8
    n_local = E // world
    rb = lambda kk: kk // 256 * 144
    gate, up = ctx.new_buffer(n_local * ff * rb(h)), ctx.new_buffer(n_local * ff * rb(h))
    down = ctx.new_buffer(n_local * h * rb(ff))
    for i, (b, rows, kk) in enumerate(((gate, n_local * ff, h), (up, n_local * ff, h), (down, n_local * h, ff))):
        R.fill_weights(ctx, 2, b, rows * (kk // 256), 77 + i + 10 * rank, 0.01)
    router = torch.randn(E, h, dtype=torch.float32, device="cuda") * 0.02
    if world > 1:
        dist.broadcast(router, 0)
    be = CudaBackend(R, ctx, torch)
    be.set_experts(router, gate, up, down, E, n_local, h, ff, k, False)
    out = {}
    for T in (1, 16):
        x = torch.randn(T, h, dtype=torch.float32, device="cuda")
        ms = _time_steps(torch, dist, stream, ctx, lambda: ep_moe_forward(be, dist, torch, x, E, k, False, world, rank), steps, world)
        out["T%d_per_rank" % T] = {"us_per_layer": ms * 1e3, "tokens_per_s_all_ranks": world * T / (ms * 1e-3)}
    if world > 1:
        try:
            fused = FusedEpDecodeMoe(R, ctx, torch, dist, router, gate, up, down, E, h, ff, k, False, world, rank, max_tokens=16)
            for T in (1, 16):
                x = torch.randn(T, h, dtype=torch.float32, device="cuda")
                dist.broadcast(x, 0)
                ms = _time_steps(torch, dist, stream, ctx, lambda: fused(x), steps, world)
                out["T%d_replicated_fused_peer_stores" % T] = {"us_per_layer": ms * 1e3, "tokens_per_s": T / (ms * 1e-3)}
        except Exception as exc:   # symmetric memory unavailable on this host: keep the NCCL figures
            out["fused_unavailable"] = repr(exc)[:200]
    for b in (gate, up, down):
        b.free()
    out["qwen3_shape_prefill"] = bench_expert_parallel_prefill(R, ctx, torch, dist, stream, rank, world)
    return out


def bench_ep_decode(R, ctx, torch, dist, rank, world):
    """Full OLMoE-shaped greedy decode (16 layers, hidden 2048, 64 experts top-8, Q4_K, 128-token prompt + 64 steps) with
    the experts split 64/G per rank and the MoE combine fused over peer memory; attention, router, embeddings and lm_head
    are replicated (same seeds on every rank), every rank decodes the same token stream."""
    import ctypes as C
    import time
    import numpy as np
    import torch.distributed._symmetric_memory as symm
    L, h, E, ff, k, V = 16, 2048, 64, 1024, 8, 50304
    nl = E // world
    rb = lambda kk: kk // 256 * 144
    shapes = {"wq": (L * h, h), "wk": (L * h, h), "wv": (L * h, h), "wo": (L * h, h), "lm_head": (V, h),
              "gate": (L * nl * ff, h), "up": (L * nl * ff, h), "down": (L * nl * h, ff)}
    dev = {}
    for i, (name, (rows, kk)) in enumerate(shapes.items()):
        dev[name] = ctx.new_buffer(rows * rb(kk))
        seed = 90001 + i + (1000 * rank if name in ("gate", "up", "down") else 0)
        R.fill_weights(ctx, R.FMT_Q4K, dev[name], rows * (kk // 256), seed, 0.01)
    for name, n, sig in (("tok_emb", V * h, 0.02), ("router", L * E * h, 0.02)):
        dev[name] = ctx.new_buffer(4 * n)
        R.fill_normal_f32(ctx, dev[name], n, 4242 + len(name), sig)
    ones = np.ones(L * h, np.float32)
    dev["attn_norm"], dev["ffn_norm"], dev["out_norm"] = ctx.buffer_from(ones), ctx.buffer_from(ones), ctx.buffer_from(ones[:h])
    ctx.flush()
    partial = symm.empty(2 * world * h, dtype=torch.float32, device="cuda")
    pad = symm.empty(64, dtype=torch.int32, device="cuda")
    pad.zero_()
    torch.cuda.synchronize()
    hq, hp = symm.rendezvous(partial, dist.group.WORLD), symm.rendezvous(pad, dist.group.WORLD)
    pq = (C.c_void_p * world)(*[int(p) for p in hq.buffer_ptrs])
    pp = (C.c_void_p * world)(*[int(p) for p in hp.buffer_ptrs])
    dist.barrier()
    torch.cuda.synchronize()
    cfg = R.ModelCfg(n_layers=L, hidden=h, n_heads=16, n_kv_heads=16, head_dim=128, vocab=V, n_experts=E, top_k=k, ff=ff,
                     max_seq=2048, renorm=0, eps=1e-5, theta=10000.0)
    model = R.Model(ctx, cfg, dev, ep=(world, rank, pq, pp))
    prompt = np.random.default_rng(1004).integers(0, V, 128).astype(np.int32)
    dist.barrier()
    model.generate_greedy(prompt, 8)
    dist.barrier()
    t0 = time.perf_counter()
    toks = model.generate_greedy(prompt, 64)
    dt_all = time.perf_counter() - t0
    dist.barrier()
    t0 = time.perf_counter()
    model.generate_greedy(prompt, 0)
    dt_prompt = time.perf_counter() - t0
    t = torch.tensor([dt_all, dt_prompt], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    same = torch.tensor(toks[127:].astype(np.int64), device="cuda")
    ref = same.clone()
    dist.broadcast(ref, 0)
    agree = torch.tensor([int(torch.equal(same, ref))], device="cuda")
    dist.all_reduce(agree, op=dist.ReduceOp.MIN)
    dt_all, dt_prompt = float(t[0].item()), float(t[1].item())
    res = {"decode_tok_s": 64 / max(dt_all - dt_prompt, 1e-9), "prompt_tok_s": 128 / dt_prompt, "tokens_total_s": 192 / dt_all,
           "launches_per_token": int(model.launches_per_token), "experts_per_rank": nl, "ranks_agree_on_tokens": bool(agree.item()),
           "note": "one token stream over the whole group; wall clock (max over ranks) around one call of 192 recorded steps"}
    dist.barrier()
    model.close()
    for b in dev.values():
        b.free()
    return res


def bench_expert_parallel_prefill(R, ctx, torch, dist, stream, rank, world, steps=5, T_total=4096):
    """Qwen3-MoE-shaped batched block (hidden 2048, 128 experts, top-8, intermediate 768, Q4_K -> bf16 tensor-core
    GEMMs), 4096 tokens in all (4096/G per rank), experts split 128/G per rank, Zipf(1.1) expert popularity,
    count-exchanged all-to-all dispatch and combine.  Reports the straggler's load beside the mean."""
    E, h, ff, k = 128, 2048, 768, 8
    n_local, T = E // world, T_total // world
    rb = lambda kk: kk // 256 * 144
    gate, up = ctx.new_buffer(n_local * ff * rb(h)), ctx.new_buffer(n_local * ff * rb(h))
    down = ctx.new_buffer(n_local * h * rb(ff))
    for i, (b, rows, kk) in enumerate(((gate, n_local * ff, h), (up, n_local * ff, h), (down, n_local * h, ff))):
        R.fill_weights(ctx, 2, b, rows * (kk // 256), 177 + i + 10 * rank, 0.01)
    g = torch.Generator(device="cuda").manual_seed(1 + rank)
    p = 1.0 / torch.arange(1, E + 1, device="cuda", dtype=torch.float64) ** 1.1
    idx = torch.multinomial((p / p.sum()).float().expand(T, E).contiguous(), k, replacement=False, generator=g).to(torch.int32)
    w = torch.rand(T, k, device="cuda", generator=g)
    x = torch.randn(T, h, device="cuda", generator=g)

    class GivenRouting(CudaBackend):
        def route(self, _x):
            return idx, w
    be = GivenRouting(R, ctx, torch, grouped_min_slots=256)
    be.set_experts(None, gate, up, down, E, n_local, h, ff, k, False)
    ms = _time_steps(torch, dist, stream, ctx, lambda: ep_moe_forward_counted(be, dist, torch, x, E, k, False, world, rank), steps, world)
    recv = torch.bincount((idx // n_local).flatten().long(), minlength=world).to(torch.float64)
    if world > 1:
        dist.all_reduce(recv)
    return {"ms_per_layer": ms, "tokens_per_s_all_ranks": T_total / (ms * 1e-3), "tokens_per_rank": T,
            "slots_per_rank_max": float(recv.max().item()), "slots_per_rank_mean": float(recv.mean().item())}
