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

import os

import numpy as np

# The kernels here reach peer memory with plain loads and stores only.  Left to its default, torch binds symmetric
# memory to an NVLink multicast object as well; a rank that exits while bound to one can raise NVLink faults on the
# other ranks' GPUs, so the binding is switched off before the first rendezvous (NCCL's in-switch reduction likewise).
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")


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
    `sharded_gemv`.

    Two output vectors alternate from call to call.  Passing barrier n only means that every rank has ANNOUNCED epoch
    n, not that it has finished reading the result of call n, so a fast rank's call n+1 must not write where a slow
    rank still reads: it writes the other vector.  The vector of call n is written again by call n+2, which a rank can
    only reach after barrier n+1, and every rank announces n+1 in stream order after its own reads of result n."""

    def __init__(self, R, ctx, torch, dist, fmt, w_local, rows_total, k, world, rank):
        import ctypes as C
        import torch.distributed._symmetric_memory as symm
        self.R, self.ctx, self.torch, self.C = R, ctx, torch, C
        self.fmt, self.w, self.rows_total, self.k, self.world, self.rank = fmt, w_local, rows_total, k, world, rank
        self.y = symm.empty(2 * rows_total, dtype=torch.float32, device="cuda")
        self.pad = symm.empty(64, dtype=torch.int32, device="cuda")
        self.pad.zero_()
        torch.cuda.synchronize()
        group = dist.group.WORLD
        self._hy = symm.rendezvous(self.y, group)
        self._hp = symm.rendezvous(self.pad, group)
        base = [int(p) for p in self._hy.buffer_ptrs]
        self.y_ptrs = [(C.c_void_p * world)(*[b + half * 4 * rows_total for b in base]) for half in (0, 1)]
        self.pad_ptrs = (C.c_void_p * world)(*[int(p) for p in self._hp.buffer_ptrs])
        self.epoch = 0
        dist.barrier()        # every pad is zero and mapped before the first flag is written
        torch.cuda.synchronize()

    def __call__(self, x):
        """Returns this rank's full-length output vector of this call (valid once the stream has passed the barrier
        kernel; it stays untouched until the call after the next one)."""
        self.epoch += 1
        half = self.epoch & 1
        self.R.gemv_allgather_f32(self.ctx, self.fmt, self.w, x, self.y_ptrs[half], self.world, self.rank, self.rows_total, self.k)
        self.R.peer_barrier(self.ctx, self.pad_ptrs, self.world, self.rank, self.epoch)
        return self.y[half * self.rows_total:(half + 1) * self.rows_total]


class FusedGreedyLmHead:
    """Row-sharded greedy lm_head: every rank multiplies its rows, finds its own (largest logit, global row) pair in the
    GEMV's epilogue and stores the 8 bytes into every rank's pair table (peer stores into symmetric memory); one barrier
    kernel, whose warp then reduces the `world` pairs to the token.  8 bytes per rank cross NVLink instead of the logits.
    Two pair tables alternate from call to call, for the reason given in FusedAllGatherGemv."""

    def __init__(self, R, ctx, torch, dist, fmt, w_local, rows_total, k, world, rank):
        import ctypes as C
        import torch.distributed._symmetric_memory as symm
        self.R, self.ctx, self.torch = R, ctx, torch
        self.fmt, self.w, self.rows_total, self.k, self.world, self.rank = fmt, w_local, rows_total, k, world, rank
        self.pairs = symm.empty(2 * 2 * 8, dtype=torch.int32, device="cuda")     # two tables of 8 (value bits, index) pairs
        self.pad = symm.empty(64, dtype=torch.int32, device="cuda")
        self.pairs.zero_()
        self.pad.zero_()
        torch.cuda.synchronize()
        group = dist.group.WORLD
        self._hq = symm.rendezvous(self.pairs, group)
        self._hp = symm.rendezvous(self.pad, group)
        base = [int(p) for p in self._hq.buffer_ptrs]
        self.pair_ptrs = [(C.c_void_p * world)(*[b + half * 64 for b in base]) for half in (0, 1)]
        self.pad_ptrs = (C.c_void_p * world)(*[int(p) for p in self._hp.buffer_ptrs])
        self.logits_local = torch.empty(rows_total // world, dtype=torch.float32, device="cuda")
        self.token = torch.empty(1, dtype=torch.int32, device="cuda")
        self.epoch = 0
        dist.barrier()
        torch.cuda.synchronize()

    def __call__(self, x):
        """Returns the device word holding the token of this call (the same on every rank)."""
        self.epoch += 1
        half = self.epoch & 1
        self.R.gemv_argmax_allgather(self.ctx, self.fmt, self.w, x, self.logits_local, self.pair_ptrs[half], self.world, self.rank,
                                     self.rows_total, self.k)
        self.R.peer_barrier_argmax(self.ctx, self.pad_ptrs, self.world, self.rank, self.epoch, self.pairs.data_ptr() + half * 64, self.token)
        return self.token


class FusedEpPrefillMoe:
    """Expert-parallel MoE block for prefill-sized batches with the exchange done by the library's own kernels: every
    rank routes its T tokens, stores each (token, expert) row into the receive buffer of the expert's owner (peer stores
    into symmetric memory), the owners run the grouped tensor-core GEMMs over what they received and store the outputs
    back into the senders' slots; two barrier kernels, no host read, no collective library call.  The NCCL variant with
    torch indexing is `ep_moe_forward_counted`.  placement 1 puts expert e on rank e % world (spreads a popularity that
    falls with the expert index), 0 on rank e // (E / world)."""

    def __init__(self, R, ctx, torch, dist, router, gate_local, up_local, down_local, E, h, ff, k, renorm, world, rank, T, placement=0):
        import ctypes as C
        import torch.distributed._symmetric_memory as symm
        self.R, self.ctx, self.torch = R, ctx, torch
        self.w = (router, gate_local, up_local, down_local)
        self.E, self.h, self.ff, self.k, self.renorm, self.world, self.rank, self.T = E, h, ff, k, renorm, world, rank, T
        self.placement = placement
        S = T * k
        self.recv_rows = symm.empty(world * S * h, dtype=torch.bfloat16, device="cuda")
        self.recv_meta = symm.empty(world * S * 2, dtype=torch.int32, device="cuda")
        self.recv_counts = symm.empty(64, dtype=torch.int32, device="cuda")
        self.return_rows = symm.empty(S * h, dtype=torch.float32, device="cuda")
        self.pad = symm.empty(64, dtype=torch.int32, device="cuda")
        self.pad.zero_()
        self.recv_counts.zero_()
        torch.cuda.synchronize()
        group = dist.group.WORLD
        self._handles = [symm.rendezvous(t, group) for t in (self.recv_rows, self.recv_meta, self.recv_counts, self.return_rows, self.pad)]
        self.tables = [(C.c_void_p * world)(*[int(p) for p in hnd.buffer_ptrs]) for hnd in self._handles]
        self.scratch_bytes = ctx.lib.runit_moe_ep_prefill_scratch_bytes(T, h, ff, E, k, world)
        self.scratch = ctx.new_buffer(self.scratch_bytes)
        self.out = torch.empty(T, h, dtype=torch.float32, device="cuda")
        self.idx = torch.empty(T, k, dtype=torch.int32, device="cuda")
        self.wts = torch.empty(T, k, dtype=torch.float32, device="cuda")
        self.epoch = 0
        dist.barrier()
        torch.cuda.synchronize()

    def __call__(self, x, residual=None):
        """x: f32 [T][h], this rank's tokens.  Returns (out [T][h], idx [T][k], weights [T][k])."""
        assert x.shape[0] == self.T
        self.epoch += 1
        router, gate, up, down = self.w
        rows, meta, counts, ret, pads = self.tables
        self.R.moe_layer_q4k_bf16_ep(self.ctx, router, gate, up, down, x, residual, self.out, self.idx, self.wts, self.scratch,
                                     self.scratch_bytes, rows, meta, counts, ret, pads, self.T, self.h, self.ff, self.E, self.k,
                                     int(self.renorm), self.world, self.rank, self.epoch, self.placement)
        return self.out, self.idx, self.wts


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
