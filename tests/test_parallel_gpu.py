"""GPU check of the sharded paths through the C ABI: with one visible GPU the schemes run with world size 1
(same host logic, CUDA backend); with two or more GPUs two NCCL ranks are spawned (NVLS disabled, plain
collectives) and compared with the single-GPU MoE block and the oracle."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
H, FF, E, K_TOP = 512, 256, 8, 2
M_ROWS, K_IN = 256, 512


def make_data(O):
    rng = np.random.default_rng(321)
    return {"lm": O.rand_q4k(rng, M_ROWS, K_IN).reshape(-1), "router": rng.normal(0, 0.02, (E, H)).astype(np.float32),
            "gate": O.rand_q4k(rng, E * FF, H).reshape(-1), "up": O.rand_q4k(rng, E * FF, H).reshape(-1),
            "down": O.rand_q4k(rng, E * H, FF).reshape(-1), "x_lm": rng.normal(0, 1, K_IN).astype(np.float32),
            "x": rng.normal(0, 1, (8, H)).astype(np.float32)}


def run_rank(rank, world, port, q):
    import torch
    import torch.distributed as dist
    import oracle as O
    import runit_mac_b200 as R
    from runit_mac_b200 import parallel as P
    torch.cuda.set_device(rank)
    if world > 1:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    ctx = R.Context(rank, stream=stream.cuda_stream)
    d = make_data(O)
    be = P.CudaBackend(R, ctx, torch)
    rb_in, rb_h, rb_ff = O.row_bytes(O.Q4K, K_IN), O.row_bytes(O.Q4K, H), O.row_bytes(O.Q4K, FF)
    r0, n = P.shard_rows(M_ROWS, world, rank)
    be.set_lm_head(2, torch.from_numpy(d["lm"].reshape(M_ROWS, rb_in)[r0:r0 + n].copy()).cuda(), n, K_IN)
    y = P.sharded_gemv(be, dist, torch, torch.from_numpy(d["x_lm"]).cuda(), M_ROWS, world, rank)
    nl = E // world
    sl = lambda a, per: torch.from_numpy(a.reshape(E, per)[rank * nl:(rank + 1) * nl].copy()).cuda()
    be.set_experts(torch.from_numpy(d["router"]).cuda(), sl(d["gate"], FF * rb_h), sl(d["up"], FF * rb_h), sl(d["down"], H * rb_ff),
                   E, nl, H, FF, K_TOP, False)
    T = d["x"].shape[0] // world
    xs = torch.from_numpy(d["x"][rank * T:(rank + 1) * T]).cuda()
    out, idx, w = P.ep_moe_forward(be, dist, torch, xs, E, K_TOP, False, world, rank)
    torch.cuda.synchronize()
    ctx.flush()
    out_c, idx_c, _ = P.ep_moe_forward_counted(be, dist, torch, xs, E, K_TOP, False, world, rank)   # true-count exchange
    torch.cuda.synchronize()
    ctx.flush()
    assert torch.equal(idx_c, idx) and torch.allclose(out_c, out, rtol=1e-6, atol=1e-6 * float(out.abs().max()))
    y_fused = None
    if world > 1:
        # the same sharded product with the all-gather fused into the GEMV epilogue (peer stores + barrier kernel): four
        # calls in a row with a different input each and no host synchronisation between them (the two output vectors
        # alternate, so a rank that runs ahead cannot overwrite what a slower rank still reads); every call must give the
        # NCCL result bit for bit
        fused = P.FusedAllGatherGemv(R, ctx, torch, dist, 2, be.w_local, M_ROWS, K_IN, world, rank)
        xs_lm = [torch.from_numpy(d["x_lm"] * (1.0 + 0.5 * i)).cuda() for i in range(4)]
        want = [P.sharded_gemv(be, dist, torch, xi, M_ROWS, world, rank).clone() for xi in xs_lm]
        got = [fused(xi).clone() for xi in xs_lm]     # the clone is stream-ordered before the next call's barrier
        ctx.flush()
        for yf, yw in zip(got, want):
            assert torch.equal(yf, yw), "fused all-gather differs from the NCCL all-gather"
        assert torch.equal(want[0], y)
        y_fused = got[0].cpu().numpy()
    if world > 1:
        # greedy variant: every rank finds the (largest logit, row) pair of its slice in the GEMV's epilogue, 8 bytes per rank
        # are exchanged; four calls in a row with different inputs, each must give the argmax of the gathered logits
        greedy = P.FusedGreedyLmHead(R, ctx, torch, dist, 2, be.w_local, M_ROWS, K_IN, world, rank)
        toks = [greedy(xi).clone() for xi in xs_lm]
        ctx.flush()
        for tk, yw in zip(toks, want):
            assert int(tk.item()) == int(torch.argmax(yw).item()), "sharded greedy lm_head differs from argmax of the gathered logits"
    if world > 1:
        # prefill-size block with the library's own dispatch (peer stores, two barrier kernels): this rank's tokens through
        # the expert-parallel block, twice per placement, against the single-GPU batched block over all experts: same bits
        T2, rb2 = 96, O.row_bytes(O.Q4K, H)
        rngp = np.random.default_rng(77 + rank)
        xp = torch.from_numpy(rngp.normal(0, 1, (T2, H)).astype(np.float32)).cuda()
        resp = torch.from_numpy(rngp.normal(0, 1, (T2, H)).astype(np.float32)).cuda()
        full = {n: torch.from_numpy(d[n]).cuda() for n in ("gate", "up", "down")}
        router_t = torch.from_numpy(d["router"]).cuda()
        nbg = R.moe_grouped_scratch_bytes(ctx, T2, H, FF, E, K_TOP)
        sg = ctx.new_buffer(nbg)
        ref_out = torch.empty(T2, H, device="cuda")
        ref_idx = torch.empty(T2, K_TOP, dtype=torch.int32, device="cuda")
        R.moe_layer_q4k_bf16(ctx, router_t, full["gate"], full["up"], full["down"], xp, resp, ref_out, ref_idx, None, sg, nbg, T2, H, FF, E,
                             K_TOP, 0)
        ctx.flush()
        for placement in (0, 1):
            own = [e for e in range(E) if (e % world if placement else e // nl) == rank]
            pick = lambda a, per: torch.from_numpy(np.concatenate([a.reshape(E, per)[e] for e in own])).cuda()
            epp = P.FusedEpPrefillMoe(R, ctx, torch, dist, router_t, pick(d["gate"], FF * rb_h), pick(d["up"], FF * rb_h),
                                      pick(d["down"], H * rb_ff), E, H, FF, K_TOP, False, world, rank, T2, placement=placement)
            for _ in range(2):
                o, i_p, _w = epp(xp, resp)
                ctx.flush()
                assert torch.equal(i_p, ref_idx), "expert-parallel prefill block routes differently"
                assert torch.equal(o, ref_out), "expert-parallel prefill block differs from the single-GPU batched block"
            dist.barrier()
    out_ep = None
    if world > 1:
        # decode-size block with replicated tokens and the combine fused over peer memory: three calls in a row give the
        # same bits (the parent checks them against the oracle and that all ranks hold identical bits)
        ep = P.FusedEpDecodeMoe(R, ctx, torch, dist, torch.from_numpy(d["router"]).cuda(), sl(d["gate"], FF * rb_h), sl(d["up"], FF * rb_h),
                                sl(d["down"], H * rb_ff), E, H, FF, K_TOP, False, world, rank, max_tokens=d["x"].shape[0])
        x_all = torch.from_numpy(d["x"]).cuda()
        res_all = torch.from_numpy(d["x"][::-1].copy()).cuda()
        prev = None
        for _ in range(3):
            o, i_ep, _w = ep(x_all, res_all)
            ctx.flush()
            o = o.clone()
            assert prev is None or torch.equal(o, prev)
            prev = o
        out_ep = (o.cpu().numpy(), i_ep.cpu().numpy())
        dist.barrier()
        # hidden 512: the exchange as launches of its own; hidden 1024 with the opt-in exchange inside the GEMVs (partial sums
        # pushed by the down projection's epilogue, summed in the prologue of the next GEMV): the same launch count as one GPU
        out_ep = out_ep + ([ep_decode_tokens(R, P, O, ctx, torch, dist, world, rank, hidden) for hidden in (512, 1024)],)
    res = (rank, y.cpu().numpy(), out.cpu().numpy(), idx.cpu().numpy(), out_ep)
    if world > 1:
        dist.destroy_process_group()
    if q is not None:
        q.put(res)
    return res


def ep_decode_tokens(R, P, O, ctx, torch, dist, world, rank, hidden=512):
    """Small OLMoE-shaped decoder twice on this rank: all experts local, and experts split over the ranks with the
    fused peer-memory combine.  Returns both greedy token sequences."""
    import ctypes as C
    import torch.distributed._symmetric_memory as symm
    from test_decode_gpu import SMALL, rand_q4k_zero_mean
    c = dict(SMALL)
    c["hidden"] = hidden
    c["n_heads"] = hidden // c["head_dim"]
    L, h, E, ff, V = c["n_layers"], c["hidden"], c["n_experts"], c["ff"], c["vocab"]
    q_dim, kv_dim = c["n_heads"] * c["head_dim"], c["n_kv_heads"] * c["head_dim"]
    rb = lambda k: k // 256 * 144
    shapes = {"wq": (L * q_dim, h), "wk": (L * kv_dim, h), "wv": (L * kv_dim, h), "wo": (L * h, q_dim),
              "gate": (L * E * ff, h), "up": (L * E * ff, h), "down": (L * E * h, ff), "lm_head": (V, h)}
    rng = np.random.default_rng(21)          # same seed on every rank: replicated weights
    host = {n: rand_q4k_zero_mean(O, rng, rows, k).reshape(-1) for n, (rows, k) in shapes.items()}
    host.update({"tok_emb": rng.normal(0, 0.02, (V, h)).astype(np.float32), "attn_norm": np.ones((L, h), np.float32),
                 "ffn_norm": np.ones((L, h), np.float32), "out_norm": np.ones(h, np.float32),
                 "router": rng.normal(0, 0.02, (L, E, h)).astype(np.float32)})
    prompt = np.random.default_rng(22).integers(0, V, 8).astype(np.int32)
    full = R.Model(ctx, R.ModelCfg(**c), {n: ctx.buffer_from(a) for n, a in host.items()})
    tok_full = full.generate_greedy(prompt, 24)
    full.close()
    nl = E // world
    local = dict(host)
    for n, per in (("gate", ff * rb(h)), ("up", ff * rb(h)), ("down", h * rb(ff))):
        local[n] = np.ascontiguousarray(host[n].reshape(L, E, per)[:, rank * nl:(rank + 1) * nl]).reshape(-1)
    partial = symm.empty(2 * world * h, dtype=torch.float32, device="cuda")
    pad = symm.empty(64, dtype=torch.int32, device="cuda")
    pad.zero_()
    torch.cuda.synchronize()
    hq, hp = symm.rendezvous(partial, dist.group.WORLD), symm.rendezvous(pad, dist.group.WORLD)
    pq = (C.c_void_p * world)(*[int(p) for p in hq.buffer_ptrs])
    pp = (C.c_void_p * world)(*[int(p) for p in hp.buffer_ptrs])
    dist.barrier()
    torch.cuda.synchronize()
    ctx.set_tuning("ep_fused_exchange", 1 if hidden == 1024 else 0)     # read when the model is created
    model = R.Model(ctx, R.ModelCfg(**c), {n: ctx.buffer_from(a) for n, a in local.items()}, ep=(world, rank, pq, pp))
    ctx.set_tuning("ep_fused_exchange", 0)
    dist.barrier()
    tok_ep = model.generate_greedy(prompt, 24)
    tok_ep2 = model.generate_greedy(prompt, 24)       # a second run on the same model: epochs keep growing
    assert (tok_ep == tok_ep2).all()
    lpt = int(model.launches_per_token)
    # the single-GPU decoder's count for the same shape: 1 + L * (q|k|v, attention, o-proj, [norm,] MoE block) + 2
    lpt_one = 1 + L * (3 + (3 if hidden in (1024, 2048, 4096) else 6)) + 2
    dist.barrier()
    model.close()
    return tok_full, tok_ep, lpt, lpt_one


def test_sharded_paths_match_oracle(oracle):
    import torch
    O = oracle
    world = 2 if torch.cuda.device_count() >= 2 else 1
    if world == 1:
        res = [run_rank(0, 1, 0, None)]
    else:
        import torch.multiprocessing as mp
        s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
        ctxm = mp.get_context("spawn")
        q = ctxm.Queue()
        procs = [ctxm.Process(target=run_rank, args=(r, world, port, q)) for r in range(world)]
        for p in procs:
            p.start()
        try:
            res = sorted([q.get(timeout=300) for _ in range(world)], key=lambda t: t[0])
            for p in procs:
                p.join(timeout=60)
                assert p.exitcode == 0
        finally:
            # whatever failed (an assert in one child, a time-out here), no child is left behind inside a collective
            for p in procs:
                if p.is_alive():
                    p.terminate()
            for p in procs:
                p.join(timeout=30)
    d = make_data(O)
    full = O.gemv(O.Q4K, d["lm"], d["x_lm"], M_ROWS, K_IN)
    for r in res:
        st = O.compare(full, r[1], rel_tol=1e-3)
        assert st.n_mismatch_rel == 0, st
    ref, ridx, _ = O.moe_layer_q4k(d["router"], d["gate"], d["up"], d["down"], d["x"], h=H, ff=FF, E=E, top_k=K_TOP, renorm=False)
    out = np.concatenate([r[2] for r in res])
    idx = np.concatenate([r[3] for r in res])
    assert (idx == ridx).all()
    st = O.compare(ref, out, rel_tol=1e-3)
    assert st.n_mismatch_rel == 0, st
    if world > 1:
        ref_res = ref + d["x"][::-1]
        for r in res:
            assert (r[4][1] == ridx).all()
            st = O.compare(ref_res, r[4][0], rel_tol=1e-3)
            assert st.n_mismatch_rel == 0, st
            assert np.array_equal(r[4][0], res[0][4][0]), "ranks disagree on the bits of the fused expert-parallel block"
            for case, (tok_full, tok_ep, lpt, lpt_one) in enumerate(r[4][2]):
                assert (tok_ep == tok_full).all(), ("expert-parallel decode differs from the single-GPU decode", case, tok_full, tok_ep)
                assert (tok_ep == res[0][4][2][case][1]).all() and len(set(tok_ep[7:].tolist())) > 3
                # hidden 512: the exchange costs launches; hidden 1024: none
                assert (lpt > lpt_one) if case == 0 else (lpt == lpt_one), (case, lpt, lpt_one)


def test_partitioned_kernels_with_one_rank(ctx, oracle):
    """The kernels of the partitioned paths with a group of one (every "peer" table points at this GPU's own buffers), so
    that a single-GPU run still executes them: the greedy lm_head (pair pushed into the own table, barrier kernel that
    reduces it) and the expert-parallel prefill block (dispatch, counts, barrier, grouped GEMMs with the return fused into
    the epilogue, barrier, weighted sum), each against its single-GPU counterpart."""
    import ctypes as C
    import torch
    import runit_mac_b200 as R
    O = oracle
    d = make_data(O)
    tab = lambda t: (C.c_void_p * 1)(t.data_ptr())
    # greedy lm_head
    w = torch.from_numpy(d["lm"]).cuda()
    x = torch.from_numpy(d["x_lm"]).cuda()
    logits = torch.empty(M_ROWS, device="cuda")
    pairs = torch.zeros(16, dtype=torch.int32, device="cuda")
    pad = torch.zeros(64, dtype=torch.int32, device="cuda")
    tok = torch.full((4,), -1, dtype=torch.int32, device="cuda")
    for epoch in (1, 2, 3):
        R.gemv_argmax_allgather(ctx, 2, w, x, logits, tab(pairs), 1, 0, M_ROWS, K_IN)
        R.peer_barrier_argmax(ctx, tab(pad), 1, 0, epoch, pairs, tok)
        ctx.flush()
        assert int(tok[0].item()) == int(torch.argmax(logits).item())
    st = O.compare(O.gemv(O.Q4K, d["lm"], d["x_lm"], M_ROWS, K_IN), logits.cpu().numpy(), rel_tol=1e-3)
    assert st.n_mismatch_rel == 0, st
    # expert-parallel prefill block, world = 1, against the plain batched block: same bits
    T = 80
    rng = np.random.default_rng(9)
    xp = torch.from_numpy(rng.normal(0, 1, (T, H)).astype(np.float32)).cuda()
    res = torch.from_numpy(rng.normal(0, 1, (T, H)).astype(np.float32)).cuda()
    router = torch.from_numpy(d["router"]).cuda()
    gate, up, down = (torch.from_numpy(d[n]).cuda() for n in ("gate", "up", "down"))
    nbg = R.moe_grouped_scratch_bytes(ctx, T, H, FF, E, K_TOP)
    sg = ctx.new_buffer(nbg)
    ref_out = torch.empty(T, H, device="cuda")
    ref_idx = torch.empty(T, K_TOP, dtype=torch.int32, device="cuda")
    R.moe_layer_q4k_bf16(ctx, router, gate, up, down, xp, res, ref_out, ref_idx, None, sg, nbg, T, H, FF, E, K_TOP, 0)
    S = T * K_TOP
    rows = torch.empty(S * H, dtype=torch.bfloat16, device="cuda")
    meta = torch.empty(S * 2, dtype=torch.int32, device="cuda")
    cnt = torch.zeros(64, dtype=torch.int32, device="cuda")
    ret = torch.empty(S * H, dtype=torch.float32, device="cuda")
    pad2 = torch.zeros(64, dtype=torch.int32, device="cuda")
    nb = ctx.lib.runit_moe_ep_prefill_scratch_bytes(T, H, FF, E, K_TOP, 1)
    scratch = ctx.new_buffer(nb)
    out = torch.empty(T, H, device="cuda")
    idx = torch.empty(T, K_TOP, dtype=torch.int32, device="cuda")
    for epoch in (1, 2):
        for placement in (0, 1):
            R.moe_layer_q4k_bf16_ep(ctx, router, gate, up, down, xp, res, out, idx, None, scratch, nb, tab(rows), tab(meta), tab(cnt),
                                    tab(ret), tab(pad2), T, H, FF, E, K_TOP, 0, 1, 0, 2 * epoch - 1 + placement, placement)
            ctx.flush()
            assert torch.equal(idx, ref_idx) and torch.equal(out, ref_out)


def test_peer_barrier_times_out_without_a_peer(ctx):
    """Failure detection without a fault: a two-rank barrier whose second rank never signals (its flag word is a
    local buffer nothing writes) gives up after its time limit; the next flush reports the time-out and the
    context keeps working."""
    import ctypes as C
    import runit_mac_b200 as R
    pads = [ctx.new_buffer(256), ctx.new_buffer(256)]
    for p in pads:
        p.upload(np.zeros(64, np.uint32))
    table = (C.c_void_p * 2)(pads[0].ptr, pads[1].ptr)
    import time
    t0 = time.perf_counter()
    R.peer_barrier(ctx, table, 2, 0, 1)
    with pytest.raises(R.KernelError) as e:
        ctx.flush()
    one_limit = time.perf_counter() - t0
    assert "TIMEOUT" in str(e.value)
    assert pads[1].download(np.uint32, 2)[0] == 1          # our own announcement did reach the peer's pad
    # the give-up is sticky on the device: a queue of barriers behind the missing rank costs about ONE time limit,
    # not one each (a recorded decode step holds one barrier per layer), and each still announces its epoch
    t0 = time.perf_counter()
    for epoch in range(2, 10):
        R.peer_barrier(ctx, table, 2, 0, epoch)
    with pytest.raises(R.KernelError):
        ctx.flush()
    eight = time.perf_counter() - t0
    assert eight < 2.5 * one_limit + 0.2, (one_limit, eight)
    assert pads[1].download(np.uint32, 2)[0] == 9
    # the report cleared the flag: the next barrier waits again (and gives up again); world size 1 completes at once
    R.peer_barrier(ctx, table, 2, 0, 10)
    with pytest.raises(R.KernelError):
        ctx.flush()
    one = (C.c_void_p * 1)(pads[0].ptr)
    R.peer_barrier(ctx, one, 1, 0, 11)
    ctx.flush()
