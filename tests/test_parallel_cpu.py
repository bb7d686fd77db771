"""Host logic of the two multi-GPU schemes (row-sharded GEMV + all-gather; expert-parallel MoE with
fixed-capacity and count-exchanged all-to-all dispatch/combine) on CPU: two gloo ranks, arithmetic supplied by the oracle.
Checks shard offsets, slot placement, the round trip through both all-to-alls and the weighted combine
against the single-process oracle."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from runit_mac_b200 import parallel as P

H, FF, E, K_TOP, M_ROWS, K_IN = 256, 256, 8, 2, 64, 512


class OracleBackend:
    """CPU stand-in for the kernels (test infrastructure): the oracle on this rank's shard."""

    def __init__(self, O, world, rank, data):
        self.O, self.world, self.rank, self.d = O, world, rank, data
        self.n_local = E // world

    def local_gemv(self, x):
        r0, n = P.shard_rows(M_ROWS, self.world, self.rank)
        rb = self.O.row_bytes(self.O.Q4K, K_IN)
        w = self.d["lm"].reshape(M_ROWS, rb)[r0:r0 + n]
        return torch.from_numpy(self.O.gemv(self.O.Q4K, w, x.numpy(), n, K_IN))

    def route(self, x):
        idx, w = [], []
        for t in range(x.shape[0]):
            lg = self.O.gemv_f32w(self.d["router"], x[t].numpy(), E, H)
            i_, w_, _ = self.O.topk_softmax(lg, K_TOP, False)
            idx.append(i_); w.append(w_)
        return torch.from_numpy(np.stack(idx)), torch.from_numpy(np.stack(w))

    def experts(self, x_slots, local_expert):
        O = self.O
        rb_h, rb_ff = O.row_bytes(O.Q4K, H), O.row_bytes(O.Q4K, FF)
        y = torch.zeros(x_slots.shape[0], H)
        e0 = self.rank * self.n_local
        for s in range(x_slots.shape[0]):
            le = int(local_expert[s])
            if le < 0:
                continue
            assert 0 <= le < self.n_local
            e = e0 + le
            xs = x_slots[s].numpy()
            g = O.gemv(O.Q4K, self.d["gate"].reshape(E, FF * rb_h)[e], xs, FF, H)
            u = O.gemv(O.Q4K, self.d["up"].reshape(E, FF * rb_h)[e], xs, FF, H)
            y[s] = torch.from_numpy(O.gemv(O.Q4K, self.d["down"].reshape(E, H * rb_ff)[e], O.silu_mul_f32(g, u), H, FF))
        return y


def make_data(O):
    rng = np.random.default_rng(99)
    return {"lm": O.rand_q4k(rng, M_ROWS, K_IN).reshape(-1), "router": rng.normal(0, 0.02, (E, H)).astype(np.float32),
            "gate": O.rand_q4k(rng, E * FF, H).reshape(-1), "up": O.rand_q4k(rng, E * FF, H).reshape(-1),
            "down": O.rand_q4k(rng, E * H, FF).reshape(-1),
            "x_lm": rng.normal(0, 1, K_IN).astype(np.float32), "x": rng.normal(0, 1, (6, H)).astype(np.float32),
            "res": rng.normal(0, 1, (6, H)).astype(np.float32)}


def worker(rank, world, port, q):
    import oracle as O
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        O.set_num_threads(1)
        d = make_data(O)
        be = OracleBackend(O, world, rank, d)
        y = P.sharded_gemv(be, dist, torch, torch.from_numpy(d["x_lm"]), M_ROWS, world, rank)
        T = d["x"].shape[0] // world                     # tokens are data-parallel: 3 per rank
        xs = torch.from_numpy(d["x"][rank * T:(rank + 1) * T])
        rs = torch.from_numpy(d["res"][rank * T:(rank + 1) * T])
        out, idx, w = P.ep_moe_forward(be, dist, torch, xs, E, K_TOP, False, world, rank, residual=rs)
        out2, idx2, _ = P.ep_moe_forward_counted(be, dist, torch, xs, E, K_TOP, False, world, rank, residual=rs)   # true counts
        assert (idx2 == idx).all()
        q.put((rank, y.numpy(), out.numpy(), idx.numpy(), w.numpy(), out2.numpy()))
    finally:
        dist.destroy_process_group()


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_two_ranks_match_the_single_process_oracle(oracle):
    O = oracle
    world = 2
    ctxm = mp.get_context("spawn")
    q = ctxm.Queue()
    port = free_port()
    procs = [ctxm.Process(target=worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=120) for _ in range(world)], key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    d = make_data(O)
    full = O.gemv(O.Q4K, d["lm"], d["x_lm"], M_ROWS, K_IN)
    for r in range(world):
        assert (res[r][1] == full).all()                       # every rank holds the same gathered logits
    ref, ridx, rw = O.moe_layer_q4k(d["router"], d["gate"], d["up"], d["down"], d["x"], h=H, ff=FF, E=E, top_k=K_TOP, renorm=False,
                                    residual=d["res"])
    out = np.concatenate([res[r][2] for r in range(world)])
    idx = np.concatenate([res[r][3] for r in range(world)])
    assert (idx == ridx).all()
    assert np.allclose(out, ref, rtol=1e-5, atol=1e-5 * np.abs(ref).max())
    out2 = np.concatenate([res[r][5] for r in range(world)])      # the count-exchanged variant gives the same block
    assert np.allclose(out2, ref, rtol=1e-5, atol=1e-5 * np.abs(ref).max())


def test_shard_and_pack_helpers():
    assert P.shard_rows(152064, 8, 3) == (57024, 19008) and P.shard_rows(50304, 4, 0) == (0, 12576)
    with pytest.raises(ValueError):
        P.shard_rows(10, 4, 0)
    idx = torch.tensor([[0, 5], [6, 1], [7, 4]], dtype=torch.int32)   # E=8, 2 ranks: owners 0,1 | 1,0 | 1,1
    dest, pos, cap = P.ep_pack(torch, idx, 8, 2)
    assert dest.tolist() == [0, 1, 1, 0, 1, 1] and pos.tolist() == [0, 0, 1, 1, 2, 3] and cap == 6
    # single rank degenerates to the plain block
    assert P.expert_owner(torch.tensor([0, 63]), 64, 1).tolist() == [0, 0]
