"""GPU parity tests of the MoE block (router, softmax/top-k routing, grouped expert products, weighted
combine), through the C ABI, against the CPU oracle.

Bars: router expert indices bit-exact (set and order) except where the decisive probabilities are
closer than 1e-6 (ties excluded, and counted); routing weights and block outputs within
|gpu - oracle| <= 1e-3 * max(|ref|, rms(ref)) (f32 accumulation)."""
from pathlib import Path

import numpy as np
import pytest

from helpers import assert_close

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).parent / "golden" / "path_golden.npz"


def check_routing(O, logits, k, renorm, gidx, gw, tie=1e-6):
    """Compare device routing with the oracle token by token; returns the number of excluded ties."""
    excluded = 0
    for t in range(logits.shape[0]):
        ridx, rw, probs = O.topk_softmax(logits[t], k, renorm)
        srt = np.sort(probs)[::-1]
        gaps = srt[:k] - srt[1:k + 1]           # gap between consecutive ranks up to the k/(k+1) boundary
        if (ridx != gidx[t]).any():
            assert gaps.min() <= tie, ("routing differs without a near-tie", t, ridx, gidx[t], gaps.min())
            excluded += 1
            continue
        assert np.allclose(gw[t], rw, rtol=1e-5, atol=1e-8), (t, gw[t], rw)
    return excluded


@pytest.mark.parametrize("E,k", [(64, 8), (128, 8), (8, 2), (256, 32), (40, 3)])
def test_route_topk_matches_oracle(ctx, oracle, E, k):
    import runit_mac_b200 as R
    O = oracle
    rng = np.random.default_rng(E * 100 + k)
    T = 300
    logits = rng.normal(0, 1.5, (T, E)).astype(np.float32)
    for renorm in (0, 1):
        idx, w = ctx.new_buffer(T * k * 4), ctx.new_buffer(T * k * 4)
        R.moe_route_topk(ctx, ctx.buffer_from(logits), 0, E, k, renorm, T, idx, w)
        ctx.flush()
        gi = idx.download(np.int32, T * k).reshape(T, k)
        gw = w.download(np.float32, T * k).reshape(T, k)
        assert check_routing(O, logits, k, bool(renorm), gi, gw) <= 2
        if renorm:
            assert np.allclose(gw.sum(1), 1.0, atol=1e-5)
    # f16 logits, the reference's router output dtype (forward.rs:1650, 2421-2422)
    l16 = logits.astype(np.float16)
    idx, w = ctx.new_buffer(T * k * 4), ctx.new_buffer(T * k * 4)
    R.moe_route_topk(ctx, ctx.buffer_from(l16), 1, E, k, 1, T, idx, w)
    ctx.flush()
    gi = idx.download(np.int32, T * k).reshape(T, k)
    gw = w.download(np.float32, T * k).reshape(T, k)
    assert check_routing(O, l16.astype(np.float32), k, True, gi, gw) <= T // 10   # f16 logits collide often


def test_route_topk_ties_pick_lowest_index(ctx):
    import runit_mac_b200 as R
    idx, w = ctx.new_buffer(16), ctx.new_buffer(16)
    R.moe_route_topk(ctx, ctx.buffer_from(np.zeros(16, np.float32)), 0, 16, 4, 0, 1, idx, w)
    ctx.flush()
    assert list(idx.download(np.int32, 4)) == [0, 1, 2, 3]
    assert np.allclose(w.download(np.float32, 4), 1.0 / 16)


def test_router_gemv_f32(ctx, oracle):
    import runit_mac_b200 as R
    O = oracle
    rng = np.random.default_rng(3)
    for E, h, T in ((64, 2048, 5), (128, 2048, 3), (8, 256, 2), (64, 1024, 70)):
        w = rng.normal(0, 0.02, (E, h)).astype(np.float32)
        x = rng.normal(0, 1, (T, h)).astype(np.float32)
        lg = ctx.new_buffer(T * E * 4)
        R.moe_router_f32(ctx, ctx.buffer_from(w), ctx.buffer_from(x), lg, E, h, T)
        ctx.flush()
        got = lg.download(np.float32, T * E).reshape(T, E)
        ref = np.stack([O.gemv_f32w(w, x[t], E, h) for t in range(T)])
        assert_close(O, ref, got, rel_tol=1e-5, what="router")


@pytest.mark.parametrize("variant", [0, 1, 2, 3])
def test_router_gemm_many_tokens(ctx, oracle, variant):
    """The f32 router for prefill sizes: the kernel chosen by size (0), one warp per expert (1), the tiled GEMM (2) and the
    GEMM with K split over the warps of a CTA (3), ragged token and expert counts included, against the same f64-exact
    product; logits of one token do not depend on how many tokens ride along."""
    import runit_mac_b200 as R
    O = oracle
    rng = np.random.default_rng(30 + variant)
    ctx.set_tuning("router_variant", variant)
    try:
        for E, h, T in ((64, 2048, 300), (128, 2048, 131), (60, 1024, 129), (64, 512, 16)):
            w = rng.normal(0, 0.02, (E, h)).astype(np.float32)
            x = rng.normal(0, 1, (T, h)).astype(np.float32)
            wb, lg = ctx.buffer_from(w), ctx.new_buffer(T * E * 4)
            R.moe_router_f32(ctx, wb, ctx.buffer_from(x), lg, E, h, T)
            ctx.flush()
            got = lg.download(np.float32, T * E).reshape(T, E)
            ref = (x.astype(np.float64) @ w.astype(np.float64).T).astype(np.float32)
            assert_close(O, ref, got, rel_tol=1e-5, what="router, variant %d" % variant)
            if variant == 3 and T >= 117:
                lg2 = ctx.new_buffer(17 * E * 4)
                R.moe_router_f32(ctx, wb, ctx.buffer_from(x[100:117]), lg2, E, h, 17)
                ctx.flush()
                assert np.array_equal(lg2.download(np.float32, 17 * E).reshape(17, E), got[100:117])
    finally:
        ctx.set_tuning("router_variant", 0)


def test_moe_golden_fixture(ctx, oracle):
    import runit_mac_b200 as R
    G = np.load(GOLD)
    h, ff, E, k = map(int, G["moe_dims"])
    out, idx, w = R.moe_layer_q4k_host(ctx, G["moe_router"], G["moe_gate"], G["moe_up"], G["moe_down"], G["moe_x"], h=h, ff=ff,
                                       E=E, top_k=k, renorm=False)
    assert (idx == G["moe_idx"]).all()
    assert np.allclose(w, G["moe_w"], rtol=1e-5)
    assert_close(oracle, G["moe_y"], out, what="moe golden")


def make_olmoe_layer(O, rng, E=64, h=2048, ff=1024):
    router = rng.normal(0, 0.02, (E, h)).astype(np.float32)
    gate = O.rand_q4k(rng, E * ff, h)
    up = O.rand_q4k(rng, E * ff, h)
    down = O.rand_q4k(rng, E * h, ff)
    return router, gate, up, down


@pytest.fixture(scope="module")
def olmoe_layer(oracle):
    return make_olmoe_layer(oracle, np.random.default_rng(1003))


@pytest.mark.parametrize("T", [1, 16])
def test_moe_layer_olmoe_shape(ctx, oracle, olmoe_layer, T):
    """Single OLMoE-1B-7B-shaped layer: hidden 2048, 64 experts, top-8, expert intermediate 1024, f32
    router ~N(0,0.02), softmax then top-8 without renormalisation, Q4_K experts, x ~ N(0,1)."""
    import runit_mac_b200 as R
    O = oracle
    router, gate, up, down = olmoe_layer
    rng = np.random.default_rng(10 + T)
    x = rng.normal(0, 1, (T, 2048)).astype(np.float32)
    res = rng.normal(0, 1, (T, 2048)).astype(np.float32)
    ref, ridx, rw = O.moe_layer_q4k(router, gate, up, down, x, h=2048, ff=1024, E=64, top_k=8, renorm=False, residual=res)
    out, idx, w = R.moe_layer_q4k_host(ctx, router, gate, up, down, x, h=2048, ff=1024, E=64, top_k=8, renorm=False, residual=res)
    logits = np.stack([O.gemv_f32w(router, x[t], 64, 2048) for t in range(T)])
    excluded = check_routing(O, logits, 8, False, idx, w)
    assert excluded == 0 or T > 1
    ok = [(idx[t] == ridx[t]).all() for t in range(T)]
    assert_close(O, ref[ok], out[ok], what="moe layer T=%d" % T)
    # renormalised variant (the reference's behaviour, forward.rs:2438-2445)
    ref, _, rw = O.moe_layer_q4k(router, gate, up, down, x, h=2048, ff=1024, E=64, top_k=8, renorm=True)
    out, idx2, w2 = R.moe_layer_q4k_host(ctx, router, gate, up, down, x, h=2048, ff=1024, E=64, top_k=8, renorm=True)
    assert np.allclose(w2.sum(1), 1.0, atol=1e-5)
    ok = [(idx2[t] == ridx[t]).all() for t in range(T)]
    assert_close(O, ref[ok], out[ok], what="moe layer renorm T=%d" % T)


def test_moe_layer_256_tokens_sampled(ctx, oracle, olmoe_layer):
    """T=256: every token is routed on the device; a sample of tokens is recomputed by the oracle
    (tokens are independent), and the block is checked for linearity in the residual."""
    import runit_mac_b200 as R
    O = oracle
    router, gate, up, down = olmoe_layer
    T = 256
    rng = np.random.default_rng(256)
    x = rng.normal(0, 1, (T, 2048)).astype(np.float32)
    out, idx, w = R.moe_layer_q4k_host(ctx, router, gate, up, down, x, h=2048, ff=1024, E=64, top_k=8, renorm=False)
    assert len(np.unique(idx)) == 64                      # with 2048 assignments every expert is hit
    assert (np.sort(idx, 1)[:, 1:] != np.sort(idx, 1)[:, :-1]).all()   # 8 distinct experts per token
    sample = [0, 1, 17, 100, 255] + list(rng.integers(0, T, 7))
    ref, ridx, _ = O.moe_layer_q4k(router, gate, up, down, x[sample], h=2048, ff=1024, E=64, top_k=8, renorm=False)
    for j, t in enumerate(sample):
        if (ridx[j] == idx[t]).all():
            assert_close(O, ref[j], out[t], what="token %d" % t)
    res = rng.normal(0, 1, (T, 2048)).astype(np.float32)
    out2, _, _ = R.moe_layer_q4k_host(ctx, router, gate, up, down, x, h=2048, ff=1024, E=64, top_k=8, renorm=False, residual=res)
    assert_close(O, out + res, out2, rel_tol=1e-5, what="residual")


def test_moe_bad_arguments(ctx):
    import runit_mac_b200 as R
    b = ctx.new_buffer(1 << 20)
    with pytest.raises(R.KernelError) as e:   # scratch too small
        R.moe_layer_q4k(ctx, b, b, b, b, b, None, b, None, None, b, 1024, 4, 2048, 1024, 64, 8, 0)
    assert e.value.status == 3
    with pytest.raises(R.KernelError):        # hidden not a multiple of 256
        R.moe_layer_q4k(ctx, b, b, b, b, b, None, b, None, None, b, 1 << 20, 1, 2000, 1024, 64, 8, 0)
    with pytest.raises(R.KernelError):        # more experts per token than experts
        R.moe_route_topk(ctx, b, 0, 4, 8, 0, 1, b, b)
    ctx.flush()


def test_expert_parallel_entry_with_one_rank(ctx, oracle):
    """runit_moe_layer_q4k_ep with world = 1 (own buffers stand in for the peer-mapped ones): same block as
    runit_moe_layer_q4k up to the order of the final additions; two calls alternate the halves of the partial buffer."""
    import ctypes as C
    import runit_mac_b200 as R
    O = oracle
    h, ff, E, k, T = 512, 256, 8, 2, 5
    rng = np.random.default_rng(31)
    router = rng.normal(0, 0.02, (E, h)).astype(np.float32)
    gate = np.stack([O.rand_q4k(rng, ff, h) for _ in range(E)])
    up = np.stack([O.rand_q4k(rng, ff, h) for _ in range(E)])
    down = np.stack([O.rand_q4k(rng, h, ff) for _ in range(E)])
    x = rng.normal(0, 1, (T, h)).astype(np.float32)
    res = rng.normal(0, 1, (T, h)).astype(np.float32)
    ref, ridx, _ = O.moe_layer_q4k(router, gate, up, down, x, h=h, ff=ff, E=E, top_k=k, renorm=False, residual=res)
    bufs = [ctx.buffer_from(a) for a in (router, gate, up, down, x, res)]
    out, idx, w = ctx.new_buffer(T * h * 4), ctx.new_buffer(T * k * 4), ctx.new_buffer(T * k * 4)
    nbytes = R.moe_scratch_bytes(ctx, T, h, ff, E, k)
    scratch = ctx.new_buffer(nbytes)
    partial = ctx.buffer_from(np.full(2 * T * h, np.nan, np.float32))
    pad = ctx.buffer_from(np.zeros(64, np.uint32))
    pt, pp = (C.c_void_p * 1)(partial.ptr), (C.c_void_p * 1)(pad.ptr)
    for epoch in (1, 2):
        R.moe_layer_q4k_ep(ctx, *bufs, out, idx, w, scratch, nbytes, pt, pp, T, h, ff, E, k, 0, 1, 0, epoch)
        ctx.flush()
        assert (idx.download(np.int32, T * k).reshape(T, k) == ridx).all()
        assert_close(O, ref, out.download(np.float32, T * h).reshape(T, h), what="ep entry, one rank, epoch %d" % epoch)
    halves = partial.download(np.float32, 2 * T * h).reshape(2, T * h)
    assert np.isfinite(halves).all() and np.array_equal(halves[0], halves[1])     # both halves were used, same sums
    with pytest.raises(R.KernelError):
        R.moe_layer_q4k_ep(ctx, *bufs, out, idx, w, scratch, nbytes, pt, pp, T, h, ff, E, k, 0, 3, 0, 3)   # 8 experts / 3 ranks
    ctx.flush()


def rand_q4k_small_zero_mean(O, rng, rows, k, sigma):
    """Q4_K rows with zero-mean weights of a scale that keeps every f16 intermediate of the reference's block far from
    overflow (d*sc*(q - 7.5): dmin = 7.5 d, min index = scale index)."""
    nb = k // 256
    d = np.abs(rng.normal(0.0, sigma, (rows, nb)))
    sc = rng.integers(0, 64, (rows, nb, 8), dtype=np.uint8)
    nib = rng.integers(0, 16, (rows, nb, 256), dtype=np.uint8)
    return O.pack_q4k(d, 7.5 * d, sc, sc, nib)


def test_reference_op_sequence_with_f16_twins(ctx, oracle):
    """The literal drop-in use: the reference's own MoE op sequence (crates/engine/src/forward.rs:1644-1679) issued
    call by call through the twins, with the reference's dtypes — f16 router weights and f16 logits
    (gemv_f16w_f32in), renormalised top-k, gate/up through the f16 twin of the Q4_K weights with f32 input and f16
    output (WeightBuf::gemv_f32in for Q4K, forward.rs:164-180: dequant_q4k_f16 at load, then gemv_f16w_f32in),
    silu_mul_f16, down from the packed weights with f16 in/out (gemv_q4k_f16), the f16 accumulator
    (scale_accumulate_f16 in routing order) and add_f16_into_f32 — against the oracle's REF_F16 mode, which places
    the same f16 roundings.  Tolerance: the reference's own for f16 kernels, abs 1e-2 (dispatch.rs:1782)."""
    import runit_mac_b200 as R
    O = oracle
    rng = np.random.default_rng(1644)
    E, h, ff, k, T = 64, 2048, 1024, 8, 3
    rb_h, rb_ff = O.row_bytes(O.Q4K, h), O.row_bytes(O.Q4K, ff)
    router16 = rng.normal(0, 0.02, (E, h)).astype(np.float16)
    gate = rand_q4k_small_zero_mean(O, rng, E * ff, h, 2e-4)
    up = rand_q4k_small_zero_mean(O, rng, E * ff, h, 2e-4)
    down = rand_q4k_small_zero_mean(O, rng, E * h, ff, 2e-4)
    x = rng.normal(0, 1, (T, h)).astype(np.float32)
    res = rng.normal(0, 1, (T, h)).astype(np.float32)
    ref, ridx, rw = O.moe_layer_q4k(router16.astype(np.float32), gate, up, down, x, h=h, ff=ff, E=E, top_k=k, renorm=True,
                                    mode=O.MOE_REF_F16, residual=res)
    assert np.isfinite(ref).all() and np.abs(ref - res).max() > 0.1      # the block contributes, nothing overflowed f16

    # load time: packed weights as stored + the f16 twins of gate and up (forward.rs:1137-1222 keeps both)
    gate_b, up_b, down_b = ctx.buffer_from(gate), ctx.buffer_from(up), ctx.buffer_from(down)
    gate16, up16 = ctx.new_buffer(E * ff * h * 2), ctx.new_buffer(E * ff * h * 2)
    R.dequant_q4k_f16(ctx, gate_b, gate16, E * ff * (h // 256))
    R.dequant_q4k_f16(ctx, up_b, up16, E * ff * (h // 256))
    router_b = ctx.buffer_from(router16)
    logits = ctx.new_buffer(E * 2)
    idx_b, w_b = ctx.new_buffer(k * 4), ctx.new_buffer(k * 4)
    g16, u16, act16, ffn16, moe16 = (ctx.new_buffer(n * 2) for n in (ff, ff, ff, h, h))
    ties = 0
    for t in range(T):
        xb = ctx.buffer_from(x[t])
        xres = ctx.buffer_from(res[t])                     # s.x: the f32 hidden state the block adds into
        R.gemv_f16w_f32in(ctx, router_b, xb, logits, E, h)
        R.moe_route_topk(ctx, logits, 1, E, k, 1, 1, idx_b, w_b)
        ctx.flush()                                        # the reference reads the logits on the host here (forward.rs:1654)
        eids, ew = idx_b.download(np.int32, k), w_b.download(np.float32, k)
        if (eids != ridx[t]).any():
            # f16 logits one rounding apart can swap two experts: only a near-tie of the oracle's own logits excuses it
            lg = O.gemv_f32w(router16.astype(np.float32), x[t], E, h).astype(np.float16).astype(np.float32)
            srt = np.sort(lg)[::-1]
            assert (srt[:k] - srt[1:k + 1]).min() <= 2 * np.spacing(np.float16(abs(srt[0]))), (t, eids, ridx[t])
            ties += 1
            continue
        assert np.allclose(ew, rw[t], rtol=1e-4)
        ctx.call("memset", moe16, 0, h * 2)
        for i in range(k):
            e = int(eids[i])
            R.gemv_f16w_f32in(ctx, gate16.ptr + e * ff * h * 2, xb, g16, ff, h)
            R.gemv_f16w_f32in(ctx, up16.ptr + e * ff * h * 2, xb, u16, ff, h)
            R.silu_mul_f16(ctx, g16, u16, act16, ff)
            R.gemv_q4k_f16(ctx, down_b.ptr + e * h * rb_ff, act16, ffn16, h, ff)
            R.scale_accumulate_f16(ctx, ffn16, moe16, float(ew[i]), h)
        R.add_f16_into_f32(ctx, moe16, xres, h)
        ctx.flush()
        got = xres.download(np.float32, h)
        assert np.isfinite(got).all()
        assert np.abs(got - ref[t]).max() <= 1e-2, (t, float(np.abs(got - ref[t]).max()))
    assert ties <= 1
