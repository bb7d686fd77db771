"""GPU parity tests of recorded command lists whose consecutive GEMVs run as one persistent launch (opt-in knob
stream_fuse).

The recorded ops must behave exactly like the same calls issued one by one (the reference commits a token's dispatches
in one command buffer and its GPU runs them in order, crates/kernels/src/context.rs:248-296): every output is compared
with the oracle at the path's tolerance (1e-3 of the output scale) and with the list recorded without the folding."""
import numpy as np
import pytest

from helpers import assert_close

pytestmark = pytest.mark.gpu
FMT_NAME = {1: "q4_0", 2: "q4k"}


class Layer:
    """Weights and vectors of one decoder layer's GEMVs at a small shape (same op pattern as a 7B layer)."""

    def __init__(self, ctx, O, rng, fmt, hidden, inter, q_dim, kv_dim):
        self.fmt, self.hidden, self.inter, self.q_dim, self.kv_dim = fmt, hidden, inter, q_dim, kv_dim
        self.host = {"q": O.rand_weights(fmt, rng, q_dim, hidden), "k": O.rand_weights(fmt, rng, kv_dim, hidden),
                     "v": O.rand_weights(fmt, rng, kv_dim, hidden), "o": O.rand_weights(fmt, rng, hidden, q_dim),
                     "gate": O.rand_weights(fmt, rng, inter, hidden), "up": O.rand_weights(fmt, rng, inter, hidden),
                     "down": O.rand_weights(fmt, rng, hidden, inter)}
        self.dev = {n: ctx.buffer_from(w) for n, w in self.host.items()}


def record_token(ctx, R, layers, lm, bufs, vocab):
    """The GEMVs of one token: per layer fused Q|K|V (reads xn), o-proj + residual into x (reads q), fused gate/up + SiLU
    (reads xn), down + residual into x (reads act); then the output matrix on xn."""
    n = FMT_NAME[layers[0].fmt]
    for L in layers:
        getattr(R, "fused_qkv_%s_f32" % n)(ctx, L.dev["q"], L.dev["k"], L.dev["v"], bufs["xn"], bufs["q"], bufs["k"], bufs["v"],
                                            L.q_dim, L.kv_dim, L.hidden)
        getattr(R, "gemv_%s_add_f32_f32in" % n)(ctx, L.dev["o"], bufs["q"], bufs["x"], bufs["x"], L.hidden, L.q_dim)
        getattr(R, "fused_ffn_%s_f32" % n)(ctx, L.dev["gate"], L.dev["up"], bufs["xn"], bufs["act"], L.inter, L.hidden)
        getattr(R, "gemv_%s_add_f32_f32in" % n)(ctx, L.dev["down"], bufs["act"], bufs["x"], bufs["x"], L.hidden, L.inter)
    getattr(R, "gemv_%s_f32in_f32out" % n)(ctx, lm, bufs["xn"], bufs["logits"], vocab, layers[0].hidden)


def oracle_token(O, layers, lm_host, xn, x0, vocab):
    x = x0.astype(np.float64)
    f = layers[0].fmt
    for L in layers:
        q = O.gemv(f, L.host["q"], xn, L.q_dim, L.hidden)
        x = x + O.gemv(f, L.host["o"], q.astype(np.float32), L.hidden, L.q_dim)
        g, u = O.gemv(f, L.host["gate"], xn, L.inter, L.hidden), O.gemv(f, L.host["up"], xn, L.inter, L.hidden)
        act = O.silu_mul_f32(g.astype(np.float32), u.astype(np.float32))
        x = x + O.gemv(f, L.host["down"], act, L.hidden, L.inter)
    return x.astype(np.float32), O.gemv(f, lm_host, xn, vocab, layers[0].hidden)


@pytest.mark.parametrize("fmt", [2, 1])
@pytest.mark.parametrize("cfg", [0, 1, 2, 3])
def test_recorded_token_runs_as_one_launch_and_matches(ctx, oracle, fmt, cfg):
    import runit_mac_b200 as R
    O = oracle
    rng = np.random.default_rng(50 + fmt)
    hidden, inter, q_dim, kv_dim, vocab = 512, 1280, 512, 96, 1000      # ragged last tile in the output matrix
    layers = [Layer(ctx, O, rng, fmt, hidden, inter, q_dim, kv_dim) for _ in range(3)]
    lm_host = O.rand_weights(fmt, rng, vocab, hidden)
    lm = ctx.buffer_from(lm_host)
    xn = rng.normal(0, 1, hidden).astype(np.float32)
    x0 = rng.normal(0, 1, hidden).astype(np.float32)
    f4 = lambda n: ctx.new_buffer(4 * n)
    bufs = {"xn": ctx.buffer_from(xn), "x": ctx.buffer_from(x0), "q": f4(q_dim), "k": f4(kv_dim), "v": f4(kv_dim), "act": f4(inter),
            "logits": f4(vocab)}
    ref_x, ref_logits = oracle_token(O, layers, lm_host, xn, x0, vocab)

    def run(fuse):
        ctx.set_tuning("stream_fuse", fuse)
        ctx.set_tuning("stream_cfg", cfg)
        try:
            record_token(ctx, R, layers, lm, bufs, vocab)          # eager once: kernels configured before the recording
            ctx.flush()
            ctx.graph_begin()
            record_token(ctx, R, layers, lm, bufs, vocab)
            g = ctx.graph_end()
        finally:
            ctx.set_tuning("stream_fuse", 0)
            ctx.set_tuning("stream_cfg", 0)
        outs = []
        bufs["x"].upload(x0)
        for _ in range(3):                                          # replays: the counters of the program return to rest
            g.launch()
            ctx.flush()
            outs.append((bufs["x"].download(np.float32, hidden), bufs["logits"].download(np.float32, vocab),
                         bufs["act"].download(np.float32, inter)))
        info = (g.fused_launches, g.kernel_launches)
        g.destroy()
        return outs, info
    fused, (nf, nk) = run(1)
    plain, (pf, pk) = run(0)
    assert (nf, nk) == (13, 1) and (pf, pk) == (0, 13)
    assert_close(O, ref_x, fused[0][0], what="hidden state after one token")
    assert_close(O, ref_logits, fused[0][1], what="logits")
    for a, b in zip(fused, plain):
        for va, vb in zip(a, b):
            scale = np.sqrt(np.mean(vb.astype(np.float64) ** 2))
            assert np.abs(va - vb).max() <= 2e-4 * scale    # same arithmetic, another summation order over the K-slices
    # the fused list gives the same bits on every run from the same state
    again, _ = run(1)
    for a, b in zip(fused, again):
        assert all(np.array_equal(va, vb) for va, vb in zip(a, b))


def test_recorded_order_is_kept_across_overwrites(ctx, oracle):
    """Write-after-read and write-after-write between folded GEMVs: B overwrites A's input, C reads what B wrote over it,
    D overwrites A's output.  The list must behave like the calls in order."""
    import runit_mac_b200 as R
    O = oracle
    rng = np.random.default_rng(9)
    n = 512
    W = [O.rand_weights(2, rng, n, n) for _ in range(4)]
    Wd = [ctx.buffer_from(w) for w in W]
    x0 = rng.normal(0, 1, n).astype(np.float32)
    xb, yb, zb = ctx.buffer_from(x0), ctx.new_buffer(4 * n), ctx.new_buffer(4 * n)

    def calls():
        R.gemv_q4k_f32in_f32out(ctx, Wd[0], xb, yb, n, n)       # A: y = W0 x
        R.gemv_q4k_f32in_f32out(ctx, Wd[1], yb, xb, n, n)       # B: x = W1 y      (overwrites A's input)
        R.gemv_q4k_f32in_f32out(ctx, Wd[2], xb, zb, n, n)       # C: z = W2 x
        R.gemv_q4k_f32in_f32out(ctx, Wd[3], zb, yb, n, n)       # D: y = W3 z      (overwrites A's output, which B read)
    y = O.gemv(2, W[0], x0, n, n).astype(np.float32)
    x1 = O.gemv(2, W[1], y, n, n).astype(np.float32)
    z = O.gemv(2, W[2], x1, n, n).astype(np.float32)
    y2 = O.gemv(2, W[3], z, n, n).astype(np.float32)
    calls()
    ctx.flush()
    xb.upload(x0)
    ctx.set_tuning("stream_fuse", 1)
    try:
        ctx.graph_begin()
        calls()
        g = ctx.graph_end()
    finally:
        ctx.set_tuning("stream_fuse", 0)
    assert g.fused_launches == 4 and g.kernel_launches == 1
    g.launch()
    ctx.flush()
    # four chained products of matrices with a positive mean: compare at the scale of each vector
    assert_close(O, x1, xb.download(np.float32, n), rel_tol=2e-3, what="x after B")
    assert_close(O, z, zb.download(np.float32, n), rel_tol=3e-3, what="z after C")
    assert_close(O, y2, yb.download(np.float32, n), rel_tol=4e-3, what="y after D")
    g.destroy()


def test_mixed_formats_and_long_lists_split_into_several_launches(ctx, oracle):
    import runit_mac_b200 as R
    O = oracle
    rng = np.random.default_rng(10)
    m, k = 96, 512
    w4k, w40 = O.rand_weights(2, rng, m, k), O.rand_weights(1, rng, m, k)
    a, b = ctx.buffer_from(w4k), ctx.buffer_from(w40)
    x = rng.normal(0, 1, k).astype(np.float32)
    xb = ctx.buffer_from(x)
    ys = [ctx.new_buffer(4 * m) for _ in range(140)]
    w8 = ctx.buffer_from(O.rand_weights(0, rng, 8, 64))

    def calls():
        for i in range(3):
            R.gemv_q4k_f32in_f32out(ctx, a, xb, ys[i], m, k)
        for i in range(3, 6):
            R.gemv_q4_0_f32in_f32out(ctx, b, xb, ys[i], m, k)
        R.gemv_q4k_f32in_f32out(ctx, a, xb, ys[6], m, k)         # a single one between two other formats stays as it is
        R.gemv_q8_0_f32in_f32out(ctx, w8, xb, ys[7], 8, 64)
        for i in range(8, 140):                                   # more GEMVs than one program holds
            R.gemv_q4k_f32in_f32out(ctx, a, xb, ys[i], m, k)
    calls()
    ctx.flush()
    ctx.set_tuning("stream_fuse", 1)
    try:
        ctx.graph_begin()
        calls()
        g = ctx.graph_end()
    finally:
        ctx.set_tuning("stream_fuse", 0)
    assert g.fused_launches == 3 + 3 + 132 and g.kernel_launches == 1 + 1 + 1 + 1 + 2
    g.launch()
    ctx.flush()
    r4k, r40 = O.gemv(2, w4k, x, m, k), O.gemv(1, w40, x, m, k)
    for i in list(range(3)) + [6, 8, 70, 135, 139]:
        assert_close(O, r4k, ys[i].download(np.float32, m), what="q4k output %d" % i)
    for i in range(3, 6):
        assert_close(O, r40, ys[i].download(np.float32, m), what="q4_0 output %d" % i)
    g.destroy()


def test_decode_shapes_over_several_layers_match_the_separate_launches(ctx):
    """Three layers of the 7B-shaped GEMV set (fused Q|K|V, o + residual, fused gate/up, down + residual) plus the output
    matrix, weights generated on the device: every CTA walks more items than its per-item bookkeeping has slots, through
    GEMVs with 14, 2 and 16 warps per tile (some warps have no part in some items).  The folded list must reproduce the
    separate launches (same arithmetic, other summation order over the K-slices)."""
    import runit_mac_b200 as R
    hidden, inter, q_dim, kv_dim, vocab, layers = 3584, 18944, 3584, 512, 32000, 3
    rb = lambda k: k // 256 * 144
    mats = {"q": (q_dim, hidden), "k": (kv_dim, hidden), "v": (kv_dim, hidden), "o": (hidden, q_dim), "gate": (inter, hidden),
            "up": (inter, hidden), "down": (hidden, inter)}
    W = []
    for l in range(layers):
        d = {}
        for i, (n, (m, k)) in enumerate(mats.items()):
            d[n] = ctx.new_buffer(m * rb(k))
            R.fill_weights_q4k_zero_mean(ctx, d[n], m * (k // 256), 1000 + 16 * l + i, 2e-4)
        W.append(d)
    lm = ctx.new_buffer(vocab * rb(hidden))
    R.fill_weights_q4k_zero_mean(ctx, lm, vocab * (hidden // 256), 77, 2e-4)
    f4 = lambda n: ctx.new_buffer(4 * n)
    xn, x, q, kk, v, act, logits = f4(hidden), f4(hidden), f4(q_dim), f4(kv_dim), f4(kv_dim), f4(inter), f4(vocab)
    R.fill_normal_f32(ctx, xn, hidden, 5, 1.0)
    x0 = np.random.default_rng(3).normal(0, 1, hidden).astype(np.float32)

    def calls():
        for w in W:
            R.fused_qkv_q4k_f32(ctx, w["q"], w["k"], w["v"], xn, q, kk, v, q_dim, kv_dim, hidden)
            R.gemv_q4k_add_f32_f32in(ctx, w["o"], q, x, x, hidden, q_dim)
            R.fused_ffn_q4k_f32(ctx, w["gate"], w["up"], xn, act, inter, hidden)
            R.gemv_q4k_add_f32_f32in(ctx, w["down"], act, x, x, hidden, inter)
        R.gemv_q4k_f32in_f32out(ctx, lm, xn, logits, vocab, hidden)

    def run(fuse):
        ctx.set_tuning("stream_fuse", fuse)
        try:
            calls()
            ctx.flush()
            ctx.graph_begin()
            calls()
            g = ctx.graph_end()
        finally:
            ctx.set_tuning("stream_fuse", 0)
        x.upload(x0)
        outs = []
        for _ in range(2):
            g.launch()
            ctx.flush()
            outs.append((x.download(np.float32, hidden), act.download(np.float32, inter), logits.download(np.float32, vocab)))
        n = (g.fused_launches, g.kernel_launches)
        g.destroy()
        return outs, n
    fused, nf = run(1)
    plain, npl = run(0)
    assert nf == (4 * layers + 1, 1) and npl == (0, 4 * layers + 1)
    for a, b in zip(fused, plain):
        for va, vb in zip(a, b):
            assert np.isfinite(va).all()
            scale = np.sqrt(np.mean(vb.astype(np.float64) ** 2))
            assert np.abs(va - vb).max() <= 3e-4 * scale
