"""GPU parity tests of the fused-dequant GEMV family, called through the C ABI and compared with
the CPU oracle on the same seeded inputs.

Tolerance (floating point): |gpu - oracle_f64| <= 1e-3 * max(|ref|, rms(ref)) — the bound the
path's specification states for GEMV outputs with f32 accumulation; f16 outputs must match the
rounded oracle to 1 ulp.  The reference's own test tolerances (absolute 1e-2 / 3e-2,
crates/kernels/src/dispatch.rs:1782-1783) are looser."""
from pathlib import Path

import numpy as np
import pytest

from helpers import REL_TOL, assert_close, f16_ulp_close

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).parent / "golden" / "path_golden.npz"
FMT_NAME = {0: "q8_0", 1: "q4_0", 2: "q4k"}


def run_gemv(ctx, R, name, w, x, m, k, out_dtype=np.float32, residual=None):
    wb, xb = ctx.buffer_from(w), ctx.buffer_from(x)
    yb = ctx.new_buffer(max(16, m * np.dtype(out_dtype).itemsize))
    if residual is None:
        getattr(R, name)(ctx, wb, xb, yb, m, k)
    else:
        rb = ctx.buffer_from(residual)
        getattr(R, name)(ctx, wb, xb, yb, rb, m, k)
    ctx.flush()
    return yb.download(out_dtype, m)


# shapes: benchmark decode shapes scaled down in M, plus ragged tiles/units/stages
SHAPES = {
    0: [(1152, 896), (37, 896), (896, 4864), (5, 32), (64, 96), (33, 1024), (70, 2080)],
    1: [(512, 3584), (37, 3584), (40, 18944), (5, 256), (33, 512), (31, 2304), (70, 2080), (5, 32), (64, 96), (40, 2176)],
    2: [(512, 3584), (37, 2048), (40, 18944), (3, 256), (65, 1024), (1024, 2048)],
}


@pytest.mark.parametrize("fmt", [0, 1, 2])
def test_gemv_f32in_f32out_matches_oracle(ctx, oracle, fmt):
    import runit_mac_b200 as R
    O = oracle
    for m, k in SHAPES[fmt]:
        rng = np.random.default_rng(1000 + fmt * 100 + m + k)
        w = O.rand_weights(fmt, rng, m, k)
        x = rng.normal(0, 1, k).astype(np.float32)
        ref = O.gemv(fmt, w, x, m, k, O.TIER_F64)
        got = run_gemv(ctx, R, "gemv_%s_f32in_f32out" % FMT_NAME[fmt], w, x, m, k)
        st = assert_close(O, ref, got, what="%s %dx%d" % (FMT_NAME[fmt], m, k))
        # well inside the tolerance: all three formats round the activations to 16-bit block fixed point (2^-16 .. 2^-15 of
        # a 32-block's maximum) for the integer dot products (Q8_0: dp4a; the 4-bit formats: tensor-core MMAs)
        assert st.max_rel < 2e-4, (fmt, m, k, st)


@pytest.mark.parametrize("math", [1, 2])
@pytest.mark.parametrize("fmt", [1, 2])
def test_gemv_other_arithmetic_paths_match_oracle(ctx, oracle, fmt, math):
    """The packed-f32 (1) and dp4a (2) arithmetic of the batch-1 kernel stay selectable and correct."""
    import runit_mac_b200 as R
    O = oracle
    ctx.set_tuning("gemv_math", math)
    try:
        for m, k in SHAPES[fmt][:4]:
            rng = np.random.default_rng(2000 + fmt * 100 + m + k)
            w = O.rand_weights(fmt, rng, m, k)
            x = rng.normal(0, 1, k).astype(np.float32)
            ref = O.gemv(fmt, w, x, m, k, O.TIER_F64)
            got = run_gemv(ctx, R, "gemv_%s_f32in_f32out" % FMT_NAME[fmt], w, x, m, k)
            st = assert_close(O, ref, got, what="%s %dx%d math %d" % (FMT_NAME[fmt], m, k, math))
            assert st.max_rel < 2e-5, (fmt, m, k, math, st)
    finally:
        ctx.set_tuning("gemv_math", 0)


@pytest.mark.parametrize("fmt", [0, 1, 2])
def test_staged_and_simple_kernels_agree(ctx, oracle, fmt):
    """Two independently written kernels (shared-memory staged, and warp-per-row scalar) agree."""
    import runit_mac_b200 as R
    O = oracle
    m, k = {0: (129, 896), 1: (129, 3584), 2: (129, 2048)}[fmt]
    rng = np.random.default_rng(77 + fmt)
    w = O.rand_weights(fmt, rng, m, k)
    x = rng.normal(0, 1, k).astype(np.float32)
    name = "gemv_%s_f32in_f32out" % FMT_NAME[fmt]
    a = run_gemv(ctx, R, name, w, x, m, k)
    ctx.set_tuning("gemv_variant", 1)
    try:
        b = run_gemv(ctx, R, name, w, x, m, k)
    finally:
        ctx.set_tuning("gemv_variant", 0)
    ref = O.gemv(fmt, w, x, m, k, O.TIER_F64)
    assert_close(O, ref, a, what="staged")
    assert_close(O, ref, b, what="simple")


def test_residual_and_dtype_variants(ctx, oracle):
    import runit_mac_b200 as R
    O = oracle
    for fmt, (m, k) in ((0, (96, 896)), (1, (70, 3584)), (2, (70, 2048))):
        rng = np.random.default_rng(50 + fmt)
        fn = FMT_NAME[fmt]
        w = O.rand_weights(fmt, rng, m, k)
        x = rng.normal(0, 1, k).astype(np.float32)
        x16 = x.astype(np.float16)
        res = rng.normal(0, 1, m).astype(np.float32)
        res16 = res.astype(np.float16)
        y = O.gemv(fmt, w, x, m, k, O.TIER_F64)
        y_h = O.gemv(fmt, w, x16.astype(np.float32), m, k, O.TIER_F64)
        # + f32 residual, f32 in (gemv_*_add_f32_f32in)
        got = run_gemv(ctx, R, "gemv_%s_add_f32_f32in" % fn, w, x, m, k, residual=res)
        assert_close(O, y + res, got, what=fn + " add_f32")
        if fmt != 2:
            # f32 in -> f16 out (gemv_q8_0_f32in / gemv_q4_0_f32in)
            got = run_gemv(ctx, R, "gemv_%s_f32in" % fn, w, x, m, k, out_dtype=np.float16)
            assert f16_ulp_close(y.astype(np.float16), got), fn + " f32in->f16"
        # f16 in -> f16 out
        got = run_gemv(ctx, R, "gemv_%s_f16" % fn, w, x16, m, k, out_dtype=np.float16)
        assert f16_ulp_close(y_h.astype(np.float16), got), fn + " f16"
        # f16 in + f16 residual -> f16
        got = run_gemv(ctx, R, "gemv_%s_add_f16" % fn, w, x16, m, k, out_dtype=np.float16, residual=res16)
        assert f16_ulp_close((y_h + res16.astype(np.float32)).astype(np.float16), got), fn + " add_f16"
        if fmt != 1:
            # f16 in + f32 residual -> f32
            got = run_gemv(ctx, R, "gemv_%s_add_f32res_f16" % fn, w, x16, m, k, residual=res)
            assert_close(O, y_h + res, got, what=fn + " add_f32res_f16")


def test_inplace_residual_aliasing(ctx, oracle):
    """The engine calls the +residual kernels with output == residual (forward.rs:1619,1702)."""
    import runit_mac_b200 as R
    O = oracle
    m, k = 200, 2048
    rng = np.random.default_rng(5)
    w = O.rand_q4k(rng, m, k)
    x = rng.normal(0, 1, k).astype(np.float32)
    res = rng.normal(0, 1, m).astype(np.float32)
    wb, xb, yb = ctx.buffer_from(w), ctx.buffer_from(x), ctx.buffer_from(res)
    R.gemv_q4k_add_f32_f32in(ctx, wb, xb, yb, yb, m, k)
    ctx.flush()
    assert_close(O, O.gemv(O.Q4K, w, x, m, k) + res, yb.download(np.float32, m))


def test_launch_shape_aliases(ctx, oracle):
    import runit_mac_b200 as R
    O = oracle
    m, k = 130, 896
    rng = np.random.default_rng(6)
    w = O.rand_q8_0(rng, m, k)
    x = rng.normal(0, 1, k).astype(np.float32)
    ref = O.gemv(O.Q8_0, w, x, m, k)
    for name in ("gemv_q8_0_f32in_f32out_mr", "gemv_q8_0_f32in_f32out_wide"):
        assert_close(O, ref, run_gemv(ctx, R, name, w, x, m, k), what=name)
    res = rng.normal(0, 1, m).astype(np.float32)
    for name in ("gemv_q8_0_add_f32_f32in_mr", "gemv_q8_0_add_f32_f32in_wide"):
        assert_close(O, ref + res, run_gemv(ctx, R, name, w, x, m, k, residual=res), what=name)
    assert f16_ulp_close(ref.astype(np.float16), run_gemv(ctx, R, "gemv_q8_0_f32in_wide", w, x, m, k, out_dtype=np.float16))


def test_fused_qkv_q8_0(ctx, oracle):
    """Qwen2.5-0.5B decode shape: q_dim 896, kv_dim 128, k 896, with bias (fused_qkv.metal:13-119)."""
    import runit_mac_b200 as R
    O = oracle
    q_dim, kv_dim, k = 896, 128, 896
    rng = np.random.default_rng(1001)
    ws = [O.rand_q8_0(rng, n, k) for n in (q_dim, kv_dim, kv_dim)]
    x = rng.normal(0, 1, k).astype(np.float32)
    bias = [rng.normal(0, 0.02, n).astype(np.float32) for n in (q_dim, kv_dim, kv_dim)]
    refs = [O.gemv(O.Q8_0, w, x, n, k) for w, n in zip(ws, (q_dim, kv_dim, kv_dim))]
    wb = [ctx.buffer_from(w) for w in ws]
    xb = ctx.buffer_from(x)
    outs = [ctx.new_buffer(n * 4) for n in (q_dim, kv_dim, kv_dim)]
    R.fused_qkv_q8_0_f32(ctx, *wb, xb, *outs, q_dim, kv_dim, k)
    ctx.flush()
    for o, r, n in zip(outs, refs, (q_dim, kv_dim, kv_dim)):
        assert_close(O, r, o.download(np.float32, n), what="fused_qkv")
    # f16 bias (the reference's dtype) and f32 bias (the benchmark configuration's)
    b16 = [ctx.buffer_from(b.astype(np.float16)) for b in bias]
    R.fused_qkv_bias_q8_0_f32(ctx, *wb, xb, *outs, *b16, q_dim, kv_dim, k)
    ctx.flush()
    for o, r, b, n in zip(outs, refs, bias, (q_dim, kv_dim, kv_dim)):
        assert_close(O, r + b.astype(np.float16).astype(np.float32), o.download(np.float32, n), what="fused_qkv f16 bias")
    b32 = [ctx.buffer_from(b) for b in bias]
    R.fused_qkv_f32bias_q8_0_f32(ctx, *wb, xb, *outs, *b32, q_dim, kv_dim, k)
    ctx.flush()
    for o, r, b, n in zip(outs, refs, bias, (q_dim, kv_dim, kv_dim)):
        assert_close(O, r + b, o.download(np.float32, n), what="fused_qkv f32 bias")


@pytest.mark.parametrize("fmt", [1, 2])
def test_fused_qkv_4bit(ctx, oracle, fmt):
    """Q|K|V in one launch for Q4_0 / Q4_K (Qwen2.5-7B shapes: q 3584, kv 512, k 3584), also with dependent launch."""
    import runit_mac_b200 as R
    O = oracle
    q_dim, kv_dim, k = 3584, 512, 3584
    rng = np.random.default_rng(40 + fmt)
    ws = [O.rand_weights(fmt, rng, n, k) for n in (q_dim, kv_dim, kv_dim)]
    x = rng.normal(0, 1, k).astype(np.float32)
    refs = [O.gemv(fmt, w, x, n, k) for w, n in zip(ws, (q_dim, kv_dim, kv_dim))]
    wb = [ctx.buffer_from(w) for w in ws]
    outs = [ctx.new_buffer(n * 4) for n in (q_dim, kv_dim, kv_dim)]
    for pdl in (0, 1):
        ctx.set_tuning("pdl", pdl)
        try:
            getattr(R, "fused_qkv_%s_f32" % FMT_NAME[fmt])(ctx, *wb, ctx.buffer_from(x), *outs, q_dim, kv_dim, k)
            ctx.flush()
        finally:
            ctx.set_tuning("pdl", 0)
        for o, r, n in zip(outs, refs, (q_dim, kv_dim, kv_dim)):
            assert_close(O, r, o.download(np.float32, n), what="fused_qkv 4-bit pdl=%d" % pdl)


def test_dependent_launch_chain_is_ordered(ctx, oracle):
    """A chain y1 = W1.x, y2 = W2.y1 + y2 launched with programmatic dependent launch gives the serial result."""
    import runit_mac_b200 as R
    O = oracle
    n = 1024
    rng = np.random.default_rng(8)
    w1, w2 = O.rand_q4k(rng, n, n), O.rand_q4k(rng, n, n)
    x = rng.normal(0, 1, n).astype(np.float32)
    y1 = O.gemv(O.Q4K, w1, x, n, n)
    res = rng.normal(0, 1, n).astype(np.float32)
    ref = O.gemv(O.Q4K, w2, y1, n, n) + res
    b1, b2, xb = ctx.buffer_from(w1), ctx.buffer_from(w2), ctx.buffer_from(x)
    t, out = ctx.new_buffer(n * 4), ctx.buffer_from(res)
    ctx.set_tuning("pdl", 1)
    try:
        for _ in range(3):
            ctx.call("memcpy_h2d", out, res.ctypes.data, res.nbytes)
            R.gemv_q4k_f32in_f32out(ctx, b1, xb, t, n, n)
            R.gemv_q4k_add_f32_f32in(ctx, b2, t, out, out, n, n)
            ctx.flush()
            assert_close(O, ref, out.download(np.float32, n), rel_tol=1e-3, what="pdl chain")
    finally:
        ctx.set_tuning("pdl", 0)


@pytest.mark.parametrize("fmt,ff,k", [(0, 4864, 896), (0, 40, 96), (1, 1000, 3584), (1, 17, 256), (2, 1000, 3584), (2, 33, 256)])
def test_fused_ffn(ctx, oracle, fmt, ff, k):
    """act = silu(Wg.x) * (Wu.x)  (fused_ffn.metal:36-93, gemv_q4_0.metal:254-311)."""
    import runit_mac_b200 as R
    O = oracle
    rng = np.random.default_rng(300 + ff)
    wg, wu = O.rand_weights(fmt, rng, ff, k), O.rand_weights(fmt, rng, ff, k)
    x = rng.normal(0, 1, k).astype(np.float32)
    g64, u64 = O.gemv_f64(fmt, wg, x, ff, k), O.gemv_f64(fmt, wu, x, ff, k)
    ref = (g64 / (1.0 + np.exp(-g64)) * u64).astype(np.float32)
    act = ctx.new_buffer(ff * 4)
    getattr(R, "fused_ffn_%s_f32" % FMT_NAME[fmt])(ctx, ctx.buffer_from(wg), ctx.buffer_from(wu), ctx.buffer_from(x), act, ff, k)
    ctx.flush()
    assert_close(O, ref, act.download(np.float32, ff), what="fused_ffn")


@pytest.mark.parametrize("fmt,m,k,batch", [(1, 37900, 512, 8), (2, 37900, 512, 7), (1, 200, 18944, 5), (2, 200, 18944, 8),
                                           (2, 18944, 3584, 8), (1, 18944, 3584, 8), (2, 37900, 3584, 8)])
def test_batched_gemv_tensor_core_path_shapes(ctx, oracle, fmt, m, k, batch):
    """The integer tensor-core path of the 4-bit formats: 32 rows per warp (many tiles), K split over clusters of 8
    (few tiles, long K), ragged last tile, and the FFN shape of the benchmark configuration."""
    import runit_mac_b200 as R
    O = oracle
    rng = np.random.default_rng(m + k + batch)
    w = O.rand_weights(fmt, rng, m, k)
    x = rng.normal(0, 1, (batch, k)).astype(np.float32)
    res = rng.normal(0, 1, (batch, m)).astype(np.float32)
    rows = np.unique(np.concatenate([np.arange(0, min(m, 70)), rng.integers(0, m, 200), np.arange(m - 40, m)]))
    rb = O.row_bytes(fmt, k)
    ref = O.gemv(fmt, w.reshape(m, rb)[rows].copy(), x, len(rows), k, O.TIER_F64).reshape(batch, len(rows))
    yb = ctx.new_buffer(batch * m * 4)
    R.gemv_batched_f32(ctx, fmt, ctx.buffer_from(w), ctx.buffer_from(x), yb, ctx.buffer_from(res), m, k, batch)
    ctx.flush()
    got = yb.download(np.float32, batch * m).reshape(batch, m)
    assert_close(O, ref + res[:, rows], got[:, rows], what="batched tensor-core path")
    # the same call twice gives the same bits (fixed reduction order across the cluster)
    R.gemv_batched_f32(ctx, fmt, ctx.buffer_from(w), ctx.buffer_from(x), yb, ctx.buffer_from(res), m, k, batch)
    ctx.flush()
    assert np.array_equal(got, yb.download(np.float32, batch * m).reshape(batch, m))


@pytest.mark.parametrize("fmt", [1, 2])
def test_batched_gemv_launch_shapes(ctx, oracle, fmt):
    """Every launch shape of the integer tensor-core path that the size rules can pick (rows per warp 16 / 32, cluster size
    1 / 2 / 4 / 8 over K, ring depth 2 / 3 / 6), forced on one ragged matrix: the same results to the bar, and the same bits
    whenever the reduction order is the same (same cluster size)."""
    import runit_mac_b200 as R
    O = oracle
    m, k, batch = 1000, 3584, 8
    rng = np.random.default_rng(77 + fmt)
    w = O.rand_weights(fmt, rng, m, k)
    x = rng.normal(0, 1, (batch, k)).astype(np.float32)
    ref = O.gemv(fmt, w, x, m, k, O.TIER_F64)
    wb, xb, yb = ctx.buffer_from(w), ctx.buffer_from(x), ctx.new_buffer(batch * m * 4)
    first = {}
    try:
        for rw in (16, 32):
            for cs in (1, 2, 4, 8):
                for stages in (2, 3, 6):
                    for key, val in (("imma_rw", rw), ("imma_csplit", cs), ("imma_stages", stages)):
                        ctx.set_tuning(key, val)
                    R.gemv_batched_f32(ctx, fmt, wb, xb, yb, None, m, k, batch)
                    ctx.flush()
                    got = yb.download(np.float32, batch * m)
                    assert_close(O, ref, got, what="batched, %d rows per warp, cluster of %d, %d stages" % (rw, cs, stages))
                    assert np.array_equal(first.setdefault(cs, got), got), (rw, cs, stages)
    finally:
        for key in ("imma_rw", "imma_csplit", "imma_stages"):
            ctx.set_tuning(key, 0)


@pytest.mark.parametrize("fmt", [0, 1, 2])
@pytest.mark.parametrize("batch", [1, 2, 3, 8])
def test_batched_gemv(ctx, oracle, fmt, batch):
    import runit_mac_b200 as R
    O = oracle
    m, k = {0: (100, 896), 1: (100, 3584), 2: (100, 3584)}[fmt]
    rng = np.random.default_rng(900 + fmt * 10 + batch)
    w = O.rand_weights(fmt, rng, m, k)
    x = rng.normal(0, 1, (batch, k)).astype(np.float32)
    res = rng.normal(0, 1, (batch, m)).astype(np.float32)
    ref = O.gemv(fmt, w, x, m, k, O.TIER_F64)
    yb = ctx.new_buffer(batch * m * 4)
    R.gemv_batched_f32(ctx, fmt, ctx.buffer_from(w), ctx.buffer_from(x), yb, None, m, k, batch)
    ctx.flush()
    assert_close(O, ref, yb.download(np.float32, batch * m), what="batched")
    R.gemv_batched_f32(ctx, fmt, ctx.buffer_from(w), ctx.buffer_from(x), yb, ctx.buffer_from(res), m, k, batch)
    ctx.flush()
    assert_close(O, ref + res, yb.download(np.float32, batch * m), what="batched+res")


def test_known_answer_blocks_on_gpu(ctx, oracle):
    """The hand-derived block cases and the all-zero Q4_K fixture of the reference's integration
    test (crates/engine/tests/qwen2_load_test.rs:104-118) through the CUDA kernels."""
    import runit_mac_b200 as R
    O = oracle
    w = O.pack_q8_0(np.ones((1, 1)), (np.arange(32) - 16).reshape(1, 1, 32))
    assert run_gemv(ctx, R, "gemv_q8_0_f32in_f32out", w, np.ones(32, np.float32), 1, 32)[0] == -16.0
    raw = np.zeros((1, 18), np.uint8)
    raw[0, 0:2] = np.frombuffer(np.float16(1.0).tobytes(), np.uint8)
    raw[0, 2:] = 0xF0
    x = np.zeros(32, np.float32); x[0::2] = 1.0
    assert run_gemv(ctx, R, "gemv_q4_0_f32in_f32out", raw, x, 1, 32)[0] == -128.0
    x = np.zeros(32, np.float32); x[1::2] = 1.0
    assert run_gemv(ctx, R, "gemv_q4_0_f32in_f32out", raw, x, 1, 32)[0] == 112.0
    for j in range(8):
        sc = np.zeros((1, 1, 8), np.uint8); mn = np.zeros((1, 1, 8), np.uint8)
        sc[0, 0, j] = 49 if j >= 4 else 1
        w = O.pack_q4k(np.ones((1, 1)), np.zeros((1, 1)), sc, mn, np.full((1, 1, 256), 3, np.uint8))
        x = np.arange(256, dtype=np.float32)
        pair, hi = (j - 4, 1) if j >= 4 else (j, 0)
        lo = 64 * pair + 32 * hi
        want = 3.0 * sc[0, 0, j] * x[lo:lo + 32].sum()
        assert run_gemv(ctx, R, "gemv_q4k_f32in_f32out", w, x, 1, 256)[0] == want, j
    m, k = 40, 512
    w = np.zeros((m, k // 256, 144), np.uint8)
    w[:, :, 0:2] = np.frombuffer(np.float16(1.0).tobytes(), np.uint8)
    x = np.random.default_rng(3).normal(0, 1, k).astype(np.float32)
    assert (run_gemv(ctx, R, "gemv_q4k_f32in_f32out", w, x, m, k) == 0).all()
    res = np.arange(m, dtype=np.float32)
    assert (run_gemv(ctx, R, "gemv_q4k_add_f32_f32in", w, x, m, k, residual=res) == res).all()


def test_golden_fixtures_on_gpu(ctx, oracle):
    import runit_mac_b200 as R
    O = oracle
    G = np.load(GOLD)
    i = 0
    while "gemv%d_fmt" % i in G:
        fmt, m, k = map(int, G["gemv%d_fmt" % i])
        x = G["gemv%d_x" % i]
        yb = ctx.new_buffer(2 * m * 4)
        R.gemv_batched_f32(ctx, fmt, ctx.buffer_from(G["gemv%d_w" % i]), ctx.buffer_from(x), yb, None, m, k, 2)
        ctx.flush()
        assert_close(O, G["gemv%d_y" % i], yb.download(np.float32, 2 * m), what="golden %d" % i)
        i += 1


def test_dequant_and_glue_ops(ctx, oracle):
    import runit_mac_b200 as R
    O = oracle
    rng = np.random.default_rng(21)
    nb = 37
    w = O.rand_q4k(rng, 1, nb * 256)
    out = ctx.new_buffer(nb * 256 * 2)
    R.dequant_q4k_f16(ctx, ctx.buffer_from(w), out, nb)
    ctx.flush()
    assert (out.download(np.uint16, nb * 256) == O.dequant_q4k_f16(w, nb).view(np.uint16)).all()   # bit-exact
    n = 1000
    g = rng.normal(0, 2, n).astype(np.float32); u = rng.normal(0, 2, n).astype(np.float32)
    o = ctx.new_buffer(n * 4)
    R.silu_mul_f32(ctx, ctx.buffer_from(g), ctx.buffer_from(u), o, n)
    ctx.flush()
    assert np.allclose(o.download(np.float32, n), O.silu_mul_f32(g, u), rtol=2e-6, atol=1e-7)
    g16, u16 = g.astype(np.float16), u.astype(np.float16)
    R.silu_mul_f16(ctx, ctx.buffer_from(g16), ctx.buffer_from(u16), o, n)
    ctx.flush()
    assert f16_ulp_close(O.silu_mul_f16(g16, u16), o.download(np.float16, n))
    acc = rng.normal(0, 1, n).astype(np.float16)
    ab = ctx.buffer_from(acc)
    R.scale_accumulate_f16(ctx, ctx.buffer_from(g16), ab, 0.37, n)
    ctx.flush()
    assert (ab.download(np.uint16, n) == O.scale_accumulate_f16(g16, acc, 0.37).view(np.uint16)).all()   # bit-exact
    a32 = rng.normal(0, 1, n).astype(np.float32)
    ab = ctx.buffer_from(a32)
    R.add_f16_into_f32(ctx, ctx.buffer_from(g16), ab, n)
    ctx.flush()
    assert (ab.download(np.float32, n) == O.add_f16_into_f32(g16, a32)).all()   # bit-exact


def test_router_gemv_known_answers(ctx, oracle):
    """The reference's smoke binary (crates/engine/src/bin/test_gemv.rs:10-136) through the CUDA kernel."""
    import runit_mac_b200 as R

    def run(w16, x, m, k):
        y = ctx.new_buffer(max(16, m * 2))
        R.gemv_f16w_f32in(ctx, ctx.buffer_from(w16), ctx.buffer_from(x), y, m, k)
        ctx.flush()
        return y.download(np.float16, m).astype(np.float32)

    assert np.abs(run(np.eye(4, dtype=np.float16), np.array([1, 2, 3, 4], np.float32), 4, 4) - [1, 2, 3, 4]).max() < 0.01
    assert np.abs(run(np.ones((32, 32), np.float16), np.arange(1, 33, dtype=np.float32), 32, 32) - 528).max() < 1.0
    m = k = 896
    i = np.arange(m * k)
    w = (((i % 17).astype(np.float32) - 8.0) * np.float32(0.001)).astype(np.float16).reshape(m, k)
    x = ((np.arange(k) % 13).astype(np.float32) - 6.0) * np.float32(0.01)
    ref = w.astype(np.float64) @ x.astype(np.float64)
    got = run(w, x, m, k)
    assert np.abs(got - ref).max() < 0.1
    assert f16_ulp_close(oracle.gemv_f16w_f32in(w, x, m, k).astype(np.float16), got.astype(np.float16))


def test_bad_arguments_return_status_not_faults(ctx):
    import runit_mac_b200 as R
    b = ctx.new_buffer(4096)
    for args in ((b, b, b, 0, 256), (b, b, b, 4, 100), (None, b, b, 4, 256), (b, None, b, 4, 256), (b, b, None, 4, 256)):
        with pytest.raises(R.KernelError) as e:
            R.gemv_q4k_f32in_f32out(ctx, *args)
        assert e.value.status == 2
    with pytest.raises(R.KernelError):
        R.gemv_q8_0_f32in_f32out(ctx, b, b, b, 4, 48)          # k not a multiple of 32
    with pytest.raises(R.KernelError):
        R.gemv_batched_f32(ctx, 2, b, b, b, None, 4, 256, 9)   # batch > 8
    with pytest.raises(R.KernelError):
        R.gemv_q4k_f32in_f32out(ctx, b.ptr + 2, b, b, 4, 256)  # misaligned weight pointer
    ctx.flush()   # context still healthy


def test_full_size_lm_head_sampled_rows(ctx, oracle):
    """Benchmark-size matrices (Qwen2.5-7B lm_head 152064x3584, device-generated weights): a random
    sample of rows is copied back and checked against the oracle, plus linearity y(a*x1+x2) =
    a*y(x1)+y(x2), which holds at any size."""
    import runit_mac_b200 as R
    O = oracle
    m, k = 152064, 3584
    for fmt in (1, 2):
        rb = R.row_bytes(fmt, k)
        wb = ctx.new_buffer(m * rb)
        R.fill_weights(ctx, fmt, wb, m * (k // R.BLOCK_ELEMS[fmt]), 1002 + fmt, 0.02 if fmt == 1 else 0.01)
        rng = np.random.default_rng(4 + fmt)
        x1 = rng.normal(0, 1, k).astype(np.float32); x2 = rng.normal(0, 1, k).astype(np.float32)
        ys = []
        for x in (x1, x2, np.float32(0.5) * x1 + x2):
            yb = ctx.new_buffer(m * 4)
            getattr(R, "gemv_%s_f32in_f32out" % FMT_NAME[fmt])(ctx, wb, ctx.buffer_from(x), yb, m, k)
            ctx.flush()
            ys.append(yb.download(np.float32, m))
        rows = np.unique(np.concatenate([[0, 1, 31, 32, m - 1, m - 32, m - 33], rng.integers(0, m, 200)]))
        for r in rows:
            wr = wb.download(np.uint8, rb, offset=int(r) * rb)
            ref = O.gemv(fmt, wr, x1, 1, k, O.TIER_F64)[0]
            scale = max(abs(ref), float(np.sqrt(np.mean(ys[0] ** 2))))
            assert abs(ys[0][r] - ref) <= REL_TOL * scale, (fmt, r)
        lin = np.float32(0.5) * ys[0] + ys[1]
        # the three products round their activations to 16-bit block fixed point independently
        assert_close(O, lin, ys[2], rel_tol=5e-4, what="linearity")
        wb.free()


@pytest.mark.parametrize("fmt", [0, 1, 2])
def test_non_finite_activations_are_not_masked(ctx, oracle, fmt):
    """A NaN or an Inf in the activations must reach the output, as it does through the reference's f32 multiply-add
    chain (gemv_q8_0.metal:24-36, gemv_q4_0.metal:26-49, gemv_q4k.metal:85-122): every row whose dot product includes
    the bad element ends non-finite.  The integer paths quantise activations per 32-block, so their rule is: a block
    that holds a non-finite value makes every row NaN.  Host-made inputs only; batch 1 (integer tensor-core / dp4a
    paths) and batch 8 (batched integer tensor-core path, only the bad activation row is affected)."""
    import runit_mac_b200 as R
    O = oracle
    m, k = {0: (96, 896), 1: (96, 3584), 2: (96, 2048)}[fmt]
    rng = np.random.default_rng(77 + fmt)
    w = O.rand_weights(fmt, rng, m, k)
    wb = ctx.buffer_from(w)
    name = "gemv_%s_f32in_f32out" % FMT_NAME[fmt]
    for bad, pos in ((np.nan, 5), (np.inf, k - 3), (-np.inf, k // 2)):
        x = rng.normal(0, 1, k).astype(np.float32)
        x[pos] = bad
        yb = ctx.new_buffer(m * 4)
        getattr(R, name)(ctx, wb, ctx.buffer_from(x), yb, m, k)
        ctx.flush()
        got = yb.download(np.float32, m)
        assert not np.isfinite(got).any(), (FMT_NAME[fmt], bad, int(np.isfinite(got).sum()))
        # the other arithmetic paths of the batch-1 kernel agree
        for math in (1, 2):
            ctx.set_tuning("gemv_math", math)
            try:
                getattr(R, name)(ctx, wb, ctx.buffer_from(x), yb, m, k)
                ctx.flush()
            finally:
                ctx.set_tuning("gemv_math", 0)
            assert not np.isfinite(yb.download(np.float32, m)).any(), (FMT_NAME[fmt], bad, math)
        xs = rng.normal(0, 1, (8, k)).astype(np.float32)
        xs[3, pos] = bad
        y8 = ctx.new_buffer(8 * m * 4)
        R.gemv_batched_f32(ctx, fmt, wb, ctx.buffer_from(xs), y8, None, m, k, 8)
        ctx.flush()
        got8 = y8.download(np.float32, 8 * m).reshape(8, m)
        assert not np.isfinite(got8[3]).any() and np.isfinite(np.delete(got8, 3, 0)).all()
        ref = O.gemv(fmt, w, np.delete(xs, 3, 0), m, k, O.TIER_F64)
        assert_close(O, ref, np.delete(got8, 3, 0), what="finite rows beside a non-finite one")
    # a finite input still gives a finite, correct result afterwards
    x = rng.normal(0, 1, k).astype(np.float32)
    assert_close(O, O.gemv(fmt, w, x, m, k, O.TIER_F64), run_gemv(ctx, R, name, w, x, m, k), what="after non-finite")


@pytest.mark.parametrize("fmt", [0, 1, 2])
def test_rms_norm_inside_the_gemv(ctx, oracle, fmt):
    """RMSNorm (norm.metal:95-154, f32 gamma) fused into the GEMV and into Q|K|V: compared with the oracle's norm followed by
    its GEMV; staged kernel with and without dependent launch, the other arithmetic paths, and the simple kernel."""
    import runit_mac_b200 as R
    O = oracle
    eps = 1e-5
    for m, k in ((512, 2048), (37, 1024), (70, 2080 if fmt != 2 else 2304)):
        rng = np.random.default_rng(7000 + fmt * 10 + m)
        w = O.rand_weights(fmt, rng, m, k)
        x = rng.normal(0, 3.0, k).astype(np.float32)
        gamma = rng.normal(1, 0.2, k).astype(np.float32)
        res = rng.normal(0, 1, m).astype(np.float32)
        xn = O.rms_norm_f32(x, gamma, eps)
        ref = O.gemv(fmt, w, xn, m, k)
        wb, xb, gb, rb = ctx.buffer_from(w), ctx.buffer_from(x), ctx.buffer_from(gamma), ctx.buffer_from(res)
        yb = ctx.new_buffer(m * 4)
        for knob, val in (("pdl", 0), ("pdl", 1), ("gemv_math", 1), ("gemv_math", 2), ("gemv_variant", 1)):
            ctx.set_tuning(knob, val)
            try:
                R.rms_norm_gemv_f32(ctx, fmt, wb, xb, gb, eps, yb, None, m, k)
                ctx.flush()
                assert_close(O, ref, yb.download(np.float32, m), what="norm+gemv fmt=%d %dx%d %s=%d" % (fmt, m, k, knob, val))
                R.rms_norm_gemv_f32(ctx, fmt, wb, xb, gb, eps, yb, rb, m, k)
                ctx.flush()
                assert_close(O, ref + res, yb.download(np.float32, m), what="norm+gemv+res fmt=%d %dx%d" % (fmt, m, k))
            finally:
                ctx.set_tuning(knob, 0)
    # Q|K|V with the norm inside
    q_dim, kv_dim, k = 1024, 256, 2048
    rng = np.random.default_rng(7100 + fmt)
    ws = [O.rand_weights(fmt, rng, n, k) for n in (q_dim, kv_dim, kv_dim)]
    x = rng.normal(0, 0.5, k).astype(np.float32)
    gamma = rng.normal(1, 0.2, k).astype(np.float32)
    xn = O.rms_norm_f32(x, gamma, eps)
    outs = [ctx.new_buffer(n * 4) for n in (q_dim, kv_dim, kv_dim)]
    R.rms_norm_fused_qkv_f32(ctx, fmt, *[ctx.buffer_from(w) for w in ws], ctx.buffer_from(x), ctx.buffer_from(gamma), eps, *outs,
                             q_dim, kv_dim, k)
    ctx.flush()
    for o, w, n in zip(outs, ws, (q_dim, kv_dim, kv_dim)):
        assert_close(O, O.gemv(fmt, w, xn, n, k), o.download(np.float32, n), what="norm+qkv fmt=%d" % fmt)


@pytest.mark.parametrize("fmt", [1, 2])
def test_greedy_epilogue_of_the_gemv(ctx, oracle, fmt):
    """lm_head with the argmax inside the launch (argmax after lm_head, forward.rs:1967-1973): the token equals the argmax of
    the logits the same launch wrote (lowest index among equal values), with and without the RMSNorm prologue, on ragged
    row counts, repeatedly (the ticket counter returns to zero), and with duplicated rows (a tie)."""
    import runit_mac_b200 as R
    O = oracle
    for m, k in ((50304 // 8, 2048), (1000, 512), (31, 256)):
        rng = np.random.default_rng(8800 + fmt + m)
        w = O.rand_weights(fmt, rng, m, k)
        rb = w.size // m
        w = w.reshape(m, rb)
        w[m // 2] = w[3]                       # rows 3 and m/2 give the same logit: a tie if it is the maximum
        x = rng.normal(0, 1, k).astype(np.float32)
        gamma = rng.normal(1, 0.1, k).astype(np.float32)
        wb, xb, gb = ctx.buffer_from(w.reshape(-1)), ctx.buffer_from(x), ctx.buffer_from(gamma)
        lb, tb = ctx.new_buffer(m * 4), ctx.new_buffer(16)
        for g in (None, gb):
            for rep in range(3):
                R.gemv_argmax_f32(ctx, fmt, wb, xb, g, 1e-5, lb, tb, m, k)
                ctx.flush()
                logits = lb.download(np.float32, m)
                assert int(tb.download(np.int32, 1)[0]) == int(np.argmax(logits)), (fmt, m, k, g is not None, rep)
            xin = x if g is None else O.rms_norm_f32(x, gamma, 1e-5)
            assert_close(O, O.gemv(fmt, w.reshape(-1), xin, m, k), logits, what="gemv_argmax logits")
        # force the tie to be the maximum: one input that aligns with row 3
        xt = np.zeros(k, np.float32)
        xt[:] = O.dequant_rows(fmt, w[3].copy(), 1, k).reshape(-1)
        ctx.call("memcpy_h2d", xb, xt.ctypes.data, xt.nbytes)
        R.gemv_argmax_f32(ctx, fmt, wb, xb, None, 0.0, lb, tb, m, k)
        ctx.flush()
        logits = lb.download(np.float32, m)
        assert int(tb.download(np.int32, 1)[0]) == int(np.argmax(logits))
        assert logits[3] == logits[m // 2]


@pytest.mark.parametrize("fold", [0, 1])
@pytest.mark.parametrize("batch", [8, 3])
@pytest.mark.parametrize("fmt", [1, 2])
def test_batched_gemv_of_several_matrices_in_one_launch(ctx, oracle, fmt, batch, fold):
    """q | k | v and gate | up at batch 2..8: one launch over up to three matrices that share the activations (prepared once)
    gives what the single-matrix launches give, and the oracle's values."""
    import runit_mac_b200 as R
    O = oracle
    ctx.set_tuning("imma_fold", fold)      # 1: the activation pre-pass inside the GEMV launch (opt-in variant)
    try:
        _multi_cases(ctx, R, O, fmt, batch)
    finally:
        ctx.set_tuning("imma_fold", 0)


def _multi_cases(ctx, R, O, fmt, batch):
    for rows, k in (((3584, 512, 512), 3584), ((1000, 37), 2048), ((96,), 512)):
        rng = np.random.default_rng(9000 + fmt + batch + len(rows))
        ws = [O.rand_weights(fmt, rng, m, k) for m in rows]
        x = rng.normal(0, 1, (batch, k)).astype(np.float32)
        wb, xb = [ctx.buffer_from(w) for w in ws], ctx.buffer_from(x)
        outs = [ctx.new_buffer(batch * m * 4) for m in rows]
        R.gemv_batched_multi_f32(ctx, fmt, wb, xb, outs, rows, k, batch)
        ctx.flush()
        for w, m, o, b1 in zip(ws, rows, outs, wb):
            got = o.download(np.float32, batch * m)
            assert_close(O, O.gemv(fmt, w, x, m, k), got, what="multi batched fmt=%d %dx%d batch=%d" % (fmt, m, k, batch))
            single = ctx.new_buffer(batch * m * 4)
            R.gemv_batched_f32(ctx, fmt, b1, xb, single, None, m, k, batch)
            ctx.flush()
            assert np.array_equal(single.download(np.float32, batch * m), got)
