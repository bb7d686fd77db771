"""GPU parity tests of the fused-dequant GEMVs for Q5_0, Q5_K and Q6_K (formats the reference only dequantises on the
CPU, crates/engine/src/forward.rs:900-949, 979-1012) against the oracle's restatement of those formulas."""
import numpy as np
import pytest

from helpers import assert_close

pytestmark = pytest.mark.gpu
NAME = {3: "q5_0", 4: "q5k", 5: "q6k"}
SHAPES = {3: [(5, 32), (64, 96), (37, 3584), (200, 2080), (1, 18944)], 4: [(3, 256), (65, 1024), (37, 3584), (300, 2048), (2, 18944)],
          5: [(3, 256), (65, 1024), (37, 3584), (301, 2048), (2, 18944), (33, 768)]}


@pytest.mark.parametrize("fmt", [3, 4, 5])
def test_gemv_matches_oracle(ctx, oracle, fmt):
    import runit_mac_b200 as R
    O = oracle
    for m, k in SHAPES[fmt]:
        rng = np.random.default_rng(fmt * 1000 + m + k)
        w = O.rand_weights(fmt, rng, m, k)
        x = rng.normal(0, 1, k).astype(np.float32)
        res = rng.normal(0, 1, m).astype(np.float32)
        ref = O.gemv(fmt, w, x, m, k, O.TIER_F64)
        wb, xb, yb = ctx.buffer_from(w), ctx.buffer_from(x), ctx.new_buffer(max(16, 4 * m))
        getattr(R, "gemv_%s_f32in_f32out" % NAME[fmt])(ctx, wb, xb, yb, m, k)
        ctx.flush()
        st = assert_close(O, ref, yb.download(np.float32, m), what="%s %dx%d" % (NAME[fmt], m, k))
        assert st.max_rel < 2e-5
        rb = ctx.buffer_from(res)
        getattr(R, "gemv_%s_add_f32_f32in" % NAME[fmt])(ctx, wb, xb, rb, rb, m, k)      # in place, like the engine's residual adds
        ctx.flush()
        assert_close(O, ref + res, rb.download(np.float32, m), what="%s + residual" % NAME[fmt])


def test_rows_that_start_off_word_boundaries(ctx, oracle):
    """Q6_K rows of an odd number of superblocks are 210 * odd bytes long: every other row starts two bytes off a word
    boundary; a weight pointer into the middle of a buffer (16-byte aligned) works as well."""
    import runit_mac_b200 as R
    O = oracle
    rng = np.random.default_rng(6)
    m, k = 41, 768
    w = O.rand_weights(5, rng, m + 8, k).reshape(-1)
    x = rng.normal(0, 1, k).astype(np.float32)
    rb = O.row_bytes(5, k)
    assert rb % 4 == 2
    wb, xb, yb = ctx.buffer_from(w), ctx.buffer_from(x), ctx.new_buffer(4 * m)
    R.gemv_q6k_f32in_f32out(ctx, wb.ptr + 8 * rb, xb, yb, m, k)     # 8 rows in: 5040 bytes, a multiple of 16
    ctx.flush()
    assert_close(O, O.gemv(5, w[8 * rb:], x, m, k), yb.download(np.float32, m), what="q6k offset rows")


def test_known_answer_blocks_and_argument_checks(ctx, oracle):
    import runit_mac_b200 as R
    y = ctx.new_buffer(16)
    # Q6_K block of the oracle test: d = 1, scales 1..16, every q = 1: row . ones = 32 * (1+3+5+7+9+11+13+15) = 2048
    blk = np.zeros(210, np.uint8)
    blk[0:128] = 0x11
    blk[128:192] = 0xAA
    blk[192:208] = np.arange(1, 17, dtype=np.uint8)
    blk[208:210] = np.array([1.0], np.float16).view(np.uint8)
    R.gemv_q6k_f32in_f32out(ctx, ctx.buffer_from(blk), ctx.buffer_from(np.ones(256, np.float32)), y, 1, 256)
    ctx.flush()
    assert y.download(np.float32, 1)[0] == 2048.0
    # Q5_0 block: d = 1, qs = 0x10, qh = 0x0000FFFF: elements 0..15 are 0, 16..31 are -15: dot with 1..32 = -15 * sum(17..32)
    blk = np.zeros(22, np.uint8)
    blk[0:2] = np.array([1.0], np.float16).view(np.uint8)
    blk[2:4] = 0xFF
    blk[6:] = 0x10
    R.gemv_q5_0_f32in_f32out(ctx, ctx.buffer_from(blk), ctx.buffer_from(np.arange(1, 33, dtype=np.float32)), y, 1, 32)
    ctx.flush()
    assert y.download(np.float32, 1)[0] == -15.0 * sum(range(17, 33))
    w = ctx.new_buffer(4096)
    x = ctx.new_buffer(4096)
    for bad in (lambda: R.gemv_q6k_f32in_f32out(ctx, w, x, y, 1, 200), lambda: R.gemv_q5k_f32in_f32out(ctx, w, x, y, 0, 256),
                lambda: R.gemv_q5_0_f32in_f32out(ctx, w, x, y, 1, 48), lambda: R.gemv_q5k_add_f32_f32in(ctx, w, x, y, None, 1, 256)):
        with pytest.raises(R.KernelError):
            bad()


@pytest.mark.parametrize("fmt,tag", [(5, "q6k"), (4, "q5k"), (3, "q5_0")])
def test_kquant_tile_kernel(ctx, oracle, fmt, tag):
    """The Q6_K, Q5_K and Q5_0 tile kernels (lane = row, 32-row tiles, dp4a against three 8-bit limbs of the activations; forced here also on
    shapes it would leave to the first kernel; (130, 18944) and (301, 2048) split K over several CTAs per tile, the others
    over the four warps of one): the oracle's values at the bar of the other kernel, rows that start two bytes off a word boundary (Q6_K), the in-place residual, a non-finite activation, and agreement
    with the first kernel."""
    import runit_mac_b200 as R
    O = oracle
    gemv, gemv_add = getattr(R, "gemv_%s_f32in_f32out" % tag), getattr(R, "gemv_%s_add_f32_f32in" % tag)
    ctx.set_tuning("kquant_variant", 2)
    try:
        for m, k in ((3, 256), (65, 1024), (37, 3584), (301, 2048), (130, 18944), (41, 768), (129, 1280)):
            rng = np.random.default_rng(6000 + m + k)
            w = O.rand_weights(fmt, rng, m, k)
            x = rng.normal(0, 1, k).astype(np.float32)
            x[rng.integers(0, k, 3)] *= 300.0              # outliers: the limbs keep 23 bits per 32-block
            res = rng.normal(0, 1, m).astype(np.float32)
            ref = O.gemv(fmt, w, x, m, k, O.TIER_F64)
            wb, xb, yb = ctx.buffer_from(w), ctx.buffer_from(x), ctx.new_buffer(max(16, 4 * m))
            gemv(ctx, wb, xb, yb, m, k)
            ctx.flush()
            got = yb.download(np.float32, m)
            st = assert_close(O, ref, got, what=tag + " tile kernel %dx%d" % (m, k))
            assert st.max_rel < 2e-5, st
            rb = ctx.buffer_from(res)
            gemv_add(ctx, wb, xb, rb, rb, m, k)
            ctx.flush()
            assert_close(O, ref + res, rb.download(np.float32, m), what=tag + " tile kernel + residual")
            ctx.set_tuning("kquant_variant", 1)
            gemv(ctx, wb, xb, yb, m, k)
            ctx.flush()
            ctx.set_tuning("kquant_variant", 2)
            assert_close(O, yb.download(np.float32, m), got, rel_tol=1e-5, what=tag + " tile kernel against the first kernel")
        # a NaN and an Inf among the activations reach every output as non-finite values
        m, k = 40, 1024
        w = O.rand_weights(fmt, np.random.default_rng(1), m, k)
        for bad in (np.nan, np.inf):
            x = np.ones(k, np.float32)
            x[517] = bad
            yb = ctx.new_buffer(4 * m)
            gemv(ctx, ctx.buffer_from(w), ctx.buffer_from(x), yb, m, k)
            ctx.flush()
            assert not np.isfinite(yb.download(np.float32, m)).any()
    finally:
        ctx.set_tuning("kquant_variant", 0)
