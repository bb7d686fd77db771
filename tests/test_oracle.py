"""CPU tests of the oracle: every known answer the reference's own tests hold for this path, the
hand-derived single-block cases that follow from the block layouts documented in the shaders,
agreement of the three accumulation tiers, and the committed golden vectors.

(The reference has no golden vector for any quantized operator — parity for them is unpinned;
what it does pin is exercised here.)"""
from pathlib import Path

import numpy as np
import pytest

GOLD = Path(__file__).parent / "golden" / "path_golden.npz"


def test_f16_conversion_is_ieee_rne(oracle):
    O = oracle
    rng = np.random.default_rng(1)
    x = np.concatenate([rng.normal(0, 1, 50000), rng.normal(0, 1e-6, 5000), rng.normal(0, 3e4, 5000),
                        [0.0, -0.0, 65504, 65519.99, 65520, 1e-8, 5.96e-8, 2.98e-8, 2.99e-8, 6.1e-5]]).astype(np.float32)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert (O.f32_to_f16_bits(x) == want).all()
    h = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    f, g = O.f16_bits_to_f32(h), h.view(np.float16).astype(np.float32)
    assert ((f == g) | (np.isnan(f) & np.isnan(g))).all()


# ── known answers of crates/engine/src/bin/test_gemv.rs (f16-weight GEMV = the router GEMV) ──
def test_router_gemv_identity_4x4(oracle):
    # test_gemv.rs:10-56
    y = oracle.gemv_f16w_f32in(np.eye(4, dtype=np.float16), np.array([1, 2, 3, 4], np.float32), 4, 4)
    assert np.abs(y - [1, 2, 3, 4]).max() < 0.01


def test_router_gemv_ones_32x32(oracle):
    # test_gemv.rs:58-85: all-ones x [1..32] = 528
    y = oracle.gemv_f16w_f32in(np.ones((32, 32), np.float16), np.arange(1, 33, dtype=np.float32), 32, 32)
    assert np.abs(y - 528.0).max() < 1.0 and y[0] == 528.0


def test_router_gemv_896_pattern(oracle):
    # test_gemv.rs:87-136: w=((i%17)-8)*1e-3, x=((i%13)-6)*1e-2, |gpu - f64 cpu| < 0.1
    m = k = 896
    i = np.arange(m * k)
    w = (((i % 17).astype(np.float32) - 8.0) * np.float32(0.001)).astype(np.float16).reshape(m, k)
    x = ((np.arange(k) % 13).astype(np.float32) - 6.0) * np.float32(0.01)
    ref = w.astype(np.float64) @ x.astype(np.float64)
    y = oracle.gemv_f16w_f32in(w, x, m, k)
    assert np.abs(y - ref).max() < 0.1
    assert np.abs(y - ref).max() < 1e-4   # and in fact far closer


# ── crates/engine/tests/qwen2_load_test.rs:104-118: Q4_K blocks d=1, everything else zero ──
def test_q4k_zero_blocks_give_exact_zero(oracle):
    O = oracle
    m, k = 6, 512
    w = np.zeros((m, k // 256, 144), np.uint8)
    w[:, :, 0:2] = np.frombuffer(np.float16(1.0).tobytes(), np.uint8)
    x = np.random.default_rng(3).normal(0, 1, k).astype(np.float32)
    for tier in (O.TIER_SHADER, O.TIER_DEQUANT, O.TIER_F64):
        assert (O.gemv(O.Q4K, w, x, m, k, tier) == 0).all()


# ── hand-derived single-block cases from the documented layouts ──
def test_q8_0_single_block(oracle):
    O = oracle
    # gemv_q8_0.metal:11-14: value = d*qs; d=1, qs=i-16, x=1 -> sum = -16
    w = O.pack_q8_0(np.ones((1, 1)), (np.arange(32) - 16).reshape(1, 1, 32))
    assert w.shape == (1, 34) and w[0, 0] == 0x00 and w[0, 1] == 0x3C   # f16(1.0) little-endian, scale first
    for tier in range(3):
        assert O.gemv(O.Q8_0, w, np.ones(32, np.float32), 1, 32, tier)[0] == -16.0
    # d=0.5, x = e_5 picks qs[5]*0.5
    w = O.pack_q8_0(np.full((1, 1), 0.5), (np.arange(32) * 3 - 40).reshape(1, 1, 32))
    x = np.zeros(32, np.float32); x[5] = 2.0
    assert O.gemv(O.Q8_0, w, x, 1, 32, O.TIER_SHADER)[0] == 0.5 * (15 - 40) * 2.0


def test_q4_0_interleaved_nibbles(oracle):
    O = oracle
    # gemv_q4_0.metal:10-15: low nibble = element 2i, high nibble = element 2i+1, value = d*(nib-8)
    raw = np.zeros((1, 18), np.uint8)
    raw[0, 0:2] = np.frombuffer(np.float16(1.0).tobytes(), np.uint8)
    raw[0, 2:] = 0xF0   # low nibble 0 -> -8 at even elements, high nibble 15 -> +7 at odd elements
    deq = O.dequant_rows(O.Q4_0, raw, 1, 32)[0]
    assert (deq[0::2] == -8).all() and (deq[1::2] == 7).all()
    x = np.zeros(32, np.float32); x[0::2] = 1.0
    assert O.gemv(O.Q4_0, raw, x, 1, 32, O.TIER_SHADER)[0] == -8.0 * 16
    x = np.zeros(32, np.float32); x[1::2] = 1.0
    assert O.gemv(O.Q4_0, raw, x, 1, 32, O.TIER_F64)[0] == 7.0 * 16
    # packer agrees with the layout
    nib = np.zeros((1, 1, 32), np.uint8); nib[0, 0, 1::2] = 15
    assert (O.pack_q4_0(np.ones((1, 1)), nib) == raw).all()


def test_q4k_scale_unpack_and_nibble_mapping(oracle):
    O = oracle
    # dequant.metal:42-51,74-82: sub-block j<4 -> low nibbles of qs[32j..] (elements 64j..64j+31);
    # sub-block j+4 -> high nibbles (elements 64j+32..64j+63); 6-bit scales, upper two bits of
    # scale j+4 live in scales[j]>>6.
    for j in range(8):
        sc = np.zeros((1, 1, 8), np.uint8); mn = np.zeros((1, 1, 8), np.uint8)
        sc[0, 0, j] = 49 if j >= 4 else 1      # 49 needs the two high bits
        nib = np.full((1, 1, 256), 3, np.uint8)
        w = O.pack_q4k(np.ones((1, 1)), np.zeros((1, 1)), sc, mn, nib)
        deq = O.dequant_rows(O.Q4K, w, 1, 256)[0]
        pair, hi = (j - 4, 1) if j >= 4 else (j, 0)
        lo_el = 64 * pair + 32 * hi
        want = np.zeros(256, np.float32); want[lo_el:lo_el + 32] = 3.0 * sc[0, 0, j]
        assert (deq == want).all(), j
    # min term: dmin*m subtracted
    sc = np.zeros((1, 1, 8), np.uint8); mn = np.zeros((1, 1, 8), np.uint8); mn[0, 0, 6] = 37
    w = O.pack_q4k(np.zeros((1, 1)), np.full((1, 1), 0.5), sc, mn, np.zeros((1, 1, 256), np.uint8))
    deq = O.dequant_rows(O.Q4K, w, 1, 256)[0]
    assert (deq[64 * 2 + 32:64 * 2 + 64] == -18.5).all() and np.count_nonzero(deq) == 32
    # dequant_q4k_f16 agrees with the row dequant rounded to f16
    rng = np.random.default_rng(5)
    w = O.rand_q4k(rng, 3, 512)
    assert (O.dequant_q4k_f16(w, 6).view(np.uint16) ==
            O.dequant_rows(O.Q4K, w, 3, 512).astype(np.float16).reshape(-1).view(np.uint16)).all()


@pytest.mark.parametrize("fmt,m,k", [(0, 19, 896), (0, 4, 4864), (1, 21, 3584), (1, 7, 96), (2, 13, 2048), (2, 5, 18944)])
def test_tiers_agree(oracle, fmt, m, k):
    """Shader-order f32, dequant-then-dot f32 and f64 accumulation agree to f32 rounding; this
    cross-checks the packers against three independently written decoders."""
    O = oracle
    rng = np.random.default_rng(100 + fmt * 7 + m)
    w = O.rand_weights(fmt, rng, m, k)
    x = rng.normal(0, 1, (2, k)).astype(np.float32)
    y64 = O.gemv_f64(fmt, w, x, m, k)
    mag = np.abs(O.dequant_rows(fmt, w, m, k)) @ np.abs(x).T   # [m, batch] sum |w||x|
    for tier in (O.TIER_SHADER, O.TIER_DEQUANT):
        y = O.gemv(fmt, w, x, m, k, tier)
        assert (np.abs(y - y64) <= 4e-6 * mag.T + 1e-30).all()
    # and against a numpy restatement of the dequantised matrix
    ref = x.astype(np.float64) @ O.dequant_rows(fmt, w, m, k).astype(np.float64).T
    assert np.allclose(y64, ref, rtol=1e-12, atol=1e-12)


def test_topk_softmax_semantics(oracle):
    O = oracle
    rng = np.random.default_rng(9)
    lg = rng.normal(0, 1, 64).astype(np.float32)
    idx, w, probs = O.topk_softmax(lg, 8, False)
    order = np.argsort(-probs, kind="stable")[:8]
    assert (idx == order).all()                       # descending probability
    assert np.allclose(probs.sum(), 1.0, atol=1e-6)   # softmax over ALL experts first (forward.rs:2424-2428)
    assert np.allclose(w, probs[idx]) and w.sum() < 1.0
    _, wr, _ = O.topk_softmax(lg, 8, True)            # renormalised (forward.rs:2438-2445)
    assert np.allclose(wr.sum(), 1.0, atol=1e-6) and np.allclose(wr, w / w.sum(), rtol=1e-6)
    # ties: lowest index first
    idx, _, _ = O.topk_softmax(np.zeros(16, np.float32), 4, False)
    assert list(idx) == [0, 1, 2, 3]
    with pytest.raises(ValueError):
        O.topk_softmax(lg, 65, False)


def test_moe_glue_ops(oracle):
    O = oracle
    rng = np.random.default_rng(11)
    g = rng.normal(0, 2, 300).astype(np.float32); u = rng.normal(0, 2, 300).astype(np.float32)
    want = g / (1 + np.exp(-g.astype(np.float64))) * u
    assert np.allclose(O.silu_mul_f32(g, u), want, rtol=1e-6, atol=1e-7)
    g16, u16 = g.astype(np.float16), u.astype(np.float16)
    want16 = (g16.astype(np.float64) / (1 + np.exp(-g16.astype(np.float64))) * u16.astype(np.float64)).astype(np.float16)
    got16 = O.silu_mul_f16(g16, u16)
    assert np.abs(got16.astype(np.float32) - want16.astype(np.float32)).max() <= 2e-3 * np.abs(want16).max()
    acc = rng.normal(0, 1, 300).astype(np.float16)
    out = O.scale_accumulate_f16(g16, acc, 0.37)
    want = (acc.astype(np.float32) + (g16.astype(np.float32) * np.float32(0.37)).astype(np.float16).astype(np.float32)).astype(np.float16)
    assert (out.view(np.uint16) == want.view(np.uint16)).all()
    a32 = rng.normal(0, 1, 300).astype(np.float32)
    assert (O.add_f16_into_f32(g16, a32) == a32 + g16.astype(np.float32)).all()


def test_moe_layer_modes(oracle):
    O = oracle
    rng = np.random.default_rng(13)
    h, ff, E, k = 256, 256, 4, 2
    router = rng.normal(0, 0.02, (E, h)).astype(np.float32)
    gate, up, down = O.rand_q4k(rng, E * ff, h), O.rand_q4k(rng, E * ff, h), O.rand_q4k(rng, E * h, ff)
    x = rng.normal(0, 1, (2, h)).astype(np.float32)
    y, idx, w = O.moe_layer_q4k(router, gate, up, down, x, h=h, ff=ff, E=E, top_k=k, renorm=False)
    # rebuild token 0 from the primitive oracle ops
    lg = O.gemv_f32w(router, x[0], E, h)
    i0, w0, _ = O.topk_softmax(lg, k, False)
    assert (i0 == idx[0]).all() and np.allclose(w0, w[0])
    acc = np.zeros(h, np.float64)
    rb_h, rb_ff = O.row_bytes(O.Q4K, h), O.row_bytes(O.Q4K, ff)
    for e, we in zip(i0, w0):
        g = O.gemv(O.Q4K, gate.reshape(-1)[e * ff * rb_h:], x[0], ff, h)
        u = O.gemv(O.Q4K, up.reshape(-1)[e * ff * rb_h:], x[0], ff, h)
        a = O.silu_mul_f32(g, u)
        acc += np.float32(we) * O.gemv(O.Q4K, down.reshape(-1)[e * h * rb_ff:], a, h, ff)
    assert np.allclose(y[0], acc, rtol=2e-6, atol=1e-6 * np.abs(acc).max())
    # residual is added on top; renorm rescales the combine
    yr, _, wr = O.moe_layer_q4k(router, gate, up, down, x, h=h, ff=ff, E=E, top_k=k, renorm=True, residual=x)
    assert np.allclose(wr.sum(1), 1.0, atol=1e-6)
    # the reference's f16 rounding points stay within its own tolerance scale of the f32 mode
    y16, idx16, _ = O.moe_layer_q4k(router, gate, up, down, x, h=h, ff=ff, E=E, top_k=k, renorm=False,
                                    mode=O.MOE_REF_F16)
    if (idx16 == idx).all():
        finite = np.isfinite(y16)
        assert np.abs(y16[finite] - y[finite]).max() <= 2e-2 * np.abs(y).max()


def test_bf16_block_mode(oracle):
    """bf16 rounding is round-to-nearest-even on the top 16 bits; the bf16-operand block stays near the f32 block and
    gives the same result whether it routes itself or is handed that routing."""
    O = oracle
    v = np.array([1.0, 1.00390625, 1.01171875, 1.0078125, -3.14159, 0.0, 65504.0, 1e-30], np.float32)
    r = O.bf16_round(v)
    assert r.tolist()[:4] == [1.0, 1.0, 1.015625, 1.0078125]     # ties go to the even mantissa
    assert (r.view(np.uint32) & 0xFFFF == 0).all() and np.abs(r - v).max() <= np.abs(v).max() * 2.0 ** -8
    assert all(O.lib().ro_bf16_round(float(a)) == float(b) for a, b in zip(v, r))
    rng = np.random.default_rng(21)
    h, ff, E, k, T = 256, 256, 4, 2, 5
    router = rng.normal(0, 0.02, (E, h)).astype(np.float32)
    gate, up, down = O.rand_q4k(rng, E * ff, h), O.rand_q4k(rng, E * ff, h), O.rand_q4k(rng, E * h, ff)
    x = rng.normal(0, 1, (T, h)).astype(np.float32)
    y32, i32, w32 = O.moe_layer_q4k(router, gate, up, down, x, h=h, ff=ff, E=E, top_k=k, renorm=False)
    yb, ib, wb = O.moe_grouped_q4k_bf16(router, gate, up, down, x, h=h, ff=ff, E=E, top_k=k)
    assert (ib == i32).all() and np.array_equal(wb, w32)
    assert np.abs(yb - y32).max() <= 3e-2 * np.sqrt(np.mean(y32 ** 2))
    yg, _, _ = O.moe_grouped_q4k_bf16(None, gate, up, down, x, h=h, ff=ff, E=E, top_k=k, routing=(ib, wb))
    assert np.array_equal(yg, yb)
    # rebuild one output element from the primitive ops: dequantised rows rounded to bf16, x rounded to bf16
    rb_h, rb_ff = O.row_bytes(O.Q4K, h), O.row_bytes(O.Q4K, ff)
    xb = O.bf16_round(x[0]).astype(np.float64)
    acc = np.float32(0)
    for e, we in zip(ib[0], wb[0]):
        wg = O.bf16_round(O.dequant_rows(O.Q4K, gate.reshape(-1)[e * ff * rb_h:(e + 1) * ff * rb_h], ff, h)).astype(np.float64)
        wu = O.bf16_round(O.dequant_rows(O.Q4K, up.reshape(-1)[e * ff * rb_h:(e + 1) * ff * rb_h], ff, h)).astype(np.float64)
        wd = O.bf16_round(O.dequant_rows(O.Q4K, down.reshape(-1)[e * h * rb_ff:(e + 1) * h * rb_ff], h, ff)).astype(np.float64)
        g, u = (wg @ xb).astype(np.float32), (wu @ xb).astype(np.float32)
        act = O.bf16_round(O.silu_mul_f32(g, u)).astype(np.float64)
        acc = np.float32(acc + np.float32(we) * np.float32(wd[3] @ act))
    assert abs(acc - yb[0, 3]) <= 2e-6 * abs(yb[0]).max()


def test_decode_ops(oracle):
    O = oracle
    rng = np.random.default_rng(17)
    x = rng.normal(0, 1, (3, 128)).astype(np.float32); g = rng.normal(1, 0.1, 128).astype(np.float32)
    want = x / np.sqrt((x.astype(np.float64) ** 2).mean(1, keepdims=True) + 1e-5) * g
    assert np.allclose(O.rms_norm_f32(x, g, 1e-5), want, rtol=1e-6)
    # rope: position 0 is the identity; norm is preserved; pairs are (d, d+hd/2)
    q = rng.normal(0, 1, 4 * 64).astype(np.float32); kk = rng.normal(0, 1, 2 * 64).astype(np.float32)
    q0, k0 = O.rope_qk_f32(q, kk, 64, 4, 2, 0, 10000.0)
    assert (q0 == q).all() and (k0 == kk).all()
    q5, _ = O.rope_qk_f32(q, kk, 64, 4, 2, 5, 10000.0)
    assert np.allclose(np.linalg.norm(q5), np.linalg.norm(q), rtol=1e-6)
    ang = 5.0 / 10000.0 ** (2 * 3 / 64)
    assert np.allclose(q5[3], q[3] * np.cos(ang) - q[3 + 32] * np.sin(ang), rtol=1e-5, atol=1e-6)
    # attention against a plain softmax
    heads, kvh, hd, max_seq, L = 4, 2, 64, 16, 9
    kc = rng.normal(0, 1, (kvh, max_seq, hd)).astype(np.float16); vc = rng.normal(0, 1, (kvh, max_seq, hd)).astype(np.float16)
    out = O.decode_attention_f32q_f16kv(q, kc, vc, L, heads, kvh, hd, max_seq).reshape(heads, hd)
    for hq in range(heads):
        s = kc[hq // 2, :L].astype(np.float64) @ q[hq * hd:(hq + 1) * hd].astype(np.float64) / np.sqrt(hd)
        p = np.exp(s - s.max()); p /= p.sum()
        assert np.allclose(out[hq], p @ vc[hq // 2, :L].astype(np.float64), rtol=1e-5, atol=1e-6)
    assert O.argmax_f32(np.array([1, 7, 7, 3], np.float32)) == 1


def test_comparator_semantics(oracle):
    # crates/reference/src/lib.rs:116-153: identical -> 0 mismatches; one element off by 0.5 at tol 1e-3 -> 1
    O = oracle
    a = np.array([1.0, 2.0, 3.0], np.float32)
    assert O.compare(a, a).n_mismatch_abs == 0
    st = O.compare(a, np.array([1.0, 2.5, 3.0], np.float32), abs_tol=1e-3)
    assert st.n_mismatch_abs == 1 and abs(st.max_abs - 0.5) < 1e-7
    st = O.compare(a, a + 1e-4, abs_tol=1e-3)
    assert st.n_mismatch_abs == 0
    assert O.compare(np.zeros(0, np.float32), np.zeros(0, np.float32)).n == 0


def test_lcg_matches_reference_generator(oracle):
    # crates/kernels/src/dispatch.rs:1805-1813
    v = oracle.lcg_random_f32(4, 42)
    s = 42
    for i in range(4):
        s = (s * 6364136223846793005 + 1442695040888963407) % 2 ** 64
        assert v[i] == np.float32(np.float32(s >> 33) / np.float32(4294967295.0) * np.float32(2) - np.float32(1))
    assert (np.abs(oracle.lcg_random_f32(1000, 7)) <= 1).all()


def test_golden_vectors_regression(oracle):
    """The committed fixtures reproduce bit-for-bit on this host (f64 tier, -ffp-contract=off)."""
    O = oracle
    G = np.load(GOLD)
    i = 0
    while "gemv%d_fmt" % i in G:
        fmt, m, k = map(int, G["gemv%d_fmt" % i])
        y = O.gemv(fmt, G["gemv%d_w" % i], G["gemv%d_x" % i], m, k, O.TIER_F64)
        assert (y == G["gemv%d_y" % i]).all(), i
        i += 1
    assert i == 6
    for r in range(G["route_logits"].shape[0]):
        idx, w, _ = O.topk_softmax(G["route_logits"][r], 8, False)
        assert (idx == G["route_idx"][r]).all() and np.allclose(w, G["route_w"][r], rtol=1e-6)
    h, ff, E, k = map(int, G["moe_dims"])
    y, idx, w = O.moe_layer_q4k(G["moe_router"], G["moe_gate"], G["moe_up"], G["moe_down"], G["moe_x"], h=h, ff=ff,
                                E=E, top_k=k, renorm=False)
    assert (idx == G["moe_idx"]).all() and np.allclose(y, G["moe_y"], rtol=1e-6, atol=1e-6 * np.abs(y).max())


def test_q5_0_q5k_q6k_decoders_follow_the_reference_formulas(oracle):
    """The three formats the reference only dequantises on the CPU (crates/engine/src/forward.rs:900-949, 979-1012):
    the oracle's decoders against values computed here straight from the logical fields, plus single-block cases worked
    out by hand from the byte layouts."""
    O = oracle
    rng = np.random.default_rng(900)
    m, k = 3, 512
    # Q5_0: value = d * (q - 16)
    d = np.abs(rng.normal(0, 0.02, (m, k // 32))).astype(np.float16)
    q = rng.integers(0, 32, (m, k // 32, 32), dtype=np.uint8)
    w = O.pack_q5_0(d.astype(np.float64), q)
    want = (d.astype(np.float32)[..., None] * (q.astype(np.float32) - 16)).reshape(m, k)
    assert np.array_equal(O.dequant_rows(O.Q5_0, w, m, k), want)
    # Q5_K: value = d * sc * q - dmin * mn, sub-block j = elements 32j..32j+31 with scale index: pair p = j // 2 holds
    # elements 64p..64p+31 (scale p) and 64p+32..64p+63 (scale p + 4)
    nb = k // 256
    d = np.abs(rng.normal(0, 0.01, (m, nb))).astype(np.float16)
    dm = np.abs(rng.normal(0, 0.01, (m, nb))).astype(np.float16)
    sc = rng.integers(0, 64, (m, nb, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, (m, nb, 8), dtype=np.uint8)
    q = rng.integers(0, 32, (m, nb, 256), dtype=np.uint8)
    w = O.pack_q5k(d.astype(np.float64), dm.astype(np.float64), sc, mn, q)
    idx = np.array([(e // 64) + (4 if (e % 64) >= 32 else 0) for e in range(256)])
    dl = d.astype(np.float32)[..., None] * sc[..., idx].astype(np.float32)
    ml = dm.astype(np.float32)[..., None] * mn[..., idx].astype(np.float32)
    want = (dl * q.astype(np.float32) - ml).reshape(m, k)
    assert np.array_equal(O.dequant_rows(O.Q5K, w, m, k), want)
    # Q6_K: value = d * sc[8 * half + 2 * group] * q, half = e // 128, group = (e % 128) // 32
    d = np.abs(rng.normal(0, 0.001, (m, nb))).astype(np.float16)
    sc = rng.integers(-128, 128, (m, nb, 16)).astype(np.int8)
    q = rng.integers(-32, 32, (m, nb, 256)).astype(np.int8)
    w = O.pack_q6k(d.astype(np.float64), sc, q)
    idx = np.array([8 * (e // 128) + 2 * ((e % 128) // 32) for e in range(256)])
    want = ((d.astype(np.float32)[..., None] * sc[..., idx].astype(np.float32)) * q.astype(np.float32)).reshape(m, k)
    assert np.array_equal(O.dequant_rows(O.Q6K, w, m, k), want)
    # hand-made blocks.  Q5_0, d = 1: qs all 0x10 and qh = 0x0000FFFF -> elements 0..15 = (0 | 16) - 16 = 0,
    # elements 16..31 = (1 | 0) - 16 = -15
    blk = np.zeros(22, np.uint8)
    blk[0:2] = np.array([1.0], np.float16).view(np.uint8)
    blk[2:4] = 0xFF
    blk[6:] = 0x10
    assert O.dequant_rows(O.Q5_0, blk, 1, 32)[0].tolist() == [0.0] * 16 + [-15.0] * 16
    # Q6_K, d = 1, scales = 1..16, every 6-bit value 33 (ql nibbles 1, qh = 0xAA: upper bits 2) -> q = 1: the block is
    # the scale of each group: 1, 3, 5, 7 for the first 128 elements, 9, 11, 13, 15 for the second
    blk = np.zeros(210, np.uint8)
    blk[0:128] = 0x11
    blk[128:192] = 0xAA
    blk[192:208] = np.arange(1, 17, dtype=np.uint8)
    blk[208:210] = np.array([1.0], np.float16).view(np.uint8)
    got = O.dequant_rows(O.Q6K, blk, 1, 256)[0]
    assert got.reshape(8, 32)[:, 0].tolist() == [1.0, 3.0, 5.0, 7.0, 9.0, 11.0, 13.0, 15.0] and (got.reshape(8, 32).std(1) == 0).all()
    # Q5_K, d = 1, dmin = 0, scale bytes: sc_0 = 1, sc_5 = 2 (5 >= 4: low nibble of byte 9), qs[0] = 0xF1 and bit 0 of
    # qh[0] set -> element 0 = 1 * (1 | 16) = 17; element 96 + 0 belongs to pair 1 high half (scale 5): qs[32] = 0x30 and
    # bit 96 (qh[12] bit 0) set -> 2 * (3 | 16) = 38
    blk = np.zeros(176, np.uint8)
    blk[0:2] = np.array([1.0], np.float16).view(np.uint8)
    blk[4] = 1
    blk[4 + 9] = 2
    blk[16] = 1
    blk[16 + 12] = 1
    blk[48] = 0xF1
    blk[48 + 32] = 0x30
    got = O.dequant_rows(O.Q5K, blk, 1, 256)[0]
    assert got[0] == 17.0 and got[96] == 38.0 and got[32] == 0.0   # element 32: high nibble 15 of qs[0] but scale 4 = 0
    # GEMV tiers agree on the new formats
    for fmt in (O.Q5_0, O.Q5K, O.Q6K):
        w = O.rand_weights(fmt, rng, 5, 512)
        x = rng.normal(0, 1, 512).astype(np.float32)
        a, b = O.gemv(fmt, w, x, 5, 512, O.TIER_DEQUANT), O.gemv(fmt, w, x, 5, 512, O.TIER_F64)
        assert np.allclose(a, b, rtol=2e-5, atol=1e-6 * np.abs(b).max())
        assert np.allclose(b, O.dequant_rows(fmt, w, 5, 512).astype(np.float64) @ x.astype(np.float64), rtol=1e-6)


def test_sampler_restatement_against_the_reference_tests():
    """The three tests the reference holds for its sampler (crates/engine/src/sampler.rs:163-190) and an independent
    restatement of its generator (sampler.rs:12-27) in Python integers."""
    import oracle as O
    # greedy_picks_max
    assert O.sampler_argmax_last(np.array([0.1, 5.0, 2.0], np.float32)) == 1
    # temperature_zero_is_greedy: SamplerConfig::greedy() = temperature 0, top_k 40, top_p 0.95, penalty 1.1, min_tokens 1
    greedy = O.SamplerCfg(0.0, 40, 0.95, 1.1, 1)
    assert O.sample(np.arange(10, dtype=np.float32), greedy, [], [], O.SamplerRng(42)) == 9
    # repetition_penalty_reduces_repeated: [1, 5, 3] with context [1] and penalty 2 -> 5 / 2 at index 1, the rest unchanged
    cfg = O.SamplerCfg(0.0, 0, 1.0, 2.0, 0)
    tok, scores = O.sample(np.array([1.0, 5.0, 3.0], np.float32), cfg, [1], [], O.SamplerRng(1), want_probs=True)
    assert abs(scores[1] - 2.5) < 1e-6 and abs(scores[0] - 1.0) < 1e-6 and tok == 2
    # the penalty applies once per occurrence, negative scores are multiplied
    _, scores = O.sample(np.array([-1.0, 8.0, 3.0], np.float32), cfg, [1, 0, 1], [], O.SamplerRng(1), want_probs=True)
    assert scores.tolist() == [-2.0, 2.0, 3.0]
    # Iterator::max_by keeps the last of equal maxima
    assert O.sampler_argmax_last(np.array([7.0, 1.0, 7.0, 0.0], np.float32)) == 2
    # generator: xorshift64 (13, 7, 17), seed ^ 0x9e3779b97f4a7c15, (x >> 11) as f32 / 2^53 as f32
    M = (1 << 64) - 1
    for seed in (0, 1, 42, 0xDEADBEEF):
        x = 0x9e3779b97f4a7c15 if seed == 0 else seed ^ 0x9e3779b97f4a7c15
        rng = O.SamplerRng(seed)
        for _ in range(50):
            x ^= (x << 13) & M
            x ^= x >> 7
            x ^= (x << 17) & M
            want = np.float32(np.float32(x >> 11) / np.float32(2.0 ** 53))
            assert np.float32(rng.next_f32()) == want
    # min_tokens suppresses the end-of-sequence ids; top-k keeps the first k entries in index order that reach the threshold
    cfg = O.SamplerCfg(0.0, 0, 1.0, 1.0, 3)
    assert O.sample(np.array([1.0, 9.0, 3.0], np.float32), cfg, [0, 0], [1], O.SamplerRng(1)) == 2
    assert O.sample(np.array([1.0, 9.0, 3.0], np.float32), cfg, [0, 0, 0], [1], O.SamplerRng(1)) == 1
    cfg = O.SamplerCfg(1.0, 2, 1.0, 1.0, 0)
    _, p = O.sample(np.array([2.0, 2.0, 2.0, 5.0, 1.0], np.float32), cfg, [], [], O.SamplerRng(3), want_probs=True)
    assert (p > 0).tolist() == [True, True, False, False, False]   # the threshold is p(2.0); the later, larger entry finds k taken
    # top-p: descending order until the running sum has reached p
    cfg = O.SamplerCfg(1.0, 0, 0.6, 1.0, 0)
    _, p = O.sample(np.log(np.array([0.5, 0.3, 0.15, 0.05], np.float32)), cfg, [], [], O.SamplerRng(3), want_probs=True)
    assert (p > 0).tolist() == [True, True, False, False]


def _small_host_model(O, seed=11):
    """A 2-layer decoder on the host (zero-mean Q4_K weights, the shapes of the GPU tests' small model)."""
    from test_decode_gpu import SMALL, rand_q4k_zero_mean
    c = dict(SMALL)
    L, h, E, ff, V = c["n_layers"], c["hidden"], c["n_experts"], c["ff"], c["vocab"]
    q_dim, kv_dim = c["n_heads"] * c["head_dim"], c["n_kv_heads"] * c["head_dim"]
    shapes = {"wq": (L * q_dim, h), "wk": (L * kv_dim, h), "wv": (L * kv_dim, h), "wo": (L * h, q_dim),
              "gate": (L * E * ff, h), "up": (L * E * ff, h), "down": (L * E * h, ff), "lm_head": (V, h)}
    rng = np.random.default_rng(seed)
    host = {n: rand_q4k_zero_mean(O, rng, r, k).reshape(-1) for n, (r, k) in shapes.items()}
    host.update({"tok_emb": rng.normal(0, 0.02, (V, h)).astype(np.float32), "attn_norm": np.ones((L, h), np.float32),
                 "ffn_norm": np.ones((L, h), np.float32), "out_norm": np.ones(h, np.float32),
                 "router": rng.normal(0, 0.02, (L, E, h)).astype(np.float32)})
    return c, host


def test_prefill_restatement_agrees_with_the_decode_oracle():
    """The batched prefill's restatement (bf16 GEMM operands, f16 attention operands) against the decode oracle run token by
    token in f32 over the same prompt: the same cache and logits to bf16 operand rounding (1e-2 of their spread rms, 8e-2 at
    worst), the same next token.  Ties the prefill restatement to the arithmetic that is pinned on the reference's formulas."""
    import oracle as O
    from oracle import prefill as OP
    c, host = _small_host_model(O)
    prompt = np.random.default_rng(5).integers(0, c["vocab"], 24).astype(np.int32)
    tok, logits, kc, vc = OP.prefill(c, host, prompt)
    ocfg = O.ModelCfg(**c)
    ow = O.ModelWeights(**{k: v.ctypes.data for k, v in host.items()})
    kc2 = np.zeros_like(kc)
    vc2 = np.zeros_like(vc)
    for pos, t in enumerate(prompt):
        ref_tok, ref_logits = O.decode_step(ocfg, ow, kc2, vc2, int(t), pos, want_logits=True)
    T = len(prompt)
    spread = float(np.std(ref_logits))
    # a bf16 operand carries a relative rounding of up to 2^-9: about 0.4 % rms per GEMM output, a few times that at worst
    d = np.abs(logits - ref_logits)
    assert d.max() <= 8e-2 * spread and np.sqrt((d ** 2).mean()) <= 1e-2 * spread, (d.max(), spread)
    assert tok == ref_tok or abs(ref_logits[tok] - ref_logits[ref_tok]) <= 8e-2 * spread
    for a, b in ((kc, kc2), (vc, vc2)):
        a, b = a[:, :, :T].astype(np.float32), b[:, :, :T].astype(np.float32)
        assert np.abs(a - b).max() <= 8e-2 * float(np.std(b)) and np.sqrt(((a - b) ** 2).mean()) <= 1e-2 * float(np.std(b))
    # the attention restatement alone against a plain f64 softmax
    rng = np.random.default_rng(2)
    heads, kvh, hd, T = 4, 2, 64, 70
    q = rng.normal(0, 1, (T, heads * hd)).astype(np.float32)
    kcs = rng.normal(0, 1, (kvh, 128, hd)).astype(np.float16)
    vcs = rng.normal(0, 1, (kvh, 128, hd)).astype(np.float16)
    got = OP.causal_attention_f16(q, kcs, vcs, heads, kvh, hd)
    for h in range(heads):
        K, V = kcs[h // 2, :T].astype(np.float64), vcs[h // 2, :T].astype(np.float64)
        s = q[:, h * hd:(h + 1) * hd].astype(np.float64) @ K.T / np.sqrt(hd)
        s = np.where(np.arange(T)[None, :] <= np.arange(T)[:, None], s, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        ref = (p / p.sum(axis=1, keepdims=True)) @ V
        assert np.abs(got[:, h * hd:(h + 1) * hd] - ref).max() < 5e-3


def test_decoders_against_the_upstream_definition_of_the_block_formats(oracle):
    """tests/golden/ggml_dequant.npz holds seeded blocks and what the `gguf` Python package (upstream's own numpy
    dequantisation) makes of them.  Q8_0 and Q5_0: the reference decodes like upstream, so the oracle must give the same bits.
    Q4_0 and Q4_K: the reference orders things differently (element 2i / 2i+1 from the two nibbles of byte i; scale slots j
    and j + 4 for the two nibble halves of chunk j, where upstream uses 2j and 2j + 1) - after exactly that re-ordering the
    bits agree as well, which pins the f16 fields, the 6-bit unpacking, the nibble extraction and the arithmetic order of
    the oracle to an implementation written by someone else."""
    O = oracle
    G = np.load(Path(__file__).parent / "golden" / "ggml_dequant.npz")
    for name, fmt in (("q8_0", 0), ("q5_0", 3)):
        raw, ref = G[name + "_raw"], G[name + "_ggml"]
        assert np.array_equal(O.dequant_rows(fmt, raw, raw.shape[0], ref.shape[1]), ref), name
    raw, ref = G["q4_0_raw"], G["q4_0_ggml"]
    m = raw.shape[0]
    mine = O.dequant_rows(1, raw, m, ref.shape[1]).reshape(m, -1, 32)
    up = ref.reshape(m, -1, 32)
    assert np.array_equal(mine[..., 0::2], up[..., :16]) and np.array_equal(mine[..., 1::2], up[..., 16:])
    # Q4_K: move upstream's slots (2j, 2j+1) into the reference's (j, j+4), decode with the oracle, compare with upstream
    raw, ref = G["q4k_raw"].copy(), G["q4k_ggml"]
    blk = raw.reshape(m, -1, 144)
    s = blk[..., 4:16].astype(np.uint8)
    sc = np.empty(s.shape[:-1] + (8,), np.uint8)
    mn = np.empty_like(sc)
    sc[..., :4], mn[..., :4] = s[..., 0:4] & 63, s[..., 4:8] & 63                                  # get_scale_min_k4, j < 4
    sc[..., 4:] = (s[..., 8:12] & 15) | ((s[..., 0:4] >> 6) << 4)
    mn[..., 4:] = (s[..., 8:12] >> 4) | ((s[..., 4:8] >> 6) << 4)
    perm = [0, 2, 4, 6, 1, 3, 5, 7]                  # reference slot j <- upstream slot 2j, slot j + 4 <- 2j + 1
    blk[..., 4:16] = O.pack_q4k_scales(sc[..., perm], mn[..., perm])
    assert np.array_equal(O.dequant_rows(2, blk.reshape(m, -1), m, ref.shape[1]), ref)
