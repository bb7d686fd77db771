"""Comparison helpers shared by the parity tests."""
import numpy as np

REL_TOL = 1e-3   # |gpu - ref| <= REL_TOL * max(|ref|, rms(ref)): the bound the path's spec states
ABS_TOL_F16 = 1e-2   # the reference's own tolerance for f16 kernels (dispatch.rs:1782)


def assert_close(oracle, ref, got, rel_tol=REL_TOL, what=""):
    ref = np.asarray(ref, np.float32).reshape(-1)
    got = np.asarray(got, np.float32).reshape(-1)
    assert ref.shape == got.shape, (ref.shape, got.shape)
    assert np.isfinite(got).all(), "%s: non-finite output" % what
    st = oracle.compare(ref, got, abs_tol=1e30, rel_tol=rel_tol)
    assert st.n_mismatch_rel == 0, "%s: %r" % (what, st)
    return st


def f16_ulp_close(ref16, got16, ulps=1, rel_tol=REL_TOL):
    """f16 outputs: equal to the rounded oracle up to `ulps` units in the last place, or — where the
    dot product cancels to a value far below its terms — within rel_tol of the output scale (the f32
    sum feeding the rounding differs in order between implementations)."""
    a = np.asarray(ref16, np.float16).view(np.int16).astype(np.int32)
    b = np.asarray(got16, np.float16).view(np.int16).astype(np.int32)
    a = np.where(a < 0, -(a & 0x7FFF), a)
    b = np.where(b < 0, -(b & 0x7FFF), b)
    rf = np.asarray(ref16, np.float16).astype(np.float32)
    gf = np.asarray(got16, np.float16).astype(np.float32)
    scale = np.maximum(np.abs(rf), np.sqrt(np.mean(rf.astype(np.float64) ** 2)))
    ok = (np.abs(a - b) <= ulps) | (np.abs(rf - gf) <= rel_tol * scale)
    return bool(ok.all()) and bool(np.isfinite(gf).all())


def assert_close_bf16_chain(oracle, ref, got, what=""):
    """Outputs of a chain with a bf16-rounded intermediate (act = bf16(silu(g)*u) feeding the down product): an
    intermediate within f32 rounding distance of a bf16 rounding boundary may round the other way on the two sides
    (one bf16 ulp = 2^-8 of that activation), which moves a few outputs by more than the 1e-3 bar.  Accept: every
    element within 4e-3 of the output scale and at least 99.9 % of the elements within 1e-3."""
    ref = np.asarray(ref, np.float32).reshape(-1)
    got = np.asarray(got, np.float32).reshape(-1)
    assert ref.shape == got.shape and np.isfinite(got).all(), what
    scale = np.maximum(np.abs(ref), np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    rel = np.abs(got - ref) / scale
    assert rel.max() <= 4e-3, "%s: max rel %.3e" % (what, rel.max())
    assert (rel <= REL_TOL).mean() >= 0.999, "%s: %.4f %% within 1e-3" % (what, 100 * (rel <= REL_TOL).mean())
