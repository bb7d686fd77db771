"""The MoE entry point that allocates nothing (built-in scratch region) against the regular entry point.

Collected last on purpose (file name): if it fails, a run that stops at the first failure has already
run every other test.  It builds its own context and data, so it passes alone in a fresh process as
well as after the rest of the suite."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_point_matches_regular_entry_point_twice():
    import oracle as O
    import runit_mac_b200 as R

    ctx = R.Context(0)
    lib, hnd = ctx.lib, ctx.handle
    h, ff, E, k = 512, 256, 8, 2
    rng = np.random.default_rng(4242)
    router = ctx.buffer_from(rng.normal(0, 0.02, (E, h)).astype(np.float32))
    gate = ctx.buffer_from(O.rand_q4k(rng, E * ff, h))
    up = ctx.buffer_from(O.rand_q4k(rng, E * ff, h))
    down = ctx.buffer_from(O.rand_q4k(rng, E * h, ff))
    assert lib.runit_moe_static_scratch_capacity() >= 1 << 20

    def void(b):
        return C.c_void_p(b.ptr if b is not None else None)

    for call_no, T in enumerate((5, 3)):          # two calls in a row; the second reuses the region
        x = rng.normal(0, 1, (T, h)).astype(np.float32)
        res = rng.normal(0, 1, (T, h)).astype(np.float32)
        xb, rb = ctx.buffer_from(x), ctx.buffer_from(res)
        outs = []
        for which in ("regular", "static"):
            out, idx, w = ctx.new_buffer(T * h * 4), ctx.new_buffer(T * k * 4), ctx.new_buffer(T * k * 4)
            if which == "regular":
                nb = lib.runit_moe_scratch_bytes(T, h, ff, E, k)
                scratch = ctx.new_buffer(nb)
                st = lib.runit_moe_layer_q4k(hnd, void(router), void(gate), void(up), void(down), void(xb), void(rb), void(out),
                                             void(idx), void(w), void(scratch), nb, T, h, ff, E, k, 0)
            else:
                st = lib.runit_moe_layer_q4k_static(hnd, void(router), void(gate), void(up), void(down), void(xb), void(rb),
                                                    void(out), void(idx), void(w), T, h, ff, E, k, 0)
            assert st == 0, lib.runit_last_error_string(hnd)
            ctx.flush()
            outs.append((out.download(np.float32, T * h), idx.download(np.int32, T * k), w.download(np.float32, T * k)))
        (o0, i0, w0), (o1, i1, w1) = outs
        assert (i0 == i1).all(), call_no
        assert (w0 == w1).all(), call_no
        # same kernels, same order of operations: the tolerance of the other MoE tests (1e-3 of the output
        # scale) is the bar, and in fact the results are identical
        st = O.compare(o0, o1, rel_tol=1e-3)
        assert st.n_mismatch_rel == 0 and np.isfinite(o1).all(), (call_no, st)
        assert (o0 == o1).all(), call_no

    # a shape beyond the built-in region is refused with a clear error and launches nothing
    before = ctx.launches
    big = ctx.new_buffer(64)
    st = lib.runit_moe_layer_q4k_static(hnd, void(big), void(big), void(big), void(big), void(big), None, void(big), None, None,
                                        4096, 2048, 1024, 64, 8, 0)
    assert st == 3   # RUNIT_ERR_BUFFER_SIZE
    assert b"built-in region" in lib.runit_last_error_string(hnd)
    assert ctx.launches == before
    ctx.flush()
    ctx.close()
