"""GGUF file -> packed device weights -> fused-dequant kernels: the uploaded bytes are the file's bytes, the GEMVs on
them match the oracle, a merged expert tensor feeds the MoE layer as one buffer, and a tensor larger than the staging
buffers arrives intact."""
import numpy as np
import pytest

from gguf_writer import T_F32, T_STR, T_U32, build_gguf
from helpers import assert_close

pytestmark = pytest.mark.gpu


def test_upload_and_gemv_from_a_gguf_file(ctx, oracle, tmp_path):
    import runit_mac_b200 as R
    from runit_mac_b200.gguf import GgufDtype as D, parse_gguf_file
    O = oracle
    rng = np.random.default_rng(11)
    shapes = {"blk.0.attn_q.weight": (0, D.Q8_0, 96, 896), "blk.0.attn_k.weight": (1, D.Q4_0, 70, 3584),
              "output.weight": (2, D.Q4K, 300, 2048)}
    ws = {n: O.rand_weights(f, rng, m, k) for n, (f, _, m, k) in shapes.items()}
    norm = rng.normal(1, 0.1, 2048).astype(np.float32)
    tensors = [(n, [k, m], dt, ws[n]) for n, (_, dt, m, k) in shapes.items()] + [("output_norm.weight", [2048], D.F32, norm)]
    path = tmp_path / "model.gguf"
    path.write_bytes(build_gguf([("general.architecture", T_STR, "qwen2"), ("qwen2.block_count", T_U32, 1),
                                 ("qwen2.attention.layer_norm_rms_epsilon", T_F32, 1e-6)], tensors))
    g = parse_gguf_file(path)
    assert g.metadata["qwen2.block_count"] == 1 and abs(g.metadata["qwen2.attention.layer_norm_rms_epsilon"] - 1e-6) < 1e-12
    for n, (fmt, dt, m, k) in shapes.items():
        wb = g.upload_weight(ctx, n)
        assert (wb.fmt, wb.rows, wb.k, wb.experts, wb.dtype) == (fmt, m, k, 1, dt)
        assert wb.buffer.download(np.uint8, ws[n].nbytes).tobytes() == ws[n].tobytes()
        x = rng.normal(0, 1, k).astype(np.float32)
        yb = ctx.new_buffer(m * 4)
        getattr(R, "gemv_%s_f32in_f32out" % ("q8_0", "q4_0", "q4k")[fmt])(ctx, wb.buffer, ctx.buffer_from(x), yb, m, k)
        ctx.flush()
        assert_close(O, O.gemv(fmt, ws[n], x, m, k, O.TIER_F64), yb.download(np.float32, m), what=n)
    nb = g.upload_weight(ctx, "output_norm.weight")
    assert nb.fmt is None and nb.k == 2048
    assert np.array_equal(nb.buffer.download(np.float32, 2048), norm)


def test_kquant_tensors_of_a_mixed_file_stay_packed(ctx, oracle, tmp_path):
    """A Q4_K_M file mixes Q6_K / Q5_K (and older files Q5_0) tensors among the Q4_K ones; the reference expands them to
    f16 at load (crates/engine/src/forward.rs:900-949, 979-1012).  Here they are uploaded as stored and multiplied packed."""
    import runit_mac_b200 as R
    from runit_mac_b200.gguf import GgufDtype as D, parse_gguf_file
    O = oracle
    rng = np.random.default_rng(13)
    shapes = {"blk.0.ffn_down.weight": (O.Q6K, D.Q6K, 130, 1024, "q6k"), "blk.0.attn_v.weight": (O.Q5K, D.Q5K, 64, 512, "q5k"),
              "token_embd.weight": (O.Q5_0, D.Q5_0, 100, 256, "q5_0")}
    ws = {n: O.rand_weights(f, rng, m, k) for n, (f, _, m, k, _) in shapes.items()}
    path = tmp_path / "mixed.gguf"
    path.write_bytes(build_gguf([("general.architecture", T_STR, "qwen2")], [(n, [k, m], dt, ws[n]) for n, (_, dt, m, k, _) in shapes.items()]))
    g = parse_gguf_file(path)
    for n, (fmt, dt, m, k, kname) in shapes.items():
        wb = g.upload_weight(ctx, n)
        assert (wb.fmt, wb.rows, wb.k, wb.dtype) == (fmt, m, k, dt)
        assert wb.buffer.download(np.uint8, ws[n].nbytes).tobytes() == ws[n].tobytes()
        x = rng.normal(0, 1, k).astype(np.float32)
        yb = ctx.new_buffer(m * 4)
        getattr(R, "gemv_%s_f32in_f32out" % kname)(ctx, wb.buffer, ctx.buffer_from(x), yb, m, k)
        ctx.flush()
        assert_close(O, O.gemv(fmt, ws[n], x, m, k, O.TIER_F64), yb.download(np.float32, m), what=n)


def test_merged_expert_tensors_feed_the_moe_layer(ctx, oracle, tmp_path):
    """`ffn_*_exps` tensors ([K, rows, E] in file order) stay one packed buffer each (crates/engine/src/forward.rs:1321-1418
    slices them per expert instead)."""
    from runit_mac_b200 import moe_scratch_bytes
    from runit_mac_b200.gguf import GgufDtype as D, parse_gguf_file
    O = oracle
    h, ff, E, k, T = 512, 256, 8, 2, 3
    rng = np.random.default_rng(12)
    router = rng.normal(0, 0.02, (E, h)).astype(np.float32)
    gate = np.stack([O.rand_q4k(rng, ff, h) for _ in range(E)])
    up = np.stack([O.rand_q4k(rng, ff, h) for _ in range(E)])
    down = np.stack([O.rand_q4k(rng, h, ff) for _ in range(E)])
    path = tmp_path / "moe.gguf"
    path.write_bytes(build_gguf([("general.architecture", T_STR, "olmoe"), ("olmoe.expert_count", T_U32, E),
                                 ("olmoe.expert_used_count", T_U32, k)],
                                [("blk.0.ffn_gate_inp.weight", [h, E], D.F32, router),
                                 ("blk.0.ffn_gate_exps.weight", [h, ff, E], D.Q4K, gate),
                                 ("blk.0.ffn_up_exps.weight", [h, ff, E], D.Q4K, up),
                                 ("blk.0.ffn_down_exps.weight", [ff, h, E], D.Q4K, down)]))
    g = parse_gguf_file(path)
    assert (g.metadata["olmoe.expert_count"], g.metadata["olmoe.expert_used_count"]) == (E, k)
    rb, gb, ub, db = (g.upload_weight(ctx, "blk.0.ffn_%s.weight" % n) for n in ("gate_inp", "gate_exps", "up_exps", "down_exps"))
    assert (gb.rows, gb.k, gb.experts) == (ff, h, E) and (db.rows, db.k, db.experts) == (h, ff, E)
    x = rng.normal(0, 1, (T, h)).astype(np.float32)
    out, idx, w = ctx.new_buffer(T * h * 4), ctx.new_buffer(T * k * 4), ctx.new_buffer(T * k * 4)
    nbytes = moe_scratch_bytes(ctx, T, h, ff, E, k)
    scratch = ctx.new_buffer(nbytes)
    ctx.call("moe_layer_q4k", rb.buffer, gb.buffer, ub.buffer, db.buffer, ctx.buffer_from(x), None, out, idx, w, scratch, nbytes,
             T, h, ff, E, k, 0)
    ctx.flush()
    ref, ridx, _ = O.moe_layer_q4k(router, gate, up, down, x, h=h, ff=ff, E=E, top_k=k, renorm=False)
    got_idx = idx.download(np.int32, T * k).reshape(T, k)
    assert (got_idx == ridx).all()
    assert_close(O, ref, out.download(np.float32, T * h).reshape(T, h), what="moe layer from gguf")


def test_upload_larger_than_the_staging_buffers(ctx, tmp_path):
    """80 MB tensor: three chunks through the two 32 MB pinned buffers; also the size check of the destination."""
    from runit_mac_b200.gguf import GgufDtype as D, GgufError, parse_gguf_file
    rows, k = 40000, 3584
    rng = np.random.default_rng(13)
    raw = rng.integers(0, 256, rows * (k // 256) * 144, dtype=np.uint8)
    path = tmp_path / "big.gguf"
    path.write_bytes(build_gguf([], [("pad", [3], D.F32, np.zeros(3, np.float32)), ("big.weight", [k, rows], D.Q4K, raw)]))
    g = parse_gguf_file(path)
    wb = g.upload_weight(ctx, "big.weight")
    got = wb.buffer.download(np.uint8, raw.nbytes)
    assert np.array_equal(got, raw)
    import ctypes as C
    from runit_mac_b200 import gguf as G
    small = ctx.new_buffer(1024)
    st = G._api().runit_gguf_upload_tensor(ctx.handle, g._h, b"big.weight", C.c_void_p(small.ptr), small.nbytes)
    assert st == 11
    with pytest.raises(GgufError) as e:
        G._check(st)
    assert e.value.kind == "BufferSize"
