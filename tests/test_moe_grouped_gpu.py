"""GPU parity tests of the batched (prefill-sized) MoE block on the tensor cores, through the C ABI.

Oracle: the bf16-operand restatement of the block (weights = bf16 of the Q4_K value, activations bf16,
f64 accumulation rounded to f32).  Bar: |gpu - oracle| <= 1e-3 * max(|ref|, rms(ref)) for at least 99.9 % of the outputs and
4e-3 for all of them: the residue comes from the f32 accumulation order inside the MMA and from intermediate
activations that land on the other side of a bf16 rounding boundary (helpers.assert_close_bf16_chain).  Routing indices must be identical (ties closer than 1e-6 excluded)."""
import numpy as np
import pytest

from helpers import assert_close, assert_close_bf16_chain

pytestmark = pytest.mark.gpu


def make_layer(O, rng, E, h, ff):
    router = rng.normal(0, 0.02, (E, h)).astype(np.float32)
    return router, O.rand_q4k(rng, E * ff, h), O.rand_q4k(rng, E * ff, h), O.rand_q4k(rng, E * h, ff)


@pytest.mark.parametrize("T,E,k,h,ff", [(1, 4, 2, 256, 256), (64, 4, 2, 256, 256), (100, 4, 2, 512, 256),
                                        (300, 8, 2, 512, 512), (777, 16, 4, 1024, 768)])
def test_grouped_block_with_router(ctx, oracle, T, E, k, h, ff):
    import runit_mac_b200 as R
    O = oracle
    rng = np.random.default_rng(T * 7 + E)
    router, gate, up, down = make_layer(O, rng, E, h, ff)
    x = rng.normal(0, 1, (T, h)).astype(np.float32)
    ref, ridx, rw = O.moe_grouped_q4k_bf16(router, gate, up, down, x, h=h, ff=ff, E=E, top_k=k)
    out, idx, w = R.moe_layer_q4k_bf16_host(ctx, router, gate, up, down, x, h=h, ff=ff, E=E, top_k=k)
    same = (idx == ridx).all(1)
    assert same.sum() >= T - max(1, T // 100), "routing differs on %d tokens" % (T - same.sum())
    assert np.allclose(w[same], rw[same], rtol=1e-5, atol=1e-8)
    assert_close_bf16_chain(O, ref[same], out[same], what="grouped block T=%d" % T)
    # the bf16 block stays close to the f32 block (bf16 operands: ~2^-9 per product, averaged over the sum)
    ref32, i32, _ = O.moe_layer_q4k(router, gate, up, down, x[:4], h=h, ff=ff, E=E, top_k=k, renorm=False)
    ok = (i32 == idx[:4]).all(1)
    scale = np.sqrt(np.mean(ref32 ** 2))
    assert np.abs(out[:4][ok] - ref32[ok]).max() <= 3e-2 * scale


def test_grouped_block_given_routing_edge_cases(ctx, oracle):
    """Routing supplied by the caller: an expert without tokens, an expert with exactly one full tile, slots with
    ids outside [0, E) (skipped), residual added."""
    import runit_mac_b200 as R
    O = oracle
    rng = np.random.default_rng(77)
    T, E, k, h, ff = 256, 6, 2, 512, 256
    _, gate, up, down = make_layer(O, rng, E, h, ff)
    x = rng.normal(0, 1, (T, h)).astype(np.float32)
    res = rng.normal(0, 1, (T, h)).astype(np.float32)
    idx = np.empty((T, k), np.int32)
    idx[:128] = [0, 1]            # expert 0 and 1: exactly 128 slots each from these tokens
    idx[128:] = [2, 3]            # expert 4: none; expert 5: see below
    idx[200:, 1] = 5
    idx[250:, 0] = -1             # skipped slots
    idx[255, 1] = E + 3
    w = rng.random((T, k)).astype(np.float32)
    ref, _, _ = O.moe_grouped_q4k_bf16(None, gate, up, down, x, h=h, ff=ff, E=E, top_k=k, residual=res, routing=(idx, w))
    out, _, _ = R.moe_layer_q4k_bf16_host(ctx, None, gate, up, down, x, h=h, ff=ff, E=E, top_k=k, residual=res, routing=(idx, w))
    assert_close_bf16_chain(O, ref - res, out - res, what="given routing")
    assert np.array_equal(out[255], res[255])     # both slots of the last token are skipped


@pytest.fixture(scope="module")
def qwen3_moe_block():
    """Qwen3-MoE-shaped block: hidden 2048, 128 experts, top-8, expert intermediate 768, 4096 tokens ~ N(0,1), routing
    with expert popularity ~ Zipf(s = 1.1) (8 distinct experts per token)."""
    import torch
    import runit_mac_b200 as R
    ctx = R.Context(0)
    T, E, k, h, ff = 4096, 128, 8, 2048, 768
    rb = lambda kk: kk // 256 * 144
    gate, up, down = ctx.new_buffer(E * ff * rb(h)), ctx.new_buffer(E * ff * rb(h)), ctx.new_buffer(E * h * rb(ff))
    for i, (b, rows, kk) in enumerate(((gate, E * ff, h), (up, E * ff, h), (down, E * h, ff))):
        R.fill_weights(ctx, 2, b, rows * (kk // 256), 50 + i, 0.01)
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(T, h, device="cuda", generator=g)
    p = 1.0 / torch.arange(1, E + 1, device="cuda", dtype=torch.float64) ** 1.1
    idx = torch.multinomial((p / p.sum()).float().expand(T, E).contiguous(), k, replacement=False, generator=g).to(torch.int32)
    w = torch.rand(T, k, device="cuda", generator=g)
    nbytes = R.moe_grouped_scratch_bytes(ctx, T, h, ff, E, k)
    scratch = ctx.new_buffer(nbytes)
    torch.cuda.synchronize()
    return dict(ctx=ctx, T=T, E=E, k=k, h=h, ff=ff, gate=gate, up=up, down=down, x=x, idx=idx, w=w, scratch=scratch, nbytes=nbytes)


def run_block(b, x, idx, w, res=None):
    import torch
    import runit_mac_b200 as R
    out = torch.empty(b["T"], b["h"], device="cuda")
    torch.cuda.synchronize()
    R.moe_experts_grouped_q4k_bf16(b["ctx"], b["gate"], b["up"], b["down"], x, idx, w, res, out, b["scratch"], b["nbytes"],
                                   b["T"], b["h"], b["ff"], b["E"], b["k"])
    b["ctx"].flush()
    return out


def test_full_size_block_sampled_and_properties(oracle, qwen3_moe_block):
    import torch
    b = qwen3_moe_block
    O = oracle
    T, E, k, h, ff = b["T"], b["E"], b["k"], b["h"], b["ff"]
    out = run_block(b, b["x"], b["idx"], b["w"])
    assert torch.isfinite(out).all()
    # (1) a sample of tokens recomputed by the oracle (tokens are independent)
    rbh, rbf = h // 256 * 144, ff // 256 * 144
    gate = b["gate"].download(np.uint8, E * ff * rbh)
    up = b["up"].download(np.uint8, E * ff * rbh)
    down = b["down"].download(np.uint8, E * h * rbf)
    sample = [0, 1, 2047, 4095]
    xs = b["x"][sample].cpu().numpy()
    ref, _, _ = O.moe_grouped_q4k_bf16(None, gate, up, down, xs, h=h, ff=ff, E=E, top_k=k,
                                       routing=(b["idx"][sample].cpu().numpy(), b["w"][sample].cpu().numpy()))
    assert_close_bf16_chain(O, ref, out[sample].cpu().numpy(), what="sampled tokens of the full-size block")
    # (2) permuting the tokens permutes the outputs bit for bit (no token sees another token's data)
    perm = torch.randperm(T, device="cuda", generator=torch.Generator(device="cuda").manual_seed(9))
    out_p = run_block(b, b["x"][perm].contiguous(), b["idx"][perm].contiguous(), b["w"][perm].contiguous())
    assert torch.equal(out_p, out[perm])
    # (3) doubling the routing weights doubles the output exactly; the residual is added on top
    res = torch.randn(T, h, device="cuda")
    out2 = run_block(b, b["x"], b["idx"], (2.0 * b["w"]).contiguous(), res)
    assert torch.allclose(out2 - res, 2.0 * out, rtol=0, atol=2e-6 * float(out.abs().max()))
    # (4) every expert received tokens, the most popular one many tiles of them
    cnt = torch.bincount(b["idx"].flatten().long(), minlength=E)
    assert cnt.min() > 0 and cnt.max() > 1024


def test_grouped_bad_arguments(ctx):
    import runit_mac_b200 as R
    b = ctx.new_buffer(1 << 20)
    with pytest.raises(R.KernelError) as e:   # scratch too small
        R.moe_layer_q4k_bf16(ctx, b, b, b, b, b, None, b, None, None, b, 1024, 64, 2048, 768, 128, 8, 0)
    assert e.value.status == 3
    with pytest.raises(R.KernelError):        # intermediate size not a multiple of 256
        R.moe_layer_q4k_bf16(ctx, b, b, b, b, b, None, b, None, None, b, 1 << 20, 1, 2048, 700, 8, 2, 0)
    with pytest.raises(R.KernelError):        # too many experts
        R.moe_experts_grouped_q4k_bf16(ctx, b, b, b, b, b, b, None, b, b, 1 << 20, 1, 256, 256, 300, 2)
    ctx.flush()


def test_grouped_experts_one_slot_per_row_and_command_list(ctx, oracle):
    """The form expert-parallel owners use: k = 1, weight 1, negative ids for unused rows; and the same call recorded
    as a command list and replayed gives the same bits."""
    import runit_mac_b200 as R
    O = oracle
    rng = np.random.default_rng(5)
    n, E, h, ff = 333, 4, 512, 256
    _, gate, up, down = make_layer(O, rng, E, h, ff)
    x = rng.normal(0, 1, (n, h)).astype(np.float32)
    ids = rng.integers(-1, E, (n, 1)).astype(np.int32)
    w = np.ones((n, 1), np.float32)
    ref, _, _ = O.moe_grouped_q4k_bf16(None, gate, up, down, x, h=h, ff=ff, E=E, top_k=1, routing=(ids, w))
    bufs = [ctx.buffer_from(a) for a in (gate, up, down, x, ids, w)]
    out = ctx.new_buffer(n * h * 4)
    nbytes = R.moe_grouped_scratch_bytes(ctx, n, h, ff, E, 1)
    scratch = ctx.new_buffer(nbytes)
    R.moe_experts_grouped_q4k_bf16(ctx, *bufs, None, out, scratch, nbytes, n, h, ff, E, 1)
    ctx.flush()
    got = out.download(np.float32, n * h).reshape(n, h)
    assert_close_bf16_chain(O, ref, got, what="k = 1 slots")
    assert (got[ids[:, 0] < 0] == 0).all()
    ctx.graph_begin()
    R.moe_experts_grouped_q4k_bf16(ctx, *bufs, None, out, scratch, nbytes, n, h, ff, E, 1)
    g = ctx.graph_end()
    out.upload(np.zeros(n * h, np.float32))
    g.launch()
    ctx.flush()
    assert np.array_equal(got, out.download(np.float32, n * h).reshape(n, h))
    g.destroy()
