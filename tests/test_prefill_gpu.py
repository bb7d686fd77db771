"""GPU parity tests of the batched prefill (crates/engine/src/prefill.rs:29-255) through the C ABI.

The device path rounds GEMM operands to bf16 and attention operands to f16; oracle/prefill.py restates exactly that
arithmetic (f64 accumulation).  Single kernels are held to it at 1e-3 of the output scale (5e-3 for the bf16-rounded
attention output: one bf16 ulp is 2^-8 of the value), the whole pass over several tokens at 5e-3 rms (see the test).  Against the f32 decode oracle, which the reference's formulas pin, the same
quantities agree to bf16 operand rounding; tests/test_oracle.py holds that comparison."""
import numpy as np
import pytest

from helpers import assert_close

pytestmark = pytest.mark.gpu


def bf16_bits_to_f32(u16):
    return (u16.astype(np.uint32) << 16).view(np.float32)


@pytest.mark.parametrize("hd", [128, 64])
@pytest.mark.parametrize("T,start", [(1, 0), (63, 0), (64, 0), (65, 0), (200, 0), (70, 37)])
def test_causal_attention_kernel(ctx, oracle, hd, T, start):
    import runit_mac_b200 as R
    from oracle import prefill as OP
    heads, kvh, max_seq = 4, 2, 320
    rng = np.random.default_rng(T * 7 + hd + start)
    q = rng.normal(0, 1, (T, heads * hd)).astype(np.float32)
    kc = np.zeros((kvh, max_seq, hd), np.float16)
    vc = np.zeros((kvh, max_seq, hd), np.float16)
    kc[:, :start + T] = rng.normal(0, 1, (kvh, start + T, hd)).astype(np.float16)
    vc[:, :start + T] = rng.normal(0, 1, (kvh, start + T, hd)).astype(np.float16)
    kc[:, start + T:] = np.float16(1e4)        # rows past the data must never contribute
    vc[:, start + T:] = np.float16(1e4)
    ob = ctx.new_buffer(T * heads * hd * 2)
    R.prefill_attention_f16kv(ctx, ctx.buffer_from(q), ctx.buffer_from(kc), ctx.buffer_from(vc), ob, T, heads, kvh, hd, max_seq, start)
    ctx.flush()
    got = bf16_bits_to_f32(ob.download(np.uint16, T * heads * hd)).reshape(T, heads * hd)
    ref = OP.causal_attention_f16(q, kc, vc, heads, kvh, hd, start_pos=start)
    assert_close(oracle, ref, got, rel_tol=5e-3, what="prefill attention hd=%d T=%d start=%d" % (hd, T, start))


def test_small_model_prefill_matches_restatement_and_decode(ctx, oracle):
    import runit_mac_b200 as R
    from oracle import prefill as OP
    from test_decode_gpu import SMALL, build_model
    O = oracle
    model, ocfg, ow, host = build_model(ctx, R, O, SMALL, 11, device_fill=False, zero_mean=True)
    hostw = {k: v for k, v in host.items() if not k.startswith("_")}
    for n in (1, 5, 40, 57):
        prompt = np.random.default_rng(n).integers(0, SMALL["vocab"], n).astype(np.int32)
        tok = model.prefill(prompt)
        logits = model.logits()
        rtok, rlogits, kc, vc = OP.prefill(SMALL, hostw, prompt)
        spread = float(np.std(rlogits))
        if n == 1:
            # one token: attention is the value row itself, every GEMM and the MoE block are compared at the kernel bar
            assert_close(O, rlogits, logits, rel_tol=1e-3, what="prefill logits, 1 token")
        else:
            # several stages in a row: where the device's f32 sum and the restatement's f64 sum fall on different sides of a
            # bf16 (or f16) rounding boundary the operand of the next stage differs by one ulp (2^-8 of its value); a few
            # per cent of the operands do, which adds about 6e-4 rms per stage.  Held to 5e-3 rms / 2e-2 at worst.
            d = np.abs(logits - rlogits)
            assert np.sqrt((d ** 2).mean()) <= 5e-3 * spread and d.max() <= 2e-2 * spread, (n, d.max(), np.sqrt((d ** 2).mean()), spread)
        assert tok == rtok or abs(rlogits[tok] - rlogits[rtok]) <= 2e-2 * spread
        # decoding continues from the cache the prefill filled: the next steps agree with the decode oracle run on the
        # restatement's cache (f16 rounding of k and v can differ in the last bit where bf16 sums differ: logits at 1e-2)
        out = model.generate_greedy(np.array([tok], np.int32), 4, start_pos=n)
        kc = kc.copy(); vc = vc.copy()
        t = tok
        for step in range(3):
            t_ref, l_ref = O.decode_step(ocfg, ow, kc, vc, int(t), n + step, want_logits=True)
            if step == 0:
                model.generate_greedy(np.array([tok], np.int32), 0, start_pos=n)      # one step: logits of position n
                d = np.abs(model.logits() - l_ref)
                assert d.max() <= 2e-2 * float(np.std(l_ref)), (n, d.max(), float(np.std(l_ref)))
            t = t_ref
        # against the decoder run token by token on the device (f32 path): same next token unless the logits are that close
        model2 = R.Model(ctx, host["_cfg"], host["_dev"])
        o2 = model2.generate_greedy(prompt, 1, skip_prompt_logits=False)
        if o2[n - 1] != tok:
            assert abs(rlogits[tok] - rlogits[o2[n - 1]]) <= 8e-2 * spread
        model2.close()
        assert out[0] >= 0
    with pytest.raises(R.KernelError):
        model.prefill(np.array([SMALL["vocab"]], np.int32))                  # InvalidTokenId, prefill.rs:55-57
    with pytest.raises(R.KernelError):
        model.prefill(np.zeros(SMALL["max_seq"] + 1, np.int32))
    model.close()


def test_olmoe_shaped_prefill_128_tokens(ctx, oracle):
    """The 128-token prompt of the decode benchmark through the batched pass at the full OLMoE shape: the logits of the
    last position against the f32 decode oracle fed token by token (bf16 operand rounding: 1e-2 of the spread rms)."""
    import runit_mac_b200 as R
    from test_decode_gpu import OLMOE_EMB_SIGMA, OLMOE_WEIGHT_SIGMA, build_model
    O = oracle
    cfg = dict(n_layers=16, hidden=2048, n_heads=16, n_kv_heads=16, head_dim=128, vocab=50304, n_experts=64, top_k=8, ff=1024,
               max_seq=2048, renorm=0, eps=1e-5, theta=10000.0)
    model, ocfg, ow, host = build_model(ctx, R, O, cfg, 1004, device_fill=True, zero_mean=True, weight_sigma=OLMOE_WEIGHT_SIGMA,
                                        emb_sigma=OLMOE_EMB_SIGMA)
    prompt = np.random.default_rng(1004).integers(0, 50304, 128).astype(np.int32)
    tok = model.prefill(prompt)
    logits = model.logits()
    L, kvh, S, hd = 16, 16, 2048, 128
    kc = np.zeros((L, kvh, S, hd), np.float16)
    vc = np.zeros_like(kc)
    for pos, t in enumerate(prompt[:-1]):
        O.decode_step(ocfg, ow, kc, vc, int(t), pos)
    ref_tok, ref_logits = O.decode_step(ocfg, ow, kc, vc, int(prompt[-1]), len(prompt) - 1, want_logits=True)
    spread = float(np.std(ref_logits))
    d = np.abs(logits - ref_logits)
    assert np.sqrt((d ** 2).mean()) <= 1e-2 * spread and d.max() <= 8e-2 * spread, (d.max(), np.sqrt((d ** 2).mean()), spread)
    assert tok == ref_tok or abs(ref_logits[tok] - ref_logits[ref_tok]) <= 8e-2 * spread
    # and the decoder continues from that cache
    out = model.generate_greedy(np.array([tok], np.int32), 8, start_pos=128)
    assert (out >= 0).all()
    model.close()


@pytest.mark.parametrize("T", [1, 100, 300])
def test_dense_ffn_block(ctx, oracle, T):
    """The dense feed-forward block of a prefill pass (prefill.rs:217-227) on the tensor cores, with and without the RMSNorm in
    front and the residual, against the bf16-operand restatement (the batched block's oracle with one expert, weight 1)."""
    import runit_mac_b200 as R
    O = oracle
    h, ff = 512, 768
    rng = np.random.default_rng(40 + T)
    wg, wu, wd = O.rand_q4k(rng, ff, h), O.rand_q4k(rng, ff, h), O.rand_q4k(rng, h, ff)
    x = rng.normal(0, 1, (T, h)).astype(np.float32)
    res = rng.normal(0, 1, (T, h)).astype(np.float32)
    gamma = rng.normal(1, 0.1, h).astype(np.float32)
    nb = ctx.lib.runit_ffn_q4k_bf16_scratch_bytes(T, h, ff)
    scratch = ctx.new_buffer(nb)
    wb = [ctx.buffer_from(w) for w in (wg, wu, wd)]
    ob = ctx.new_buffer(T * h * 4)
    routing = (np.zeros((T, 1), np.int32), np.ones((T, 1), np.float32))
    for use_gamma, use_res in ((False, False), (True, True), (False, True)):
        xin = O.rms_norm_f32(x, gamma, 1e-5) if use_gamma else x
        ref, _, _ = O.moe_grouped_q4k_bf16(None, wg, wu, wd, xin, h=h, ff=ff, E=1, top_k=1, residual=res if use_res else None, routing=routing)
        R.ffn_q4k_bf16(ctx, *wb, ctx.buffer_from(x), ctx.buffer_from(gamma) if use_gamma else None, 1e-5,
                       ctx.buffer_from(res) if use_res else None, ob, scratch, nb, T, h, ff)
        ctx.flush()
        got = ob.download(np.float32, T * h).reshape(T, h)
        scale = np.maximum(np.abs(ref), np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
        rel = float((np.abs(got - ref) / scale).max())
        assert rel <= 4e-3, (T, use_gamma, use_res, rel)
