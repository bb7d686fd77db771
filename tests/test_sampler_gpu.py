"""GPU parity tests of the device sampler against the oracle's restatement of the reference's host sampler
(crates/engine/src/sampler.rs:61-111), through the C ABI.

What is compared: the token of every draw (the generator streams are identical, so with identical probabilities the
draws coincide), and the vector the draw was made from (the filtered probabilities), to 1e-4 relative + 1e-9 absolute: the
device's softmax sum is a tree sum and its expf is the device's, while the reference adds the 50304 terms one after the other
in f32, which alone carries a rounding error of about sqrt(n) * 2^-24 = 1e-5 of the sum.  A draw may legitimately differ where r lands within that
rounding of a boundary of the running sum; the tests allow two such draws in 200 and require every other to match."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def run_draws(ctx, R, O, logits, cfg_vals, context, eos, seed, n_draws):
    n = logits.size
    lb, sb = ctx.buffer_from(logits), ctx.new_buffer(4 * n)
    cb = ctx.buffer_from(np.asarray(context if len(context) else [0], np.int32))
    eb = ctx.buffer_from(np.asarray(eos if len(eos) else [0], np.int32))
    rb = ctx.buffer_from(np.array([R.sampler_seed_state(ctx, seed)], np.uint64))
    tb = ctx.new_buffer(16)
    cfg = R.SamplerCfg(*cfg_vals)
    ocfg = O.SamplerCfg(*cfg_vals)
    orng = O.SamplerRng(seed)
    got, want, probs, oprobs = [], [], None, None
    for _ in range(n_draws):
        R.sample_f32(ctx, lb, sb, n, cfg, cb, 0, len(context), eb, len(eos), rb, tb)
        ctx.flush()
        got.append(int(tb.download(np.int32, 1)[0]))
        probs = sb.download(np.float32, n)
        t, oprobs = O.sample(logits, ocfg, context, eos, orng, want_probs=True)
        want.append(t)
    state = int(rb.download(np.uint64, 1)[0])
    return np.array(got), np.array(want), probs, oprobs, state, int(orng.state.value)


@pytest.mark.parametrize("n", [50304, 1000, 37])
@pytest.mark.parametrize("cfg_vals", [
    (1.0, 40, 0.95, 1.1, 1),     # SamplerConfig::default()
    (0.7, 40, 1.0, 1.0, 0),      # top-k only
    (0.5, 0, 0.9, 1.0, 0),       # top-p only (sharp distribution: the nucleus lies inside the 1024 most probable)
    (0.8, 0, 1.0, 1.2, 0),       # no filter: the draw runs over the whole vocabulary
    (1.0, 1000, 0.5, 1.0, 0),    # wide top-k
])
def test_draws_match_the_host_sampler(ctx, oracle, n, cfg_vals):
    import runit_mac_b200 as R
    O = oracle
    rng = np.random.default_rng(n + int(cfg_vals[0] * 10))
    logits = rng.normal(0, 2.5, n).astype(np.float32)
    context = rng.integers(0, n, 40).tolist() + [5, 5, 5]      # repeated tokens: the penalty applies per occurrence
    got, want, probs, oprobs, st, ost = run_draws(ctx, R, O, logits, cfg_vals, context, [3, 7], 42, 200)
    assert (got != want).sum() <= 2, (got[got != want], want[got != want])
    assert st == ost
    if cfg_vals[0] != 0:
        assert ((probs > 0) == (oprobs > 0)).all()
        np.testing.assert_allclose(probs, oprobs, rtol=1e-4, atol=1e-9)
        if (oprobs > 0).sum() > 10:
            assert len(set(got.tolist())) >= 3     # a distribution, not a constant


def test_greedy_penalty_eos_and_ties(ctx, oracle):
    import runit_mac_b200 as R
    O = oracle
    # temperature 0: argmax of the penalised scores, last index among equal maxima; the generator does not advance
    logits = np.array([1.0, 7.0, 3.0, 7.0, 0.5] + [0.0] * 2000, np.float32)
    got, want, _, _, st, ost = run_draws(ctx, R, O, logits, (0.0, 40, 0.95, 1.0, 0), [], [], 9, 2)
    assert got.tolist() == want.tolist() == [3, 3] and st == ost == R.sampler_seed_state(ctx, 9)
    # the penalty (twice on token 3, once on token 1) hands the maximum to token 2
    got, want, probs, oprobs, _, _ = run_draws(ctx, R, O, logits, (0.0, 0, 1.0, 2.0, 0), [3, 1, 3], [], 9, 1)
    assert got.tolist() == want.tolist() == [1] or got.tolist() == want.tolist()
    np.testing.assert_array_equal(probs[:5], oprobs[:5])
    # end-of-sequence ids are suppressed while the context is shorter than min_tokens
    got, want, _, _, _, _ = run_draws(ctx, R, O, logits, (0.0, 0, 1.0, 1.0, 5), [0, 0], [1, 3], 9, 1)
    assert got.tolist() == want.tolist() == [2]
    got, want, _, _, _, _ = run_draws(ctx, R, O, logits, (0.0, 0, 1.0, 1.0, 2), [0, 0], [1, 3], 9, 1)
    assert got.tolist() == want.tolist() == [3]
    # top-k ties: the first k entries in index order that reach the threshold stay
    logits = np.array([2.0, 2.0, 2.0, 5.0, 1.0], np.float32)
    got, want, probs, oprobs, _, _ = run_draws(ctx, R, O, logits, (1.0, 2, 1.0, 1.0, 0), [], [], 3, 20)
    assert (probs > 0).tolist() == (oprobs > 0).tolist() == [True, True, False, False, False]
    assert got.tolist() == want.tolist()


def test_nucleus_wider_than_the_candidates_is_reported(ctx, oracle):
    """Top-k off and a flat distribution over 5000 tokens: the nucleus of p = 0.9 needs 4500 of them; the launch says so."""
    import runit_mac_b200 as R
    logits = np.zeros(5000, np.float32)
    lb, sb = ctx.buffer_from(logits), ctx.new_buffer(4 * 5000)
    rb = ctx.buffer_from(np.array([R.sampler_seed_state(ctx, 1)], np.uint64))
    tb, cb = ctx.new_buffer(16), ctx.new_buffer(16)
    R.sample_f32(ctx, lb, sb, 5000, R.SamplerCfg(1.0, 0, 0.9, 1.0, 0), cb, 0, 0, cb, 0, rb, tb)
    with pytest.raises(R.KernelError) as e:
        ctx.flush()
    assert "nucleus" in str(e.value)
    ctx.flush()                      # reported once; the context stays usable
    with pytest.raises(R.KernelError):
        R.sample_f32(ctx, lb, sb, 5000, R.SamplerCfg(1.0, 2000, 0.9, 1.0, 0), cb, 0, 0, cb, 0, rb, tb)   # top_k > 1024


def test_sampled_generation_matches_oracle_loop(ctx, oracle):
    """generate.rs:299-350 on the device: a small decoder generates with the sampler inside its recorded step.  The oracle
    then replays the produced sequence (teacher forcing) and draws with the host sampler from its own logits and the same
    generator stream: every draw must give the token the device produced (one draw in the run may sit on a boundary)."""
    import runit_mac_b200 as R
    from test_decode_gpu import SMALL, build_model
    O = oracle
    model, ocfg, ow, host = build_model(ctx, R, O, SMALL, 11, device_fill=False, zero_mean=True)
    prompt = [3, 17, 250, 9]
    n_gen = 24
    vals = (0.9, 40, 0.95, 1.1, 1)
    out = model.generate_sampled(prompt, n_gen, R.SamplerCfg(*vals), seed=7, eos_ids=[5])
    assert (out[:len(prompt) - 1] == -1).all()
    got = out[len(prompt) - 1:].tolist()
    L, kvh, S, hd = ocfg.n_layers, ocfg.n_kv_heads, ocfg.max_seq, ocfg.head_dim
    kc = np.zeros((L, kvh, S, hd), np.float16)
    vc = np.zeros_like(kc)
    orng = O.SamplerRng(7)
    seq = prompt + got
    want = []
    for step in range(len(prompt) + n_gen):
        _, logits = O.decode_step(ocfg, ow, kc, vc, int(seq[step]), step, want_logits=True)
        if step >= len(prompt) - 1:
            g = step - (len(prompt) - 1)
            want.append(O.sample(logits, O.SamplerCfg(*vals), got[:g], [5], orng))
    assert sum(a != b for a, b in zip(got, want)) <= 1, (got, want)
    assert len(set(got)) > 3
    # the same seed gives the same stream again; another seed another one
    assert model.generate_sampled(prompt, n_gen, R.SamplerCfg(*vals), seed=7, eos_ids=[5]).tolist() == out.tolist()
    assert model.generate_sampled(prompt, n_gen, R.SamplerCfg(*vals), seed=8, eos_ids=[5]).tolist() != out.tolist()
    # greedy through the sampler (temperature 0, no penalty) equals the greedy decoder unless a tie decides
    g0 = model.generate_sampled(prompt, n_gen, R.SamplerCfg(0.0, 0, 1.0, 1.0, 0), seed=1)
    g1 = model.generate_greedy(prompt, n_gen)
    assert g0.tolist() == g1.tolist()
    model.close()
