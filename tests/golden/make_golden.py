"""Generates tests/golden/path_golden.npz — frozen input/output vectors of the CPU oracle.

The reference project cannot be built or run outside macOS (Rust + Metal) and holds no golden
vectors for the quantized operators, so these fixtures are produced by the oracle
(oracle/runit_oracle.c, f64-accumulation tier) on seeded inputs and committed; the tests check
both the oracle (regression) and the CUDA library against them.  Run from the repository root:

    python tests/golden/make_golden.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import oracle as O  # noqa: E402


def main():
    O.build_oracle()
    rng = np.random.default_rng(20240607)
    out = {}
    # GEMV cases: (format, m, k) with ragged tile / unit counts
    cases = [(O.Q8_0, 37, 896), (O.Q8_0, 5, 96), (O.Q4_0, 33, 512), (O.Q4_0, 9, 160), (O.Q4K, 40, 1024),
             (O.Q4K, 3, 256)]
    for i, (fmt, m, k) in enumerate(cases):
        w = O.rand_weights(fmt, rng, m, k)
        x = rng.normal(0, 1, (2, k)).astype(np.float32)
        y = O.gemv(fmt, w, x, m, k, O.TIER_F64)
        out["gemv%d_fmt" % i] = np.array([fmt, m, k], np.int32)
        out["gemv%d_w" % i] = w
        out["gemv%d_x" % i] = x
        out["gemv%d_y" % i] = y
    # routing
    logits = rng.normal(0, 1, (6, 64)).astype(np.float32)
    idx, wts, wts_rn = [], [], []
    for r in range(6):
        i_, w_, _ = O.topk_softmax(logits[r], 8, False)
        _, wr, _ = O.topk_softmax(logits[r], 8, True)
        idx.append(i_); wts.append(w_); wts_rn.append(wr)
    out["route_logits"] = logits
    out["route_idx"] = np.stack(idx)
    out["route_w"] = np.stack(wts)
    out["route_w_renorm"] = np.stack(wts_rn)
    # one small MoE block: h=256, ff=256, E=4, top-2, T=3
    h, ff, E, k = 256, 256, 4, 2
    router = rng.normal(0, 0.02, (E, h)).astype(np.float32)
    gate = O.rand_q4k(rng, E * ff, h)
    up = O.rand_q4k(rng, E * ff, h)
    down = O.rand_q4k(rng, E * h, ff)
    x = rng.normal(0, 1, (3, h)).astype(np.float32)
    y, mi, mw = O.moe_layer_q4k(router, gate, up, down, x, h=h, ff=ff, E=E, top_k=k, renorm=False)
    out.update(moe_router=router, moe_gate=gate, moe_up=up, moe_down=down, moe_x=x, moe_y=y, moe_idx=mi,
               moe_w=mw, moe_dims=np.array([h, ff, E, k], np.int32))
    np.savez_compressed(Path(__file__).with_name("path_golden.npz"), **out)
    print("wrote", Path(__file__).with_name("path_golden.npz"))


if __name__ == "__main__":
    main()
