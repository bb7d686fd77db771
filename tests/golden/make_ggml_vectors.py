"""Writes tests/golden/ggml_dequant.npz: seeded blocks of four weight formats together with what the `gguf` Python
package (the block formats' upstream definition, gguf.quants.dequantize; version recorded in the file) makes of them.

Run where that package is installed:  python tests/golden/make_ggml_vectors.py
The parity tests only read the file.  It pins the oracle's decoders to an implementation written by someone else for the
formats where the reference decodes like upstream (Q8_0, Q5_0) and, through the stated re-ordering, for Q4_0 and Q4_K,
whose element order / scale slots differ in the reference (crates/kernels/shaders/gemv_q4_0.metal:26-49,
crates/engine/src/forward.rs:1039-1054)."""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

import gguf                                             # noqa: E402
from gguf import GGMLQuantizationType as T, quants     # noqa: E402

from oracle import packing as P                         # noqa: E402

# (Q5_K and Q6_K are left out: the reference's decoders for them, forward.rs:920-949 and 979-1012, index the high bits and
# the scales differently from upstream, and no simple re-ordering of a block maps one onto the other.)
FORMATS = {"q8_0": (0, T.Q8_0, 32), "q4_0": (1, T.Q4_0, 32), "q4k": (2, T.Q4_K, 256), "q5_0": (3, T.Q5_0, 32)}


def main():
    rng = np.random.default_rng(20240611)
    out = {"gguf_version": np.array(getattr(gguf, "__version__", "0.19.0"))}
    for name, (fmt, qt, be) in FORMATS.items():
        m, k = 3, be * 4
        raw = np.asarray(P.rand_weights(fmt, rng, m, k), np.uint8).reshape(m, -1)
        out[name + "_raw"] = raw
        out[name + "_ggml"] = quants.dequantize(raw, qt).astype(np.float32)
    np.savez_compressed(Path(__file__).with_name("ggml_dequant.npz"), **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
