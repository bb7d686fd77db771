"""CPU checks of the drop-in boundary: the shared library loads, exports every symbol that
include/runit_cuda.h declares (no compute call is made without a GPU), and the host-side mirror of
the reference's dispatch layer exposes the reference's operator names."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    from runit_mac_b200 import _lib
    protos = _lib.parse_header()
    assert len(protos) >= 45
    lib = _lib.load()   # raises ImportError listing the missing names
    for name in protos:
        assert hasattr(lib, name), name


def test_header_cites_the_reference_interface():
    text = (ROOT / "include" / "runit_cuda.h").read_text()
    # every twin of a dispatch.rs function carries its file:line
    for name in ("gemv_q8_0_f32in_f32out", "gemv_q4_0_f32in_f32out", "gemv_q4k_f32in_f32out", "fused_qkv_bias_q8_0_f32",
                 "fused_ffn_q8_0_f32", "scale_accumulate_f16", "dequant_q4k_f16"):
        i = text.index("runit_" + name + "(")
        assert re.search(r"dispatch\.rs:\d+", text[max(0, i - 400):i]), name


def test_python_mirror_has_the_reference_operator_names():
    import runit_mac_b200 as R
    ref_names = ["gemv_q8_0_f32in_f32out", "gemv_q8_0_add_f32_f32in", "gemv_q8_0_f32in", "gemv_q8_0_f16", "gemv_q8_0_add_f16",
                 "gemv_q8_0_add_f32res_f16", "gemv_q4_0_f32in_f32out", "gemv_q4_0_add_f32_f32in", "gemv_q4_0_f32in",
                 "gemv_q4_0_f16", "gemv_q4_0_add_f16", "fused_ffn_q4_0_f32", "gemv_q4k_f32in_f32out", "gemv_q4k_add_f32_f32in",
                 "gemv_q4k_f16", "gemv_q4k_add_f16", "gemv_q4k_add_f32res_f16", "dequant_q4k_f16", "fused_qkv_q8_0_f32",
                 "fused_qkv_bias_q8_0_f32", "fused_ffn_q8_0_f32", "gemv_f16w_f32in", "silu_mul_f16", "silu_mul_f32",
                 "scale_accumulate_f16", "add_f16_into_f32"]
    for n in ref_names:
        assert callable(getattr(R, n)), n
    assert R.row_bytes(R.FMT_Q8_0, 896) == 952 and R.row_bytes(R.FMT_Q4_0, 3584) == 2016 and R.row_bytes(R.FMT_Q4K, 2048) == 1152


def test_status_strings_and_null_context_are_rejected_without_a_gpu():
    from runit_mac_b200 import _lib
    lib = _lib.load()
    assert lib.runit_status_string(0) == b"RUNIT_OK"
    assert lib.runit_status_string(2) == b"RUNIT_ERR_BAD_ARG"
    # a null context is a host-side argument error, never a launch
    assert lib.runit_flush(None) == 2
    assert lib.runit_gemv_q4k_f32in_f32out(None, None, None, None, 1, 256) == 2


def test_no_product_file_touches_the_oracle():
    """The product path must not import, link or call anything under oracle/."""
    for p in list((ROOT / "runit_mac_b200").rglob("*.py")) + list((ROOT / "runit_mac_b200" / "csrc").glob("*")):
        if p.is_file() and p.suffix in (".py", ".cu", ".cuh", ".h"):
            t = p.read_text()
            assert "oracle" not in t.lower() or p.name == "__never__", p


def test_rust_shim_covers_the_whole_boundary(tmp_path):
    """crates/kernels-cuda (source a maintainer adds to the reference workspace; no Rust toolchain here): ffi.rs declares
    every function of both headers, dispatch.rs wraps every operator, both are exactly what gen_bindings.py writes, and
    KernelError has the reference's variants with their shapes (crates/kernels/src/error.rs:4-22)."""
    import importlib.util
    shim = ROOT / "crates" / "kernels-cuda"
    spec = importlib.util.spec_from_file_location("gen_bindings", shim / "gen_bindings.py")
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    ffi, disp = (shim / "src" / "ffi.rs").read_text(), (shim / "src" / "dispatch.rs").read_text()
    fns = [f for h in gen.HEADERS for f in gen.parse(h)]
    assert len(fns) >= 120
    for _ret, name, _args in fns:
        assert "pub fn %s(" % name in ffi, name
    for name in ("gemv_q8_0_f32in_f32out", "gemv_q4k_add_f32_f32in", "fused_qkv_bias_q8_0_f32", "fused_ffn_q4_0_f32", "scale_accumulate_f16",
                 "moe_layer_q4k", "moe_layer_q4k_ep", "gemv_allgather_f32", "gemv_q6k_f32in_f32out", "decode_attention_f32", "argmax_f16"):
        assert "pub fn %s(ctx: &CudaContext" % name in disp, name
    # regenerate into a scratch copy and compare
    gen.HERE = tmp_path
    (tmp_path / "src").mkdir()
    gen.gen()
    assert (tmp_path / "src" / "ffi.rs").read_text() == ffi and (tmp_path / "src" / "dispatch.rs").read_text() == disp
    err = (shim / "src" / "error.rs").read_text()
    for variant in ("NoDevice,", "LibraryLoad { path: String, reason: String }", "PipelineNotFound(String)",
                    "PipelineCreate { name: String, reason: String }", "Dispatch(String)", "BufferSize { expected: usize, actual: usize }"):
        assert variant in err, variant
