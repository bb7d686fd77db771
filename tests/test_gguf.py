"""GGUF reader behind the C ABI of include/runit_gguf.h: the cases of the reference's parser tests
(crates/gguf/src/parser.rs:240-348: minimal file, invalid magic, unsupported version, tensor data size, alignment)
plus every metadata type, truncation and the data-region check.  No GPU is touched."""
import re
import struct
from pathlib import Path

import numpy as np
import pytest

from gguf_writer import (T_ARR, T_BOOL, T_F32, T_F64, T_I8, T_I16, T_I32, T_I64, T_STR, T_U8, T_U16, T_U32, T_U64,
                         build_gguf)

ROOT = Path(__file__).resolve().parents[1]


def minimal():
    # the reference's build_test_gguf: one metadata string, one 4 x 8 F32 tensor
    data = np.arange(32, dtype=np.float32)
    return build_gguf([("general.architecture", T_STR, "qwen2")], [("test.weight", [4, 8], 0, data)]), data


def test_header_symbols_are_exported():
    from runit_mac_b200 import _lib, gguf
    text = (ROOT / "include" / "runit_gguf.h").read_text()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    names = set(re.findall(r"\b(runit_gguf_\w+)\s*\(", text))
    assert len(names) >= 28
    lib = _lib.load()
    for n in names:
        assert hasattr(lib, n), n
    gguf._api()
    head = (ROOT / "include" / "runit_gguf.h").read_text()
    for cite in ("crates/gguf/src/parser.rs:22", "crates/gguf/src/types.rs:69-199", "crates/gguf/src/error.rs:4-31"):
        assert cite in head


def test_parse_minimal_gguf():
    from runit_mac_b200.gguf import GgufDtype, GgufParser
    img, data = minimal()
    g = GgufParser(img).parse()
    assert g.version == 3
    assert len(g.tensors) == 1
    t = g.tensors[0]
    assert t.name == "test.weight" and t.shape == [4, 8] and t.dtype == GgufDtype.F32 and t.data_offset == 0
    assert g.data_offset % 32 == 0 and g.data_offset <= len(img)
    assert g.metadata["general.architecture"] == "qwen2"
    assert t.num_elements() == 32 and t.data_size() == 128
    assert np.array_equal(np.frombuffer(g.read_tensor("test.weight"), np.float32), data)
    g.close()


def test_parse_from_a_file(tmp_path):
    from runit_mac_b200.gguf import parse_gguf_file, GgufError
    img, data = minimal()
    p = tmp_path / "m.gguf"
    p.write_bytes(img)
    g = parse_gguf_file(p)
    assert g.version == 3 and g.tensors[0].shape == [4, 8]
    assert np.array_equal(np.frombuffer(g.read_tensor("test.weight"), np.float32), data)
    with pytest.raises(GgufError) as e:
        g.tensor("missing.weight")
    assert e.value.kind == "NotFound"
    with pytest.raises(GgufError) as e:
        parse_gguf_file(tmp_path / "absent.gguf")
    assert e.value.kind == "Io"


def test_invalid_magic():
    from runit_mac_b200.gguf import GgufError, GgufParser
    img, _ = minimal()
    bad = struct.pack("<I", 0xDEADBEEF) + img[4:]
    with pytest.raises(GgufError) as e:
        GgufParser(bad).parse()
    assert e.value.kind == "InvalidMagic" and "0xDEADBEEF" in str(e.value)


def test_unsupported_version():
    from runit_mac_b200.gguf import GgufError, GgufParser
    with pytest.raises(GgufError) as e:
        GgufParser(build_gguf([], [], version=99)).parse()
    assert e.value.kind == "UnsupportedVersion" and "99" in str(e.value)
    assert GgufParser(build_gguf([], [], version=2)).parse().version == 2


def test_tensor_data_size_and_dtype_table():
    from runit_mac_b200.gguf import GgufDtype as D
    # the reference's case: Q4_K, 4096 x 4096 -> 65536 blocks of 144 bytes
    n = 4096 * 4096
    assert D.tensor_data_size(D.Q4K, n) == (n // 256) * 144
    table = {D.F32: (1, 4), D.F16: (1, 2), D.BF16: (1, 2), D.Q4_0: (32, 18), D.Q4_1: (32, 20), D.Q5_0: (32, 22),
             D.Q5_1: (32, 24), D.Q8_0: (32, 34), D.Q8_1: (32, 40), D.Q2K: (256, 84), D.Q3K: (256, 110), D.Q4K: (256, 144),
             D.Q5K: (256, 176), D.Q6K: (256, 210), D.Q8K: (256, 292)}
    for dt, (bs, ts) in table.items():
        assert (D.block_size(dt), D.type_size(dt)) == (bs, ts), dt
    assert D.tensor_data_size(D.Q8_0, 33) == 2 * 34          # partial blocks round up
    assert D.name(D.Q4K) == "Q4_K" and D.name(D.Q6K) == "Q6_K" and D.name(D.F32) == "F32"
    assert D.from_u32(12) == 12 and D.from_u32(4) is None and D.from_u32(5) is None and D.from_u32(31) is None


def test_align_offset_and_custom_alignment():
    from runit_mac_b200.gguf import GgufParser, align_offset
    assert [align_offset(o, 32) for o in (0, 1, 31, 32, 33)] == [0, 32, 32, 32, 64]
    a = np.arange(5, dtype=np.float32)
    b = np.arange(7, dtype=np.float32) + 100
    g = GgufParser(build_gguf([], [("a", [5], 0, a), ("b", [7], 0, b)], alignment=64)).parse()
    assert g.alignment == 64 and g.data_offset % 64 == 0
    assert g.tensor("b").data_offset == 64
    assert np.array_equal(np.frombuffer(g.read_tensor("b"), np.float32), b)
    assert np.array_equal(np.frombuffer(g.read_tensor("a"), np.float32), a)


def test_every_metadata_type():
    from runit_mac_b200.gguf import GgufParser
    md = [("u8", T_U8, 200), ("i8", T_I8, -5), ("u16", T_U16, 60000), ("i16", T_I16, -30000), ("u32", T_U32, 4000000000),
          ("i32", T_I32, -2000000000), ("f32", T_F32, 1.5), ("yes", T_BOOL, 1), ("no", T_BOOL, 0), ("s", T_STR, "héllo ✓"),
          ("u64", T_U64, 2 ** 63 + 5), ("i64", T_I64, -2 ** 62), ("f64", T_F64, 1e-300),
          ("tokens", T_ARR, (T_STR, ["a", "", "ccc"])), ("ids", T_ARR, (T_I32, [-1, 0, 7])), ("scores", T_ARR, (T_F32, [0.5, -2.0])),
          ("flags", T_ARR, (T_BOOL, [1, 0])), ("empty", T_ARR, (T_U8, []))]
    g = GgufParser(build_gguf(md, [])).parse()
    m = g.metadata
    assert list(m) == [k for k, _, _ in md]            # file order
    assert (m["u8"], m["i8"], m["u16"], m["i16"], m["u32"], m["i32"]) == (200, -5, 60000, -30000, 4000000000, -2000000000)
    assert m["f32"] == 1.5 and m["yes"] is True and m["no"] is False and m["s"] == "héllo ✓"
    assert m["u64"] == 2 ** 63 + 5 and m["i64"] == -2 ** 62 and m["f64"] == 1e-300
    assert m["tokens"] == ["a", "", "ccc"] and m["ids"] == [-1, 0, 7] and m["scores"] == [0.5, -2.0]
    assert m["flags"] == [True, False] and m["empty"] == []


def test_malformed_files_report_the_reference_error_kinds():
    from runit_mac_b200.gguf import GgufError, GgufParser
    img, _ = minimal()

    def kind(image):
        with pytest.raises(GgufError) as e:
            GgufParser(image).parse()
        return e.value.kind

    assert kind(img[:10]) == "UnexpectedEof"                       # inside the header
    assert kind(img[:40]) == "UnexpectedEof"                       # inside the metadata
    assert kind(b"") == "UnexpectedEof"
    assert kind(img[:-8]) == "DataRegionOverflow"                  # tensor bytes cut short
    assert kind(build_gguf([("k", 13, 0)], []) if False else struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + struct.pack("<Q", 1) + b"k" + struct.pack("<I", 13)) == "UnknownMetadataType"
    assert kind(build_gguf([], [("t", [8], 4, b"\0" * 64)])) == "UnknownDtype"      # ggml id 4 was removed from the format
    bad_utf8 = struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + struct.pack("<Q", 2) + b"\xff\xfe" + struct.pack("<I", T_U8) + b"\0"
    assert kind(bad_utf8) == "InvalidUtf8"
    huge = struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + struct.pack("<Q", 1 << 60) + b"k"
    assert kind(huge) == "UnexpectedEof"                           # a string length beyond the file


def test_quantized_tensor_index_matches_the_packers(oracle):
    """Shapes and byte sizes of Q8_0 / Q4_0 / Q4_K tensors and of a merged expert tensor, read back bit-exactly."""
    from runit_mac_b200.gguf import GgufDtype as D, GgufParser
    O = oracle
    rng = np.random.default_rng(7)
    w8, w4, wk = O.rand_q8_0(rng, 6, 64), O.rand_q4_0(rng, 5, 96), O.rand_q4k(rng, 3, 512)
    ex = np.stack([O.rand_q4k(rng, 4, 256) for _ in range(3)])   # [E][rows][K/256 * 144]
    g = GgufParser(build_gguf([("general.architecture", T_STR, "olmoe")],
                              [("blk.0.attn_q.weight", [64, 6], D.Q8_0, w8), ("blk.0.attn_k.weight", [96, 5], D.Q4_0, w4),
                               ("blk.0.attn_v.weight", [512, 3], D.Q4K, wk), ("blk.0.ffn_gate_exps.weight", [256, 4, 3], D.Q4K, ex)])).parse()
    for name, arr in (("blk.0.attn_q.weight", w8), ("blk.0.attn_k.weight", w4), ("blk.0.attn_v.weight", wk),
                      ("blk.0.ffn_gate_exps.weight", ex)):
        t = g.tensor(name)
        assert t.data_size() == arr.nbytes, name
        assert g.read_tensor(name) == arr.tobytes(), name
    assert g.tensor("blk.0.ffn_gate_exps.weight").shape == [256, 4, 3]
