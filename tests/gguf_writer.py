"""Test-side GGUF writer (the product only reads GGUF): builds a little-endian v2/v3 image from Python values."""
from __future__ import annotations

import struct

import numpy as np

T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 = range(13)
_FMT = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i", T_F32: "<f", T_BOOL: "<B",
        T_U64: "<Q", T_I64: "<q", T_F64: "<d"}


def _string(s) -> bytes:
    b = s if isinstance(s, bytes) else s.encode()
    return struct.pack("<Q", len(b)) + b


def _value(vtype: int, v) -> bytes:
    if vtype == T_STR:
        return _string(v)
    if vtype == T_ARR:
        et, items = v
        return struct.pack("<IQ", et, len(items)) + b"".join(_value(et, x) for x in items)
    return struct.pack(_FMT[vtype], v)


def build_gguf(metadata, tensors, version: int = 3, alignment: int | None = None, magic: int = 0x46554747) -> bytes:
    """metadata: list of (key, type, value); tensors: list of (name, dims in file order, ggml type id, bytes)."""
    metadata = list(metadata)
    if alignment is not None:
        metadata.append(("general.alignment", T_U32, alignment))
    align = alignment or 32
    out = struct.pack("<IIQQ", magic, version, len(tensors), len(metadata))
    for key, vtype, v in metadata:
        out += _string(key) + struct.pack("<I", vtype) + _value(vtype, v)
    tensors = [(n, d, t, data.tobytes() if isinstance(data, np.ndarray) else bytes(data)) for n, d, t, data in tensors]
    offsets, off = [], 0
    for _name, _dims, _dt, data in tensors:
        offsets.append(off)
        off = (off + len(data) + align - 1) // align * align
    for (name, dims, dt, _data), o in zip(tensors, offsets):
        out += _string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        out += struct.pack("<IQ", dt, o)
    out += b"\0" * ((len(out) + align - 1) // align * align - len(out))
    base = len(out)
    for (_name, _dims, _dt, data), o in zip(tensors, offsets):
        out += b"\0" * (base + o - len(out)) + data
    return out
