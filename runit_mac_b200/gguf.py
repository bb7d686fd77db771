"""Host-side mirror of the reference's GGUF crate over the C ABI of ``include/runit_gguf.h``.

Names follow ``crates/gguf/src`` of the reference: ``parse_gguf_file`` / ``GgufParser.parse`` (parser.rs:22,229),
``GgufFile`` / ``GgufTensorInfo`` (types.rs:18-63), ``GgufDtype`` (types.rs:69-199), ``GgufError`` (error.rs:4-31).
Parsing and the tables run in the library (no GPU needed); ``upload_weight`` copies a tensor's packed bytes into
device memory for the fused-dequant kernels (the reference's ``upload_weight_wb``, crates/engine/src/forward.rs:1137-1222,
and its per-expert slicing of merged ``*_exps`` tensors, forward.rs:1321-1418 — here the merged tensor stays one buffer).
"""
from __future__ import annotations

import ctypes as C
from collections import namedtuple
from pathlib import Path

from . import _lib

GGUF_MAGIC = 0x46554747
GGUF_DEFAULT_ALIGNMENT = 32

_KINDS = {
    1: "Io", 2: "InvalidMagic", 3: "UnsupportedVersion", 4: "UnknownDtype", 5: "UnknownMetadataType",
    6: "UnexpectedEof", 7: "InvalidUtf8", 8: "DataRegionOverflow", 9: "NotFound", 10: "BadArg", 11: "BufferSize", 12: "Cuda",
}

# ggml type id -> kernel format id of include/runit_cuda.h (RUNIT_FMT_*)
KERNEL_FORMATS = {8: 0, 2: 1, 12: 2, 6: 3, 13: 4, 14: 5}     # Q8_0, Q4_0, Q4_K, Q5_0, Q5_K, Q6_K


class GgufError(RuntimeError):
    """One kind per variant of the reference's ``GgufError`` (plus lookups of this ABI)."""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status
        self.kind = _KINDS.get(status, "Unknown")


class _Info(C.Structure):
    _fields_ = [("name", C.c_char_p), ("dtype", C.c_uint32), ("n_dims", C.c_uint32), ("ne", C.c_uint64 * 4),
                ("data_offset", C.c_uint64), ("num_elements", C.c_uint64), ("data_size", C.c_uint64)]


_bound = None


def _api():
    """The GGUF entry points of librunit_cuda.so with their prototypes."""
    global _bound
    if _bound is not None:
        return _bound
    lib = _lib.load()
    vp, u32, u64, i32, cp = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int32, C.c_char_p
    P = C.POINTER
    sigs = {
        "runit_gguf_open": (i32, [cp, P(vp)]),
        "runit_gguf_open_memory": (i32, [vp, u64, P(vp)]),
        "runit_gguf_close": (None, [vp]),
        "runit_gguf_last_error": (cp, []),
        "runit_gguf_version": (u32, [vp]),
        "runit_gguf_alignment": (u64, [vp]),
        "runit_gguf_data_offset": (u64, [vp]),
        "runit_gguf_tensor_count": (u64, [vp]),
        "runit_gguf_metadata_count": (u64, [vp]),
        "runit_gguf_tensor_at": (i32, [vp, u64, P(_Info)]),
        "runit_gguf_tensor_find": (i32, [vp, cp, P(_Info)]),
        "runit_gguf_dtype_block_size": (u64, [u32]),
        "runit_gguf_dtype_type_size": (u64, [u32]),
        "runit_gguf_dtype_tensor_data_size": (u64, [u32, u64]),
        "runit_gguf_dtype_name": (cp, [u32]),
        "runit_gguf_meta_key_at": (i32, [vp, u64, P(cp)]),
        "runit_gguf_meta_type": (i32, [vp, cp, P(u32), P(u32), P(u64)]),
        "runit_gguf_meta_u64": (i32, [vp, cp, P(u64)]),
        "runit_gguf_meta_i64": (i32, [vp, cp, P(C.c_int64)]),
        "runit_gguf_meta_f64": (i32, [vp, cp, P(C.c_double)]),
        "runit_gguf_meta_bool": (i32, [vp, cp, P(i32)]),
        "runit_gguf_meta_str": (i32, [vp, cp, P(vp), P(u64)]),
        "runit_gguf_meta_array_u64": (i32, [vp, cp, u64, P(u64)]),
        "runit_gguf_meta_array_i64": (i32, [vp, cp, u64, P(C.c_int64)]),
        "runit_gguf_meta_array_f64": (i32, [vp, cp, u64, P(C.c_double)]),
        "runit_gguf_meta_array_str": (i32, [vp, cp, u64, P(vp), P(u64)]),
        "runit_gguf_read_tensor": (i32, [vp, cp, vp, u64]),
        "runit_gguf_upload_tensor": (i32, [vp, vp, cp, vp, u64]),
    }
    for name, (ret, args) in sigs.items():
        fn = getattr(lib, name)   # AttributeError = the library does not export what the header declares
        fn.restype, fn.argtypes = ret, args
    _bound = lib
    return lib


class GgufDtype:
    """ggml tensor type id with the reference's table methods (types.rs:142-199)."""

    F32, F16, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q8_1 = 0, 1, 2, 3, 6, 7, 8, 9
    Q2K, Q3K, Q4K, Q5K, Q6K, Q8K = 10, 11, 12, 13, 14, 15
    BF16 = 30

    @staticmethod
    def from_u32(v: int):
        return v if _api().runit_gguf_dtype_name(v) is not None else None

    @staticmethod
    def block_size(dtype: int) -> int:
        return _api().runit_gguf_dtype_block_size(dtype)

    @staticmethod
    def type_size(dtype: int) -> int:
        return _api().runit_gguf_dtype_type_size(dtype)

    @staticmethod
    def tensor_data_size(dtype: int, num_elements: int) -> int:
        return _api().runit_gguf_dtype_tensor_data_size(dtype, num_elements)

    @staticmethod
    def name(dtype: int) -> str:
        n = _api().runit_gguf_dtype_name(dtype)
        return n.decode() if n is not None else "?"


class GgufTensorInfo(namedtuple("GgufTensorInfo", "name shape dtype data_offset num_elements_ data_size_")):
    """``shape`` lists the dimensions in file order (``shape[0]`` = row length K)."""

    def num_elements(self) -> int:
        return self.num_elements_

    def data_size(self) -> int:
        return self.data_size_


WeightBuf = namedtuple("WeightBuf", "buffer fmt rows k experts dtype")


class GgufFile:
    """Parsed file: ``version``, ``metadata`` (dict), ``tensors`` (file order), ``data_offset``."""

    def __init__(self, handle, keep=None):
        self._h = handle
        self._keep = keep   # the memory image, if parsed from bytes
        api = _api()
        self.version = api.runit_gguf_version(handle)
        self.alignment = api.runit_gguf_alignment(handle)
        self.data_offset = api.runit_gguf_data_offset(handle)
        self.tensors = []
        info = _Info()
        for i in range(api.runit_gguf_tensor_count(handle)):
            _check(api.runit_gguf_tensor_at(handle, i, C.byref(info)))
            self.tensors.append(GgufTensorInfo(info.name.decode(), [int(info.ne[d]) for d in range(info.n_dims)], int(info.dtype),
                                               int(info.data_offset), int(info.num_elements), int(info.data_size)))
        self._by_name = {t.name: t for t in self.tensors}
        self.metadata = {}
        key = C.c_char_p()
        for i in range(api.runit_gguf_metadata_count(handle)):
            _check(api.runit_gguf_meta_key_at(handle, i, C.byref(key)))
            self.metadata[key.value.decode()] = self._value(key.value)

    def _value(self, key: bytes):
        api = _api()
        t, et, n = C.c_uint32(), C.c_uint32(), C.c_uint64()
        _check(api.runit_gguf_meta_type(self._h, key, C.byref(t), C.byref(et), C.byref(n)))
        if t.value == 9:
            return [self._scalar(key, et.value, i) for i in range(n.value)]
        return self._scalar(key, t.value, None)

    def _scalar(self, key: bytes, t: int, index):
        api = _api()
        pre = (self._h, key) if index is None else (self._h, key, index)
        sfx = "" if index is None else "array_"
        if t in (0, 2, 4, 10):
            v = C.c_uint64()
            _check(getattr(api, "runit_gguf_meta_%su64" % sfx)(*pre, C.byref(v)))
            return int(v.value)
        if t in (1, 3, 5, 11):
            v = C.c_int64()
            _check(getattr(api, "runit_gguf_meta_%si64" % sfx)(*pre, C.byref(v)))
            return int(v.value)
        if t in (6, 12):
            v = C.c_double()
            _check(getattr(api, "runit_gguf_meta_%sf64" % sfx)(*pre, C.byref(v)))
            return float(v.value)
        if t == 7:
            if index is not None:
                v = C.c_uint64()
                _check(api.runit_gguf_meta_array_u64(*pre, C.byref(v)))
                return bool(v.value)
            v = C.c_int32()
            _check(api.runit_gguf_meta_bool(*pre, C.byref(v)))
            return bool(v.value)
        if t == 8:
            p, n = C.c_void_p(), C.c_uint64()
            _check(getattr(api, "runit_gguf_meta_%sstr" % sfx)(*pre, C.byref(p), C.byref(n)))
            return C.string_at(p.value, n.value).decode()
        return None   # nested arrays are not flattened here

    def tensor(self, name: str) -> GgufTensorInfo:
        if name not in self._by_name:
            info = _Info()
            _check(_api().runit_gguf_tensor_find(self._h, name.encode(), C.byref(info)))
        return self._by_name[name]

    def read_tensor(self, name: str) -> bytes:
        """The tensor's bytes as stored in the file."""
        t = self.tensor(name)
        buf = (C.c_uint8 * max(1, t.data_size()))()
        _check(_api().runit_gguf_read_tensor(self._h, name.encode(), buf, t.data_size()))
        return bytes(buf[: t.data_size()])

    def upload_weight(self, ctx, name: str) -> WeightBuf:
        """Packed bytes of ``name`` in a new device buffer.  ``fmt`` is the kernel format id for Q8_0 / Q4_0 / Q4_K / Q5_0 /
        Q5_K / Q6_K tensors and None for the others (F32 / F16 norms, router, embeddings are uploaded as they are)."""
        t = self.tensor(name)
        buf = ctx.new_buffer(max(16, t.data_size()))
        _check(_api().runit_gguf_upload_tensor(ctx.handle, self._h, name.encode(), C.c_void_p(buf.ptr), buf.nbytes))
        k = t.shape[0] if t.shape else 1
        rows = t.shape[1] if len(t.shape) > 1 else 1
        experts = t.shape[2] if len(t.shape) > 2 else 1
        return WeightBuf(buf, KERNEL_FORMATS.get(t.dtype), rows, k, experts, t.dtype)

    def close(self):
        if self._h:
            _api().runit_gguf_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _check(status: int):
    if status != 0:
        raise GgufError(status, _api().runit_gguf_last_error().decode())


def parse_gguf_file(path) -> GgufFile:
    h = C.c_void_p()
    _check(_api().runit_gguf_open(str(Path(path)).encode(), C.byref(h)))
    return GgufFile(h)


class GgufParser:
    """``GgufParser(reader).parse()`` of the reference, over an in-memory image (bytes)."""

    def __init__(self, image: bytes):
        self._image = bytes(image)

    def parse(self) -> GgufFile:
        keep = C.create_string_buffer(self._image, max(1, len(self._image)))
        h = C.c_void_p()
        _check(_api().runit_gguf_open_memory(keep, len(self._image), C.byref(h)))
        return GgufFile(h, keep=keep)


def align_offset(offset: int, alignment: int) -> int:
    """parser.rs: next multiple of ``alignment`` at or after ``offset``."""
    return (offset + alignment - 1) // alignment * alignment
