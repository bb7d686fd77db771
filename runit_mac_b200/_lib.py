"""Loader of ``librunit_cuda.so`` — the C-ABI library declared in ``include/runit_cuda.h``.

The library is the product; this module only finds it, checks that every declared symbol is
exported and gives each one a ctypes prototype parsed from the header.  There is no fallback:
if the library is missing or a symbol is absent, import fails loudly.
"""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

PKG = Path(__file__).resolve().parent
HEADER = PKG.parent / "include" / "runit_cuda.h"
LIB_PATH = PKG / "librunit_cuda.so"

_CTYPES = {
    "int32_t": C.c_int32, "uint32_t": C.c_uint32, "uint64_t": C.c_uint64, "int64_t": C.c_int64,
    "size_t": C.c_size_t, "float": C.c_float, "void*": C.c_void_p, "const void*": C.c_void_p,
    "const char*": C.c_char_p, "runit_ctx_t*": C.c_void_p, "runit_ctx_t**": C.POINTER(C.c_void_p),
    "void**": C.POINTER(C.c_void_p), "int32_t*": C.POINTER(C.c_int32), "uint32_t*": C.POINTER(C.c_uint32),
    "const int32_t*": C.POINTER(C.c_int32), "const uint64_t*": C.POINTER(C.c_uint64), "const uint32_t*": C.POINTER(C.c_uint32),
    "const runit_model_cfg*": C.c_void_p, "const runit_sampler_cfg*": C.c_void_p, "const runit_model_weights*": C.c_void_p, "runit_model_t*": C.c_void_p,
    "int32_t*": C.POINTER(C.c_int32),
    "runit_model_t**": C.POINTER(C.c_void_p), "const void* const*": C.POINTER(C.c_void_p),
    "void* const*": C.POINTER(C.c_void_p), "float*": C.POINTER(C.c_float),
    "uint64_t*": C.POINTER(C.c_uint64), "runit_graph_t*": C.c_void_p, "runit_graph_t**": C.POINTER(C.c_void_p),
}


def parse_header(path: Path = HEADER):
    """Return {name: (restype, [argtypes])} for every function declared in the header."""
    text = path.read_text()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    protos = {}
    for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(runit_\w+)\s*\(([^;{]*?)\)\s*;", text):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        ret = re.sub(r"\s+", " ", ret).replace(" *", "*")
        argt = []
        if args and args != "void":
            for a in args.split(","):
                a = re.sub(r"\s+", " ", a.strip())
                a = re.sub(r"\s*\*\s*", "* ", a).strip()
                # drop the parameter name if there is one
                parts = a.split(" ")
                if len(parts) > 1 and not parts[-1].endswith("*") and parts[-1] not in _CTYPES:
                    parts = parts[:-1]
                t = " ".join(parts).replace("* *", "**").replace(" *", "*")
                t = re.sub(r"\*\s+\*", "**", t)
                t = t.replace("* const*", "* const*")
                argt.append(t)
        protos[name] = (ret, argt)
    return protos


def _ctype(t: str):
    t = t.strip()
    if t not in _CTYPES:
        raise KeyError("no ctypes mapping for C type %r (add it to runit_mac_b200/_lib.py)" % t)
    return _CTYPES[t]


_lib = None
_protos = None


def prototypes():
    global _protos
    if _protos is None:
        _protos = parse_header()
    return _protos


def load():
    """dlopen the library and type every exported function; raise if anything is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            "%s is missing: build it with `python -m runit_mac_b200.build` (needs nvcc). "
            "There is no CPU or PyTorch fallback for this library." % LIB_PATH)
    lib = C.CDLL(str(LIB_PATH), mode=C.RTLD_GLOBAL)
    missing = []
    for name, (ret, args) in prototypes().items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            missing.append(name)
            continue
        fn.restype = _ctype(ret)
        fn.argtypes = [_ctype(a) for a in args]
    if missing:
        raise ImportError("librunit_cuda.so does not export: %s" % ", ".join(missing))
    _lib = lib
    return lib
