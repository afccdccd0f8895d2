"""The C ABI: the shared library loads, exports every function the header declares, and the
ctypes prototypes agree with the header's parameter lists (no compute calls: runs without a GPU)."""
import ctypes as C
import os
import re

import pytest

from omnimem_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "omnimem_b200.h")


def _declarations():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = text[text.index("const char* nsa_last_error"):]
    decls = {}
    for m in re.finditer(r"([A-Za-z_0-9\* ]+?)\s*\b(nsa_[a-z_0-9]+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S):
        ret, name, params = m.group(1).strip(), m.group(2), m.group(3)
        plist = [] if params.strip() in ("", "void") else [p.strip() for p in params.split(",")]
        decls[name] = (ret, plist)
    return decls


def _kind_of_c(param: str) -> str:
    if "*" in param or "[" in param:
        return "ptr"
    for key, kind in (("int32_t", "i32"), ("int64_t", "i64"), ("size_t", "size"), ("float", "f32")):
        if key in param:
            return kind
    raise AssertionError(f"unknown C parameter type: {param}")


def _kind_of_ctypes(t) -> str:
    if t in (C.c_void_p, C.c_char_p) or hasattr(t, "contents") or (isinstance(t, type) and issubclass(t, C._Pointer)):
        return "ptr"
    return {C.c_int32: "i32", C.c_int64: "i64", C.c_size_t: "size", C.c_float: "f32"}[t]


def test_library_is_built_and_loads():
    assert os.path.exists(_lib.LIB_PATH), "build with python -m omnimem_b200.build"
    lib = _lib.load()
    assert b"sm_100a" in lib.nsa_version()


def test_every_declared_symbol_is_exported_and_bound():
    decls = _declarations()
    assert len(decls) >= 20
    lib = _lib.load()
    for name in decls:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert set(decls) == set(_lib.PROTOTYPES)


def test_ctypes_prototypes_match_the_header():
    for name, (ret, params) in _declarations().items():
        res, args = _lib.PROTOTYPES[name]
        assert len(args) == len(params), f"{name}: {len(args)} ctypes args vs {len(params)} in the header"
        for i, (a, p) in enumerate(zip(args, params)):
            assert _kind_of_ctypes(a) == _kind_of_c(p), f"{name} arg {i}: {a} vs '{p}'"
        if "char*" in ret.replace(" ", ""):
            assert res is C.c_char_p
        elif "size_t" in ret:
            assert res is C.c_size_t
        else:
            assert res is C.c_int32


def test_struct_layouts_match_the_header():
    # nsa_kv_source: int32, 2 ptr, 2x3 int64, int64, ptr, 2 int32, 2 ptr, int64
    assert C.sizeof(_lib.KVSource) == 8 + 16 + 48 + 8 + 8 + 8 + 16 + 8 + 8
    assert C.sizeof(_lib.TopkMask) == 12 * 4
    # nsa_rope: 3 pointers, 9 int32 (padded to 8 bytes)
    assert C.sizeof(_lib.Rope) == 24 + 40


def test_bad_arguments_return_a_status_not_a_crash():
    lib = _lib.load()
    # topk with a negative head dim is rejected before anything touches the device
    with pytest.raises(_lib.NSABackendError, match="head dim"):
        _lib.call("nsa_topk", None, None, None, None, 1, 1, 1, -5, 4, 1, 1.0, None, None, None, None, 0, 0, None)
    assert b"head dim" in lib.nsa_last_error()
    with pytest.raises(_lib.NSABackendError, match="group_size"):
        _lib.call("nsa_sel_fwd", None, None, None, None, None, None, None, None, 1, 1, 1, 128, 1, 64, 1, 0, 500,
                  1.0, 0, None)
