"""ctypes argument lists against the prototypes of the public header: same number of arguments, and
integer widths / pointers in the same places (a c_int where the header says int64_t corrupts the call)."""
import ctypes as C
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _prototypes():
    text = open(os.path.join(ROOT, "include", "atenia_moe.h")).read()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    out = {}
    for m in re.finditer(r"ATENIA_API\s+([\w\s\*]+?)\s*\b(atenia_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
        ret, name, args = m.group(1).strip(), m.group(2), " ".join(m.group(3).split())
        params = [] if args in ("void", "") else [a.strip() for a in args.split(",")]
        out[name] = (ret, params)
    return out


def _kind(decl):
    if "*" in decl:
        return "ptr"
    base = decl.replace("const ", "").split()[0]
    return {"int": "i32", "int32_t": "i32", "int64_t": "i64", "size_t": "u64", "float": "f32", "uint64_t": "u64",
            "double": "f64"}[base]  # LP64: size_t is 64 bits


def _ckind(t):
    if t in (C.c_void_p, C.c_char_p) or (isinstance(t, type) and issubclass(t, C._Pointer)):
        return "ptr"
    return {C.c_int: "i32", C.c_int32: "i32", C.c_int64: "i64", C.c_size_t: "u64", C.c_float: "f32",
            C.c_uint64: "u64", C.c_double: "f64"}[t]


def test_argtypes_follow_the_header():
    import __graft_entry__ as ge
    ge.build()
    from ateniaengine_b200 import _lib
    lib = _lib.lib()
    protos = _prototypes()
    assert set(protos) == set(_lib.EXPORTS)
    checked = 0
    for name, (ret, params) in protos.items():
        fn = getattr(lib, name)
        if fn.argtypes is None:
            continue
        assert len(fn.argtypes) == len(params), f"{name}: {len(fn.argtypes)} ctypes arguments, header has {len(params)}"
        for i, (t, p) in enumerate(zip(fn.argtypes, params)):
            assert _ckind(t) == _kind(p), f"{name} argument {i} ({p}): ctypes {t}"
        checked += 1
    assert checked >= 15
