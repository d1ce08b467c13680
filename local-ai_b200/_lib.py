"""ctypes binding of liblocal_cuda.so.

Signatures are derived from include/local_cuda.h itself, so the Python side can
never drift from the C ABI: every `LC_API` declaration becomes a ctypes
function with matching argument and result types.  Loading fails loudly when
the library cannot be built or a declared symbol is missing; nothing here
computes on the CPU.
"""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

from . import build

HEADER = build.ROOT / "include" / "local_cuda.h"

_SCALARS = {
    "int": C.c_int,
    "uint32_t": C.c_uint32,
    "uint64_t": C.c_uint64,
    "size_t": C.c_size_t,
    "float": C.c_float,
}


def _ctype(decl: str):
    """Map one C parameter / return declaration to a ctypes type."""
    d = decl.replace("const", " ").strip()
    stars = d.count("*")
    base = d.replace("*", " ").split()
    base = base[0] if base else "void"
    if stars == 0:
        if base == "void":
            return None
        return _SCALARS[base]
    if stars == 1 and base == "char":
        return C.c_char_p
    if stars == 2:
        return C.POINTER(C.c_void_p)
    return C.c_void_p


def parse_header(path: Path = HEADER) -> dict[str, tuple]:
    """name -> (restype, [argtypes], [argnames]) for every LC_API declaration."""
    text = re.sub(r"/\*.*?\*/", " ", path.read_text(), flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    out = {}
    for m in re.finditer(r"LC_API\s+([^;()]+?)\b(lc_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
        ret, name, args = m.group(1).strip(), m.group(2), " ".join(m.group(3).split())
        argtypes, argnames = [], []
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                nm = re.search(r"(\w+)\s*$", a).group(1)
                argtypes.append(_ctype(a[: a.rfind(nm)]))
                argnames.append(nm)
        out[name] = (_ctype(ret), argtypes, argnames)
    return out


_lib = None
_decls = None


def declarations() -> dict[str, tuple]:
    global _decls
    if _decls is None:
        _decls = parse_header()
    return _decls


def load() -> C.CDLL:
    """Build (if stale) and load the library, binding every declared symbol."""
    global _lib
    if _lib is not None:
        return _lib
    path = build.build_library()
    lib = C.CDLL(str(path))
    missing = []
    for name, (restype, argtypes, _) in declarations().items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            missing.append(name)
            continue
        fn.restype = restype
        fn.argtypes = argtypes
    if missing:
        raise RuntimeError(f"liblocal_cuda.so does not export: {', '.join(missing)}")
    _lib = lib
    return lib
