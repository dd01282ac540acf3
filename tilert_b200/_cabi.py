"""ctypes binding of the C ABI declared in ``include/tilert_b200.h``.

The prototypes are read from the header itself, so the Python side cannot drift from the
declarations: every function the header declares must be exported by the library, and is
bound with argument types derived from its C signature.
"""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

HEADER = Path(__file__).resolve().parent.parent / "include" / "tilert_b200.h"

_SCALARS = {
    "int": ctypes.c_int,
    "long long": ctypes.c_longlong,
    "float": ctypes.c_float,
    "size_t": ctypes.c_size_t,
}


def _ctype(decl: str):
    decl = decl.replace("const", " ").replace("unsigned", " ").strip()
    decl = re.sub(r"\s+", " ", decl)
    if "[" in decl or "*" in decl:
        return ctypes.c_void_p  # every pointer (device or host) travels as an address
    base = decl.rsplit(" ", 1)[0] if " " in decl else decl
    return _SCALARS[base.strip()]


def parse_header(path: Path = HEADER) -> dict[str, tuple[object, list[object]]]:
    """``{function name: (restype, [argtypes])}`` for every prototype in the header."""
    text = re.sub(r"/\*.*?\*/", " ", path.read_text(), flags=re.S)
    text = re.sub(r"#.*", " ", text)
    protos = {}
    for m in re.finditer(r"(const char\*|long long|int|size_t)\s+(tilert_\w+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S):
        ret, name, args = m.group(1), m.group(2), m.group(3).strip()
        restype = {"int": ctypes.c_int, "size_t": ctypes.c_size_t, "const char*": ctypes.c_char_p,
                   "long long": ctypes.c_longlong}[ret]
        argtypes = [] if args in ("", "void") else [_ctype(a) for a in args.split(",")]
        protos[name] = (restype, argtypes)
    return protos


def bind(lib_path: Path) -> ctypes.CDLL:
    lib = ctypes.CDLL(str(lib_path), mode=ctypes.RTLD_GLOBAL)
    for name, (restype, argtypes) in parse_header().items():
        fn = getattr(lib, name)  # AttributeError here = header/library mismatch
        fn.restype = restype
        fn.argtypes = argtypes
    return lib
