"""Signatures of the C ABI, read from include/knet_sm100.h.

The header declares its entry points through X-macros, so it is run through the C
preprocessor and the resulting prototypes are parsed into ctypes argument lists.  The
parsed table is cached as JSON next to the shared library.
"""
import ctypes as C
import json
import os
import re
import subprocess

_PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(_PKG)                      # .../knet.jl_b200
HEADER = os.path.join(os.path.dirname(ROOT), "include", "knet_sm100.h")
CACHE = os.path.join(ROOT, "build", "abi.json")

_SCALARS = {
    "int": "c_int", "int32_t": "c_int32", "int64_t": "c_int64", "uint64_t": "c_uint64", "uint32_t": "c_uint32",
    "size_t": "c_size_t", "float": "c_float", "double": "c_double", "void": None,
    "cudaStream_t": "c_void_p",
}


def _ctype_name(decl):
    """'const float *x' -> 'c_void_p'; 'int n' -> 'c_int'; 'float' -> 'c_float'."""
    decl = decl.strip()
    if "*" in decl:
        return "c_void_p"
    toks = [t for t in re.split(r"\s+", decl) if t not in ("const", "struct")]
    for t in toks:
        if t in _SCALARS:
            return _SCALARS[t]
    raise ValueError(f"cannot map C declaration {decl!r}")


def parse_header(header=HEADER):
    """Return {name: [restype_name, [argtype_names]]} for every declared function."""
    out = subprocess.run(["gcc", "-E", "-P", "-DKNET_API=KNET_API_MARK", header],
                         check=True, capture_output=True, text=True).stdout
    out = re.sub(r"\s+", " ", out)
    sigs = {}
    for m in re.finditer(r"KNET_API_MARK\s+([\w\s\*]+?)\s*\b(\w+)\s*\(([^()]*)\)\s*;", out):
        ret, name, args = m.group(1), m.group(2), m.group(3).strip()
        argl = [] if args in ("", "void") else [_ctype_name(a) for a in args.split(",")]
        sigs[name] = [_ctype_name(ret) if ret.strip() != "void" else None, argl]
    return sigs


def signatures(refresh=False):
    if not refresh and os.path.exists(CACHE) and os.path.getmtime(CACHE) >= os.path.getmtime(HEADER):
        with open(CACHE) as f:
            return json.load(f)
    sigs = parse_header()
    try:
        os.makedirs(os.path.dirname(CACHE), exist_ok=True)
        with open(CACHE, "w") as f:
            json.dump(sigs, f)
    except OSError:
        pass
    return sigs


def bind(lib, sigs=None):
    """Attach argtypes/restype to every declared symbol of a loaded ctypes library."""
    sigs = sigs or signatures()
    for name, (ret, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype = getattr(C, ret) if ret else None
        fn.argtypes = [getattr(C, a) for a in args]
    return lib
