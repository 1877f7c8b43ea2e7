"""ctypes binding of librwkvb200.so.

The prototypes are read from include/rwkvb200.h, so the Python side can never drift from the
C ABI.  There is no fallback: if the shared library is missing or a call fails, an exception
is raised.
"""
import ctypes
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(HERE, "..", "include", "rwkvb200.h")
LIBPATH = os.path.join(HERE, "librwkvb200.so")

F32, BF16 = 0, 1

_CTYPES = {"int": ctypes.c_int, "float": ctypes.c_float, "size_t": ctypes.c_size_t}


def prototypes(header=HEADER):
    """[(return type, name, [(type, argname)])] of every function the header declares."""
    text = open(header).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    text = re.sub(r"^\s*#[^\n]*", "", text, flags=re.M)
    out = []
    for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(rwkvb200_\w+)\s*\(([^)]*)\)\s*;", text):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        parsed = []
        if args and args != "void":
            for a in args.split(","):
                a = " ".join(a.split())
                mm = re.match(r"(.*?)(\w+)$", a)
                parsed.append((mm.group(1).strip(), mm.group(2)))
        out.append((ret, name, parsed))
    return out


def _ctype(t):
    if "*" in t:
        return ctypes.c_char_p if t.replace(" ", "") == "constchar*" else ctypes.c_void_p
    return _CTYPES[t.replace("const", "").strip()]


_lib = None


def lib():
    """The loaded library (loads on first use).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIBPATH):
            raise RuntimeError(
                f"{LIBPATH} not found: the CUDA library is not built "
                "(run `python rwkv-cuda_b200/build.py`); there is no CPU fallback")
        L = ctypes.CDLL(LIBPATH)
        for ret, name, args in prototypes():
            fn = getattr(L, name)  # AttributeError here = header/library mismatch
            fn.restype = _ctype(ret)
            fn.argtypes = [_ctype(t) for t, _ in args]
        _lib = L
    return _lib


class RwkvB200Error(RuntimeError):
    pass


def call(name, *args):
    """Call an int-returning entry point; non-zero status becomes RwkvB200Error."""
    L = lib()
    rc = getattr(L, name)(*args)
    if rc != 0:
        raise RwkvB200Error(
            f"{name}: {L.rwkvb200_strerror(rc).decode()} ({rc}): {L.rwkvb200_last_error().decode()}")
