"""ctypes binding of libswc_b200.so.  Loading fails loudly: there is no other implementation."""
from __future__ import annotations

import ctypes as C
import os
import re

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libswc_b200.so")
HEADER = os.path.join(os.path.dirname(PKG), "include", "swc_b200.h")

OK, ERR_BAD_ARG, ERR_BAD_SHAPE, ERR_MISALIGNED, ERR_UNSUPPORTED, ERR_CUDA, ERR_NCCL, ERR_TIMEOUT, ERR_NO_DEVICE, \
    ERR_TOO_LARGE = range(10)
STRICT_F32, TC_BF16 = 0, 1
F32, BF16, I32 = 0, 1, 2
ACT_NONE, ACT_RELU, ACT_TANH = 0, 1, 2
MAX_PEERS = 8

_lib = None


class SwcError(RuntimeError):
    def __init__(self, status: int, what: str, detail: str = ""):
        self.status = status
        super().__init__(f"{what}: status {status} ({status_string(status)}){': ' + detail if detail else ''}")


def declared_symbols() -> list[str]:
    """Every function the public header declares."""
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(swcb200_[A-Za-z0-9_]+)\s*\(", text)))


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m swcompiler_b200.build` "
                "(there is no fallback implementation)")
        l = C.CDLL(LIB_PATH)
        l.swcb200_status_string.restype = C.c_char_p
        l.swcb200_last_error.restype = C.c_char_p
        l.swcb200_last_error.argtypes = [C.c_void_p]
        l.swcb200_stream.restype = C.c_void_p
        l.swcb200_stream.argtypes = [C.c_void_p]
        l.swcb200_launch_count.restype = C.c_uint64
        l.swcb200_launch_count.argtypes = [C.c_void_p]
        _lib = l
    return _lib


def status_string(status: int) -> str:
    return lib().swcb200_status_string(C.c_int(status)).decode()
