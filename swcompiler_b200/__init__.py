"""swcompiler_b200 -- B200 (sm_100a) kernels for the operator calls SWCompiler's code generator emits.

The product is the C-ABI library ``libswc_b200.so`` (``include/swc_b200.h``); this package builds it,
loads it and mirrors the reference's kernel interface on torch CUDA tensors (``kernels.Backend``).
"""
from . import _lib
from ._lib import (ACT_NONE, ACT_RELU, ACT_TANH, BF16, F32, STRICT_F32, TC_BF16, SwcError)

__all__ = ["Backend", "_lib", "SwcError", "STRICT_F32", "TC_BF16", "F32", "BF16", "ACT_NONE", "ACT_RELU", "ACT_TANH"]


def __getattr__(name):
    if name == "Backend":
        from .kernels import Backend
        return Backend
    raise AttributeError(name)
