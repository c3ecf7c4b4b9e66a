"""numpy front end to the two CPU checkers.

TEST INFRASTRUCTURE.  Only the test-suite, the smoke check and the benchmark's
CPU-baseline / reference arm load this module; the shipped package never does.

* ``Oracle``    -- ``libswc_oracle.so``, the C restatement in ``swc_oracle.c``.
* ``Reference`` -- ``_ref/libswc_ref.so``, SWCompiler's own ``kernels.h`` behind
  ``extern "C"`` (``ref_shim.cpp``); exists only where it was built from a
  reference checkout (the prebuilt file is carried along, not tracked).

Both expose the same methods, named after the reference functions
(``src/codegen/utils/kernels.h``), taking and returning C-contiguous numpy
arrays.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_F = C.POINTER(C.c_float)
_I = C.POINTER(C.c_int)
_Z = C.POINTER(C.c_size_t)


def build(quiet: bool = True) -> None:
    """Compile the restatement (always) and the reference shim (if a checkout is present)."""
    subprocess.run(["make", "-C", _HERE], check=True,
                   stdout=subprocess.DEVNULL if quiet else None)


def _fp(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(_F)


def _dims(t):
    return (C.c_size_t * len(t))(*[int(x) for x in t])


def conv_out_dims(idims, fdims, kernels, strides, pads):
    """Output NHWC shape of Conv2d; Conv2dOp shape inference, src/op/dlOp.cpp:195-196."""
    n, h, w, _ = idims
    oh = (h + pads[0] + pads[2] - kernels[0]) // strides[0] + 1
    ow = (w + pads[1] + pads[3] - kernels[1]) // strides[1] + 1
    return (n, oh, ow, fdims[0])


def pool_out_dims(idims, kernels, strides, pads):
    """Output NHWC shape of MaxPool/AvgPool; same formula as Conv2d (src/op/dlOp.cpp)."""
    n, h, w, c = idims
    oh = (h + pads[0] + pads[2] - kernels[0]) // strides[0] + 1
    ow = (w + pads[1] + pads[3] - kernels[1]) // strides[1] + 1
    return (n, oh, ow, c)


class _Base:
    _names: dict

    def __init__(self, path: str):
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.path = path
        self.lib = C.CDLL(path)
        self._f = {k: getattr(self.lib, v) for k, v in self._names.items()}
        for f in self._f.values():
            f.restype = None

    # ---- dense ------------------------------------------------------------
    def matrixMatrixMul_f(self, a: np.ndarray, b: np.ndarray) -> np.ndarray:
        m, k = a.shape
        k2, n = b.shape
        assert k == k2
        c = np.empty((m, n), np.float32)
        self._f["mm"](C.c_int(m), C.c_int(n), C.c_int(k), _fp(a), C.c_int(k), _fp(b),
                      C.c_int(n), _fp(c), C.c_int(n))
        return c

    def batchedadd_f(self, batch: np.ndarray, slice_: np.ndarray) -> np.ndarray:
        rows, cols = batch.shape
        out = np.empty_like(batch)
        self._f["badd"](_fp(out), _fp(batch), _fp(slice_), C.c_size_t(rows), C.c_size_t(cols))
        return out

    def matrixTanh_f(self, a: np.ndarray) -> np.ndarray:
        m, n = a.shape
        b = np.empty_like(a)
        self._f["tanh"](C.c_int(m), C.c_int(n), _fp(a), C.c_int(n), _fp(b), C.c_int(n))
        return b

    def relu_f(self, a: np.ndarray) -> np.ndarray:
        b = np.empty_like(a)
        self._f["relu"](_fp(a), _fp(b), C.c_size_t(a.size))
        return b

    def vecAdd_f(self, a: np.ndarray, b: np.ndarray) -> np.ndarray:
        c = np.empty_like(a)
        self._f["add"](C.c_int(a.size), _fp(a), _fp(b), _fp(c))
        return c

    def matrixSoftmax_f(self, a: np.ndarray) -> np.ndarray:
        m, n = a.shape
        b = np.empty_like(a)
        self._f["softmax"](C.c_int(m), C.c_int(n), _fp(a), C.c_int(n), _fp(b), C.c_int(n))
        return b

    def argMax_i(self, a: np.ndarray, top_k: int) -> np.ndarray:
        m, n = a.shape
        idx = np.empty((m, top_k), np.int32)
        self._f["argmax"](_fp(a), idx.ctypes.data_as(_I), C.c_int(m), C.c_int(n), C.c_int(top_k))
        return idx

    def accuracy_i(self, pred: np.ndarray, label: np.ndarray, accum: np.ndarray | None = None) -> np.ndarray:
        """accum [2] int32 = (rows whose label is among their predictions, rows), added to `accum` if given."""
        pred = np.ascontiguousarray(pred, np.int32)
        label = np.ascontiguousarray(label, np.int32)
        m, n = pred.shape
        accum = np.zeros(2, np.int32) if accum is None else np.ascontiguousarray(accum, np.int32).copy()
        self._f["accuracy"](pred.ctypes.data_as(_I), label.ctypes.data_as(_I), accum.ctypes.data_as(_I), C.c_int(m), C.c_int(n))
        return accum

    # ---- NHWC -------------------------------------------------------------
    def conv2d_f(self, x, filt, bias, kernels, strides, pads, group=1) -> np.ndarray:
        odims = conv_out_dims(x.shape, filt.shape, kernels, strides, pads)
        out = np.empty(odims, np.float32)
        self._f["conv"](_fp(out), _fp(x), _fp(filt), _fp(bias), _dims(odims), _dims(x.shape),
                        _dims(filt.shape), _dims(bias.shape), _dims(kernels), _dims(strides),
                        _dims(pads), C.c_size_t(group))
        return out

    def maxpool_f(self, x, kernels, strides, pads) -> np.ndarray:
        odims = pool_out_dims(x.shape, kernels, strides, pads)
        out = np.empty(odims, np.float32)
        self._f["maxpool"](_fp(x), _fp(out), _dims(x.shape), _dims(odims), _dims(kernels),
                           _dims(strides), _dims(pads))
        return out

    def avgpool_f(self, x, kernels, strides, pads) -> np.ndarray:
        odims = pool_out_dims(x.shape, kernels, strides, pads)
        out = np.empty(odims, np.float32)
        self._f["avgpool"](_fp(x), _fp(out), _dims(x.shape), _dims(odims), _dims(kernels),
                           _dims(strides), _dims(pads))
        return out

    def batchnormalization_f(self, x, mean, var, scale, bias, eps) -> np.ndarray:
        out = np.empty_like(x)
        self._f["bn"](_fp(out), _fp(x), _fp(mean), _fp(var), _fp(scale), _fp(bias),
                      _dims(x.shape), C.c_float(eps))
        return out

    def transpose2d_f(self, x, shuffle) -> np.ndarray:
        odims = tuple(x.shape[s] for s in shuffle)
        out = np.empty(odims, np.float32)
        self._f["t2"](_fp(x), _fp(out), _dims(x.shape), _dims(odims), _dims(shuffle))
        return out

    def transpose4d_f(self, x, shuffle) -> np.ndarray:
        odims = tuple(x.shape[s] for s in shuffle)
        out = np.empty(odims, np.float32)
        self._f["t4"](_fp(x), _fp(out), _dims(x.shape), _dims(odims), _dims(shuffle))
        return out

    # ---- whole forward passes, as the emitted program chains them ---------
    def fc(self, x, w, b=None):
        """FC lowers to MatrixMatrixMul then MatrixVectorAdd (src/op/dlOp/dlOpEinsum.cpp:154-237)."""
        y = self.matrixMatrixMul_f(np.ascontiguousarray(x.reshape(x.shape[0], -1)), w)
        return y if b is None else self.batchedadd_f(y, b)

    def mlp_forward(self, x, w0, b0, w1, b1):
        """FC -> Tanh -> FC -> Softmax, the graph of test/engine/testEngineMLPInfer.cpp."""
        h = self.matrixTanh_f(self.fc(x, w0, b0))
        return self.matrixSoftmax_f(self.fc(h, w1, b1))


class Oracle(_Base):
    _names = dict(mm="orc_matmul_f32", badd="orc_bias_add_f32", tanh="orc_tanh_f32",
                  relu="orc_relu_f32", add="orc_add_f32", softmax="orc_softmax_f32",
                  argmax="orc_argmax_i32", accuracy="orc_accuracy_i32", conv="orc_conv2d_f32", maxpool="orc_maxpool_f32",
                  avgpool="orc_avgpool_f32", bn="orc_batchnorm_f32", t2="orc_transpose2d_f32",
                  t4="orc_transpose4d_f32")

    def __init__(self, path: str | None = None):
        path = path or os.path.join(_HERE, "libswc_oracle.so")
        if not os.path.exists(path):
            build()
        super().__init__(path)
        self.lib.orc_num_threads.restype = C.c_int

    kind = "port"

    @property
    def threads(self) -> int:
        return int(self.lib.orc_num_threads())

    def set_threads(self, n: int) -> None:
        self.lib.orc_set_num_threads(C.c_int(n))


class Reference(_Base):
    _names = dict(mm="ref_matrixMatrixMul_f", badd="ref_batchedadd_f", tanh="ref_matrixTanh_f",
                  relu="ref_relu_f", add="ref_vecAdd_f", softmax="ref_matrixSoftmax_f",
                  argmax="ref_argMax_i", accuracy="ref_accuracy_i", conv="ref_conv2d_f", maxpool="ref_maxpool_f",
                  avgpool="ref_avgpool_f", bn="ref_batchnormalization_f", t2="ref_transpose2d_f",
                  t4="ref_transpose4d_f")
    kind = "reference"
    threads = 1

    def __init__(self, path: str | None = None):
        super().__init__(path or os.path.join(_HERE, "_ref", "libswc_ref.so"))

    @staticmethod
    def available() -> bool:
        return os.path.exists(os.path.join(_HERE, "_ref", "libswc_ref.so"))
