"""Adapter giving the CUDA backend the same numpy-in / numpy-out face as the CPU oracle, so that the
same seeded cases (tests/cases.py) run through both.  All compute goes through the C-ABI library."""
import numpy as np
import torch

import swcompiler_b200 as swc


class GpuImpl:
    def __init__(self, precision=swc.STRICT_F32):
        self.be = swc.Backend(0, precision)

    def _t(self, a):
        return torch.from_numpy(np.ascontiguousarray(a)).cuda()

    def _n(self, t):
        self.be.sync()
        return t.cpu().numpy()

    def matrixMatrixMul_f(self, a, b):
        return self._n(self.be.matrixMatrixMul_f(self._t(a), self._t(b)))

    def batchedadd_f(self, x, s):
        return self._n(self.be.batchedadd_f(self._t(x), self._t(s)))

    def matrixTanh_f(self, a):
        return self._n(self.be.matrixTanh_f(self._t(a)))

    def relu_f(self, a):
        return self._n(self.be.relu_f(self._t(a)))

    def vecAdd_f(self, a, b):
        return self._n(self.be.vecAdd_f(self._t(a), self._t(b)))

    def matrixSoftmax_f(self, a):
        return self._n(self.be.matrixSoftmax_f(self._t(a)))

    def argMax_i(self, a, k):
        return self._n(self.be.argMax_i(self._t(a), k))

    def accuracy_i(self, pred, label, accum=None):
        return self._n(self.be.accuracy_i(self._t(pred), self._t(label), None if accum is None else self._t(accum)))

    def conv2d_f(self, x, w, b, kernels, strides, pads, group=1):
        return self._n(self.be.conv2d_f(self._t(x), self._t(w), self._t(b), kernels, strides, pads, group))

    def maxpool_f(self, x, kernels, strides, pads):
        return self._n(self.be.maxpool_f(self._t(x), kernels, strides, pads))

    def avgpool_f(self, x, kernels, strides, pads):
        return self._n(self.be.avgpool_f(self._t(x), kernels, strides, pads))

    def batchnormalization_f(self, x, mean, var, scale, bias, eps):
        return self._n(self.be.batchnormalization_f(self._t(x), self._t(mean), self._t(var), self._t(scale),
                                                    self._t(bias), eps))

    def transpose2d_f(self, x, shuffle):
        return self._n(self.be.transpose2d_f(self._t(x), shuffle))

    def transpose4d_f(self, x, shuffle):
        return self._n(self.be.transpose4d_f(self._t(x), shuffle))

    def fc(self, x, w, b=None):
        y = self.matrixMatrixMul_f(np.ascontiguousarray(x.reshape(x.shape[0], -1)), w)
        return y if b is None else self.batchedadd_f(y, b)

    def mlp_forward(self, x, w0, b0, w1, b1):
        return self.matrixSoftmax_f(self.fc(self.matrixTanh_f(self.fc(x, w0, b0)), w1, b1))
