"""Host-side mirror of the reference's kernel interface, on torch CUDA tensors.

`Backend` owns one library context (device + stream) and exposes one method per function of the
reference's kernel header (src/codegen/utils/kernels.h), same name, same argument meaning, with
tensors in place of raw pointers and shapes taken from the tensors.  Every method only validates,
allocates the output with torch and calls through the C-ABI; all arithmetic happens in the CUDA
library.  torch is used for device memory and streams, nothing else.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L


def _p(t):
    return C.c_void_p(t.data_ptr() if t is not None else 0)


def _dims(seq):
    return (C.c_size_t * len(seq))(*[int(x) for x in seq])


def conv_out_dims(idims, fdims, kernels, strides, pads):
    """Conv2dOp shape inference, src/op/dlOp.cpp:195-196."""
    n, h, w, _ = idims
    return (n, (h + pads[0] + pads[2] - kernels[0]) // strides[0] + 1,
            (w + pads[1] + pads[3] - kernels[1]) // strides[1] + 1, fdims[0])


def pool_out_dims(idims, kernels, strides, pads):
    n, h, w, c = idims
    return (n, (h + pads[0] + pads[2] - kernels[0]) // strides[0] + 1,
            (w + pads[1] + pads[3] - kernels[1]) // strides[1] + 1, c)


class Backend:
    def __init__(self, device: int | torch.device = 0, precision: int = L.STRICT_F32, own_stream: bool = False,
                 stream: "torch.cuda.Stream | None" = None):
        """Work is issued on `stream` if given, else on torch's current stream of the device (own_stream=True:
        on a stream the library creates, which torch knows nothing about -- synchronise with `sync()`)."""
        if not torch.cuda.is_available():
            raise RuntimeError("swcompiler_b200 needs a CUDA device; there is no CPU path")
        self.lib = L.lib()
        self.device = torch.device("cuda", device if isinstance(device, int) else device.index or 0)
        self._ctx = C.c_void_p()
        self.torch_stream = None
        with torch.cuda.device(self.device):
            if own_stream:
                rc = self.lib.swcb200_init(C.c_int(self.device.index), C.c_int(precision), C.byref(self._ctx))
            else:
                self.torch_stream = stream if stream is not None else torch.cuda.current_stream(self.device)
                rc = self.lib.swcb200_init_on_stream(C.c_int(self.device.index), C.c_int(precision),
                                                     C.c_void_p(self.torch_stream.cuda_stream), C.byref(self._ctx))
        if rc != L.OK:
            raise L.SwcError(rc, "swcb200_init")
        self.precision = precision

    # ---- plumbing -----------------------------------------------------------
    def close(self):
        if self._ctx:
            self.lib.swcb200_destroy(self._ctx)
            self._ctx = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int, what: str):
        if rc != L.OK:
            raise L.SwcError(rc, what, self.lib.swcb200_last_error(self._ctx).decode())

    def _call(self, name: str, *args):
        self._check(getattr(self.lib, "swcb200_" + name)(self._ctx, *args), name)

    def sync(self):
        self._call("sync")

    def set_wait_limit(self, cycles: int):
        """Limit, in SM clock cycles, of every wait inside the tensor-core kernels launched through this context."""
        self._call("set_wait_limit", C.c_longlong(cycles))

    def set_sm_limit(self, sms: int):
        """The persistent tensor-core kernels of this context take at most `sms` SMs (0 = all): leaves room for a
        collective of another stream to run beside them."""
        self._call("set_sm_limit", C.c_int(sms))

    def selftest_wait_timeout(self):
        """Launches a kernel whose bounded wait can only run out; `sync()` then raises with status ERR_TIMEOUT."""
        self._call("selftest_wait_timeout")

    def set_precision(self, precision: int):
        self._call("set_precision", C.c_int(precision))
        self.precision = precision

    @property
    def launches(self) -> int:
        return int(self.lib.swcb200_launch_count(self._ctx))

    def _f32(self, *ts):
        for t in ts:
            if t is None:
                continue
            if not (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()):
                raise ValueError("expected a contiguous fp32 CUDA tensor")

    def _new(self, shape, dtype=torch.float32):
        return torch.empty(tuple(int(s) for s in shape), dtype=dtype, device=self.device)

    # ---- dense --------------------------------------------------------------
    def matrixMatrixMul_f(self, a, b, out=None):
        self._f32(a, b)
        (m, k), (k2, n) = a.shape, b.shape
        if k != k2:
            raise ValueError("inner dimensions differ")
        c = out if out is not None else self._new((m, n))
        self._call("matrixMatrixMul_f", C.c_int(m), C.c_int(n), C.c_int(k), _p(a), C.c_int(k), _p(b), C.c_int(n),
                   _p(c), C.c_int(n))
        return c

    def batchedadd_f(self, batch, slice_, out=None):
        self._f32(batch, slice_)
        rows, cols = batch.shape
        out = out if out is not None else torch.empty_like(batch)
        self._call("batchedadd_f", _p(out), _p(batch), _p(slice_), C.c_size_t(rows), C.c_size_t(cols))
        return out

    def matrixTanh_f(self, a, out=None):
        self._f32(a)
        m, n = a.shape
        out = out if out is not None else torch.empty_like(a)
        self._call("matrixTanh_f", C.c_int(m), C.c_int(n), _p(a), C.c_int(n), _p(out), C.c_int(n))
        return out

    def matrixSoftmax_f(self, a, out=None):
        self._f32(a)
        m, n = a.shape
        out = out if out is not None else torch.empty_like(a)
        self._call("matrixSoftmax_f", C.c_int(m), C.c_int(n), _p(a), C.c_int(n), _p(out), C.c_int(n))
        return out

    def argMax_i(self, a, top_k: int):
        self._f32(a)
        m, n = a.shape
        idx = self._new((m, top_k), torch.int32)
        self._call("argMax_i", _p(a), _p(idx), C.c_int(m), C.c_int(n), C.c_int(top_k))
        return idx

    def accuracy_i(self, pred, label, accum=None):
        """accum [2] int32 += (rows whose label is among their predictions pred[i, :], rows); a fresh zeroed
        counter pair if `accum` is None."""
        m, n = pred.shape
        if accum is None:
            accum = torch.zeros(2, dtype=torch.int32, device=self.device)
            if self.torch_stream is None:  # the library's own stream knows nothing of torch's fill kernel
                torch.cuda.current_stream(self.device).synchronize()
        self._call("accuracy_i", _p(pred), _p(label), _p(accum), C.c_int(m), C.c_int(n))
        return accum

    def relu_f(self, a, out=None):
        self._f32(a)
        out = out if out is not None else torch.empty_like(a)
        self._call("relu_f", _p(a), _p(out), C.c_size_t(a.numel()))
        return out

    def vecAdd_f(self, a, b, out=None):
        self._f32(a, b)
        out = out if out is not None else torch.empty_like(a)
        self._call("vecAdd_f", C.c_int(a.numel()), _p(a), _p(b), _p(out))
        return out

    # ---- NHWC ---------------------------------------------------------------
    def conv2d_f(self, x, filt, bias, kernels, strides, pads, group=1, out=None):
        self._f32(x, filt, bias)
        odims = conv_out_dims(x.shape, filt.shape, kernels, strides, pads)
        out = out if out is not None else self._new(odims)
        self._call("conv2d_f", _p(out), _p(x), _p(filt), _p(bias), _dims(odims), _dims(x.shape), _dims(filt.shape),
                   _dims(bias.shape), _dims(kernels), _dims(strides), _dims(pads), C.c_size_t(group))
        return out

    def maxpool_f(self, x, kernels, strides, pads, out=None):
        self._f32(x)
        odims = pool_out_dims(x.shape, kernels, strides, pads)
        out = out if out is not None else self._new(odims)
        self._call("maxpool_f", _p(x), _p(out), _dims(x.shape), _dims(odims), _dims(kernels), _dims(strides),
                   _dims(pads))
        return out

    def avgpool_f(self, x, kernels, strides, pads, out=None):
        self._f32(x)
        odims = pool_out_dims(x.shape, kernels, strides, pads)
        out = out if out is not None else self._new(odims)
        self._call("avgpool_f", _p(x), _p(out), _dims(x.shape), _dims(odims), _dims(kernels), _dims(strides),
                   _dims(pads))
        return out

    def batchnormalization_f(self, x, mean, var, scale, bias, eps, out=None):
        self._f32(x, mean, var, scale, bias)
        out = out if out is not None else torch.empty_like(x)
        self._call("batchnormalization_f", _p(out), _p(x), _p(mean), _p(var), _p(scale), _p(bias), _dims(x.shape),
                   C.c_float(eps))
        return out

    def transpose2d_f(self, x, shuffle):
        self._f32(x)
        odims = tuple(x.shape[s] for s in shuffle)
        out = self._new(odims)
        self._call("transpose2d_f", _p(x), _p(out), _dims(x.shape), _dims(odims), _dims(shuffle))
        return out

    def transpose4d_f(self, x, shuffle):
        self._f32(x)
        odims = tuple(x.shape[s] for s in shuffle)
        out = self._new(odims)
        self._call("transpose4d_f", _p(x), _p(out), _dims(x.shape), _dims(odims), _dims(shuffle))
        return out

    # ---- chains as the lowered graph has them ---------------------------------
    def fc(self, x, w, b=None):
        """MatrixMatrixMul then MatrixVectorAdd (src/op/dlOp/dlOpEinsum.cpp:154-237); a 4-D NHWC input is
        viewed as [N, H*W*C] (src/tensor/tensor.cpp:128-138)."""
        y = self.matrixMatrixMul_f(x.reshape(x.shape[0], -1), w)
        return y if b is None else self.batchedadd_f(y, b)

    def mlp_forward(self, x, w0, b0, w1, b1):
        return self.matrixSoftmax_f(self.fc(self.matrixTanh_f(self.fc(x, w0, b0)), w1, b1))

    # ---- bf16 storage / tensor-core path ---------------------------------------
    def cast_f32_to_bf16(self, x, out=None):
        self._f32(x)
        out = out if out is not None else self._new(x.shape, torch.bfloat16)
        self._call("cast_f32_to_bf16", _p(x), _p(out), C.c_size_t(x.numel()))
        return out

    def cast_bf16_to_f32(self, x, out=None):
        out = out if out is not None else self._new(x.shape, torch.float32)
        self._call("cast_bf16_to_f32", _p(x), _p(out), C.c_size_t(x.numel()))
        return out

    def pack_weight_bf16(self, w):
        """fp32 W[k, n] -> bf16 Wp[n, k]."""
        self._f32(w)
        k, n = w.shape
        wp = self._new((n, k), torch.bfloat16)
        self._call("pack_weight_bf16", _p(w), C.c_int(k), C.c_int(n), C.c_int(n), _p(wp))
        return wp

    def fc_bf16(self, a, wp, bias=None, act=L.ACT_NONE, out_dtype=torch.bfloat16, out=None, a_lo=None, out_lo=None):
        """act(A[m,k] . Wp[n,k]^T + bias) in one launch; A, Wp bf16.  With `a_lo` the input is a split activation
        (A = a + a_lo, two bf16 terms); with `out_lo` (bf16 outputs) the output's second term is written there."""
        if a.dtype != torch.bfloat16 or wp.dtype != torch.bfloat16 or not (a.is_contiguous() and wp.is_contiguous()):
            raise ValueError("fc_bf16 wants contiguous bf16 operands")
        (m, k), (n, k2) = a.shape, wp.shape
        if k != k2:
            raise ValueError("inner dimensions differ")
        out = out if out is not None else self._new((m, n), out_dtype)
        dt = C.c_int(L.BF16 if out.dtype == torch.bfloat16 else L.F32)
        if a_lo is None and out_lo is None:
            self._call("fc_bf16", C.c_int(m), C.c_int(n), C.c_int(k), _p(a), C.c_int(k), _p(wp), C.c_int(k), _p(bias),
                       C.c_int(act), _p(out), dt, C.c_int(n))
            return out
        for t in (a_lo, out_lo):
            if t is not None and not (t.dtype == torch.bfloat16 and t.is_contiguous()):
                raise ValueError("the second term of a split activation is a contiguous bf16 tensor")
        if (a_lo is not None and a_lo.shape != a.shape) or (out_lo is not None and out_lo.shape != out.shape):
            raise ValueError("the two terms of a split activation have the same shape")
        self._call("fc_bf16_split", C.c_int(m), C.c_int(n), C.c_int(k), _p(a), _p(a_lo), C.c_int(k), _p(wp), C.c_int(k),
                   _p(bias), C.c_int(act), _p(out), _p(out_lo), dt, C.c_int(n))
        return out

    def fc_bf16_scatter_rows(self, a, wp, slot_table, nranks: int, rank: int, ld_slot: int):
        """A[m,k] . Wp[n,k]^T with fp32 rows scattered to the ranks that own them: row i goes into slot `rank` of the
        slot array of rank i // (m // nranks) (`slot_table` from `NcclComm.peer_slots_setup`)."""
        if a.dtype != torch.bfloat16 or wp.dtype != torch.bfloat16 or not (a.is_contiguous() and wp.is_contiguous()):
            raise ValueError("fc_bf16_scatter_rows wants contiguous bf16 operands")
        (m, k), (n, k2) = a.shape, wp.shape
        if k != k2:
            raise ValueError("inner dimensions differ")
        self._call("fc_bf16_scatter_rows", C.c_int(m), C.c_int(n), C.c_int(k), _p(a), C.c_int(k), _p(wp), C.c_int(k),
                   slot_table, C.c_int(nranks), C.c_int(rank), C.c_int(ld_slot))

    def sum_slots(self, slots, out):
        """out = slots[0] + slots[1] + ... in that order; slots [p, ...] fp32 contiguous, out one slot's shape."""
        self._f32(slots, out)
        n = out.numel()
        self._call("sum_slots", _p(slots), C.c_size_t(n), C.c_int(slots.shape[0]), _p(out), C.c_size_t(n))
        return out

    def pack_filter_bf16(self, filt):
        """fp32 filter [oC, kh, kw, iC] -> bf16, same layout."""
        self._f32(filt)
        fp = self._new(filt.shape, torch.bfloat16)
        self._call("pack_filter_bf16", _p(filt), _dims(filt.shape), _p(fp))
        return fp

    def conv2d_bf16(self, x, fp, bias, kernels, strides, pads, bn=None, residual=None, relu=False, out=None, pool=False):
        """Conv2d [-> BatchNormalization] [-> ElementAdd(residual)] [-> Relu] [-> MaxPool 2x2/2] in one tensor-core
        launch.  x, fp (packed filter), residual, out: bf16 NHWC.  bn = (scale, bias, mean, var, eps) or None.
        With `pool` the result is [N, OH/2, OW/2, oC] (3x3 filters over 64 -> 64 channels only)."""
        odims = conv_out_dims(x.shape, fp.shape, kernels, strides, pads)
        out_shape = (odims[0], odims[1] // 2, odims[2] // 2, odims[3]) if pool else odims
        out = out if out is not None else self._new(out_shape, torch.bfloat16)

        class Ep(C.Structure):
            _fields_ = [("bn_scale", C.c_void_p), ("bn_bias", C.c_void_p), ("bn_mean", C.c_void_p),
                        ("bn_var", C.c_void_p), ("bn_eps", C.c_float), ("residual", C.c_void_p), ("relu", C.c_int),
                        ("pool2x2", C.c_int)]

        ep = Ep()
        if bn is not None:
            ep.bn_scale, ep.bn_bias, ep.bn_mean, ep.bn_var = (t.data_ptr() for t in bn[:4])
            ep.bn_eps = float(bn[4])
        ep.residual = residual.data_ptr() if residual is not None else None
        ep.relu = 1 if relu else 0
        ep.pool2x2 = 1 if pool else 0
        self._call("conv2d_bf16", _p(out), _p(x), _p(fp), _p(bias), _dims(odims), _dims(x.shape), _dims(fp.shape),
                   _dims(kernels), _dims(strides), _dims(pads), C.byref(ep))
        return out

    def maxpool_bf16(self, x, kernels, strides, pads, out=None):
        odims = pool_out_dims(x.shape, kernels, strides, pads)
        out = out if out is not None else self._new(odims, torch.bfloat16)
        self._call("maxpool_bf16", _p(x), _p(out), _dims(x.shape), _dims(odims), _dims(kernels), _dims(strides),
                   _dims(pads))
        return out
