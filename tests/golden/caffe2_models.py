"""Two small synthetic Caffe2 models, written in protobuf wire format without protobuf.

The reference's importer tests read pretrained model archives (lenet_mnist, resnet50, vgg19) that are downloads and
are not available here; these stand in for them with the same operator vocabulary and Caffe2's own weight layouts
(filters oihw, FC weights [out, in] over (c, h, w)), seeded random values:

  c2lenet   data[4,28,28,1] -> Conv 5x5 1->8 -> Relu -> MaxPool 2/2 -> Conv 5x5 8->16 pad 2 -> Relu -> MaxPool 2/2
            -> FC 576->32 -> Relu -> Dropout -> FC 32->10 -> Softmax
  c2resnet  data[2,8,8,64] -> Conv 3x3 pad 1 -> SpatialBN -> Relu -> Conv 3x3 pad 1 (no bias blob) -> SpatialBN
            -> Sum(skip = data) -> Relu -> AveragePool 2/2 -> FC 1024->10 -> Softmax

`model(name)` returns the two serialized nets, the weights as numpy arrays in Caffe2 layout, and the input.
`reference_forward` runs a model through an implementation of the kernel interface (the CPU oracle) with the weights
re-laid out by numpy -- independently of the importer's C++ -- and `weight_files` gives the files an emitted program
expects (what the importer writes at import time).
"""
import struct

import numpy as np

F = np.float32


# ---- protobuf wire format (NetDef / OperatorDef / Argument of caffe2.proto)
def _varint(v):
    out = bytearray()
    v &= (1 << 64) - 1
    while True:
        b = v & 0x7F
        v >>= 7
        out.append(b | (0x80 if v else 0))
        if not v:
            return bytes(out)


def _key(field, wire):
    return _varint(field << 3 | wire)


def _ld(field, payload):
    return _key(field, 2) + _varint(len(payload)) + payload


def _arg(name, f=None, i=None, s=None, floats=None, ints=None, packed=False):
    b = _ld(1, name.encode())
    if f is not None:
        b += _key(2, 5) + struct.pack("<f", f)
    if i is not None:
        b += _key(3, 0) + _varint(i)
    if s is not None:
        b += _ld(4, s)
    if floats is not None:
        fl = np.asarray(floats, F).reshape(-1)
        b += _ld(5, fl.tobytes()) if packed else b"".join(_key(5, 5) + struct.pack("<f", float(x)) for x in fl)
    if ints is not None:
        b += _ld(6, b"".join(_varint(int(x)) for x in ints)) if packed else b"".join(_key(6, 0) + _varint(int(x)) for x in ints)
    return b


def _op(type_, inputs, outputs, args=(), name=""):
    b = b"".join(_ld(1, x.encode()) for x in inputs) + b"".join(_ld(2, x.encode()) for x in outputs)
    if name:
        b += _ld(3, name.encode())
    b += _ld(4, type_.encode()) + b"".join(_ld(5, a) for a in args)
    return b


def _net(name, ops, external_input=(), external_output=()):
    return (_ld(1, name.encode()) + b"".join(_ld(2, o) for o in ops) + b"".join(_ld(7, x.encode()) for x in external_input) +
            b"".join(_ld(8, x.encode()) for x in external_output))


def _fill(blob, arr, packed=False):
    return _op("GivenTensorFill", [], [blob], [_arg("shape", ints=arr.shape, packed=packed), _arg("values", floats=arr, packed=packed)])


def model(name, packed=False):
    """(predict_net bytes, init_net bytes, weights {blob: array in Caffe2 layout}, input array NHWC)."""
    if name == "c2lenet":
        r = np.random.default_rng(2001)
        w = {"conv1_w": (r.standard_normal((8, 1, 5, 5)) * 0.2).astype(F), "conv1_b": (r.standard_normal(8) * 0.1).astype(F),
             "conv2_w": (r.standard_normal((16, 8, 5, 5)) * 0.07).astype(F), "conv2_b": (r.standard_normal(16) * 0.1).astype(F),
             "fc3_w": (r.standard_normal((32, 576)) * 0.04).astype(F), "fc3_b": (r.standard_normal(32) * 0.1).astype(F),
             "pred_w": (r.standard_normal((10, 32)) * 0.2).astype(F), "pred_b": (r.standard_normal(10) * 0.1).astype(F)}
        x = r.random((4, 28, 28, 1)).astype(F)
        ops = [_op("Conv", ["data", "conv1_w", "conv1_b"], ["conv1"], [_arg("kernel", i=5), _arg("stride", i=1), _arg("order", s=b"NCHW")]),
               _op("Relu", ["conv1"], ["conv1"]),
               _op("MaxPool", ["conv1"], ["pool1"], [_arg("kernel", i=2), _arg("stride", i=2)]),
               _op("Conv", ["pool1", "conv2_w", "conv2_b"], ["conv2"], [_arg("kernel", i=5), _arg("pad", i=2)]),
               _op("Relu", ["conv2"], ["conv2"]),
               _op("MaxPool", ["conv2"], ["pool2"], [_arg("kernel", i=2), _arg("stride", i=2)]),
               _op("FC", ["pool2", "fc3_w", "fc3_b"], ["fc3"]),
               _op("Relu", ["fc3"], ["fc3"]),
               _op("Dropout", ["fc3"], ["drop3"], [_arg("ratio", f=0.5), _arg("is_test", i=1)]),
               _op("FC", ["drop3", "pred_w", "pred_b"], ["pred"]),
               _op("Softmax", ["pred"], ["softmax"])]
    elif name == "c2resnet":
        r = np.random.default_rng(2002)
        w = {"res_conv1_w": (r.standard_normal((64, 64, 3, 3)) * np.sqrt(2.0 / 576)).astype(F),
             "res_conv1_b": (r.standard_normal(64) * 0.1).astype(F),
             "res_conv2_w": (r.standard_normal((64, 64, 3, 3)) * np.sqrt(2.0 / 576)).astype(F),
             "fc_w": (r.standard_normal((10, 1024)) * 0.05).astype(F), "fc_b": (r.standard_normal(10) * 0.1).astype(F)}
        for i in (1, 2):
            w[f"bn{i}_s"] = r.uniform(0.5, 1.5, 64).astype(F)
            w[f"bn{i}_b"] = (r.standard_normal(64) * 0.1).astype(F)
            w[f"bn{i}_rm"] = (r.standard_normal(64) * 0.1).astype(F)
            w[f"bn{i}_riv"] = r.uniform(0.5, 1.5, 64).astype(F)
        x = r.standard_normal((2, 8, 8, 64)).astype(F)
        bn = lambda i, src, dst: _op("SpatialBN", [src, f"bn{i}_s", f"bn{i}_b", f"bn{i}_rm", f"bn{i}_riv"], [dst],
                                     [_arg("epsilon", f=1e-5), _arg("order", s=b"NCHW"), _arg("is_test", i=1)])
        ops = [_op("Conv", ["data", "res_conv1_w", "res_conv1_b"], ["c1"], [_arg("kernel", i=3), _arg("pad", i=1)]),
               bn(1, "c1", "c1"),
               _op("Relu", ["c1"], ["c1"]),
               _op("Conv", ["c1", "res_conv2_w"], ["c2"], [_arg("kernel", i=3), _arg("pads", ints=[1, 1, 1, 1], packed=packed)]),
               bn(2, "c2", "c2"),
               _op("Sum", ["c2", "data"], ["c2"]),
               _op("Relu", ["c2"], ["c2"]),
               _op("AveragePool", ["c2"], ["pool"], [_arg("kernel", i=2), _arg("stride", i=2)]),
               _op("FC", ["pool", "fc_w", "fc_b"], ["fc"]),
               _op("Softmax", ["fc"], ["softmax"])]
    else:
        raise ValueError(name)
    predict = _net(name, ops, ["data"] + list(w), ["softmax"])
    init = _net(name + "_init", [_fill(k, v, packed) for k, v in w.items()])
    return predict, init, w, x


def _filter_nhwc(w):
    return np.ascontiguousarray(w.transpose(0, 2, 3, 1))          # oihw -> ohwi


def _fc_from_nhwc(w, h, wd, c):
    out = w.shape[0]                                              # [out, (c,h,w)] -> [(h,w,c), out]
    return np.ascontiguousarray(w.reshape(out, c, h, wd).transpose(2, 3, 1, 0).reshape(h * wd * c, out))


def weight_files(name):
    """{file name: array} an emitted program of this model loads: the input and every weight in the layout the forward
    pass reads (the re-layout the importer does once, done here with numpy)."""
    _, _, w, x = model(name)
    if name == "c2lenet":
        return {"c2lenet_input.bin": x, "c2lenet_conv1_w.bin": _filter_nhwc(w["conv1_w"]), "c2lenet_conv1_b.bin": w["conv1_b"],
                "c2lenet_conv2_w.bin": _filter_nhwc(w["conv2_w"]), "c2lenet_conv2_b.bin": w["conv2_b"],
                "c2lenet_fc3_w.bin": _fc_from_nhwc(w["fc3_w"], 6, 6, 16), "c2lenet_fc3_b.bin": w["fc3_b"],
                "c2lenet_pred_w.bin": np.ascontiguousarray(w["pred_w"].T), "c2lenet_pred_b.bin": w["pred_b"]}
    f = {"c2resnet_input.bin": x, "c2resnet_res_conv1_w.bin": _filter_nhwc(w["res_conv1_w"]), "c2resnet_res_conv1_b.bin": w["res_conv1_b"],
         "c2resnet_res_conv2_w.bin": _filter_nhwc(w["res_conv2_w"]), "c2resnet_fc_w.bin": _fc_from_nhwc(w["fc_w"], 4, 4, 64),
         "c2resnet_fc_b.bin": w["fc_b"]}
    for i in (1, 2):
        for k in ("s", "b", "rm", "riv"):
            f[f"c2resnet_bn{i}_{k}.bin"] = w[f"bn{i}_{k}"]
    return f


def reference_forward(impl, name, rnd=lambda a: a):
    """The model's probabilities through `impl` (the CPU oracle's kernel interface).  `rnd` is applied where a fused
    tensor-core program rounds to bf16."""
    f = weight_files(name)
    g = lambda k: f[f"{name}_{k}.bin"]
    x = rnd(g("input"))
    if name == "c2lenet":
        h = impl.relu_f(impl.conv2d_f(x, g("conv1_w"), g("conv1_b"), (5, 5), (1, 1), (0, 0, 0, 0)))
        h = impl.maxpool_f(h, (2, 2), (2, 2), (0, 0, 0, 0))
        h = impl.relu_f(impl.conv2d_f(h, g("conv2_w"), g("conv2_b"), (5, 5), (1, 1), (2, 2, 2, 2)))
        h = impl.maxpool_f(h, (2, 2), (2, 2), (0, 0, 0, 0))
        h = impl.relu_f(impl.fc(h, g("fc3_w"), g("fc3_b")))
        return impl.matrixSoftmax_f(impl.fc(h, g("pred_w"), g("pred_b")))
    bn = lambda h, i: impl.batchnormalization_f(h, g(f"bn{i}_rm"), g(f"bn{i}_riv"), g(f"bn{i}_s"), g(f"bn{i}_b"), 1e-5)
    k3, s1, p1 = (3, 3), (1, 1), (1, 1, 1, 1)
    h = rnd(impl.relu_f(bn(impl.conv2d_f(x, rnd(g("res_conv1_w")), g("res_conv1_b"), k3, s1, p1), 1)))
    h = bn(impl.conv2d_f(h, rnd(g("res_conv2_w")), np.zeros(64, F), k3, s1, p1), 2)
    h = rnd(impl.relu_f(impl.vecAdd_f(h.reshape(-1), x.reshape(-1)).reshape(h.shape)))
    h = impl.avgpool_f(h, (2, 2), (2, 2), (0, 0, 0, 0))
    return impl.matrixSoftmax_f(impl.fc(h, rnd(g("fc_w")), g("fc_b")))
