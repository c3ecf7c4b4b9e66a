"""Seeded input cases shared by the golden-vector generator, the CPU oracle tests
and the GPU parity tests.  Every case is a small dict of numpy arrays and
attributes drawn from ``numpy.random.default_rng(seed)``; nothing is read from
disk, so the same bytes are rebuilt wherever the tests run.

Edge cases follow what the reference's loops distinguish: sizes that are not a
multiple of any tile, single rows/columns, padding taps, windows that lie wholly
in the padding, ties (MaxPool first-max, ArgMax higher-index), negative zero and
NaN for ReLU, leading dimensions of one.
"""
from __future__ import annotations

import numpy as np

F = np.float32


def _rng(seed):
    return np.random.default_rng(seed)


def matmul_cases():
    out = {}
    for name, (m, n, k), seed in [
        ("mm_1x1x1", (1, 1, 1), 11), ("mm_3x5x7", (3, 5, 7), 12), ("mm_8x10x512", (8, 10, 512), 13),
        ("mm_64x512x784", (64, 512, 784), 14), ("mm_33x129x65", (33, 129, 65), 15),
        ("mm_130x70x257", (130, 70, 257), 16), ("mm_32x10x1568", (32, 10, 1568), 17),
    ]:
        r = _rng(seed)
        out[name] = dict(a=r.standard_normal((m, k)).astype(F), b=(r.standard_normal((k, n)) * 0.05).astype(F))
    return out


def rowwise_cases():
    """2-D inputs for bias-add, tanh, softmax, argmax."""
    out = {}
    for name, (m, n), seed in [("r_1x1", (1, 1), 21), ("r_8x10", (8, 10), 22), ("r_64x512", (64, 512), 23),
                               ("r_5x1000", (5, 1000), 24), ("r_7x33", (7, 33), 25), ("r_3x4099", (3, 4099), 26)]:
        r = _rng(seed)
        x = (r.standard_normal((m, n)) * 2.0).astype(F)
        out[name] = dict(x=x, bias=(r.standard_normal(n) * 0.1).astype(F))
    # small-magnitude inputs: the tanh formula cancels near zero
    r = _rng(27)
    out["r_small_16x64"] = dict(x=(r.standard_normal((16, 64)) * 1e-3).astype(F), bias=np.zeros(64, F))
    # large magnitudes: expf overflows to inf / underflows to 0 inside the tanh formula
    out["r_large_4x32"] = dict(x=(_rng(28).standard_normal((4, 32)) * 60.0).astype(F), bias=np.zeros(32, F))
    return out


def argmax_cases():
    out = {}
    r = _rng(31)
    out["am_8x10_k3"] = dict(x=r.random((8, 10)).astype(F), k=3)
    out["am_5x1000_k5"] = dict(x=r.standard_normal((5, 1000)).astype(F), k=5)
    out["am_1x1_k1"] = dict(x=np.array([[2.5]], F), k=1)
    # ties everywhere: quantised values, so equal maxima are common -> higher index must win
    out["am_ties_16x37_k4"] = dict(x=np.round(r.random((16, 37)) * 4).astype(F), k=4)
    out["am_allsame_3x9_k9"] = dict(x=np.full((3, 9), 1.0, F), k=9)
    z = np.zeros((2, 6), F)
    z[0, 1] = -0.0
    z[0, 4] = -0.0
    out["am_signedzero_2x6_k6"] = dict(x=z, k=6)
    return out


def accuracy_cases():
    """Predictions [m, n] int32 (top-n indices) against labels [m]."""
    out = {}
    r = _rng(37)
    out["acc_64x1"] = dict(pred=r.integers(0, 10, (64, 1)).astype(np.int32), label=r.integers(0, 10, 64).astype(np.int32))
    out["acc_1000x3"] = dict(pred=r.integers(0, 10, (1000, 3)).astype(np.int32), label=r.integers(0, 10, 1000).astype(np.int32))
    # a label that appears twice among a row's predictions counts once
    out["acc_dups_5x4"] = dict(pred=np.array([[1, 1, 1, 1], [0, 2, 2, 0], [3, 4, 5, 6], [7, 7, 8, 9], [9, 9, 9, 9]], np.int32),
                               label=np.array([1, 2, 0, 7, 3], np.int32))
    out["acc_1x1"] = dict(pred=np.array([[4]], np.int32), label=np.array([4], np.int32))
    return out


def flat_cases():
    """Flat vectors for relu / add; lengths around the 128-bit vector width."""
    out = {}
    for n, seed in [(1, 41), (3, 42), (4, 43), (5, 44), (1023, 45), (4096, 46), (100003, 47)]:
        r = _rng(seed)
        out[f"v_{n}"] = dict(a=r.standard_normal(n).astype(F), b=r.standard_normal(n).astype(F))
    s = np.array([0.0, -0.0, np.nan, -np.nan, np.inf, -np.inf, 1e-45, -1e-45, 3.0, -3.0], F)
    out["v_special"] = dict(a=s, b=s[::-1].copy())
    return out


def conv_cases():
    out = {}
    spec = [
        # name, idims NHWC, oC, (kh,kw), (sh,sw), pads(t,l,b,r), group, seed
        # (group is 1 throughout: the reference reads past its filter for group > 1, kernels.h:208-209)
        ("cv_lenet1", (2, 28, 28, 1), 16, (5, 5), (1, 1), (2, 2, 2, 2), 1, 51),
        ("cv_lenet2", (2, 14, 14, 16), 32, (5, 5), (1, 1), (2, 2, 2, 2), 1, 52),
        ("cv_res3x3", (1, 12, 12, 64), 64, (3, 3), (1, 1), (1, 1, 1, 1), 1, 53),
        ("cv_1x1", (3, 5, 7, 8), 4, (1, 1), (1, 1), (0, 0, 0, 0), 1, 54),
        ("cv_stride2", (2, 9, 11, 3), 5, (3, 3), (2, 2), (1, 1, 1, 1), 1, 55),
        ("cv_asym", (1, 8, 6, 2), 3, (3, 2), (1, 2), (2, 0, 2, 0), 1, 56),
        ("cv_bigpad", (1, 3, 3, 2), 2, (3, 3), (1, 1), (2, 2, 2, 2), 1, 58),
    ]
    for name, idims, oc, k, s, p, g, seed in spec:
        r = _rng(seed)
        ic = idims[3]
        fan = k[0] * k[1] * ic // g
        out[name] = dict(x=r.standard_normal(idims).astype(F),
                         w=(r.standard_normal((oc, k[0], k[1], ic // g)) * np.sqrt(2.0 / fan)).astype(F),
                         b=(r.standard_normal(oc) * 0.1).astype(F), kernels=k, strides=s, pads=p, group=g)
    return out


def pool_cases():
    out = {}
    spec = [
        ("pl_2x2", (2, 28, 28, 16), (2, 2), (2, 2), (0, 0, 0, 0), 61),
        ("pl_2x2_c64", (1, 8, 8, 64), (2, 2), (2, 2), (0, 0, 0, 0), 62),
        ("pl_3x3s2p1", (2, 9, 7, 5), (3, 3), (2, 2), (1, 1, 1, 1), 63),
        ("pl_odd", (1, 7, 7, 3), (2, 2), (2, 2), (0, 0, 0, 0), 64),
        ("pl_allpad", (1, 2, 2, 2), (2, 2), (3, 3), (2, 2, 2, 2), 65),
        ("pl_3x2s1", (2, 5, 6, 9), (3, 2), (1, 1), (1, 0, 1, 0), 66),
    ]
    for name, idims, k, s, p, seed in spec:
        r = _rng(seed)
        out[name] = dict(x=r.standard_normal(idims).astype(F), kernels=k, strides=s, pads=p)
    # ties and negatives: quantised, all-negative (a padded tap must never contribute a 0)
    r = _rng(67)
    out["pl_ties"] = dict(x=(np.round(r.random((2, 6, 6, 4)) * 3) - 5).astype(F), kernels=(2, 2), strides=(2, 2),
                          pads=(0, 0, 0, 0))
    out["pl_neg_pad"] = dict(x=(-1 - r.random((1, 5, 5, 3))).astype(F), kernels=(3, 3), strides=(2, 2),
                             pads=(1, 1, 1, 1))
    return out


def bn_cases():
    out = {}
    for name, idims, seed in [("bn_64", (2, 7, 7, 64), 71), ("bn_3", (1, 5, 4, 3), 72), ("bn_1", (3, 2, 2, 1), 73),
                              ("bn_130", (1, 3, 3, 130), 74)]:
        r = _rng(seed)
        c = idims[3]
        out[name] = dict(x=r.standard_normal(idims).astype(F), scale=r.uniform(0.5, 1.5, c).astype(F),
                         bias=(r.standard_normal(c) * 0.1).astype(F), mean=(r.standard_normal(c) * 0.1).astype(F),
                         var=r.uniform(0.5, 1.5, c).astype(F), eps=1e-5)
    return out


def transpose_cases():
    out = {}
    r = _rng(81)
    out["t2_5x7"] = dict(x=r.standard_normal((5, 7)).astype(F), shuffle=(1, 0))
    out["t2_id"] = dict(x=r.standard_normal((4, 3)).astype(F), shuffle=(0, 1))
    out["t4_nhwc_nchw"] = dict(x=r.standard_normal((2, 5, 6, 3)).astype(F), shuffle=(0, 3, 1, 2))
    out["t4_nchw_nhwc"] = dict(x=r.standard_normal((2, 3, 5, 6)).astype(F), shuffle=(0, 2, 3, 1))
    out["t4_rev"] = dict(x=r.standard_normal((2, 3, 4, 5)).astype(F), shuffle=(3, 2, 1, 0))
    return out


def run_all(impl, accuracy=True):
    """Outputs of every case through ``impl`` (an Oracle/Reference-shaped object), keyed by case name."""
    res = {}
    for k, c in matmul_cases().items():
        res[k] = impl.matrixMatrixMul_f(c["a"], c["b"])
    for k, c in rowwise_cases().items():
        res[k + "/badd"] = impl.batchedadd_f(c["x"], c["bias"])
        res[k + "/tanh"] = impl.matrixTanh_f(c["x"])
        res[k + "/softmax"] = impl.matrixSoftmax_f(c["x"])
    for k, c in argmax_cases().items():
        res[k] = impl.argMax_i(c["x"], c["k"])
    for k, c in (accuracy_cases() if accuracy else {}).items():
        res[k] = impl.accuracy_i(c["pred"], c["label"])
    for k, c in flat_cases().items():
        res[k + "/relu"] = impl.relu_f(c["a"])
        res[k + "/add"] = impl.vecAdd_f(c["a"], c["b"])
    for k, c in conv_cases().items():
        res[k] = impl.conv2d_f(c["x"], c["w"], c["b"], c["kernels"], c["strides"], c["pads"], c["group"])
    for k, c in pool_cases().items():
        res[k + "/max"] = impl.maxpool_f(c["x"], c["kernels"], c["strides"], c["pads"])
        res[k + "/avg"] = impl.avgpool_f(c["x"], c["kernels"], c["strides"], c["pads"])
    for k, c in bn_cases().items():
        res[k] = impl.batchnormalization_f(c["x"], c["mean"], c["var"], c["scale"], c["bias"], c["eps"])
    for k, c in transpose_cases().items():
        res[k] = (impl.transpose2d_f if c["x"].ndim == 2 else impl.transpose4d_f)(c["x"], c["shuffle"])
    return res


# ---- the benchmark configurations, at their stated sizes or a bounded slice ----------------

def config1_mlp(batch=64, seed=1001):
    """MLP forward: X[B,784]~U[0,1); W1[784,512]~N(0,.05^2), b1=0; W2[512,10]~N(0,.05^2), b2=0."""
    r = _rng(seed)
    return dict(x=r.random((batch, 784)).astype(F), w0=(r.standard_normal((784, 512)) * 0.05).astype(F),
                b0=np.zeros(512, F), w1=(r.standard_normal((512, 10)) * 0.05).astype(F), b1=np.zeros(10, F),
                labels=r.integers(0, 10, batch).astype(np.int32))


def config2_lenet(batch=32, seed=1002):
    """LeNet-style NHWC: conv5x5 1->16 p2, ReLU, pool2; conv5x5 16->32 p2, ReLU, pool2; FC 1568->10; softmax."""
    r = _rng(seed)
    return dict(x=r.random((batch, 28, 28, 1)).astype(F),
                cw0=(r.standard_normal((16, 5, 5, 1)) * np.sqrt(2 / 25)).astype(F), cb0=np.zeros(16, F),
                cw1=(r.standard_normal((32, 5, 5, 16)) * np.sqrt(2 / 400)).astype(F), cb1=np.zeros(32, F),
                fw=(r.standard_normal((1568, 10)) * 0.02).astype(F), fb=np.zeros(10, F))


def lenet_forward(impl, c):
    k5, s1, p2 = (5, 5), (1, 1), (2, 2, 2, 2)
    k2, s2, p0 = (2, 2), (2, 2), (0, 0, 0, 0)
    h = impl.maxpool_f(impl.relu_f(impl.conv2d_f(c["x"], c["cw0"], c["cb0"], k5, s1, p2)), k2, s2, p0)
    h = impl.maxpool_f(impl.relu_f(impl.conv2d_f(h, c["cw1"], c["cb1"], k5, s1, p2)), k2, s2, p0)
    return impl.matrixSoftmax_f(impl.fc(h, c["fw"], c["fb"]))


def bf16_round(x):
    """Round fp32 to the nearest bf16 (ties to even), returned as fp32."""
    u = np.ascontiguousarray(x, F).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(F).reshape(np.shape(x))


def config3_wide_mlp(batch, width=4096, classes=1000, layers=4, seed=1003):
    """Wide MLP: X~N(0,1) bf16-representable; `layers` x (W~N(0,1/width) bf16-representable, b~N(0,.01^2) fp32,
    ReLU); final FC width->classes, softmax.  `batch` may be a slice of the stated 65536 rows."""
    r = _rng(seed)
    c = dict(x=bf16_round(r.standard_normal((batch, width)).astype(F)), w=[], b=[])
    for i in range(layers + 1):
        n = width if i < layers else classes
        c["w"].append(bf16_round((r.standard_normal((width, n)) / np.sqrt(width)).astype(F)))
        c["b"].append((r.standard_normal(n) * 0.01).astype(F))
    return c


def wide_mlp_forward(impl, c, softmax=True):
    h = c["x"]
    last = len(c["w"]) - 1
    for i, (w, b) in enumerate(zip(c["w"], c["b"])):
        h = impl.fc(h, w, b)
        if i < last:
            h = impl.relu_f(h)
    return impl.matrixSoftmax_f(h) if softmax else h


def config5_res_stage(batch, hw=56, ch=64, blocks=3, seed=1005):
    """ResNet-style stage, NHWC: `blocks` x (conv3x3-BN-ReLU-conv3x3-BN-add(skip)-ReLU), then MaxPool 2x2/2."""
    r = _rng(seed)
    c = dict(x=r.standard_normal((batch, hw, hw, ch)).astype(F), conv=[], bn=[])
    for _ in range(2 * blocks):
        c["conv"].append(dict(w=(r.standard_normal((ch, 3, 3, ch)) * np.sqrt(2 / (9 * ch))).astype(F),
                              b=np.zeros(ch, F)))
        c["bn"].append(dict(scale=r.uniform(0.5, 1.5, ch).astype(F), bias=(r.standard_normal(ch) * 0.1).astype(F),
                            mean=(r.standard_normal(ch) * 0.1).astype(F), var=r.uniform(0.5, 1.5, ch).astype(F),
                            eps=1e-5))
    return c


def res_stage_forward(impl, c):
    k3, s1, p1 = (3, 3), (1, 1), (1, 1, 1, 1)
    h = c["x"]
    for blk in range(len(c["conv"]) // 2):
        skip = h
        for j in range(2):
            cv, bn = c["conv"][2 * blk + j], c["bn"][2 * blk + j]
            h = impl.conv2d_f(h, cv["w"], cv["b"], k3, s1, p1)
            h = impl.batchnormalization_f(h, bn["mean"], bn["var"], bn["scale"], bn["bias"], bn["eps"])
            if j == 0:
                h = impl.relu_f(h)
        h = impl.relu_f(impl.vecAdd_f(h.reshape(-1), skip.reshape(-1)).reshape(h.shape))
    return impl.maxpool_f(h, (2, 2), (2, 2), (0, 0, 0, 0))
