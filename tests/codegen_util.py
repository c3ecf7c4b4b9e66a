"""Helpers shared by the CPU and GPU tests of the emitted programs (tests/golden/emitted: what B200Codegen printed for
the sample graphs of gen_driver.cpp, kept as fixtures because the GPU machine has no reference checkout to print them)."""
import os
import re
import shutil
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EMITTED = os.path.join(ROOT, "tests", "golden", "emitted")


def reference_root() -> str:
    """Where a checkout of the reference is looked for: $REFERENCE_ROOT, else a folder `reference` beside the repository."""
    return os.environ.get("REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def compile_emitted(which: str, workdir: str) -> str:
    """g++ the emitted program against the kernel library, the way its Makefile does."""
    shutil.copyfile(os.path.join(EMITTED, which + "_Graph.cpp"), os.path.join(workdir, "Graph.cpp"))
    exe = os.path.join(workdir, "net.bin")
    lib = os.path.join(ROOT, "swcompiler_b200")
    cmd = ["g++", "-O2", "-std=c++11", "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(CUDA, "include"),
           os.path.join(workdir, "Graph.cpp"), "-o", exe, "-L" + lib, "-lswc_b200", "-Wl,-rpath," + lib,
           "-L" + os.path.join(CUDA, "lib64"), "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    return exe


def convnet_inputs(seed=77):
    r = np.random.default_rng(seed)
    f = np.float32
    return {
        "cn_input.bin": r.standard_normal((4, 8, 8, 4)).astype(f),
        "cn_conv_w.bin": (r.standard_normal((4, 3, 3, 4)) * 0.3).astype(f),
        "cn_conv_b.bin": (r.standard_normal(4) * 0.1).astype(f),
        "cn_bn_scale.bin": r.uniform(0.5, 1.5, 4).astype(f),
        "cn_bn_bias.bin": (r.standard_normal(4) * 0.1).astype(f),
        "cn_bn_mean.bin": (r.standard_normal(4) * 0.1).astype(f),
        "cn_bn_var.bin": r.uniform(0.5, 1.5, 4).astype(f),
        "cn_fc_w.bin": (r.standard_normal((64, 10)) * 0.2).astype(f),
        "cn_fc_b.bin": (r.standard_normal(10) * 0.1).astype(f),
    }


def convnet_oracle(impl, t):
    h = impl.conv2d_f(t["cn_input.bin"], t["cn_conv_w.bin"], t["cn_conv_b.bin"], (3, 3), (1, 1), (1, 1, 1, 1))
    h = impl.batchnormalization_f(h, t["cn_bn_mean.bin"], t["cn_bn_var.bin"], t["cn_bn_scale.bin"], t["cn_bn_bias.bin"], 1e-5)
    h = impl.relu_f(impl.vecAdd_f(h.reshape(-1), t["cn_input.bin"].reshape(-1)).reshape(h.shape))
    h = impl.maxpool_f(h, (2, 2), (2, 2), (0, 0, 0, 0))
    return impl.matrixSoftmax_f(impl.fc(h, t["cn_fc_w.bin"], t["cn_fc_b.bin"]))


def resblock_inputs(seed=91):
    """Files of the residual-block graph (gen_driver resblock): [2,8,8,64] image, two 3x3 64->64 convolutions with
    batch-norm, FC 1024->10."""
    r = np.random.default_rng(seed)
    f = np.float32
    t = {"rb_input.bin": r.standard_normal((2, 8, 8, 64)).astype(f),
         "rb_fc_w.bin": (r.standard_normal((1024, 10)) * 0.05).astype(f),
         "rb_fc_b.bin": (r.standard_normal(10) * 0.1).astype(f)}
    for i in range(2):
        t[f"rb_conv{i}_w.bin"] = (r.standard_normal((64, 3, 3, 64)) * np.sqrt(2.0 / 576)).astype(f)
        t[f"rb_conv{i}_b.bin"] = (r.standard_normal(64) * 0.1).astype(f)
        t[f"rb_bn{i}_scale.bin"] = r.uniform(0.5, 1.5, 64).astype(f)
        t[f"rb_bn{i}_bias.bin"] = (r.standard_normal(64) * 0.1).astype(f)
        t[f"rb_bn{i}_mean.bin"] = (r.standard_normal(64) * 0.1).astype(f)
        t[f"rb_bn{i}_var.bin"] = r.uniform(0.5, 1.5, 64).astype(f)
    return t


def resblock_oracle(impl, t, rnd=lambda a: a):
    """The graph op by op through the CPU oracle.  `rnd` is applied where the fused tensor-core program rounds to
    bf16 (image, filters, FC weight, stored activations), so that what is compared is the arithmetic, not the storage."""
    k3, s1, p1 = (3, 3), (1, 1), (1, 1, 1, 1)
    x = rnd(t["rb_input.bin"])

    def conv_bn(h, i):
        h = impl.conv2d_f(h, rnd(t[f"rb_conv{i}_w.bin"]), t[f"rb_conv{i}_b.bin"], k3, s1, p1)
        return impl.batchnormalization_f(h, t[f"rb_bn{i}_mean.bin"], t[f"rb_bn{i}_var.bin"], t[f"rb_bn{i}_scale.bin"],
                                         t[f"rb_bn{i}_bias.bin"], 1e-5)

    h = rnd(impl.relu_f(conv_bn(x, 0)))
    h = conv_bn(h, 1)
    h = rnd(impl.relu_f(impl.vecAdd_f(h.reshape(-1), x.reshape(-1)).reshape(h.shape)))
    h = impl.maxpool_f(h, (2, 2), (2, 2), (0, 0, 0, 0))
    return impl.matrixSoftmax_f(impl.fc(h, rnd(t["rb_fc_w.bin"]), t["rb_fc_b.bin"]))


def _conv_bn_files(r, t, prefix, tag, k):
    f = np.float32
    t[f"{prefix}conv{tag}_w.bin"] = (r.standard_normal((64, k, k, 64)) * np.sqrt(2.0 / (k * k * 64))).astype(f)
    t[f"{prefix}conv{tag}_b.bin"] = (r.standard_normal(64) * 0.1).astype(f)
    t[f"{prefix}bn{tag}_scale.bin"] = r.uniform(0.5, 1.5, 64).astype(f)
    t[f"{prefix}bn{tag}_bias.bin"] = (r.standard_normal(64) * 0.1).astype(f)
    t[f"{prefix}bn{tag}_mean.bin"] = (r.standard_normal(64) * 0.1).astype(f)
    t[f"{prefix}bn{tag}_var.bin"] = r.uniform(0.5, 1.5, 64).astype(f)


def resproj_inputs(seed=93):
    """Files of the projection-shortcut block (gen_driver resproj): [2,8,8,64] image; main branch two 3x3 convolutions
    with batch-norm, shortcut a 1x1 convolution with batch-norm; FC 1024->10."""
    r = np.random.default_rng(seed)
    f = np.float32
    t = {"rp_input.bin": r.standard_normal((2, 8, 8, 64)).astype(f),
         "rp_fc_w.bin": (r.standard_normal((1024, 10)) * 0.05).astype(f),
         "rp_fc_b.bin": (r.standard_normal(10) * 0.1).astype(f)}
    for tag, k in (("S", 1), ("0", 3), ("1", 3)):
        _conv_bn_files(r, t, "rp_", tag, k)
    return t


def resproj_oracle(impl, t, rnd=lambda a: a):
    x = rnd(t["rp_input.bin"])

    def conv_bn(h, tag, k, pad):
        h = impl.conv2d_f(h, rnd(t[f"rp_conv{tag}_w.bin"]), t[f"rp_conv{tag}_b.bin"], (k, k), (1, 1), (pad,) * 4)
        return impl.batchnormalization_f(h, t[f"rp_bn{tag}_mean.bin"], t[f"rp_bn{tag}_var.bin"], t[f"rp_bn{tag}_scale.bin"],
                                         t[f"rp_bn{tag}_bias.bin"], 1e-5)

    shortcut = rnd(conv_bn(x, "S", 1, 0))
    h = rnd(impl.relu_f(conv_bn(x, "0", 3, 1)))
    h = conv_bn(h, "1", 3, 1)
    h = rnd(impl.relu_f(impl.vecAdd_f(h.reshape(-1), shortcut.reshape(-1)).reshape(h.shape)))
    h = impl.maxpool_f(h, (2, 2), (2, 2), (0, 0, 0, 0))
    return impl.matrixSoftmax_f(impl.fc(h, rnd(t["rp_fc_w.bin"]), t["rp_fc_b.bin"]))


def convact_inputs(seed=95):
    """Files of the Conv2dWithActivation graph (gen_driver convact)."""
    r = np.random.default_rng(seed)
    f = np.float32
    return {"ca_input.bin": r.standard_normal((2, 8, 8, 64)).astype(f),
            "ca_conv_w.bin": (r.standard_normal((64, 3, 3, 64)) * np.sqrt(2.0 / 576)).astype(f),
            "ca_conv_b.bin": (r.standard_normal(64) * 0.1).astype(f),
            "ca_fc_w.bin": (r.standard_normal((1024, 10)) * 0.05).astype(f),
            "ca_fc_b.bin": (r.standard_normal(10) * 0.1).astype(f)}


def convact_oracle(impl, t, rnd=lambda a: a):
    """conv2d_f then relu_f: the chain Conv2dWithActivationOp stands for."""
    h = impl.conv2d_f(rnd(t["ca_input.bin"]), rnd(t["ca_conv_w.bin"]), t["ca_conv_b.bin"], (3, 3), (1, 1), (1, 1, 1, 1))
    h = rnd(impl.relu_f(h))
    h = impl.maxpool_f(h, (2, 2), (2, 2), (0, 0, 0, 0))
    return impl.matrixSoftmax_f(impl.fc(h, rnd(t["ca_fc_w.bin"]), t["ca_fc_b.bin"]))


def write_mnist8_records(dirname, wrong=(3,)):
    """A record file in the reference DataLoader's format, <1 label byte><784 floats> per sample: the 8 fixture images and
    2 more (a tail that batches of 4 drop); the labels listed in `wrong` are made wrong on purpose."""
    g = os.path.join(ROOT, "tests", "golden", "mnist8")
    x = np.fromfile(os.path.join(g, "mnist_images_8.bin"), np.float32).reshape(8, 784)
    labels = np.loadtxt(os.path.join(g, "mnist_images_8.meta.txt"), dtype=np.int32)
    for f in os.listdir(g):
        shutil.copyfile(os.path.join(g, f), os.path.join(dirname, f))
    with open(os.path.join(dirname, "mnist8_records.bin"), "wb") as f:
        for n, i in enumerate(list(range(8)) + [0, 1]):
            lab = int(labels[i]) if n not in wrong else (int(labels[i]) + 1) % 10
            f.write(bytes([lab]))
            f.write(x[i].tobytes())
    return 8 - len([w for w in wrong if w < 8])


def parse_printed(text: str):
    """{name: 2-D array} from the program's print_device output."""
    out, name, rows = {}, None, []
    for line in text.splitlines():
        m = re.match(r"^(\w+):$", line.strip())
        if m:
            if name:
                out[name] = np.array(rows, dtype=np.float64)
            name, rows = m.group(1), []
        elif name and line.strip():
            rows.append([float(x) for x in line.split()])
    if name:
        out[name] = np.array(rows, dtype=np.float64)
    return out
