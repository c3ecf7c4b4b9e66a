"""Helpers shared by the CPU and GPU tests of the emitted programs (swcompiler_b200/codegen/emitted)."""
import os
import re
import shutil
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EMITTED = os.path.join(ROOT, "swcompiler_b200", "codegen", "emitted")
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
