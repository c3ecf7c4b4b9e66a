import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as orc
    return orc.Oracle()


@pytest.fixture(scope="session")
def golden():
    z = np.load(os.path.join(GOLDEN, "ref_outputs.npz"))
    return {k.replace("__", "/"): z[k] for k in z.files}


@pytest.fixture(scope="session")
def mnist8():
    d = os.path.join(GOLDEN, "mnist8")
    ld = lambda f, shape: np.fromfile(os.path.join(d, f), np.float32).reshape(shape)
    return dict(x=ld("mnist_images_8.bin", (8, 784)), w0=ld("mlp_weight0.bin", (784, 512)),
                b0=ld("mlp_bias0.bin", (512,)), w1=ld("mlp_weight1.bin", (512, 10)), b1=ld("mlp_bias1.bin", (10,)),
                labels=np.loadtxt(os.path.join(d, "mnist_images_8.meta.txt"), dtype=np.int32))


def bits(a):
    """Bit pattern view for exact comparison (distinguishes -0 from +0, compares NaN payload-insensitively)."""
    a = np.ascontiguousarray(a)
    if a.dtype == np.float32:
        u = a.view(np.uint32).copy()
        u[np.isnan(a)] = 0x7FC00000
        return u
    return a
