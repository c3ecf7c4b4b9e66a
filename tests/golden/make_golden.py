"""Regenerates the committed golden vectors.  Run where a reference checkout is
mounted:  python tests/golden/make_golden.py [/path/to/reference]

1. Copies the reference's only result-pinning fixture -- the 8 MNIST images, the
   784-512-10 tanh MLP weights and the expected labels (test/input/) -- to
   tests/golden/mnist8/, because the GPU machine has no reference checkout.
2. Runs the REFERENCE's own kernels.h (oracle/_ref/libswc_ref.so, built by
   oracle/Makefile from the checkout) over every seeded case of tests/cases.py
   and over the fixture MLP, and stores the outputs in ref_outputs.npz.
"""
import os
import shutil
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path[:0] = [ROOT, os.path.join(ROOT, "tests")]

import cases  # noqa: E402
from oracle import oracle as orc  # noqa: E402


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else (os.environ.get("REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference"))
    os.environ["REFERENCE_ROOT"] = ref_root
    orc.build()
    ref = orc.Reference()
    dst = os.path.join(HERE, "mnist8")
    os.makedirs(dst, exist_ok=True)
    for f in ["mnist_images_8.bin", "mnist_images_8.meta.txt", "mlp_weight0.bin", "mlp_bias0.bin",
              "mlp_weight1.bin", "mlp_bias1.bin"]:
        shutil.copyfile(os.path.join(ref_root, "test", "input", f), os.path.join(dst, f))
    out = cases.run_all(ref)
    ld = lambda f, shape: np.fromfile(os.path.join(dst, f), np.float32).reshape(shape)
    probs = ref.mlp_forward(ld("mnist_images_8.bin", (8, 784)), ld("mlp_weight0.bin", (784, 512)),
                            ld("mlp_bias0.bin", (512,)), ld("mlp_weight1.bin", (512, 10)),
                            ld("mlp_bias1.bin", (10,)))
    out["mnist8/probs"] = probs
    out["mnist8/top3"] = ref.argMax_i(probs, 3)
    c2 = cases.config2_lenet(batch=4)
    out["config2_b4/probs"] = cases.lenet_forward(ref, c2)
    c5 = cases.config5_res_stage(batch=1, hw=12, blocks=1)
    out["config5_b1_hw12/out"] = cases.res_stage_forward(ref, c5)
    np.savez_compressed(os.path.join(HERE, "ref_outputs.npz"), **{k.replace("/", "__"): v for k, v in out.items()})
    print("wrote", len(out), "arrays;", os.path.getsize(os.path.join(HERE, "ref_outputs.npz")), "bytes")
    print("mnist8 top-1:", out["mnist8/top3"][:, 0].tolist())


if __name__ == "__main__":
    main()
