"""The Caffe2 importer (swcompiler_b200/codegen/Caffe2Import.cpp): model files -> IRGraph -> emitted program.

The pretrained archives the reference's importer tests read are downloads that are not available; two seeded synthetic
models in Caffe2's own file format and weight layouts stand in (tests/golden/caffe2_models.py).  Checked here on the
CPU: the wire-format reader (unpacked and packed repeated fields, truncated input), the weight files the import writes
against an independent numpy re-layout, an unsupported operator, and the programs the generator prints for the
imported graphs -- interpreted call by call with the CPU oracle -- against the same network computed directly.
"""
import os
import subprocess
import sys

import numpy as np
import pytest

from codegen_util import EMITTED, reference_root
from conftest import bits

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import caffe2_models as c2  # noqa: E402

REF = reference_root()
needs_reference = pytest.mark.skipif(not os.path.exists(os.path.join(REF, "include", "SWC.h")), reason="no reference checkout")


def _interpret(which, model, oracle, tmp_path):
    from emitted_interp import Interp
    for name, arr in c2.weight_files(model).items():
        arr.tofile(os.path.join(str(tmp_path), name))
    return Interp(oracle, str(tmp_path)).run(os.path.join(EMITTED, which + "_Graph.cpp"))


def test_imported_programs_compute_the_models(oracle, tmp_path):
    import cases
    got = _interpret("c2lenet", "c2lenet", oracle, tmp_path)
    want = c2.reference_forward(oracle, "c2lenet")
    assert np.array_equal(bits(got["softmax"]), bits(want))
    assert got["top1"][:, 0].astype(int).tolist() == oracle.argMax_i(want, 1)[:, 0].tolist()
    got = _interpret("c2resnet", "c2resnet", oracle, tmp_path)
    assert np.array_equal(bits(got["softmax"]), bits(c2.reference_forward(oracle, "c2resnet")))
    fused = _interpret("c2resnet_fused", "c2resnet", oracle, tmp_path)["softmax"]
    assert np.abs(fused - c2.reference_forward(oracle, "c2resnet", rnd=cases.bf16_round)).max() <= 2e-3
    assert np.abs(fused - c2.reference_forward(oracle, "c2resnet")).max() <= 5e-2


def test_imported_program_shape():
    """No Transpose nodes on the forward pass (weights are re-laid out once, at import), Dropout is an alias, a Conv
    without a bias blob gets a zero bias, the fused plan folds Conv + SpatialBN + Sum + Relu into one call."""
    text = open(os.path.join(EMITTED, "c2lenet_Graph.cpp")).read()
    body = text[text.index("int main("):]
    calls = [l.split("(swcb200_")[1].split("(")[0] for l in body.splitlines() if "SWC_CHECK(swcb200_" in l]
    assert calls == ["init", "conv2d_f", "relu_f", "maxpool_f", "conv2d_f", "relu_f", "maxpool_f", "matrixMatrixMul_f",
                     "batchedadd_f", "relu_f", "matrixMatrixMul_f", "batchedadd_f", "matrixSoftmax_f", "argMax_i", "sync", "destroy"]
    assert "transpose" not in body
    assert "drop3 = fc3_v2;" in body
    res = open(os.path.join(EMITTED, "c2resnet_Graph.cpp")).read()
    assert "fill_device<float>(conv_1_bias, 64, (float)0" in res
    fused = open(os.path.join(EMITTED, "c2resnet_fused_Graph.cpp")).read()
    assert fused.count("swcb200_conv2d_bf16(") == 2 and "data_bf16, 1}" in fused      # skip = the model's input, ReLU on


@needs_reference
def test_import_writes_the_weights_numpy_would_and_rejects_what_it_cannot_read(tmp_path):
    from swcompiler_b200.codegen import build_codegen as bc
    exe = bc.build(REF)
    work = str(tmp_path)
    for packed in (False, True):                       # proto2 writers emit unpacked repeated fields; accept both
        for name in ("c2lenet", "c2resnet"):
            predict, init, _, _ = c2.model(name, packed=packed)
            open(os.path.join(work, name + "_predict.pb"), "wb").write(predict)
            open(os.path.join(work, name + "_init.pb"), "wb").write(init)
            r = subprocess.run([exe, name, work, "x"], cwd=work, capture_output=True, text=True)
            assert r.returncode == 0, r.stderr
            assert open(os.path.join(work, name + "_Graph.cpp")).read() == open(os.path.join(EMITTED, name + "_Graph.cpp")).read()
            for fname, arr in c2.weight_files(name).items():
                if fname.endswith("_input.bin"):
                    continue
                got = np.fromfile(os.path.join(work, fname), np.float32)
                assert np.array_equal(bits(got), bits(arr.reshape(-1))), fname
    # a truncated file
    predict, init, _, _ = c2.model("c2lenet")
    open(os.path.join(work, "c2lenet_init.pb"), "wb").write(init[:len(init) // 2 + 3])
    r = subprocess.run([exe, "c2lenet", work, "x"], cwd=work, capture_output=True, text=True)
    assert r.returncode == 4 and "import of c2lenet failed" in r.stderr
    # an operator outside the importer's vocabulary
    open(os.path.join(work, "c2lenet_init.pb"), "wb").write(init)
    open(os.path.join(work, "c2lenet_predict.pb"), "wb").write(c2._net("bad", [c2._op("LRN", ["data"], ["out"], [c2._arg("size", i=5)])]))
    r = subprocess.run([exe, "c2lenet", work, "x"], cwd=work, capture_output=True, text=True)
    assert r.returncode == 4 and "unsupported Caffe2 operator LRN" in r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("which,model,tol", [("c2lenet", "c2lenet", 0.0), ("c2resnet", "c2resnet", 0.0), ("c2resnet_fused", "c2resnet", 5e-2)])
def test_imported_programs_on_the_gpu(which, model, tol, tmp_path, oracle):
    from codegen_util import compile_emitted, parse_printed
    exe = compile_emitted(which, str(tmp_path))
    for name, arr in c2.weight_files(model).items():
        arr.tofile(os.path.join(str(tmp_path), name))
    r = subprocess.run([exe], capture_output=True, text=True, cwd=str(tmp_path), timeout=120)
    assert r.returncode == 0, r.stderr
    got = parse_printed(r.stdout)
    want = c2.reference_forward(oracle, model)
    if tol == 0.0:
        assert np.abs(got["softmax"] - want).max() <= 5.1e-4        # printed with three decimals
        assert got["top1"][:, 0].astype(int).tolist() == oracle.argMax_i(want, 1)[:, 0].tolist()
    else:
        assert np.abs(got["softmax"] - want).max() <= tol
