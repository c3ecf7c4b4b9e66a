"""CPU: the programs B200Codegen emits.  They must compile and link against the kernel library as they stand,
call the table once per op node in the order the reference's lowering produced, and -- where a reference
checkout is present -- be exactly what the generator emits today."""
import os
import subprocess

import pytest

from codegen_util import EMITTED, compile_emitted

REF = os.environ.get("REFERENCE_ROOT", "/root/reference")


def _calls(which):
    text = open(os.path.join(EMITTED, which + "_Graph.cpp")).read()
    body = text[text.index("int main("):]
    return [l.split("(swcb200_")[1].split("(")[0] for l in body.splitlines() if "SWC_CHECK(swcb200_" in l]


def test_mlp8_program_calls_the_table_in_lowered_order():
    assert _calls("mlp8") == ["init", "matrixMatrixMul_f", "batchedadd_f", "matrixTanh_f", "matrixMatrixMul_f", "batchedadd_f",
                              "matrixSoftmax_f", "argMax_i", "sync", "destroy"]


def test_convnet_program_calls_the_table_in_lowered_order():
    assert _calls("convnet") == ["init", "conv2d_f", "batchnormalization_f", "vecAdd_f", "relu_f", "maxpool_f",
                                 "matrixMatrixMul_f", "batchedadd_f", "matrixSoftmax_f", "argMax_i", "sync", "destroy"]
    text = open(os.path.join(EMITTED, "convnet_Graph.cpp")).read()
    assert "pool_out_reshape = pool_out;" in text        # the Reshape node is an alias, not a copy
    # every tensor offset in the arena is 256-byte aligned
    offs = [int(l.split("gpu_arena + ")[1].split(")")[0]) for l in text.splitlines() if "gpu_arena + " in l]
    assert offs and all(o % 256 == 0 for o in offs)


@pytest.mark.parametrize("which", ["mlp8", "convnet"])
def test_emitted_programs_compile_and_link(which, tmp_path):
    exe = compile_emitted(which, str(tmp_path))
    import torch
    if not torch.cuda.is_available():
        r = subprocess.run([exe], capture_output=True, text=True, cwd=str(tmp_path))
        assert r.returncode != 0 and "no sm_100 CUDA device" in r.stderr   # fails loudly, no CPU path


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "include", "SWC.h")), reason="no reference checkout")
def test_committed_programs_are_what_the_generator_emits(tmp_path):
    from swcompiler_b200.codegen import build_codegen as bc
    exe = bc.build(REF)
    out = bc.emit(exe, str(tmp_path))
    for f in ("mlp8_Graph.cpp", "convnet_Graph.cpp", "mlp8_Makefile"):
        assert open(os.path.join(out, f)).read() == open(os.path.join(EMITTED, f)).read(), f
