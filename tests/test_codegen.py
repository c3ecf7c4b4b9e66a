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


def test_fused_mlp8_is_two_fused_calls_with_bf16_between_them():
    """Emit-time fusion: MatrixMatrixMul -> MatrixVectorAdd -> Tanh becomes one swcb200_fc_bf16; the hidden activation,
    read only by the next fused call, exists in bf16 alone; the logits, read by the fp32 softmax, are written as fp32."""
    assert _calls("mlp8_fused") == ["init", "pack_weight_bf16", "pack_weight_bf16", "cast_f32_to_bf16", "fc_bf16", "fc_bf16",
                                    "matrixSoftmax_f", "argMax_i", "sync", "destroy"]
    text = open(os.path.join(EMITTED, "mlp8_fused_Graph.cpp")).read()
    assert "SWCB200_ACT_TANH, data2_bf16, SWCB200_BF16, 512" in text and "SWCB200_ACT_NONE, data3, SWCB200_F32, 10" in text
    assert "float *data1;" not in text and "float *data2;" not in text      # chain intermediates get no storage
    assert "swcb200_init(0, SWCB200_TC_BF16" in text


def test_fused_resblock_is_five_calls():
    """Conv -> BN -> ReLU and Conv -> BN -> Add(skip) -> ReLU are one swcb200_conv2d_bf16 each, the pool runs on bf16
    storage, the FC reads the pooled bf16 tensor through the Reshape view: 15 op nodes, 5 calls and one input cast."""
    assert _calls("resblock_fused") == ["init", "pack_filter_bf16", "pack_filter_bf16", "pack_weight_bf16", "cast_f32_to_bf16",
                                        "conv2d_bf16", "conv2d_bf16", "maxpool_bf16", "fc_bf16", "matrixSoftmax_f", "argMax_i",
                                        "sync", "destroy"]
    text = open(os.path.join(EMITTED, "resblock_fused_Graph.cpp")).read()
    assert "{bn0_scale, bn0_bias, bn0_mean, bn0_var, 1e-05f, nullptr, 1}" in text
    assert "{bn1_scale, bn1_bias, bn1_mean, bn1_var, 1e-05f, image_bf16, 1}" in text   # the skip tensor, in bf16
    assert "pool_out_bf16, 1024, fc_w_packed" in text
    offs = [int(l.split("gpu_arena + ")[1].split(")")[0]) for l in text.splitlines() if "gpu_arena + " in l]
    assert offs and all(o % 256 == 0 for o in offs)
    # the same graph unfused: one call per op node
    assert _calls("resblock")[1:-2] == ["conv2d_f", "batchnormalization_f", "relu_f", "conv2d_f", "batchnormalization_f",
                                        "vecAdd_f", "relu_f", "maxpool_f", "matrixMatrixMul_f", "batchedadd_f", "matrixSoftmax_f",
                                        "argMax_i"]


def test_fused_convnet_falls_back_per_op_where_the_kernel_cannot_take_the_shape():
    """4 channels: the convolution chain is printed op by op through the fp32 table; the FC is still fused and its
    fp32 input is cast once."""
    assert _calls("convnet_fused") == ["init", "pack_weight_bf16", "conv2d_f", "batchnormalization_f", "vecAdd_f", "relu_f",
                                       "maxpool_f", "cast_f32_to_bf16", "fc_bf16", "matrixSoftmax_f", "argMax_i", "sync", "destroy"]


ALL_PROGRAMS = ["mlp8", "convnet", "resblock", "mlp8_fused", "convnet_fused", "resblock_fused"]


@pytest.mark.parametrize("which", ALL_PROGRAMS)
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
    for f in [w + "_Graph.cpp" for w in ALL_PROGRAMS] + ["mlp8_Makefile"]:
        assert open(os.path.join(out, f)).read() == open(os.path.join(EMITTED, f)).read(), f
