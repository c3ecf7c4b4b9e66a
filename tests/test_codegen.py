"""CPU: the programs B200Codegen emits.  They must compile and link against the kernel library as they stand,
call the table once per op node in the order the reference's lowering produced, and -- where a reference
checkout is present -- be exactly what the generator emits today."""
import os
import subprocess

import pytest

from codegen_util import EMITTED, compile_emitted, reference_root

REF = reference_root()


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


def test_fused_resblock_is_four_calls():
    """Conv -> BN -> ReLU is one swcb200_conv2d_bf16, Conv -> BN -> Add(skip) -> ReLU -> MaxPool 2x2/2 another (the
    pool is the last step of its epilogue: 3x3 filter, 64 -> 64 channels, even sizes), the FC reads the pooled bf16
    tensor through the Reshape view: 15 op nodes, 4 calls and one input cast."""
    assert _calls("resblock_fused") == ["init", "pack_filter_bf16", "pack_filter_bf16", "pack_weight_bf16", "cast_f32_to_bf16",
                                        "conv2d_bf16", "conv2d_bf16", "fc_bf16", "matrixSoftmax_f", "argMax_i",
                                        "sync", "destroy"]
    text = open(os.path.join(EMITTED, "resblock_fused_Graph.cpp")).read()
    assert "{bn0_scale, bn0_bias, bn0_mean, bn0_var, 1e-05f, nullptr, 1}" in text
    assert "{bn1_scale, bn1_bias, bn1_mean, bn1_var, 1e-05f, image_bf16, 1, 1}" in text   # the skip tensor in bf16; relu; pool2x2
    assert "relu1_out" not in text                                                        # the un-pooled result is never stored
    assert "swcb200_conv2d_bf16(ctx, pool_out_bf16, relu0_out_bf16" in text and "conv1_odims_9[] = {2, 8, 8, 64}" in text
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


def test_data_parallel_mlp8_scatters_gathers_and_guards_the_master():
    """config.mpi, mpi_size 2, force_data_parallel through the reference's own tiling passes: inputs are scattered
    (batch split) or broadcast (weights) once after loading, every rank runs the forward pass on its tile, the results
    are gathered on rank 0, which alone holds the un-partitioned tensors and prints."""
    calls = _calls("mlp8_dp2")
    assert calls == ["init", "comm_load", "comm_init"] + ["scatter"] * 5 + ["matrixMatrixMul_f", "batchedadd_f", "matrixTanh_f",
                                                                 "matrixMatrixMul_f", "batchedadd_f", "matrixSoftmax_f", "argMax_i",
                                                                 "gather", "gather", "sync", "comm_destroy", "destroy"]
    text = open(os.path.join(EMITTED, "mlp8_dp2_Graph.cpp")).read()
    assert "swcb200_scatter(ctx, data0, data0_tile, data0_fork_dims_0, 2, 0, SWCB200_F32, 0)" in text       # batch split
    assert "swcb200_scatter(ctx, weight0, weight0_replicate, weight0_fork_dims_1, 2, -1, SWCB200_F32, 0)" in text   # replicate
    assert "swcb200_matrixMatrixMul_f(ctx, 4, 512, 784, data0_tile" in text                                  # 8 rows / 2 ranks
    assert "top3_join_dims_6, 2, 0, SWCB200_I32, 0)" in text
    assert "data0 = rank == 0 ? reinterpret_cast<float *>(gpu_master + 0) : nullptr;" in text
    assert "MPI_Send" not in text and "MPI_Init" not in text and "mpi.h" not in text
    # with the planner: the replicated weights are packed after the load-time scatters, the tile is cast once
    assert _calls("mlp8_dp2_fused") == ["init", "comm_load", "comm_init"] + ["scatter"] * 5 + ["pack_weight_bf16"] * 2 + [
        "cast_f32_to_bf16", "fc_bf16", "fc_bf16", "matrixSoftmax_f", "argMax_i", "gather", "gather", "sync", "comm_destroy",
        "destroy"]


def test_model_parallel_fc_pair_is_column_split_row_split_and_a_reduce():
    """Strategies {-1,1,1}, {1,1}, {1,0,-2} lowered by the reference's ParallelLoweringPass: X replicated, W1 split by
    columns, W2 by rows, the hidden activation never leaves its rank, and the one collective of the forward pass is
    the Reduce of the partial outputs (MPI_Reduce in the reference, NCCL here)."""
    assert _calls("fcpair_mp2") == ["init", "comm_load", "comm_init", "scatter", "scatter", "scatter", "matrixMatrixMul_f", "relu_f",
                                    "matrixMatrixMul_f", "reduce_sum", "sync", "comm_destroy", "destroy"]
    text = open(os.path.join(EMITTED, "fcpair_mp2_Graph.cpp")).read()
    assert "swcb200_scatter(ctx, x, x_replicate, x_fork_dims_0, 2, -1, SWCB200_F32, 0)" in text
    assert "swcb200_scatter(ctx, w1, w1_tile, w1_fork_dims_1, 2, 1, SWCB200_F32, 0)" in text
    assert "swcb200_scatter(ctx, w2, w2_tile, w2_fork_dims_2, 2, 0, SWCB200_F32, 0)" in text
    assert "swcb200_matrixMatrixMul_f(ctx, 64, 256, 256, x_replicate, 256, w1_tile, 256, h_tile, 256)" in text
    assert "swcb200_matrixMatrixMul_f(ctx, 64, 128, 256, hr_tile, 256, w2_tile, 128, y_reduce, 128)" in text
    assert "swcb200_reduce_sum(ctx, y_reduce, y, 8192, SWCB200_F32, 0)" in text
    mk = open(os.path.join(EMITTED, "fcpair_mp2_Makefile")).read()
    assert "for r in 0 1; do SWCB200_RANK=$$r SWCB200_NRANKS=2" in mk
    # with the planner the row-split GEMM and the Reduce behind it become the join over peer memory: no reduce_sum, the
    # partial-sum tensor serves as the p slots, and the ranks' mappings of it are made once, before the forward pass
    calls = _calls("fcpair_mp2_fused")
    assert "reduce_sum" not in calls and calls.index("peer_slots_setup") < calls.index("fc_bf16")
    i = calls.index("fc_bf16_scatter_rows")
    assert calls[i:i + 4] == ["fc_bf16_scatter_rows", "allreduce_sum", "sum_slots", "gather"] and calls[-3] == "peer_slots_release"
    text = open(os.path.join(EMITTED, "fcpair_mp2_fused_Graph.cpp")).read()
    assert ("swcb200_fc_bf16_scatter_rows(ctx, 64, 128, 256, hr_tile_bf16, 256, w2_tile_packed, 256, y_reduce_owner_slots, "
            "nprocs, rank, 128)") in text
    assert "swcb200_sum_slots(ctx, y_reduce, 4096, nprocs, y_reduce_rows, 4096)" in text
    assert "swcb200_gather(ctx, y_reduce_rows, y, " in text


def test_batch_split_residual_block_runs_untiled_ops_on_the_master():
    """BatchNormalization and ElementAdd have no tiling descriptor in the reference (src/op/dlOp/dlOp.h:747-761, :347-355):
    its passes bracket them with Gather and Scatter and the generator prints them inside `if (rank == 0)`."""
    text = open(os.path.join(EMITTED, "resblock_dp2_Graph.cpp")).read()
    body = text[text.index("int main("):]
    guarded = [l.strip() for blk in body.split("if (rank == 0) {")[1:] for l in blk.split("\n    }")[0].splitlines()]
    assert sum("swcb200_batchnormalization_f(" in l for l in guarded) == 2 and sum("swcb200_vecAdd_f(" in l for l in guarded) == 1
    calls = _calls("resblock_dp2")
    i = calls.index("batchnormalization_f")
    assert calls[i - 1] == "gather" and calls[i + 1] == "scatter"
    assert calls.count("conv2d_f") == 2 and "swcb200_conv2d_f(ctx, conv0_out_tile, image_tile" in text   # convolutions on tiles


def test_model_parallel_mlp8_retiles_between_ops_that_disagree():
    """Column-split FC, bias-add on row tiles, tanh on column tiles, row-split FC: the lowering pass inserts Transform
    nodes (1 -> 0 and 0 -> 1), a Reduce to the master and a Scatter back out; all four kinds of communication node."""
    assert _calls("mlp8_mp2")[3:-3] == ["scatter"] * 5 + ["matrixMatrixMul_f", "transform", "batchedadd_f", "transform",
                                                          "matrixTanh_f", "matrixMatrixMul_f", "reduce_sum", "scatter",
                                                          "batchedadd_f", "matrixSoftmax_f", "argMax_i", "gather", "gather"]
    text = open(os.path.join(EMITTED, "mlp8_mp2_Graph.cpp")).read()
    assert "fc0_mm_out_transform_dims_5[] = {8, 512};" in text and "fc0_mm_out_transform_dims_5, 2, 1, 0, SWCB200_F32)" in text
    assert "data1_transform_dims_6[] = {8, 512};" in text and "data1_transform_dims_6, 2, 0, 1, SWCB200_F32)" in text


def test_cuda_graph_form(oracle, golden, tmp_path):
    """graph_replays: the calls of the forward pass sit in a closure that runs once plainly (the library's first-call
    set-up must not happen inside a capture), once under stream capture, and is then replayed as a CUDA graph."""
    import numpy as np

    from conftest import GOLDEN, bits
    from emitted_interp import Interp
    text = open(os.path.join(EMITTED, "mlp8_graph_Graph.cpp")).read()
    body = text[text.index("auto forward = [&]() {"):text.index("};\n    forward();")]
    assert body.count("SWC_CHECK(swcb200_") == 7 and "swcb200_sync" not in body     # nothing that synchronises inside
    order = [text.index(t) for t in ("forward();\n    SWC_CHECK(swcb200_sync(ctx));", "cudaStreamBeginCapture(run_stream",
                                     "cudaStreamEndCapture(run_stream, &graph)", "cudaGraphInstantiate(&graph_exec, graph, 0)",
                                     "cudaGraphLaunch(graph_exec, run_stream)", "print_device<float>")]
    assert order == sorted(order)
    d = os.path.join(GOLDEN, "mnist8")
    it = Interp(oracle, d)
    out = it.run(os.path.join(EMITTED, "mlp8_graph_Graph.cpp"))
    assert it.forward_runs == 5 and np.array_equal(bits(out["data4"]), bits(golden["mnist8/probs"]))   # 1 plain + 1 captured + 3 replays
    assert _calls("resblock_fused_graph").count("conv2d_bf16") == 2


def test_streaming_evaluation_program(oracle, tmp_path):
    """config.use_dataloader: the forward pass inside a loop over a record file, two device slots and two pinned host
    buffers for the loader-fed tensors, uploads on a second stream, AccuracyOp as swcb200_accuracy_i; the counters are
    zeroed once and accumulate over the batches; a tail the file cannot fill a batch from is dropped."""
    from codegen_util import write_mnist8_records
    from emitted_interp import Interp
    text = open(os.path.join(EMITTED, "mlp_eval_Graph.cpp")).read()
    assert 'RecordLoader loader("mnist8_records.bin", true, 10, 4, 784);' in text
    assert "data0 = data0_slot[s];" in text and "selected = selected_slot[s];" in text
    assert "cudaMemcpyAsync(data0, host_data[s], 3136 * sizeof(float), cudaMemcpyHostToDevice, copy_stream)" in text
    assert "swcb200_accuracy_i(ctx, top1, selected, accur, 4, 1)" in text
    assert text.index("fill_device<int>(accur, 2, (int)0, host_stage);") < text.index("for (int s = 0; have; s ^= 1) {")
    assert 'load_to_device<float>(data0' not in text          # the loader fills it, batch by batch
    right = write_mnist8_records(str(tmp_path), wrong=(3,))
    for which in ("mlp_eval", "mlp_eval_fused"):
        it = Interp(oracle, str(tmp_path))
        out = it.run(os.path.join(EMITTED, which + "_Graph.cpp"))
        assert it.batches == 2 and out["accur"].tolist() == [[right, 8]], which
    assert _calls("mlp_eval_fused").count("fc_bf16") == 2 and _calls("mlp_eval_fused").count("pack_weight_bf16") == 2


def _interpret(which, files, oracle, tmp_path):
    from emitted_interp import Interp
    for name, arr in files.items():
        arr.tofile(os.path.join(tmp_path, name))
    it = Interp(oracle, str(tmp_path))
    return it.run(os.path.join(EMITTED, which + "_Graph.cpp"))


def test_emitted_call_sequences_compute_the_right_thing_on_the_cpu(oracle, golden, tmp_path):
    """The emitted programs' calls, carried out one by one by the CPU oracle (tests/emitted_interp.py): operand names,
    shapes, leading dimensions, the fusion planner's storage plan and casts.  (The CUDA kernels are the GPU tests' job.)"""
    import numpy as np

    import cases
    from codegen_util import convnet_inputs, convnet_oracle, resblock_inputs, resblock_oracle
    from conftest import GOLDEN, bits
    d = os.path.join(GOLDEN, "mnist8")
    mnist = {f: np.fromfile(os.path.join(d, f), dtype=np.uint8) for f in os.listdir(d)}
    got = _interpret("mlp8", mnist, oracle, tmp_path)
    assert np.array_equal(bits(got["data4"]), bits(golden["mnist8/probs"])) and np.array_equal(got["top3"], golden["mnist8/top3"])
    got = _interpret("mlp8_fused", mnist, oracle, tmp_path)
    assert got["top3"][:, 0].tolist() == [5, 0, 4, 1, 9, 2, 1, 3] and np.abs(got["data4"] - golden["mnist8/probs"]).max() <= 2e-2
    t = convnet_inputs()
    want = convnet_oracle(oracle, t)
    assert np.array_equal(bits(_interpret("convnet", t, oracle, tmp_path)["probs"]), bits(want))
    assert np.abs(_interpret("convnet_fused", t, oracle, tmp_path)["probs"] - want).max() <= 2e-2
    t = resblock_inputs()
    assert np.array_equal(bits(_interpret("resblock", t, oracle, tmp_path)["probs"]), bits(resblock_oracle(oracle, t)))
    fused = _interpret("resblock_fused", t, oracle, tmp_path)["probs"]
    assert np.abs(fused - resblock_oracle(oracle, t, rnd=cases.bf16_round)).max() <= 1e-3   # same rounding points
    assert np.abs(fused - resblock_oracle(oracle, t)).max() <= 5e-2


def test_projection_shortcut_block_and_conv_with_activation(oracle, tmp_path):
    """Two convolution chains meet at one ElementAdd (a residual block whose shortcut is a 1x1 convolution).  The fused
    plan must give the add to the chain that is printed LAST, with the other chain's result -- already computed -- as the
    skip operand; and Conv2dWithActivationOp is conv2d_f + relu_f unfused, one conv2d_bf16 with the ReLU flag fused."""
    import numpy as np

    import cases
    from codegen_util import convact_inputs, convact_oracle, resproj_inputs, resproj_oracle
    from conftest import bits
    calls = _calls("resproj_fused")
    assert calls.count("conv2d_bf16") == 3 and "vecAdd_f" not in calls and "relu_f" not in calls
    text = open(os.path.join(EMITTED, "resproj_fused_Graph.cpp")).read()
    assert "{bnS_scale, bnS_bias, bnS_mean, bnS_var, 1e-05f, nullptr, 0}" in text             # shortcut: conv + bn only
    assert "{bn1_scale, bn1_bias, bn1_mean, bn1_var, 1e-05f, bnS_out_bf16, 1, 1}" in text     # main branch takes add + relu (+ pool)
    assert text.index("convS_epilogue") < text.index("conv1_epilogue")                         # the skip exists by then
    t = resproj_inputs()
    assert np.array_equal(bits(_interpret("resproj", t, oracle, tmp_path)["probs"]), bits(resproj_oracle(oracle, t)))
    fused = _interpret("resproj_fused", t, oracle, tmp_path)["probs"]
    assert np.abs(fused - resproj_oracle(oracle, t, rnd=cases.bf16_round)).max() <= 1e-3
    assert np.abs(fused - resproj_oracle(oracle, t)).max() <= 5e-2

    assert _calls("convact")[1:4] == ["conv2d_f", "relu_f", "maxpool_f"]
    assert _calls("convact_fused").count("conv2d_bf16") == 1 and "relu_f" not in _calls("convact_fused")
    assert "{nullptr, nullptr, nullptr, nullptr, 0.0f, nullptr, 1}" in open(os.path.join(EMITTED, "convact_fused_Graph.cpp")).read()
    t = convact_inputs()
    assert np.array_equal(bits(_interpret("convact", t, oracle, tmp_path)["probs"]), bits(convact_oracle(oracle, t)))
    fused = _interpret("convact_fused", t, oracle, tmp_path)["probs"]
    assert np.abs(fused - convact_oracle(oracle, t, rnd=cases.bf16_round)).max() <= 1e-3


from swcompiler_b200.codegen.build_codegen import PROGRAMS as ALL_PROGRAMS  # noqa: E402


@pytest.mark.parametrize("which", ALL_PROGRAMS)
def test_emitted_programs_compile_and_link(which, tmp_path):
    exe = compile_emitted(which, str(tmp_path))
    import torch
    if not torch.cuda.is_available():
        ranks = 2 if ("_dp2" in which or "_mp2" in which) else 1
        env = dict(os.environ, SWCB200_RANK="0", SWCB200_NRANKS=str(ranks), SWCB200_ID_FILE=os.path.join(str(tmp_path), "id"))
        r = subprocess.run([exe], capture_output=True, text=True, cwd=str(tmp_path), env=env)
        assert r.returncode != 0 and "no sm_100 CUDA device" in r.stderr   # fails loudly, no CPU path


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "include", "SWC.h")), reason="no reference checkout")
def test_generator_refuses_an_op_outside_the_kernel_table(tmp_path):
    """A graph with an ElementMul node: the generator records it, gen_driver exits with code 3, and the text it wrote
    holds an #error, so it cannot be compiled into a program that skips the op."""
    from swcompiler_b200.codegen import build_codegen as bc
    exe = bc.build(REF)
    r = subprocess.run([exe, "badop", str(tmp_path), "x"], cwd=bc.BUILD, capture_output=True, text=True)
    assert r.returncode == 3 and "cannot emit: mul0 : ElementMul" in r.stderr
    text = open(os.path.join(str(tmp_path), "badop_Graph.cpp")).read()
    assert '#error "swc_b200: cannot emit mul0 : ElementMul' in text
    r = subprocess.run(["g++", "-fsyntax-only", "-I" + os.path.join(os.path.dirname(EMITTED), "..", "..", "include"),
                        "-I/usr/local/cuda/include", os.path.join(str(tmp_path), "badop_Graph.cpp")], capture_output=True, text=True)
    assert r.returncode != 0 and "cannot emit" in r.stderr


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "include", "SWC.h")), reason="no reference checkout")
def test_committed_programs_are_what_the_generator_emits(tmp_path):
    from swcompiler_b200.codegen import build_codegen as bc
    exe = bc.build(REF)
    out = bc.emit(exe, str(tmp_path))
    for f in [w + "_Graph.cpp" for w in ALL_PROGRAMS] + ["mlp8_Makefile", "fcpair_mp2_Makefile"]:
        assert open(os.path.join(out, f)).read() == open(os.path.join(EMITTED, f)).read(), f
