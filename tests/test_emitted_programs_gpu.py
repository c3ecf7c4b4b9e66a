"""GPU: the programs the emit-time fusion planner prints (tensor-core precision, one call per fused chain), the
residual-block graph printed op by op in strict precision, and the programs printed for graphs the reference's tiling
passes partitioned over two ranks (one process per GPU, Scatter / Gather / Reduce over NCCL) -- compiled with g++ on
the spot and run as separate processes."""
import os
import shutil
import subprocess

import numpy as np
import pytest

import cases
from codegen_util import (compile_emitted, convnet_inputs, convnet_oracle, parse_printed, resblock_inputs, resblock_oracle)
from conftest import GOLDEN

pytestmark = pytest.mark.gpu


def _run(which, tmp_path, files):
    exe = compile_emitted(which, str(tmp_path))
    for name, arr in files.items():
        arr.tofile(os.path.join(tmp_path, name))
    r = subprocess.run([exe], capture_output=True, text=True, cwd=str(tmp_path), timeout=120)
    assert r.returncode == 0, r.stderr
    return parse_printed(r.stdout)


def _run_ranks(which, tmp_path, files, nranks):
    """One process per GPU, the way the program's Makefile starts it: rank and count in the environment, a fresh file
    for the NCCL id.  Returns what rank 0 printed."""
    import torch
    if torch.cuda.device_count() < nranks:
        pytest.skip(f"needs {nranks} GPUs")
    exe = compile_emitted(which, str(tmp_path))
    for name, arr in files.items():
        arr.tofile(os.path.join(tmp_path, name))
    env = dict(os.environ, SWCB200_NRANKS=str(nranks), SWCB200_ID_FILE=os.path.join(str(tmp_path), "nccl_id"),
               NCCL_NVLS_ENABLE="0")
    from swcompiler_b200.parallel import _find_libnccl
    if _find_libnccl():
        env["SWCB200_NCCL_LIB"] = _find_libnccl()   # the NCCL that ships with torch
    procs = [subprocess.Popen([exe], cwd=str(tmp_path), env=dict(env, SWCB200_RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.PIPE, text=True) for r in range(nranks)]
    outs = []
    try:
        for p in procs:
            outs.append(p.communicate(timeout=90))
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    for r, p in enumerate(procs):
        assert p.returncode == 0, (r, outs[r][1])
    return parse_printed(outs[0][0])


def _mnist8_files():
    d = os.path.join(GOLDEN, "mnist8")
    return {f: np.fromfile(os.path.join(d, f), dtype=np.uint8) for f in os.listdir(d)}


def test_data_parallel_mlp8_on_two_ranks(tmp_path, golden):
    got = _run_ranks("mlp8_dp2", tmp_path, _mnist8_files(), 2)
    assert got["top3"].astype(int).tolist() == golden["mnist8/top3"].tolist()
    assert np.allclose(got["data4"], golden["mnist8/probs"], atol=5.1e-4)   # strict kernels; printed with three decimals


def test_data_parallel_fused_mlp8_on_two_ranks(tmp_path, golden):
    got = _run_ranks("mlp8_dp2_fused", tmp_path, _mnist8_files(), 2)
    assert got["top3"][:, 0].astype(int).tolist() == [5, 0, 4, 1, 9, 2, 1, 3]
    assert np.abs(got["data4"] - golden["mnist8/probs"]).max() <= 2e-2


def test_model_parallel_mlp8_on_two_ranks(tmp_path, golden):
    """Transform (1 -> 0, 0 -> 1), Reduce, Scatter and Gather nodes in one forward pass."""
    got = _run_ranks("mlp8_mp2", tmp_path, _mnist8_files(), 2)
    assert got["top3"][:, 0].astype(int).tolist() == [5, 0, 4, 1, 9, 2, 1, 3]
    assert np.allclose(got["data4"], golden["mnist8/probs"], atol=6e-4)     # the second FC sums two partial products


def test_model_parallel_fc_pair_on_two_ranks(tmp_path, oracle):
    """FC1 split by output columns, ReLU on the column shards, FC2 split by input rows, partial sums joined by Reduce."""
    r = np.random.default_rng(404)
    x = r.standard_normal((64, 256)).astype(np.float32)
    w1 = (r.standard_normal((256, 512)) / 16).astype(np.float32)
    w2 = (r.standard_normal((512, 128)) / 22.6).astype(np.float32)
    got = _run_ranks("fcpair_mp2", tmp_path, {"fp_x.bin": x, "fp_w1.bin": w1, "fp_w2.bin": w2}, 2)
    want = oracle.matrixMatrixMul_f(oracle.relu_f(oracle.matrixMatrixMul_f(x, w1)), w2)
    assert np.allclose(got["y"], want, atol=6e-4)   # two partial sums instead of one k-sequential sum, three decimals printed
    # the planner's form: tensor-core GEMMs, and the Reduce done as the join over peer memory (the second GEMM's epilogue
    # stores row blocks into their owners' slots over NVLink; owners add in rank order; the master gathers the blocks)
    fused = _run_ranks("fcpair_mp2_fused", tmp_path, {"fp_x.bin": x, "fp_w1.bin": w1, "fp_w2.bin": w2}, 2)
    rb = cases.bf16_round
    part = [oracle.matrixMatrixMul_f(rb(oracle.relu_f(oracle.matrixMatrixMul_f(rb(x), rb(w1[:, c * 256:(c + 1) * 256])))),
                                     rb(w2[c * 256:(c + 1) * 256])) for c in range(2)]
    assert np.abs(fused["y"] - (part[0] + part[1])).max() <= 2e-3    # same rounding points; fp32 accumulation order differs
    assert np.abs(fused["y"] - want).max() <= 2e-2


@pytest.mark.parametrize("which", ["mlp_eval", "mlp_eval_fused"])
def test_streaming_evaluation_counts(which, tmp_path):
    from codegen_util import write_mnist8_records
    right = write_mnist8_records(str(tmp_path), wrong=(3,))
    exe = compile_emitted(which, str(tmp_path))
    r = subprocess.run([exe], capture_output=True, text=True, cwd=str(tmp_path), timeout=120)
    assert r.returncode == 0, r.stderr
    assert "batches: 2" in r.stdout
    assert parse_printed(r.stdout)["accur"].astype(int).tolist() == [[right, 8]]


def test_cuda_graph_replay_of_mlp8(tmp_path, golden):
    got = _run("mlp8_graph", tmp_path, _mnist8_files())
    assert got["top3"].astype(int).tolist() == golden["mnist8/top3"].tolist()
    assert np.allclose(got["data4"], golden["mnist8/probs"], atol=5.1e-4)


def test_cuda_graph_replay_of_the_fused_residual_block(tmp_path, oracle):
    t = resblock_inputs()
    got = _run("resblock_fused_graph", tmp_path, t)
    assert np.abs(got["probs"] - resblock_oracle(oracle, t, rnd=cases.bf16_round)).max() <= 2e-2


def test_fused_mlp8_reproduces_the_known_answer(tmp_path, golden):
    exe = compile_emitted("mlp8_fused", str(tmp_path))
    for f in os.listdir(os.path.join(GOLDEN, "mnist8")):
        shutil.copyfile(os.path.join(GOLDEN, "mnist8", f), os.path.join(tmp_path, f))
    r = subprocess.run([exe], capture_output=True, text=True, cwd=str(tmp_path), timeout=120)
    assert r.returncode == 0, r.stderr
    got = parse_printed(r.stdout)
    assert got["top3"][:, 0].astype(int).tolist() == [5, 0, 4, 1, 9, 2, 1, 3]
    assert np.abs(got["data4"] - golden["mnist8/probs"]).max() <= 2e-2     # bf16 operands, fp32 accumulation


def test_fused_convnet_matches_oracle(tmp_path, oracle):
    t = convnet_inputs()
    got = _run("convnet_fused", tmp_path, t)
    want = convnet_oracle(oracle, t)
    assert np.abs(got["probs"] - want).max() <= 2e-2


def test_resblock_strict_matches_oracle(tmp_path, oracle):
    t = resblock_inputs()
    got = _run("resblock", tmp_path, t)
    want = resblock_oracle(oracle, t)
    assert np.allclose(got["probs"], want, atol=5.1e-4)                     # printed with three decimals
    assert got["top1"][:, 0].astype(int).tolist() == oracle.argMax_i(want, 1)[:, 0].tolist()


def test_fused_resblock_matches_oracle(tmp_path, oracle):
    t = resblock_inputs()
    got = _run("resblock_fused", tmp_path, t)
    want = resblock_oracle(oracle, t, rnd=cases.bf16_round)
    assert np.abs(got["probs"] - want).max() <= 2e-2
    exact = resblock_oracle(oracle, t)
    assert np.abs(got["probs"] - exact).max() <= 5e-2
