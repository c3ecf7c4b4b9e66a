"""CPU: the C restatement against the reference's golden outputs, its known-answer fixture,
and (where the prebuilt reference library is present) the live reference, bit for bit."""
import numpy as np
import pytest

import cases
from conftest import bits
from oracle import oracle as orc


def test_restatement_matches_reference_golden_bit_exact(oracle, golden):
    got = cases.run_all(oracle)
    assert set(got) <= set(golden)
    for k, v in got.items():
        assert v.shape == golden[k].shape, k
        assert np.array_equal(bits(v), bits(golden[k])), k


def test_mnist8_known_answer(oracle, golden, mnist8):
    probs = oracle.mlp_forward(mnist8["x"], mnist8["w0"], mnist8["b0"], mnist8["w1"], mnist8["b1"])
    top3 = oracle.argMax_i(probs, 3)
    # the reference's own pinned result: test/input/mnist_images_8.meta.txt
    assert top3[:, 0].tolist() == mnist8["labels"].tolist() == [5, 0, 4, 1, 9, 2, 1, 3]
    assert np.array_equal(bits(probs), bits(golden["mnist8/probs"]))
    assert np.array_equal(top3, golden["mnist8/top3"])


def test_config_slices_match_reference_golden(oracle, golden):
    p = cases.lenet_forward(oracle, cases.config2_lenet(batch=4))
    assert np.array_equal(bits(p), bits(golden["config2_b4/probs"]))
    o = cases.res_stage_forward(oracle, cases.config5_res_stage(batch=1, hw=12, blocks=1))
    assert np.array_equal(bits(o), bits(golden["config5_b1_hw12/out"]))


@pytest.mark.skipif(not orc.Reference.available(), reason="prebuilt reference library not present")
def test_restatement_matches_live_reference(oracle):
    ref = orc.Reference()
    a, b = cases.run_all(oracle), cases.run_all(ref)
    for k in a:
        assert np.array_equal(bits(a[k]), bits(b[k])), k
    c = cases.config3_wide_mlp(batch=4, width=256, classes=100, layers=2)
    assert np.array_equal(bits(cases.wide_mlp_forward(oracle, c)), bits(cases.wide_mlp_forward(ref, c)))


def test_thread_count_does_not_change_results(oracle):
    c = cases.matmul_cases()["mm_130x70x257"]
    n = oracle.threads
    oracle.set_threads(1)
    one = oracle.matrixMatrixMul_f(c["a"], c["b"])
    oracle.set_threads(max(n, 2))
    many = oracle.matrixMatrixMul_f(c["a"], c["b"])
    oracle.set_threads(n)
    assert np.array_equal(bits(one), bits(many))


def test_semantics_spelled_out(oracle):
    # ArgMax: equal values -> higher index first (std::greater on (value, index) pairs)
    assert oracle.argMax_i(np.array([[1, 3, 3, 0]], np.float32), 3).tolist() == [[2, 1, 0]]
    # ReLU: NaN and -0 become +0
    r = oracle.relu_f(np.array([np.nan, -0.0, -1, 2], np.float32))
    assert bits(r).tolist() == [0, 0, 0, np.float32(2).view(np.uint32)]
    # MaxPool: padded taps never count; a window wholly in the padding gives 0
    x = -np.ones((1, 2, 2, 1), np.float32)
    o = oracle.maxpool_f(x, (2, 2), (3, 3), (2, 2, 2, 2))
    assert o.shape == (1, 2, 2, 1) and o.reshape(-1).tolist() == [0, 0, 0, -1]
    # AvgPool divides by the full window even when taps are padding
    a = oracle.avgpool_f(np.ones((1, 2, 2, 1), np.float32), (2, 2), (1, 1), (1, 1, 1, 1))
    assert a[0, 0, 0, 0] == 0.25 and a[0, 1, 1, 0] == 1.0
    # bf16 rounding helper: ties to even
    assert cases.bf16_round(np.array([1.00390625], np.float32))[0] == 1.0  # 1 + 2^-8 -> tie -> even
