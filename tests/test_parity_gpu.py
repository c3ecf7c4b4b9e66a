"""GPU: every kernel of the C-ABI library against the CPU oracle and the reference's golden outputs,
on the seeded cases of tests/cases.py.

Bars: bit-exact for the strict matmul and convolution, bias-add, ReLU, add, MaxPool, AvgPool, ArgMax
and the transposes; |d| <= 1e-5*|ref| + 1e-6 for tanh (its formula cancels near zero, so a pure
relative bound cannot hold against a different but correct expf) and 1e-5 relative for softmax and
batch-norm."""
import numpy as np
import pytest
import torch

import cases
from conftest import bits

pytestmark = pytest.mark.gpu

EXACT_SUFFIX = ("/badd", "/relu", "/add", "/max", "/avg")


@pytest.fixture(scope="module")
def gpu():
    from gpu_impl import GpuImpl
    return GpuImpl()


@pytest.fixture(scope="module")
def gpu_out(gpu):
    return cases.run_all(gpu, accuracy=False)   # the accuracy counters have a test of their own below


def _kind(name):
    if name.endswith("/tanh"):
        return "tanh"
    if name.endswith("/softmax") or name.startswith("bn_"):
        return "rel"
    return "exact"


def test_all_cases_against_reference_golden(gpu_out, golden):
    assert set(gpu_out) <= set(golden)
    for k, v in gpu_out.items():
        ref = golden[k]
        assert v.shape == ref.shape and v.dtype == ref.dtype, k
        kind = _kind(k)
        if kind == "exact":
            assert np.array_equal(bits(v), bits(ref)), k
        elif kind == "tanh":
            both_nan = np.isnan(v) & np.isnan(ref)
            assert np.all(both_nan | (np.abs(v - ref) <= 1e-5 * np.abs(ref) + 1e-6)), k
        else:
            both_nan = np.isnan(v) & np.isnan(ref)
            assert np.all(both_nan | (np.abs(v - ref) <= 1e-5 * np.abs(ref) + 1e-30)), k


def test_accuracy_counters(gpu, golden):
    """swcb200_accuracy_i against the reference's accuracy_i: integer counters, bit for bit, also when accumulated
    over two batches."""
    for k, c in cases.accuracy_cases().items():
        assert np.array_equal(gpu.accuracy_i(c["pred"], c["label"]), golden[k]), k
    c = cases.accuracy_cases()["acc_1000x3"]
    first = gpu.accuracy_i(c["pred"][:400], c["label"][:400])
    both = gpu.accuracy_i(c["pred"][400:], c["label"][400:], accum=first)
    assert np.array_equal(both, golden["acc_1000x3"])


def test_all_cases_against_oracle(gpu_out, oracle):
    ref = cases.run_all(oracle, accuracy=False)
    for k, v in gpu_out.items():
        if _kind(k) == "exact":
            assert np.array_equal(bits(v), bits(ref[k])), k


def test_how_close_the_tolerance_cases_really_are(gpu_out, golden):
    """Batch-norm is expected to agree bit for bit almost everywhere (double arithmetic, one rounding);
    softmax sums in a different order (shuffle tree against left-to-right) and stays within a few tens of ulp."""
    for k, v in gpu_out.items():
        if _kind(k) == "exact":
            continue
        ref = golden[k]
        if k.startswith("bn_"):
            assert np.mean(bits(v) == bits(ref)) >= 0.999, k
        elif k.endswith("/softmax"):
            ok = np.isfinite(ref) & (ref > 1e-30)
            ulps = np.abs(v[ok].view(np.int32).astype(np.int64) - ref[ok].view(np.int32).astype(np.int64))
            assert ulps.max(initial=0) <= 64, (k, int(ulps.max()))  # 1e-5 relative is ~84 ulp


def test_mnist8_known_answer(gpu, golden, mnist8):
    probs = gpu.mlp_forward(mnist8["x"], mnist8["w0"], mnist8["b0"], mnist8["w1"], mnist8["b1"])
    top3 = gpu.argMax_i(probs, 3)
    assert top3[:, 0].tolist() == [5, 0, 4, 1, 9, 2, 1, 3]
    assert np.array_equal(top3, golden["mnist8/top3"])
    assert np.allclose(probs, golden["mnist8/probs"], rtol=1e-5, atol=1e-7)


def test_config1_mlp_whole(gpu, oracle):
    c = cases.config1_mlp()
    want = oracle.mlp_forward(c["x"], c["w0"], c["b0"], c["w1"], c["b1"])
    got = gpu.mlp_forward(c["x"], c["w0"], c["b0"], c["w1"], c["b1"])
    assert np.allclose(got, want, rtol=1e-5, atol=1e-7)
    assert np.array_equal(gpu.argMax_i(got, 1), oracle.argMax_i(want, 1))
    # the hidden pre-activations (FC + bias) are bit-exact
    assert np.array_equal(bits(gpu.fc(c["x"], c["w0"], c["b0"])), bits(oracle.fc(c["x"], c["w0"], c["b0"])))


def test_config2_lenet_whole(gpu, oracle, golden):
    c = cases.config2_lenet()
    want = cases.lenet_forward(oracle, c)
    got = cases.lenet_forward(gpu, c)
    assert np.allclose(got, want, rtol=1e-5, atol=1e-7)
    assert np.array_equal(gpu.argMax_i(got, 1), oracle.argMax_i(want, 1))
    c4 = cases.config2_lenet(batch=4)
    assert np.allclose(cases.lenet_forward(gpu, c4), golden["config2_b4/probs"], rtol=1e-5, atol=1e-7)


def test_config5_res_stage_slice_strict(gpu, oracle, golden):
    c = cases.config5_res_stage(batch=1, hw=12, blocks=1)
    got = cases.res_stage_forward(gpu, c)
    assert np.allclose(got, golden["config5_b1_hw12/out"], rtol=1e-5, atol=1e-6)
    c = cases.config5_res_stage(batch=2, hw=56, blocks=3)  # two images of the stated stage
    want = cases.res_stage_forward(oracle, c)
    got = cases.res_stage_forward(gpu, c)
    assert np.allclose(got, want, rtol=1e-5, atol=1e-5)


def test_strict_matmul_with_leading_dimensions(gpu, oracle):
    """lda/ldb/ldc larger than the logical widths, as a column-sharded operand would have."""
    r = np.random.default_rng(5)
    a = r.standard_normal((70, 100)).astype(np.float32)
    b = r.standard_normal((90, 130)).astype(np.float32)
    be = gpu.be
    ta, tb = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    tc = torch.zeros((70, 140), dtype=torch.float32, device="cuda")
    import ctypes as C
    be._call("matrixMatrixMul_f", C.c_int(70), C.c_int(120), C.c_int(90), C.c_void_p(ta.data_ptr()), C.c_int(100),
             C.c_void_p(tb.data_ptr()), C.c_int(130), C.c_void_p(tc.data_ptr()), C.c_int(140))
    be.sync()
    want = oracle.matrixMatrixMul_f(np.ascontiguousarray(a[:, :90]), np.ascontiguousarray(b[:, :120]))
    assert np.array_equal(bits(tc.cpu().numpy()[:, :120]), bits(want))
    assert np.all(tc.cpu().numpy()[:, 120:] == 0)


def test_error_reporting(gpu):
    import swcompiler_b200 as swc
    x = torch.zeros((1, 4, 4, 4), device="cuda")
    w = torch.zeros((4, 3, 3, 2), device="cuda")
    b = torch.zeros(4, device="cuda")
    with pytest.raises(swc.SwcError) as e:
        gpu.be.conv2d_f(x, w, b, (3, 3), (1, 1), (1, 1, 1, 1), group=2)
    assert e.value.status == swc._lib.ERR_UNSUPPORTED
    with pytest.raises(swc.SwcError) as e:
        gpu.be.argMax_i(torch.zeros((2, 3), device="cuda"), 4)
    assert e.value.status == swc._lib.ERR_BAD_SHAPE
    # empty inputs are accepted and launch nothing
    n0 = gpu.be.launches
    gpu.be.relu_f(torch.zeros(0, device="cuda"))
    gpu.be.matrixSoftmax_f(torch.zeros((0, 5), device="cuda"))
    assert gpu.be.launches == n0


@pytest.mark.parametrize("n", [1 << 24, (1 << 24) + 3])
def test_bandwidth_kernels_at_size(gpu, n):
    """64 MiB vectors (beyond nothing the oracle cannot do in a second): exact against numpy's IEEE ops."""
    r = np.random.default_rng(9)
    a = r.standard_normal(n).astype(np.float32)
    b = r.standard_normal(n).astype(np.float32)
    assert np.array_equal(gpu.relu_f(a), np.where(a > 0, a, np.float32(0)))
    assert np.array_equal(gpu.vecAdd_f(a, b), a + b)


def test_top1_argmax_fast_path_against_oracle(gpu, oracle):
    """top_k = 1 on rows of whole float4 (the vectorised kernel): random rows at the three register budgets, and rows of
    quantised values where equal maxima are the rule, so that 'the higher index wins' is exercised in every lane."""
    r = np.random.default_rng(41)
    for (m, n) in [(300, 1000), (64, 512), (17, 256), (9, 128), (5, 1024)]:
        x = r.standard_normal((m, n)).astype(np.float32)
        assert np.array_equal(gpu.argMax_i(x, 1), oracle.argMax_i(x, 1)), (m, n)
        q = np.round(r.random((m, n)) * 3).astype(np.float32)
        q[0, :] = 2.0                    # a whole row of equal values: the last index
        q[m - 1, ::7] = -0.0
        assert np.array_equal(gpu.argMax_i(q, 1), oracle.argMax_i(q, 1)), (m, n)
    assert gpu.argMax_i(np.full((2, 128), 2.0, np.float32), 1).tolist() == [[127], [127]]


def test_maxpool_on_bf16_storage_against_oracle(gpu, oracle):
    """MaxPool on bf16 tensors: the maxima of bf16 values are bf16 values, so the result must equal the oracle's
    maxpool_f on the same (bf16-representable) numbers bit for bit -- the 2x2/2 fast path (even and odd extents,
    ties, signed zeros, all-negative windows) and the general kernel (padding, 3x3, stride 1)."""
    r = np.random.default_rng(43)
    spec = [((2, 56, 56, 64), (2, 2), (2, 2), (0, 0, 0, 0)), ((1, 8, 8, 64), (2, 2), (2, 2), (0, 0, 0, 0)),
            ((3, 7, 9, 8), (2, 2), (2, 2), (0, 0, 0, 0)), ((1, 6, 6, 24), (2, 2), (2, 2), (0, 0, 0, 0)),
            ((2, 9, 7, 16), (3, 3), (2, 2), (1, 1, 1, 1)), ((1, 5, 6, 8), (3, 2), (1, 1), (1, 0, 1, 0)),
            ((1, 6, 6, 5), (2, 2), (2, 2), (0, 0, 0, 0))]
    for idims, k, s, p in spec:
        for kind in ("normal", "ties"):
            x = r.standard_normal(idims) if kind == "normal" else np.round(r.random(idims) * 3) - 4
            x = cases.bf16_round(x.astype(np.float32))
            if kind == "ties":
                x[0, 0, :2, :] = np.float32(-0.0)
                x[0, 1, :2, :] = np.float32(0.0)
            want = oracle.maxpool_f(x, k, s, p)
            got = gpu.be.maxpool_bf16(torch.from_numpy(x).cuda().to(torch.bfloat16), k, s, p)
            gpu.be.sync()
            assert np.array_equal(bits(got.float().cpu().numpy()), bits(want)), (idims, k, s, p, kind)
