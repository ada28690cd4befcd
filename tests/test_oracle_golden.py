"""The C oracle against the golden vectors produced by the unmodified reference
(tests/golden/make_golden.py) and against the literal known answers in the
reference's own tests.  CPU only."""
import numpy as np
import pytest

from oracle_lib import nerr

GEMM_CASES = ["g_small", "g_cuda_test", "g_odd", "g_96", "g_k1", "g_skinny1", "g_skinny8"]


def _inputs(oracle, golden, name):
    M, N, K = (int(v) for v in golden[name + "_shape"])
    return (oracle.uniform((M, K), 7), oracle.uniform((K, N), 13), oracle.uniform((N,), 29),
            oracle.uniform((M, N), 5))


def test_known_answers_from_reference_tests(oracle, golden):
    # tests/test_compute.c:162-181 and tests/test_cuda.c:169-191 of the reference
    for tag in ("kat_gemm_2x3x2", "kat_gemm_2x2"):
        c = oracle.gemm(golden[tag + "_a"], golden[tag + "_b"])
        np.testing.assert_allclose(c, golden[tag + "_c"], atol=1e-4)
    eye = np.eye(2, dtype=np.float32)
    a = np.array([[1, 2], [3, 4]], np.float32)
    np.testing.assert_array_equal(oracle.gemm(a, eye), a)   # tests/test_compute.c:183-199


@pytest.mark.parametrize("name", GEMM_CASES)
def test_gemm_family_vs_reference(oracle, golden, name):
    A, B, bias, Cin = _inputs(oracle, golden, name)
    c = oracle.gemm(A, B)
    # the reference's naive backend is the same summation order: bit-exact
    np.testing.assert_array_equal(c, golden[name + "_nn_naive"])
    # the optimised backend reorders the sum: tolerance of the reference's own
    # property test (tests/test_property.c:176-209: atol 1e-3 + rtol 1e-4)
    np.testing.assert_allclose(c, golden[name + "_nn"], atol=1e-3, rtol=1e-4)
    np.testing.assert_allclose(oracle.gemm(A, np.ascontiguousarray(B.T), tb=True), golden[name + "_nt"], atol=1e-3, rtol=1e-4)
    np.testing.assert_allclose(oracle.gemm(np.ascontiguousarray(A.T), B, ta=True), golden[name + "_tn"], atol=1e-3, rtol=1e-4)
    np.testing.assert_allclose(oracle.bias_act(c, bias, "relu"), golden[name + "_relu"], atol=1e-3, rtol=1e-4)
    np.testing.assert_allclose(oracle.bias_act(c, bias, "gelu"), golden[name + "_gelu"], atol=1e-3, rtol=1e-4)
    np.testing.assert_allclose(oracle.gemm_ex(A, B, 0.5, 2.0, Cin), golden[name + "_ex"], atol=1e-3, rtol=1e-4)
    assert nerr(c, golden[name + "_nn"]) < 1e-5


def test_gelu_vs_reference(oracle, golden):
    # the reference's SIMD tanh is a polynomial: ~1e-6 absolute from libm
    np.testing.assert_allclose(oracle.gelu(golden["gelu_x"]), golden["gelu_y"], atol=2e-6)


@pytest.mark.parametrize("shape", [(1, 8, 8), (4, 16, 32), (8, 64, 128), (32, 128, 512), (16, 256, 1024)])
def test_quantiser_and_w8a32_vs_reference(oracle, golden, shape):
    M, N, K = shape
    tag = f"q_{M}_{N}_{K}"
    a, w = oracle.uniform((M, K), 7), oracle.uniform((N, K), 13)
    q, s = oracle.quantize_rows(w)
    np.testing.assert_array_equal(s, golden[tag + "_scales"])           # bit-exact scales
    if tag + "_q" in golden.files:
        np.testing.assert_array_equal(q, golden[tag + "_q"])            # bit-exact int8 rows
    sums = np.array([int(q.astype(np.int64).sum()), int(np.abs(q.astype(np.int64)).sum())])
    np.testing.assert_array_equal(sums, golden[tag + "_qsum"])
    # round trip within 1.5 quantisation steps (tests/test_quantize.c:37-69)
    assert np.all(np.abs(oracle.dequantize_rows(q, s) - w) <= 1.5 * s[:, None])
    out = oracle.qgemm_w8a32(a, q, s)
    ref = golden[tag + "_out"]
    diff = np.abs(out - ref)
    rel = diff / (np.abs(ref) + 1e-5)
    assert not np.any((diff > 1e-2) & (rel > 1e-3))                     # tests/test_quantize.c:109-113
    assert nerr(out, ref) < 1e-5


@pytest.mark.parametrize("name", ["s_test", "s_c4like"])
@pytest.mark.parametrize("causal", [0, 1])
def test_sdpa_vs_reference(oracle, golden, name, causal):
    BH, S, dk = (int(v) for v in golden[name + "_shape"])
    scale = float(golden[name + "_scale"][0])
    Q, K, V = oracle.normal((BH, S, dk), 41), oracle.normal((BH, S, dk), 43), oracle.normal((BH, S, dk), 47)
    O, L = oracle.sdpa_fwd(Q, K, V, scale, causal)
    # tests/test_attention.c:54-131 use max-abs < 1e-4
    assert np.abs(O - golden[f"{name}_c{causal}_O"]).max() < 1e-4
    assert np.abs(L - golden[f"{name}_c{causal}_L"]).max() < 1e-4
    O64, L64 = oracle.sdpa_fwd_f64(Q, K, V, scale, causal)
    assert np.abs(O - O64).max() < 1e-5 and np.abs(L - L64).max() < 1e-5


def test_w8a8_known_answers(oracle, golden):
    for i in range(3):
        a, b, bs = golden[f"w8a8_{i}_a"], golden[f"w8a8_{i}_b"], golden[f"w8a8_{i}_bs"]
        a_scale, out_scale = (float(v) for v in golden[f"w8a8_{i}_scales"])
        acc, q = oracle.qgemm_w8a8(a, a_scale, b, bs, out_scale)
        np.testing.assert_array_equal(acc, golden[f"w8a8_{i}_acc"])
        np.testing.assert_array_equal(q, golden[f"w8a8_{i}_q"])
    # ties go to even, clamp at +-127: acc * 0.5 with a_scale*b_scale/out_scale == 0.5
    acc = golden["w8a8_tie_acc"]
    a = np.zeros((1, 16), np.int8)
    # build operands whose products are the wanted accumulators: a = [v,0,..], b_n = [1,0,..] * sign
    outs = []
    for v in acc[0]:
        k = 16
        av = np.zeros((1, k), np.int8); bv = np.zeros((1, k), np.int8)
        rem, j = int(v), 0
        while rem != 0:
            step = max(-127, min(127, rem))
            av[0, j], bv[0, j] = step, 1
            rem -= step; j += 1
        accv, qv = oracle.qgemm_w8a8(av, 1.0, bv, np.array([0.5], np.float32), 1.0)
        assert int(accv[0, 0]) == int(v)
        outs.append(int(qv[0, 0]))
    np.testing.assert_array_equal(np.array(outs, np.int8), golden["w8a8_tie_q"][0])


def test_oracle_matches_live_reference(oracle, reference):
    """Where the compiled reference is present, re-check a mid-size case live."""
    A, B = oracle.uniform((130, 257), 7), oracle.uniform((257, 70), 13)
    np.testing.assert_array_equal(oracle.gemm(A, B), reference.gemm(A, B, backend="naive"))
    assert nerr(oracle.gemm(A, B), reference.gemm(A, B)) < 1e-5
    W = oracle.uniform((70, 257), 13)
    q, s = oracle.quantize_rows(W)
    q2, s2 = reference.quantize(W)
    np.testing.assert_array_equal(q, q2)
    np.testing.assert_array_equal(s, s2)
