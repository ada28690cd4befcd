"""Parity of the CUDA path with the CPU oracle, through the C ABI.

Integer work (int32 accumulators, requantised int8, the row quantiser) must be
bit-exact.  fp32 results are held to the normalised error
max|gpu - ref| / max|ref| <= 1e-5 in the split-precision modes and <= 5e-3 in
bf16 mode, against a double-precision restatement, and to the reference's own
test tolerances against its golden outputs.
"""
import numpy as np
import pytest
import torch

from oracle_lib import nerr

pytestmark = pytest.mark.gpu

TOL_SPLIT = 1e-5
TOL_BF16 = 5e-3


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def host(t):
    return t.cpu().numpy()


def run_gemm(engine, A, B, variant="nn"):
    M = A.shape[1] if variant == "tn" else A.shape[0]
    N = B.shape[0] if variant == "nt" else B.shape[1]
    out = torch.full((M, N), float("nan"), device="cuda")
    engine.gemm(dev(A), dev(B), out, variant)
    return host(out)


def test_known_answers(engine, golden):
    for tag in ("kat_gemm_2x3x2", "kat_gemm_2x2"):
        np.testing.assert_allclose(run_gemm(engine, golden[tag + "_a"], golden[tag + "_b"]), golden[tag + "_c"], atol=1e-4)


@pytest.mark.parametrize("name", ["g_small", "g_cuda_test", "g_odd", "g_96", "g_k1", "g_skinny1", "g_skinny8"])
def test_gemm_family_vs_golden(engine, oracle, golden, name):
    M, N, K = (int(v) for v in golden[name + "_shape"])
    A, B, bias, Cin = oracle.uniform((M, K), 7), oracle.uniform((K, N), 13), oracle.uniform((N,), 29), oracle.uniform((M, N), 5)
    tol = dict(atol=1e-3, rtol=1e-4)   # the reference's property-test tolerance
    np.testing.assert_allclose(run_gemm(engine, A, B), golden[name + "_nn"], **tol)
    np.testing.assert_allclose(run_gemm(engine, A, np.ascontiguousarray(B.T), "nt"), golden[name + "_nt"], **tol)
    np.testing.assert_allclose(run_gemm(engine, np.ascontiguousarray(A.T), B, "tn"), golden[name + "_tn"], **tol)
    out = torch.empty((M, N), device="cuda")
    engine.gemm_relu(dev(A), dev(B), dev(bias), out)
    np.testing.assert_allclose(host(out), golden[name + "_relu"], **tol)
    engine.gemm_bias_act(dev(A), dev(B), dev(bias), out, M, N, K, act="gelu")
    np.testing.assert_allclose(host(out), golden[name + "_gelu"], **tol)
    c = dev(Cin)
    engine.gemm_ex(dev(A), dev(B), 0.5, 2.0, c)
    np.testing.assert_allclose(host(c), golden[name + "_ex"], **tol)


@pytest.mark.parametrize("seed", range(24))
def test_gemm_property_small_shapes(engine, oracle, seed):
    # mirrors tests/test_property.c:176-209 of the reference: 1 <= M,N,K <= 96, U[-2,2]
    rng = np.random.RandomState(1000 + seed)
    M, N, K = (int(v) for v in rng.randint(1, 97, size=3))
    A, B = 2 * oracle.uniform((M, K), 11 + seed), 2 * oracle.uniform((K, N), 77 + seed)
    ref = oracle.gemm(A, B)
    for variant, a, b in (("nn", A, B), ("nt", A, np.ascontiguousarray(B.T)), ("tn", np.ascontiguousarray(A.T), B)):
        np.testing.assert_allclose(run_gemm(engine, a, b, variant), ref, atol=1e-3, rtol=1e-4)


@pytest.mark.parametrize("shape", [(128, 256, 32), (129, 257, 33), (300, 520, 1000), (257, 64, 4100), (1024, 1024, 1024)])
@pytest.mark.parametrize("mode", ["3xtf32", "bf16x3", "bf16"])
def test_gemm_modes_normalised_error(engine, oracle, shape, mode):
    M, N, K = shape
    A, B = oracle.uniform((M, K), 7), oracle.uniform((K, N), 13)
    ref64 = oracle.gemm_f64(A, B)
    engine.set_fp32_mode(mode)
    try:
        got = run_gemm(engine, A, B)
    finally:
        engine.set_fp32_mode("3xtf32")
    assert np.isfinite(got).all()
    assert nerr(got, ref64) <= (TOL_BF16 if mode == "bf16" else TOL_SPLIT), (mode, nerr(got, ref64))


def test_config1_dense_relu_1024(engine, oracle):
    """benchmark config 1: C = ReLU(A.B + bias), M=N=K=1024, U[-1,1] seeds 7/13/29."""
    A, B, bias = oracle.uniform((1024, 1024), 7), oracle.uniform((1024, 1024), 13), oracle.uniform((1024,), 29)
    ref = oracle.bias_act(oracle.gemm(A, B), bias, "relu")
    ref64 = np.maximum(oracle.gemm_f64(A, B) + bias.astype(np.float64), 0)
    out = torch.empty((1024, 1024), device="cuda")
    engine.gemm_relu(dev(A), dev(B), dev(bias), out)
    got = host(out)
    assert nerr(got, ref64) <= TOL_SPLIT
    assert nerr(got, ref) <= TOL_SPLIT
    np.testing.assert_allclose(got, ref, atol=1e-3, rtol=1e-4)


def test_gemm_is_bitwise_deterministic(engine, oracle):
    # tests/test_optimization_paths.c:265-295 of the reference: 10 runs, identical bits
    A, B = oracle.uniform((200, 300), 3), oracle.uniform((300, 170), 4)
    first = run_gemm(engine, A, B)
    for _ in range(9):
        np.testing.assert_array_equal(run_gemm(engine, A, B), first)


def test_gemm_edge_values(engine):
    # tests/test_numerical_edge.c:310-372: zeros, large values, K = 1
    z = np.zeros((7, 9), np.float32)
    np.testing.assert_array_equal(run_gemm(engine, z, np.zeros((9, 5), np.float32)), np.zeros((7, 5), np.float32))
    big = np.full((40, 64), 1e18, np.float32)
    got = run_gemm(engine, big, np.full((64, 40), 1e18, np.float32))
    np.testing.assert_allclose(got, np.full((40, 40), 64e36, np.float32), rtol=1e-5)
    a = np.arange(1, 41, dtype=np.float32).reshape(40, 1)
    b = np.arange(1, 51, dtype=np.float32).reshape(1, 50)
    np.testing.assert_allclose(run_gemm(engine, a, b), a @ b, rtol=1e-6)


def test_empty_shapes(engine):
    out = torch.zeros((0, 5), device="cuda")
    engine.gemm(torch.zeros((0, 3), device="cuda"), torch.zeros((3, 5), device="cuda"), out)
    out = torch.full((4, 5), 7.0, device="cuda")
    engine.gemm(torch.zeros((4, 0), device="cuda"), torch.zeros((0, 5), device="cuda"), out)
    np.testing.assert_array_equal(host(out), np.zeros((4, 5), np.float32))


def test_null_and_bad_arguments(engine):
    from axiom_b200.engine import EngineError
    a = torch.zeros((4, 4), device="cuda")
    with pytest.raises(EngineError) as e:
        engine.gemm(a, a, None)
    assert e.value.status == 1                      # AX_ERR_NULL_ARG
    with pytest.raises(EngineError) as e:
        engine.bias_add(a, a[0], 2, a)
    assert e.value.status == 5                      # AX_ERR_INVALID_AXIS


@pytest.mark.parametrize("M", [1, 2, 5, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("NK", [(4096, 4096), (1000, 777), (130, 257), (1000, 1028), (128, 256), (4100, 520), (512, 8192)])
def test_skinny_route(engine, oracle, M, NK):
    """benchmark config 2 (x[M,4096].W[4096,4096] + bias -> GELU, M in {1,8,32}) and ragged shapes.  M <= 8 runs the
    fp32-FMA kernels, 9..32 the tensor-core kernel when N and K are multiples of 4 (else the FMA kernels again)."""
    N, K = NK
    x = oracle.normal((M, K), 31)
    W = oracle.normal((K, N), 13, sigma=1.0 / np.sqrt(K))
    bias = oracle.uniform((N,), 29)
    pre64 = oracle.gemm_f64(x, W) + bias.astype(np.float64)
    ref = oracle.bias_act(oracle.gemm(x, W), bias, "gelu")
    out = torch.empty((M, N), device="cuda")
    xd, Wd, bd = dev(x), dev(W), dev(bias)
    engine.gemm_bias_act(xd, Wd, bd, out, M, N, K, act="gelu")
    got = host(out)
    assert nerr(got, ref) <= TOL_SPLIT
    ref64 = 0.5 * pre64 * (1 + np.tanh(0.7978845608028654 * (pre64 + 0.044715 * pre64 ** 3)))
    assert nerr(got, ref64) <= TOL_SPLIT
    # bitwise run-to-run determinism of the split-K reduction
    out2 = torch.empty((M, N), device="cuda")
    for _ in range(3):
        engine.gemm_bias_act(xd, Wd, bd, out2, M, N, K, act="gelu")
        np.testing.assert_array_equal(host(out2), got)
    # plain gemm / alpha-beta forms of the same route
    c = dev(oracle.uniform((M, N), 5))
    cin = host(c).copy()
    engine.gemm_ex(xd, Wd, 0.5, 2.0, c)
    assert nerr(host(c), 0.5 * oracle.gemm_f64(x, W) + 2.0 * cin) <= TOL_SPLIT


def test_elementwise_slots(engine, oracle, golden):
    X, bias_n, bias_m = oracle.uniform((37, 52), 3), oracle.uniform((52,), 4), oracle.uniform((37,), 6)
    out = torch.empty((37, 52), device="cuda")
    np.testing.assert_array_equal(host(engine.bias_add(dev(X), dev(bias_n), 1, out)), oracle.bias_add_axis(X, bias_n, 1))
    np.testing.assert_array_equal(host(engine.bias_add(dev(X), dev(bias_m), 0, out)), oracle.bias_add_axis(X, bias_m, 0))
    xd = dev(X)
    engine.bias_add(xd, dev(bias_n), 1, xd)          # out may alias in
    np.testing.assert_array_equal(host(xd), oracle.bias_add_axis(X, bias_n, 1))
    np.testing.assert_array_equal(host(engine.relu(dev(X), out)), oracle.relu(X))
    # any rank, any axis (the stock backend's rule, src/compute/backends/cuda/ops_fused.cu:268-292)
    X3 = oracle.uniform((5, 7, 12), 8)
    for axis in (0, 1, 2):
        b = oracle.uniform((X3.shape[axis],), 9 + axis)
        o3 = torch.empty(X3.shape, device="cuda")
        shape = [1, 1, 1]
        shape[axis] = -1
        np.testing.assert_array_equal(host(engine.bias_add_nd(dev(X3), dev(b), axis, o3)), X3 + b.reshape(shape))
    gx = golden["gelu_x"]
    g = torch.empty(gx.shape, device="cuda")
    np.testing.assert_allclose(host(engine.gelu(dev(gx), g)), golden["gelu_y"], atol=2e-6)
    np.testing.assert_allclose(host(g), oracle.gelu(gx), atol=1e-6)


def test_w8a8_known_answers_bit_exact(engine, golden):
    for i in range(3):
        a, b, bs = golden[f"w8a8_{i}_a"], golden[f"w8a8_{i}_b"], golden[f"w8a8_{i}_bs"]
        a_scale, out_scale = (float(v) for v in golden[f"w8a8_{i}_scales"])
        M, N = a.shape[0], b.shape[0]
        q = torch.zeros((M, N), dtype=torch.int8, device="cuda")
        acc = torch.zeros((M, N), dtype=torch.int32, device="cuda")
        engine.qgemm_w8a8(dev(a), a_scale, dev(b), dev(bs), out_scale, q, acc)
        np.testing.assert_array_equal(host(acc), golden[f"w8a8_{i}_acc"])
        np.testing.assert_array_equal(host(q), golden[f"w8a8_{i}_q"])


@pytest.mark.parametrize("shape", [(512, 4096, 4096), (130, 200, 1000), (128, 256, 128), (1, 64, 48), (300, 33, 4112)])
def test_w8a8_bit_exact_vs_oracle(engine, oracle, shape):
    """benchmark config 3 first: A int8 [512,4096], B int8 [4096,4096], scales U[0.001,0.02]."""
    M, N, K = shape
    a, b = oracle.int8((M, K), 7), oracle.int8((N, K), 13)
    bs = oracle.frange((N,), 17, 0.001, 0.02)
    a_scale = 0.02
    # acc has std ~ 5373*sqrt(K) (two U{-127..127} factors): scale so outputs span the int8 range, few saturate
    out_scale = float(a_scale * 0.0105 * 5373.0 * np.sqrt(K) / 50.0)
    acc_ref, q_ref = oracle.qgemm_w8a8(a, a_scale, b, bs, out_scale)
    q = torch.zeros((M, N), dtype=torch.int8, device="cuda")
    acc = torch.zeros((M, N), dtype=torch.int32, device="cuda")
    engine.qgemm_w8a8(dev(a), a_scale, dev(b), dev(bs), out_scale, q, acc)
    np.testing.assert_array_equal(host(acc), acc_ref)
    np.testing.assert_array_equal(host(q), q_ref)
    assert 0.001 < np.mean(np.abs(q_ref.astype(np.int32)) == 127) < 0.2 or M * N < 1000
    # each output alone
    q2 = torch.zeros_like(q)
    engine.qgemm_w8a8(dev(a), a_scale, dev(b), dev(bs), out_scale, q2, None)
    np.testing.assert_array_equal(host(q2), q_ref)
    acc2 = torch.zeros_like(acc)
    engine.qgemm_w8a8(dev(a), a_scale, dev(b), None, 1.0, None, acc2)
    np.testing.assert_array_equal(host(acc2), acc_ref)


@pytest.mark.parametrize("shape", [(8, 8), (128, 128), (64, 1024), (33, 1001)])
def test_quantize_rows_bit_exact(engine, oracle, shape):
    N, K = shape
    W = oracle.uniform((N, K), 42)
    W[N // 2] = 0.0                                   # an all-zero row takes scale 1
    q_ref, s_ref = oracle.quantize_rows(W)
    q = torch.zeros((N, K), dtype=torch.int8, device="cuda")
    s = torch.zeros((N,), device="cuda")
    engine.quantize_rows(dev(W), q, s)
    np.testing.assert_array_equal(host(s), s_ref)
    np.testing.assert_array_equal(host(q), q_ref)


@pytest.mark.parametrize("shape", [(1, 8, 8), (4, 16, 32), (8, 64, 128), (32, 128, 512), (16, 256, 1024), (512, 1024, 1024),
                                   (1, 4096, 4096), (3, 1000, 2048), (8, 4096, 4096), (512, 4096, 4096)])
def test_w8a32_vs_oracle_and_golden(engine, oracle, golden, shape):
    M, N, K = shape
    a, w = oracle.uniform((M, K), 7), oracle.uniform((N, K), 13)
    q, s = oracle.quantize_rows(w)
    out = torch.empty((M, N), device="cuda")
    engine.qgemm_w8a32(dev(a), dev(q), dev(s), out)
    got = host(out)
    # axiom's own argument list (a, qw, out, M) with a host ax_qweight_t-layout struct: the same call
    out_qw = torch.full((M, N), float("nan"), device="cuda")
    engine.qgemm_w8a32_qw(dev(a), dev(q), dev(s), out_qw)
    np.testing.assert_array_equal(host(out_qw), got)
    assert nerr(got, oracle.qgemm_w8a32_f64(a, q, s)) <= TOL_SPLIT
    tag = f"q_{M}_{N}_{K}_out"
    ref = golden[tag] if tag in golden.files else oracle.qgemm_w8a32(a, q, s)
    diff = np.abs(got - ref)
    rel = diff / (np.abs(ref) + 1e-5)
    assert not np.any((diff > 1e-2) & (rel > 1e-3))   # tests/test_quantize.c:109-113


@pytest.mark.parametrize("name", ["s_test", "s_c4like"])
@pytest.mark.parametrize("causal", [0, 1])
def test_sdpa_vs_golden(engine, oracle, golden, name, causal):
    BH, S, dk = (int(v) for v in golden[name + "_shape"])
    scale = float(golden[name + "_scale"][0])
    Q, K, V = oracle.normal((BH, S, dk), 41), oracle.normal((BH, S, dk), 43), oracle.normal((BH, S, dk), 47)
    O = torch.full((BH, S, dk), float("nan"), device="cuda")
    L = torch.full((BH, S), float("nan"), device="cuda")
    engine.sdpa_fwd(dev(Q), dev(K), dev(V), O, L, scale, causal)
    assert np.abs(host(O) - golden[f"{name}_c{causal}_O"]).max() < 1e-4   # tests/test_attention.c:54-131
    assert np.abs(host(L) - golden[f"{name}_c{causal}_L"]).max() < 1e-4
    O2 = torch.empty_like(O)
    engine.sdpa_fwd(dev(Q), dev(K), dev(V), O2, None, scale, causal)       # L is optional
    np.testing.assert_array_equal(host(O2), host(O))


@pytest.mark.parametrize("shape", [(4, 1024, 64), (2, 333, 64), (3, 200, 128), (2, 129, 40), (5, 64, 16),
                                   (3, 300, 16), (2, 256, 32), (2, 200, 6), (2, 1000, 24), (1, 128, 4), (2, 640, 60), (1, 513, 72)])
@pytest.mark.parametrize("causal", [0, 1])
def test_sdpa_vs_oracle(engine, oracle, shape, causal):
    """benchmark config 4 per-head shape (S=1024, dk=64, scale 1/8, causal) on a few heads, plus ragged ones."""
    BH, S, dk = shape
    Q, K, V = oracle.normal((BH, S, dk), 41), oracle.normal((BH, S, dk), 43), oracle.normal((BH, S, dk), 47)
    scale = 1.0 / np.sqrt(dk)
    O64, L64 = oracle.sdpa_fwd_f64(Q, K, V, scale, causal)
    O = torch.empty((BH, S, dk), device="cuda")
    L = torch.empty((BH, S), device="cuda")
    engine.sdpa_fwd(dev(Q), dev(K), dev(V), O, L, scale, causal)
    assert np.abs(host(O) - O64).max() < 1e-5
    assert np.abs(host(L) - L64).max() < 1e-5


@pytest.mark.parametrize("scale", [-0.2, 0.05, 1.0])
def test_sdpa_scale_sign_and_size(engine, oracle, scale):
    """A negative scale takes the fp32-FMA kernel (the tensor-core kernel takes the row maximum before scaling);
    both routes must agree with the oracle."""
    BH, S, dk = 2, 384, 32
    Q, K, V = oracle.normal((BH, S, dk), 41), oracle.normal((BH, S, dk), 43), oracle.normal((BH, S, dk), 47)
    O64, L64 = oracle.sdpa_fwd_f64(Q, K, V, scale, 1)
    O = torch.empty((BH, S, dk), device="cuda")
    L = torch.empty((BH, S), device="cuda")
    engine.sdpa_fwd(dev(Q), dev(K), dev(V), O, L, scale, 1)
    assert np.abs(host(O) - O64).max() < 1e-5
    assert np.abs(host(L) - L64).max() < 1e-5


def test_sdpa_unaligned_base_takes_fma_kernel(engine, oracle):
    """TMA needs 16-byte aligned tensors; a view that starts 4 bytes in is served by the plain-load kernel."""
    BH, S, dk = 2, 256, 64
    Q, K, V = oracle.normal((BH, S, dk), 41), oracle.normal((BH, S, dk), 43), oracle.normal((BH, S, dk), 47)
    O64, _ = oracle.sdpa_fwd_f64(Q, K, V, 0.125, 0)
    buf = torch.empty(BH * S * dk + 1, device="cuda")
    Qu = buf[1:].view(BH, S, dk)
    Qu.copy_(dev(Q))
    O = torch.empty((BH, S, dk), device="cuda")
    engine.sdpa_fwd(Qu, dev(K), dev(V), O, None, 0.125, 0)
    assert np.abs(host(O) - O64).max() < 1e-5
    assert engine.device_error() == 0


@pytest.mark.parametrize("shape,chunk", [((4096, 1024, 512), 1024), ((2500, 768, 640), 1024), ((2100, 512, 256), 0),
                                          ((8, 512, 1024), 0), ((300, 200, 100), 128), ((1030, 256, 128), 512)])
def test_gemm_host_pipelined_equals_device_gemm(engine, oracle, shape, chunk):
    """Host-operand GEMM (chunked uploads overlapped with the tensor-core work) == one device call, bit for bit,
    and both within the fp32 bound of the oracle."""
    M, N, K = shape
    A, B = oracle.uniform((M, K), 7), oracle.uniform((K, N), 13)
    hA, hB = torch.from_numpy(A).pin_memory(), torch.from_numpy(B).pin_memory()
    hC = torch.full((M, N), float("nan")).pin_memory()
    engine.gemm_host(hA, hB, hC, row_chunk=chunk)
    C = torch.empty((M, N), device="cuda")
    engine.gemm(dev(A), dev(B), C)
    np.testing.assert_array_equal(hC.numpy(), host(C))
    assert nerr(hC.numpy(), oracle.gemm_f64(A, B)) <= 1e-5
    # a second call reuses the staging and the streams
    hC2 = torch.empty((M, N)).pin_memory()
    engine.gemm_host(hA, hB, hC2, row_chunk=chunk)
    np.testing.assert_array_equal(hC2.numpy(), hC.numpy())
    assert engine.device_error() == 0


@pytest.mark.parametrize("name", ["kv_test", "kv_ragged", "kv_c4like"])
def test_kv_cache_attend_vs_golden(engine, oracle, golden, name):
    """ax_kv_cache_append x cur_len + ax_kv_cache_attend through the reference (tests/test_attention.c:268-330)."""
    BH, max_seq, cur_len, dk = (int(v) for v in golden[name + "_shape"])
    Kc, Vc, Qn = oracle.normal((BH, max_seq, dk), 43), oracle.normal((BH, max_seq, dk), 47), oracle.normal((BH, dk), 41)
    scale = float(np.float32(1.0 / np.sqrt(dk)))
    # build the cache on the device token by token, as a decode loop does
    Kd = torch.full((BH, max_seq, dk), float("nan"), device="cuda")
    Vd = torch.full((BH, max_seq, dk), float("nan"), device="cuda")
    n = 0
    for t in range(cur_len):
        n = engine.kv_cache_append(Kd, Vd, dev(np.ascontiguousarray(Kc[:, t])), dev(np.ascontiguousarray(Vc[:, t])), n)
    assert n == cur_len
    np.testing.assert_array_equal(host(Kd[:, :cur_len]), Kc[:, :cur_len])
    out = torch.full((BH, dk), float("nan"), device="cuda")
    engine.kv_cache_attend(Kd, Vd, dev(Qn), out, cur_len, scale)
    assert np.abs(host(out) - golden[name + "_out"]).max() < 1e-5
    assert np.abs(host(out) - oracle.kv_cache_attend_f64(Kc, Vc, Qn, cur_len, scale)).max() < 1e-5


@pytest.mark.parametrize("shape", [(128, 1024, 1024, 64), (16, 4096, 4095, 64), (3, 9000, 8500, 128), (5, 300, 1, 40),
                                   (2, 64, 64, 6), (7, 700, 513, 33), (4, 100, 0, 16)])
def test_kv_cache_attend_vs_oracle(engine, oracle, shape):
    """Config-4 heads at a full 1024-token cache, long caches (several segments, several chunks), odd head dims."""
    BH, max_seq, cur_len, dk = shape
    Kc, Vc, Qn = oracle.normal((BH, max_seq, dk), 43), oracle.normal((BH, max_seq, dk), 47), oracle.normal((BH, dk), 41)
    scale = float(np.float32(1.0 / np.sqrt(dk)))
    out = torch.full((BH, dk), float("nan"), device="cuda")
    Kd, Vd, Qd = dev(Kc), dev(Vc), dev(Qn)
    engine.kv_cache_attend(Kd, Vd, Qd, out, cur_len, scale)
    if cur_len == 0:
        assert np.all(host(out) == 0)
        return
    ref64 = oracle.kv_cache_attend_f64(Kc, Vc, Qn, cur_len, scale)
    assert np.abs(host(out) - ref64).max() < 1e-5
    assert np.abs(oracle.kv_cache_attend(Kc, Vc, Qn, cur_len, scale) - ref64).max() < 1e-5
    out2 = torch.empty_like(out)
    engine.kv_cache_attend(Kd, Vd, Qd, out2, cur_len, scale)       # deterministic merge of the segments
    np.testing.assert_array_equal(host(out2), host(out))
    # the last row of causal attention over the same keys is the same computation (tests/test_attention.c:300-327)
    if dk <= 128 and cur_len >= 2:
        S = min(cur_len, 256)
        Q = np.zeros((BH, S, dk), np.float32); Q[:, -1] = Qn
        O = torch.empty((BH, S, dk), device="cuda")
        engine.sdpa_fwd(dev(Q), dev(np.ascontiguousarray(Kc[:, :S])), dev(np.ascontiguousarray(Vc[:, :S])), O, None, scale, 1)
        o_s = torch.empty((BH, dk), device="cuda")
        engine.kv_cache_attend(Kd, Vd, Qd, o_s, S, scale)
        assert np.abs(host(O[:, -1]) - host(o_s)).max() < 1e-5


def test_kv_cache_errors(engine):
    from axiom_b200.engine import EngineError
    Kd = torch.zeros((2, 4, 8), device="cuda")
    q = torch.zeros((2, 8), device="cuda")
    with pytest.raises(EngineError):
        engine.kv_cache_append(Kd, Kd, q, q, 4)          # full
    with pytest.raises(EngineError):
        engine.kv_cache_attend(Kd, Kd, q, q, 5, 1.0)     # cur_len > max_seq


@pytest.mark.parametrize("name", ["qkv_64", "qkv_24", "qkv_32_nobias"])
def test_qkv_head_gemm_vs_golden(engine, oracle, golden, name):
    B, S, H, dk, with_bias = (int(v) for v in golden[name + "_shape"])
    D = H * dk
    X, W = oracle.uniform((B * S, D), 7), oracle.normal((D, 3 * D), 13, sigma=1.0 / np.sqrt(D))
    b = oracle.uniform((3 * D,), 29) if with_bias else None
    outs = [torch.full((B * H, S, dk), float("nan"), device="cuda") for _ in range(3)]
    engine.qkv_head_gemm(dev(X), dev(W), dev(b) if with_bias else None, B, S, H, dk, *outs)
    for got, key in zip(outs, "qkv"):
        assert nerr(host(got), golden[f"{name}_{key}"]) <= TOL_SPLIT


@pytest.mark.parametrize("case", [(8, 128, 16, 64, True), (2, 333, 4, 32, True), (1, 1000, 3, 96, False), (2, 50, 2, 40, True),
                                  (1, 16, 4, 64, True), (4, 64, 8, 128, True), (1, 200, 5, 8, False)])
def test_qkv_head_gemm_vs_oracle(engine, oracle, case):
    """dk % 32 == 0 with more than 32 rows stores head-major from the GEMM epilogue; other shapes go through the
    scratch matrix and the layout pass.  Both must match the oracle and leave no element unwritten."""
    B, S, H, dk, with_bias = case
    D = H * dk
    X, W = oracle.uniform((B * S, D), 7), oracle.normal((D, 3 * D), 13, sigma=1.0 / np.sqrt(D))
    b = oracle.uniform((3 * D,), 29) if with_bias else None
    outs = [torch.full((B * H, S, dk), float("nan"), device="cuda") for _ in range(3)]
    engine.qkv_head_gemm(dev(X), dev(W), dev(b) if with_bias else None, B, S, H, dk, *outs)
    want = oracle.qkv_head_gemm(X, W, b, B, S, H, dk)
    full = oracle.gemm_f64(X, W) + (b.astype(np.float64) if with_bias else 0.0)
    for i, got in enumerate(outs):
        g = host(got)
        assert not np.isnan(g).any()
        assert nerr(g, want[i]) <= TOL_SPLIT
        blk = full[:, i * D:(i + 1) * D].reshape(B, S, H, dk).transpose(0, 2, 1, 3).reshape(B * H, S, dk)
        assert nerr(g, blk) <= TOL_SPLIT
    assert engine.device_error() == 0


@pytest.mark.parametrize("name", ["s_test", "s_c4like"])
@pytest.mark.parametrize("causal", [0, 1])
def test_sdpa_bwd_vs_golden(engine, oracle, golden, name, causal):
    """ax_fused_attention_bwd[_causal] of the reference on the forward's own O and L."""
    BH, S, dk = (int(v) for v in golden[name + "_shape"])
    scale = float(golden[name + "_scale"][0])
    Q, K, V = oracle.normal((BH, S, dk), 41), oracle.normal((BH, S, dk), 43), oracle.normal((BH, S, dk), 47)
    dO = oracle.normal((BH, S, dk), 53)
    Qd, Kd, Vd, dOd = dev(Q), dev(K), dev(V), dev(dO)
    O = torch.empty((BH, S, dk), device="cuda")
    L = torch.empty((BH, S), device="cuda")
    engine.sdpa_fwd(Qd, Kd, Vd, O, L, scale, causal)
    grads = [torch.full((BH, S, dk), float("nan"), device="cuda") for _ in range(3)]
    engine.sdpa_bwd(Qd, Kd, Vd, O, dOd, L, *grads, scale, causal)
    for got, key in zip(grads, ("dQ", "dK", "dV")):
        assert np.abs(host(got) - golden[f"{name}_c{causal}_{key}"]).max() < 1e-4


@pytest.mark.parametrize("shape", [(4, 1024, 64), (2, 333, 64), (3, 200, 128), (2, 129, 40), (5, 64, 16), (2, 70, 6), (1, 513, 72)])
@pytest.mark.parametrize("causal", [0, 1])
def test_sdpa_bwd_vs_oracle(engine, oracle, shape, causal):
    BH, S, dk = shape
    Q, K, V = oracle.normal((BH, S, dk), 41), oracle.normal((BH, S, dk), 43), oracle.normal((BH, S, dk), 47)
    dO = oracle.normal((BH, S, dk), 53)
    scale = 1.0 / np.sqrt(dk)
    Qd, Kd, Vd, dOd = dev(Q), dev(K), dev(V), dev(dO)
    O = torch.empty((BH, S, dk), device="cuda")
    L = torch.empty((BH, S), device="cuda")
    engine.sdpa_fwd(Qd, Kd, Vd, O, L, scale, causal)
    grads = [torch.full((BH, S, dk), float("nan"), device="cuda") for _ in range(3)]   # outputs are overwritten
    engine.sdpa_bwd(Qd, Kd, Vd, O, dOd, L, *grads, scale, causal)
    want = oracle.sdpa_bwd_f64(Q, K, V, host(O), dO, scale, causal)
    for got, ref in zip(grads, want):
        assert nerr(host(got), ref) <= 1e-5
    again = [torch.empty((BH, S, dk), device="cuda") for _ in range(3)]
    engine.sdpa_bwd(Qd, Kd, Vd, O, dOd, L, *again, scale, causal)
    for a, b in zip(again, grads):
        np.testing.assert_array_equal(host(a), host(b))        # one writer per output, fixed order
    assert engine.device_error() == 0


@pytest.mark.parametrize("name", ["conv_3x3_same", "conv_3x3_s2", "conv_1x1", "conv_5x3_mixed"])
def test_conv_gemm_vs_golden(engine, oracle, golden, name):
    C_out, C_in, H, W, kh, kw, sh, sw, ph, pw = (int(v) for v in golden[name + "_geom"])
    w, x = oracle.uniform((C_out, C_in * kh * kw), 7), oracle.uniform((C_in, H, W), 13)
    want = golden[name + "_out"]
    out = torch.full(want.shape, float("nan"), device="cuda")
    engine.conv_gemm(dev(w), dev(x), kh, kw, sh, sw, ph, pw, out)
    assert nerr(host(out), want) <= TOL_SPLIT
    np.testing.assert_array_equal(oracle.conv_gemm(w, x, kh, kw, sh, sw, ph, pw).shape, want.shape)


@pytest.mark.parametrize("geom", [(64, 3, 224, 224, 7, 7, 2, 2, 3, 3), (128, 64, 56, 56, 3, 3, 1, 1, 1, 1), (256, 128, 28, 28, 3, 3, 2, 2, 1, 1),
                                  (10, 1, 28, 28, 5, 5, 1, 1, 0, 0), (33, 7, 17, 13, 3, 2, 2, 3, 1, 0), (512, 256, 14, 14, 1, 1, 1, 1, 0, 0)])
def test_conv_gemm_vs_oracle(engine, oracle, geom):
    """ResNet-style layers (7x7/2 stem, 3x3 same, 3x3/2, 1x1), an MNIST-size 5x5 and a ragged one."""
    C_out, C_in, H, W, kh, kw, sh, sw, ph, pw = geom
    w = oracle.normal((C_out, C_in * kh * kw), 7, sigma=1.0 / np.sqrt(C_in * kh * kw))
    x = oracle.uniform((C_in, H, W), 13)
    want = oracle.conv_gemm(w, x, kh, kw, sh, sw, ph, pw)
    out = torch.full(want.shape, float("nan"), device="cuda")
    engine.conv_gemm(dev(w), dev(x), kh, kw, sh, sw, ph, pw, out)
    assert nerr(host(out), want) <= TOL_SPLIT
    assert engine.device_error() == 0


@pytest.mark.parametrize("geom", [(256, 256, 56, 56, 3, 3, 1, 1, 1, 1),    # the benchmark layer: two 8 x 8 patches per tile, K split
                                  (96, 20, 30, 36, 5, 5, 1, 1, 2, 2),      # channels padded 20 -> 32, ragged patches on both edges
                                  (40, 33, 5, 64, 3, 3, 1, 1, 1, 1),       # flat image: 32 x 2 patches
                                  (300, 40, 20, 16, 1, 3, 1, 1, 0, 1),     # three row tiles, 1 x 3 window
                                  (64, 16, 33, 21, 2, 2, 1, 1, 0, 0),      # even window, no padding
                                  (16, 8, 6, 8, 3, 3, 1, 1, 3, 3),         # padding as wide as the window: all-zero windows
                                  (512, 32, 112, 112, 3, 3, 1, 1, 1, 1)])  # enough tiles for 128 x 256 tiles (four patches each)
@pytest.mark.parametrize("mode", ["3xtf32", "bf16x3", "bf16"])
def test_conv_implicit_gemm(engine, oracle, geom, mode):
    """Stride-1 layers whose output width is a multiple of 4 take the implicit-GEMM route (shifted TMA windows of the
    channel-innermost image, no patch matrix): every patch shape, channel padding, edge clipping, in all fp32 modes."""
    C_out, C_in, H, W, kh, kw, sh, sw, ph, pw = geom
    if mode != "3xtf32" and C_out * C_in * H * W > 1 << 28:
        pytest.skip("largest layer in the default mode only")
    w = oracle.normal((C_out, C_in * kh * kw), 7, sigma=1.0 / np.sqrt(C_in * kh * kw))
    x = oracle.uniform((C_in, H, W), 13)
    want = oracle.conv_gemm(w, x, kh, kw, sh, sw, ph, pw)
    assert ((W + 2 * pw - kw) // sw + 1) % 4 == 0 and sh == 1 and sw == 1     # the route's own conditions
    out = torch.full(want.shape, float("nan"), device="cuda")
    engine.set_fp32_mode(mode)
    try:
        engine.conv_gemm(dev(w), dev(x), kh, kw, sh, sw, ph, pw, out)
        again = torch.full(want.shape, float("nan"), device="cuda")
        engine.conv_gemm(dev(w), dev(x), kh, kw, sh, sw, ph, pw, again)
    finally:
        engine.set_fp32_mode("3xtf32")
    got = host(out)
    assert np.isfinite(got).all()
    assert nerr(got, want) <= (TOL_BF16 if mode == "bf16" else TOL_SPLIT), (mode, nerr(got, want))
    np.testing.assert_array_equal(host(again), got)      # split-K sums in slice order: repeatable
    assert engine.device_error() == 0


@pytest.mark.parametrize("shape", [(8, 1024, 16, 64), (2, 100, 5, 32), (3, 50, 4, 24), (1, 16, 2, 8), (4, 256, 8, 96)])
def test_dattn_head_gemm_nt(engine, oracle, shape):
    """dO_head = head-major(dout . Wo^T) against float64 (config-4 layer shape, ragged rows, head dims that are not
    multiples of 32, a skinny input)."""
    B, S, H, dk = shape
    D = H * dk
    dout, Wo = oracle.uniform((B * S, D), 7), oracle.normal((D, D), 13, sigma=1.0 / np.sqrt(D))
    ref = oracle.gemm_f64(dout, np.ascontiguousarray(Wo.T))                                # [B*S, D]
    want = ref.reshape(B, S, H, dk).transpose(0, 2, 1, 3).reshape(B * H, S, dk)
    out = torch.full((B * H, S, dk), float("nan"), device="cuda")
    engine.dattn_head_gemm_nt(dev(dout), dev(Wo), B, S, H, dk, out)
    assert nerr(host(out), want) <= TOL_SPLIT
    assert engine.device_error() == 0


@pytest.mark.parametrize("shape", [(8, 1024, 16, 64), (2, 100, 5, 32), (3, 50, 4, 24), (1, 16, 2, 8), (2, 300, 1, 32), (4, 256, 8, 96)])
@pytest.mark.parametrize("head_major", [False, True])
def test_dwqkv_split_acc(engine, oracle, shape, head_major):
    """dW{q,k,v} += x^T . dQKV column blocks against float64, on top of gradients that already hold values (config-4
    layer shape — split K —, ragged rows, widths that are not multiples of 32, one 32-wide tile), flat and head-major."""
    B, S, H, dk = shape
    D, rows = H * dk, B * S
    x, dqkv = oracle.uniform((rows, D), 7), oracle.normal((rows, 3 * D), 13, sigma=0.5)
    start = [oracle.uniform((D, D), 20 + i) for i in range(3)]
    grads = [dev(g.copy()) for g in start]
    if head_major:
        hm = [dev(np.ascontiguousarray(dqkv[:, i * D:(i + 1) * D].reshape(B, S, H, dk).transpose(0, 2, 1, 3)).reshape(B * H, S, dk))
              for i in range(3)]
        engine.dwqkv_split_acc_hm(dev(x), *hm, B, S, H, dk, *grads)
    else:
        engine.dwqkv_split_acc(dev(x), dev(dqkv), *grads)
    prod = oracle.gemm_f64(np.ascontiguousarray(x.T), dqkv)                                 # [D, 3D]
    for i in range(3):
        want = start[i].astype(np.float64) + prod[:, i * D:(i + 1) * D]
        assert nerr(host(grads[i]), want) <= TOL_SPLIT, (i, nerr(host(grads[i]), want))
    assert engine.device_error() == 0


@pytest.mark.parametrize("rows,D", [(8192, 1024), (200, 160), (50, 96), (16, 20), (1, 64)])
@pytest.mark.parametrize("forward", [True, False])
def test_mha_output_proj_fused(engine, oracle, rows, D, forward):
    """The attention layer's output projection, forward and backward in one call, against float64: y (with bias; skipped
    when forward is off), dattn, and dWo / dbo accumulated on top of values already there."""
    attn, dout = oracle.uniform((rows, D), 7), oracle.normal((rows, D), 13, sigma=0.5)
    Wo, bo = oracle.normal((D, D), 17, sigma=1.0 / np.sqrt(D)), oracle.uniform((D,), 19)
    dWo0, dbo0 = oracle.uniform((D, D), 23), oracle.uniform((D,), 29)
    y = torch.full((rows, D), float("nan"), device="cuda") if forward else None
    dattn = torch.full((rows, D), float("nan"), device="cuda")
    dWo, dbo = dev(dWo0.copy()), dev(dbo0.copy())
    engine.mha_output_proj_fused(dev(attn), dev(Wo), dev(bo) if forward else None, dev(dout), y, dattn, dWo, dbo)
    if forward:
        assert nerr(host(y), oracle.gemm_f64(attn, Wo) + bo.astype(np.float64)) <= TOL_SPLIT
    assert nerr(host(dattn), oracle.gemm_f64(dout, np.ascontiguousarray(Wo.T))) <= TOL_SPLIT
    assert nerr(host(dWo), dWo0.astype(np.float64) + oracle.gemm_f64(np.ascontiguousarray(attn.T), dout)) <= TOL_SPLIT
    want_dbo = dbo0.astype(np.float64) + dout.astype(np.float64).sum(axis=0)
    assert np.abs(host(dbo) - want_dbo).max() <= 1e-5 * max(1.0, np.abs(dout).sum(axis=0).max())
    assert engine.device_error() == 0


@pytest.mark.parametrize("geom", [(8, 256, 256, 56, 56, 3, 3, 1, 1, 1, 1),   # a ResNet stage at batch 8: one implicit GEMM on CTA pairs (98 tiles of 256 x 256)
                                  (3, 40, 20, 12, 20, 5, 5, 1, 1, 2, 2),      # patches of the last tile run into the next sample and past the end
                                  (5, 16, 3, 6, 8, 3, 3, 1, 1, 1, 1),         # samples smaller than one patch row
                                  (2, 24, 8, 15, 15, 3, 3, 2, 2, 1, 1),       # strided: samples one by one through the gathered form
                                  (1, 8, 4, 8, 8, 3, 3, 1, 1, 1, 1)])
def test_conv_gemm_batched(engine, oracle, geom):
    """axb_conv_gemm_batched: every sample equals the single-sample oracle; batch 0 is a no-op."""
    N, C_out, C_in, H, W, kh, kw, sh, sw, ph, pw = geom
    w = oracle.normal((C_out, C_in * kh * kw), 7, sigma=1.0 / np.sqrt(C_in * kh * kw))
    x = oracle.uniform((N, C_in, H, W), 13)
    out_h, out_w = (H + 2 * ph - kh) // sh + 1, (W + 2 * pw - kw) // sw + 1
    out = torch.full((N, C_out, out_h * out_w), float("nan"), device="cuda")
    engine.conv_gemm_batched(dev(w), dev(x), kh, kw, sh, sw, ph, pw, out)
    got = host(out)
    assert np.isfinite(got).all()
    for n in range(N):
        want = oracle.conv_gemm(w, np.ascontiguousarray(x[n]), kh, kw, sh, sw, ph, pw)
        assert nerr(got[n], want) <= TOL_SPLIT, (n, nerr(got[n], want))
    empty = torch.empty((0, C_out, out_h * out_w), device="cuda")
    engine.conv_gemm_batched(dev(w), torch.empty((0, C_in, H, W), device="cuda"), kh, kw, sh, sw, ph, pw, empty)
    assert engine.device_error() == 0


@pytest.mark.parametrize("shape", [(2, 1024, 1024), (8, 4096, 4096), (9, 1000, 2048), (16, 2048, 1040), (17, 8200, 1168),
                                   (32, 16384, 512), (33, 1024, 1024), (64, 4096, 4096), (5, 128, 8192),
                                   (2, 8192, 128), (64, 130, 8192), (7, 64, 16384), (48, 2048, 65536 // 64),
                                   (1, 16384, 4096),
                                   # up to four rows the kernel makes the digits itself: many uses of every ring stage,
                                   # a ragged N with a K tail that is not a whole k-block, four rows on one slice
                                   (3, 9728, 8192), (4, 600, 2064), (4, 16384, 1024)])
def test_w8a32_skinny_tensor_core_kernel(engine, oracle, shape):
    """2 <= M <= 64 with at least 2^20 weights (M = 1 from 2^24 weights): activations as four int8 digit planes,
    kind::i8 MMAs.  Ragged N and K
    (zero-filled tiles), one and several K-slices per tile, an outlier 1000x the other activations in one row, and a
    row with an infinity (the reference's fp32 sum is NaN or infinite there; here the row is NaN)."""
    M, N, K = shape
    a, w = oracle.uniform((M, K), 7), oracle.uniform((N, K), 13)
    a[0, 3] = 1000.0
    q, s = oracle.quantize_rows(w)
    out = torch.full((M, N), float("nan"), device="cuda")
    engine.qgemm_w8a32(dev(a), torch.from_numpy(q).cuda(), dev(s), out)
    got = host(out)
    assert engine.device_error() == 0
    assert nerr(got, oracle.qgemm_w8a32_f64(a, q, s)) <= 1e-6      # fixed point at 2^-30 of the row maximum
    ref = oracle.qgemm_w8a32(a, q, s)
    diff = np.abs(got - ref)
    assert not np.any((diff > 1e-2) & (diff / (np.abs(ref) + 1e-5) > 1e-3))   # tests/test_quantize.c:109-113
    again = torch.empty((M, N), device="cuda")
    engine.qgemm_w8a32(dev(a), torch.from_numpy(q).cuda(), dev(s), again)
    np.testing.assert_array_equal(host(again), got)
    a[M - 1, 5] = np.inf
    engine.qgemm_w8a32(dev(a), torch.from_numpy(q).cuda(), dev(s), out)
    got2 = host(out)
    assert np.all(np.isnan(got2[M - 1]))
    if M > 1:
        np.testing.assert_array_equal(got2[:M - 1], got[:M - 1])


@pytest.mark.parametrize("shape", [(65, 1024, 1024), (129, 1000, 1168), (70, 1001, 1024), (512, 2048, 512)])
def test_w8a32_digit_planes_as_gemm_operand(engine, oracle, shape):
    """M > 64: the four int8 digit rows of every activation row, interleaved, are the B operand of one int8 GEMM on the
    dense core against the weights as the A operand; the epilogue recombines the four digit sums of an output in 64-bit
    integers and stores it transposed.  Ragged M, N (also not a multiple of 4) and K, an outlier, and a row with an
    infinity."""
    M, N, K = shape
    a, w = oracle.uniform((M, K), 7), oracle.uniform((N, K), 13)
    a[1, 3] = 1000.0
    q, s = oracle.quantize_rows(w)
    bias = oracle.uniform((N,), 29)
    out = torch.full((M, N), float("nan"), device="cuda")
    engine.qdense_w8a32(dev(a), torch.from_numpy(q).cuda(), dev(s), dev(bias), out, act="relu")
    got = host(out)
    assert engine.device_error() == 0
    want = np.maximum(oracle.qgemm_w8a32_f64(a, q, s) + bias.astype(np.float64), 0.0)
    assert nerr(got, want) <= 1e-6
    a[M - 1, 5] = -np.inf
    engine.qdense_w8a32(dev(a), torch.from_numpy(q).cuda(), dev(s), dev(bias), out, act="none")
    got2 = host(out)
    assert np.all(np.isnan(got2[M - 1]))
    assert np.all(np.isfinite(got2[:M - 1]))


@pytest.mark.parametrize("shape", [(1, 4096, 4096), (8, 1000, 2048), (4, 16, 32), (32, 128, 512), (300, 512, 1024), (24, 2048, 1024)])
@pytest.mark.parametrize("act", ["none", "relu", "gelu"])
def test_qdense_w8a32(engine, oracle, shape, act):
    """Quantised dense layer = the reference's ax_qgemm_w8a32 plus the dense layer's bias and activation in one launch
    (GEMV kernel for M = 1 and small layers, integer tensor-core kernel for 2 <= M <= 64, digit planes through the
    int8 GEMM core above)."""
    M, N, K = shape
    a, w = oracle.uniform((M, K), 7), oracle.uniform((N, K), 13)
    bias = oracle.uniform((N,), 29)
    q, s = oracle.quantize_rows(w)
    pre = oracle.qgemm_w8a32_f64(a, q, s) + bias.astype(np.float64)
    want = {"none": pre, "relu": np.maximum(pre, 0.0),
            "gelu": 0.5 * pre * (1 + np.tanh(0.7978845608028654 * (pre + 0.044715 * pre ** 3)))}[act]
    out = torch.full((M, N), float("nan"), device="cuda")
    engine.qdense_w8a32(dev(a), torch.from_numpy(q).cuda(), dev(s), dev(bias), out, act=act)
    assert nerr(host(out), want) <= TOL_SPLIT
    plain = torch.empty((M, N), device="cuda")
    engine.qgemm_w8a32(dev(a), torch.from_numpy(q).cuda(), dev(s), plain)          # the reference's entry: no bias, no act
    assert nerr(host(plain), oracle.qgemm_w8a32_f64(a, q, s)) <= TOL_SPLIT


# ---- split-K of the dense tensor-core core: few output tiles, long K ----------------------------------------------

@pytest.mark.parametrize("shape", [(256, 384, 4096), (130, 200, 3000), (1024, 1024, 1024), (64, 128, 8192), (300, 96, 2052),
                                   (256, 3136, 2304), (33, 520, 1536),
                                   # two slices per tile (the pair of CTAs meets in shared memory): ragged edges,
                                   # slices of unequal length, K shorter than two chunks, 64-column tiles
                                   (1000, 900, 1100), (640, 1408, 520), (896, 1024, 300), (7000, 64, 2048),
                                   # 96 tiles of 128 x 256 on 148 SMs: three slices per tile fill two whole rounds
                                   (1024, 3072, 6144), (1000, 3000, 6200)])
def test_split_k_fp32_vs_oracle_and_repeatable(engine, oracle, shape):
    """Problems with too few 128-column tiles to fill the GPU — or with 256-column tiles that leave the last round of
    work part empty — cut K into slices.  Two slices are a thread-block cluster
    and meet in shared memory (each CTA finishes one column half); more meet in scratch, where the slice that arrives
    last adds all partial tiles in slice order.  Either way the result is inside the fp32 tolerance AND bitwise
    repeatable, with every epilogue form (bias + GELU, alpha/beta, transposed operands)."""
    M, N, K = shape
    A, B, bias, Cin = oracle.uniform((M, K), 7), oracle.uniform((K, N), 13), oracle.uniform((N,), 29), oracle.uniform((M, N), 5)
    ref = oracle.gemm_f64(A, B)
    Ad, Bd = dev(A), dev(B)
    outs = []
    for _ in range(3):
        out = torch.full((M, N), float("nan"), device="cuda")
        engine.gemm(Ad, Bd, out)
        outs.append(host(out))
    assert nerr(outs[0], ref) <= TOL_SPLIT
    np.testing.assert_array_equal(outs[0], outs[1])
    np.testing.assert_array_equal(outs[0], outs[2])
    out = torch.empty((M, N), device="cuda")
    engine.gemm_bias_act(Ad, Bd, dev(bias), out, M, N, K, act="gelu")
    assert nerr(host(out), oracle.bias_act(ref.astype(np.float32), bias, "gelu")) <= TOL_SPLIT
    c = dev(Cin)
    engine.gemm_ex(Ad, Bd, 0.5, 2.0, c)
    assert nerr(host(c), 0.5 * ref + 2.0 * Cin) <= TOL_SPLIT
    np.testing.assert_array_equal(run_gemm(engine, A, np.ascontiguousarray(B.T), "nt"), outs[0])
    np.testing.assert_array_equal(run_gemm(engine, np.ascontiguousarray(A.T), B, "tn"), outs[0])
    for mode, tol in (("bf16x3", TOL_SPLIT), ("bf16", TOL_BF16)):
        engine.set_fp32_mode(mode)
        try:
            engine.gemm(Ad, Bd, out)
        finally:
            engine.set_fp32_mode("3xtf32")
        assert nerr(host(out), ref) <= tol
    assert engine.device_error() == 0


@pytest.mark.parametrize("shape", [(64, 256, 8192), (256, 384, 4096), (130, 200, 3001), (128, 128, 16384), (512, 512, 2048)])
def test_split_k_int8_bit_exact(engine, oracle, shape):
    M, N, K = shape
    a, b, bs = oracle.int8((M, K), 7), oracle.int8((N, K), 13), oracle.frange((N,), 17, 0.001, 0.02)
    out_scale = 0.02 * 0.0105 * 73.0 * np.sqrt(K)
    acc_ref, q_ref = oracle.qgemm_w8a8(a, 0.02, b, bs, out_scale)
    q = torch.zeros((M, N), dtype=torch.int8, device="cuda")
    acc = torch.zeros((M, N), dtype=torch.int32, device="cuda")
    engine.qgemm_w8a8(dev(a), 0.02, dev(b), dev(bs), out_scale, q, acc)
    np.testing.assert_array_equal(host(acc), acc_ref)
    np.testing.assert_array_equal(host(q), q_ref)
    assert engine.device_error() == 0


def test_split_k_int8_wave_filling_sampled_rows(engine, oracle):
    """100 tiles of 128 x 256 with a long K: K is cut so that tile x slice items fill whole rounds of the 148 SMs; sampled
    rows against the oracle, bit-exact, and the whole result repeatable."""
    M, N, K = 1280, 2560, 16384
    a, b, bs = oracle.int8((M, K), 7), oracle.int8((N, K), 13), oracle.frange((N,), 17, 0.001, 0.02)
    out_scale = 0.02 * 0.0105 * 73.0 * np.sqrt(K)
    rows = np.array([0, 127, 128, 640, 1279])
    acc_ref, q_ref = oracle.qgemm_w8a8(np.ascontiguousarray(a[rows]), 0.02, b, bs, out_scale)
    q, acc = torch.zeros((M, N), dtype=torch.int8, device="cuda"), torch.zeros((M, N), dtype=torch.int32, device="cuda")
    engine.qgemm_w8a8(dev(a), 0.02, dev(b), dev(bs), out_scale, q, acc)
    np.testing.assert_array_equal(host(acc)[rows], acc_ref)
    np.testing.assert_array_equal(host(q)[rows], q_ref)
    q2 = torch.zeros((M, N), dtype=torch.int8, device="cuda")
    engine.qgemm_w8a8(dev(a), 0.02, dev(b), dev(bs), out_scale, q2, None)
    assert torch.equal(q, q2)
    assert engine.device_error() == 0


@pytest.mark.parametrize("shape", [(1024, 1024, 1024), (300, 520, 1000), (8, 4096, 4096), (20, 1000, 1028), (2560, 2560, 512),
                                   (256, 384, 4096)])
@pytest.mark.parametrize("trans_b", [False, True])
def test_prepared_weight_is_bit_identical(engine, oracle, shape, trans_b):
    """axb_gemm_prepared (operand planes of the weight made once) against axb_gemm_bias_act on the same operands: the
    same routes, so the same bits — tensor-core tiles, CTA pairs, split-K and the skinny route."""
    M, N, K = shape
    A, B, bias = oracle.uniform((M, K), 7), oracle.uniform((K, N), 13), oracle.uniform((N,), 29)
    Bd = dev(np.ascontiguousarray(B.T) if trans_b else B)
    Ad, bd = dev(A), dev(bias)
    want = torch.empty((M, N), device="cuda")
    engine.gemm_bias_act(Ad, Bd, bd, want, M, N, K, trans_b=trans_b, act="gelu")
    w = engine.weight_prepare(Bd, trans_b=trans_b)
    try:
        for _ in range(2):
            got = torch.full((M, N), float("nan"), device="cuda")
            engine.gemm_prepared(Ad, w, bd, got, M, act="gelu")
            np.testing.assert_array_equal(host(got), host(want))
        assert nerr(host(got), oracle.bias_act(oracle.gemm_f64(A, B).astype(np.float32), bias, "gelu")) <= TOL_SPLIT
        engine.set_fp32_mode("bf16")
        try:
            with pytest.raises(Exception):
                engine.gemm_prepared(Ad, w, bd, got, M)       # prepared under another arithmetic
        finally:
            engine.set_fp32_mode("3xtf32")
    finally:
        engine.weight_release(w)
