"""The C multi-GPU entry points (axb_mgpu_*): one host thread driving several devices, rows partitioned without
communication and columns partitioned with one NCCL all-gather per layer.  Needs at least two GPUs in one process
(skipped otherwise); the single-device form of every call runs anywhere a GPU is."""
import numpy as np
import pytest
import torch

from oracle_lib import nerr

pytestmark = pytest.mark.gpu


def bounds(n, g, r):
    base, rem = divmod(n, g)
    lo = r * base + min(r, rem)
    return lo, lo + base + (1 if r < rem else 0)


@pytest.fixture(scope="module")
def mg(engine):
    from axiom_b200.engine import MultiGpu
    n = min(torch.cuda.device_count(), 4)
    m = MultiGpu(engine, n)
    yield m
    m.close()
    engine.init(0)


def test_handle_and_errors(engine, mg):
    from axiom_b200.engine import EngineError, MultiGpu
    assert engine.lib.axb_mgpu_size(mg.h) == mg.n
    assert [engine.lib.axb_mgpu_device(mg.h, r) for r in range(mg.n)] == list(range(mg.n))
    with pytest.raises(EngineError):
        MultiGpu(engine, torch.cuda.device_count() + 1)
    with pytest.raises(EngineError):
        MultiGpu(engine, 0)
    assert engine.lib.axb_mgpu_synchronize(None) != 0


@pytest.mark.parametrize("shape", [(1000, 384, 512), (2048, 4096, 1024)])
def test_rows_partition_matches_single_device(engine, oracle, mg, shape):
    """Every rank's block of rows equals the oracle, and (for the shape that fills a GPU either way) the same rows of
    one call over the whole matrix bit for bit."""
    M, N, K = shape
    g = mg.n
    A, B, bias = oracle.uniform((M, K), 7), oracle.uniform((K, N), 13), oracle.uniform((N,), 29)
    rows = [bounds(M, g, r) for r in range(g)]
    Ap = [mg.upload(r, A[lo:hi]) for r, (lo, hi) in enumerate(rows)]
    Bp = [mg.upload(r, B) for r in range(g)]
    bp = [mg.upload(r, bias) for r in range(g)]
    Cp = [mg.alloc(r, (hi - lo) * N * 4) for r, (lo, hi) in enumerate(rows)]
    mg.gemm_rows(Ap, Bp, bp, Cp, [hi - lo for lo, hi in rows], N, K, act="gelu")
    mg.synchronize()
    got = np.concatenate([mg.download(r, Cp[r], (hi - lo, N), np.float32) for r, (lo, hi) in enumerate(rows)])
    want = oracle.bias_act(oracle.gemm_f64(A, B).astype(np.float32), bias, "gelu")
    assert nerr(got, want) <= 1e-5
    engine.init(0)
    whole = torch.empty((M, N), device="cuda:0")
    engine.gemm_bias_act(torch.from_numpy(A).to("cuda:0"), torch.from_numpy(B).to("cuda:0"), torch.from_numpy(bias).to("cuda:0"),
                         whole, M, N, K, act="gelu")
    assert nerr(got, whole.cpu().numpy()) <= 2e-6
    if M >= 2048:
        np.testing.assert_array_equal(got, whole.cpu().numpy())


def test_int8_rows_partition_bit_exact(engine, oracle, mg):
    M, N, K = 768, 512, 1024
    g = mg.n
    a, b, bs = oracle.int8((M, K), 7), oracle.int8((N, K), 13), oracle.frange((N,), 17, 0.001, 0.02)
    _, q_ref = oracle.qgemm_w8a8(a, 0.02, b, bs, 5.0)
    rows = [bounds(M, g, r) for r in range(g)]
    ap = [mg.upload(r, a[lo:hi]) for r, (lo, hi) in enumerate(rows)]
    bp = [mg.upload(r, b) for r in range(g)]
    sp = [mg.upload(r, bs) for r in range(g)]
    qp = [mg.alloc(r, (hi - lo) * N) for r, (lo, hi) in enumerate(rows)]
    mg.qgemm_w8a8_rows(ap, 0.02, bp, sp, 5.0, qp, [hi - lo for lo, hi in rows], N, K)
    mg.synchronize()
    got = np.concatenate([mg.download(r, qp[r], (hi - lo, N), np.int8) for r, (lo, hi) in enumerate(rows)])
    np.testing.assert_array_equal(got, q_ref)


def test_column_sharded_mlp_with_allgather(engine, oracle, mg):
    """Two chained layers, output columns partitioned, one all-gather per layer; the second layer reads the first's
    gather buffer in place.  Every rank must hold the same full activation, equal to the oracle's."""
    g = mg.n
    M, dims = 300, [256, 128 * g, 64 * g]
    x = oracle.uniform((M, dims[0]), 7)
    Ws = [oracle.normal((dims[i], dims[i + 1]), 13 + i, sigma=1.0 / np.sqrt(dims[i])) for i in range(2)]
    bs = [oracle.uniform((dims[i + 1],), 29 + i) for i in range(2)]
    h = x.astype(np.float64)
    for W, b in zip(Ws, bs):
        z = oracle.gemm_f64(np.ascontiguousarray(h.astype(np.float32)), W) + b.astype(np.float64)
        h = 0.5 * z * (1.0 + np.tanh(0.7978845608028654 * (z + 0.044715 * z ** 3)))
    X = [mg.upload(r, x) for r in range(g)]
    chunks = 1
    K = dims[0]
    for W, b in zip(Ws, bs):
        n = W.shape[1] // g
        Wp = [mg.upload(r, W[:, r * n:(r + 1) * n]) for r in range(g)]
        bp = [mg.upload(r, b[r * n:(r + 1) * n]) for r in range(g)]
        slab = [mg.alloc(r, M * n * 4) for r in range(g)]
        gathered = [mg.alloc(r, g * M * n * 4) for r in range(g)]
        mg.gemm_cols_allgather(X, chunks, Wp, bp, slab, gathered, M, n, K, act="gelu")
        X, chunks, K = gathered, g, W.shape[1]
    mg.synchronize()
    n_last = dims[-1] // g
    outs = [mg.download(r, X[r], (g, M, n_last), np.float32).transpose(1, 0, 2).reshape(M, g * n_last) for r in range(g)]
    for r in range(g):
        assert nerr(outs[r], h) <= 1e-5, r
        np.testing.assert_array_equal(outs[r], outs[0])
    engine.init(0)
