"""Drop-in proof: the UNMODIFIED reference dispatcher (oracle/_ref) drives this engine.

The vtable of libaxiom_b200_backend.so is registered with the reference's own
ax_compute_register_backend; operands reach the GPU through the reference's
ax_tensor_to_cuda (our storage_alloc / memcpy_h2d hooks); ax_compute_gemm*,
ax_compute_gemm_relu, ax_compute_gemm_ex, ax_compute_bias_add, ax_compute_relu,
ax_matmul_bias_relu, ax_compute_qkv_head_gemm and the sdpa_fwd extension slot dispatch into our kernels.
Results are compared with the same reference running its CPU backend.
"""
import ctypes

import numpy as np
import pytest

from oracle_lib import nerr

pytestmark = pytest.mark.gpu
f32p = ctypes.POINTER(ctypes.c_float)
i64 = ctypes.c_int64


def p(a):
    return None if a is None else a.ctypes.data_as(f32p)


@pytest.fixture(scope="module")
def dropin(engine, reference):
    from axiom_b200 import build
    backend = ctypes.CDLL(build.BACKEND_SO)
    lib = reference.lib
    backend.axb_backend_ops.restype = ctypes.c_void_p
    backend.axb_cuda_extension.restype = ctypes.c_void_p
    SKIP = ctypes.CFUNCTYPE(ctypes.c_int)
    ERR = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_char_p)
    cbs = (SKIP(lambda: lib.ref_skip_init_flag()), ERR(lambda st, msg: lib.ref_err_set(st, msg)))
    backend.axb_backend_set_hooks(*cbs)
    assert lib.ref_register_cuda_backend(ctypes.c_void_p(backend.axb_backend_ops()),
                                         ctypes.c_void_p(backend.axb_cuda_extension())) == 0
    lib.ref_last_error.restype = ctypes.c_char_p
    lib._keep = (backend, cbs)
    return lib


def gemm_op(lib, op, A, B, bias, C, M, N, K, alpha=1.0, beta=0.0):
    rc = lib.ref_device_gemm_op(op, p(A), p(B), p(bias), p(C), i64(M), i64(N), i64(K), ctypes.c_float(alpha), ctypes.c_float(beta))
    assert rc == 0, (rc, lib.ref_last_error())
    return C


@pytest.mark.parametrize("shape", [(2, 2, 2), (64, 32, 128), (200, 300, 170), (1, 256, 384), (8, 100, 64)])
def test_gemm_slots_through_reference_dispatcher(dropin, reference, oracle, shape):
    M, N, K = shape
    A, B, bias, C0 = oracle.uniform((M, K), 7), oracle.uniform((K, N), 13), oracle.uniform((N,), 29), oracle.uniform((M, N), 5)
    want = reference.gemm(A, B)
    tol = dict(atol=1e-3, rtol=1e-4)   # tests/test_cuda.c:213-244 of the reference uses abs 1e-3 for GPU-vs-CPU
    np.testing.assert_allclose(gemm_op(dropin, 0, A, B, None, np.zeros((M, N), np.float32), M, N, K), want, **tol)
    np.testing.assert_allclose(gemm_op(dropin, 1, A, np.ascontiguousarray(B.T), None, np.zeros((M, N), np.float32), M, N, K), want, **tol)
    np.testing.assert_allclose(gemm_op(dropin, 2, np.ascontiguousarray(A.T), B, None, np.zeros((M, N), np.float32), M, N, K), want, **tol)
    np.testing.assert_allclose(gemm_op(dropin, 3, A, B, bias, np.zeros((M, N), np.float32), M, N, K), reference.gemm_relu(A, B, bias), **tol)
    np.testing.assert_allclose(gemm_op(dropin, 4, A, B, None, C0.copy(), M, N, K, 0.5, 2.0), reference.gemm_ex(A, B, 0.5, 2.0, C0), **tol)
    # ax_gemm_set_skip_init(true): C += A.B (cpu_opt honours it; the stock CUDA backend does not)
    np.testing.assert_allclose(gemm_op(dropin, 5, A, B, None, C0.copy(), M, N, K), want + C0, **tol)
    # the dense-layer op itself: ax_matmul_bias_relu allocates its output on the device through our hook
    np.testing.assert_allclose(gemm_op(dropin, 6, A, B, bias, np.zeros((M, N), np.float32), M, N, K), reference.matmul_bias_relu(A, B, bias), **tol)
    assert nerr(gemm_op(dropin, 0, A, B, None, np.zeros((M, N), np.float32), M, N, K), oracle.gemm_f64(A, B)) <= 1e-5


def test_known_answer_of_the_reference_cuda_test(dropin):
    # tests/test_cuda.c:169-191
    A = np.array([[1, 2], [3, 4]], np.float32)
    B = np.array([[5, 6], [7, 8]], np.float32)
    C = gemm_op(dropin, 0, A, B, None, np.zeros((2, 2), np.float32), 2, 2, 2)
    np.testing.assert_allclose(C, [[19, 22], [43, 50]], atol=1e-3)


def test_elementwise_slots_through_reference_dispatcher(dropin, oracle):
    X, bn, bm = oracle.uniform((37, 52), 3), oracle.uniform((52,), 4), oracle.uniform((37,), 6)
    out = np.zeros_like(X)
    for axis, b in ((1, bn), (0, bm)):
        rc = dropin.ref_device_elementwise(0, p(X), p(b), axis, p(out), i64(37), i64(52))
        assert rc == 0, dropin.ref_last_error()
        np.testing.assert_array_equal(out, oracle.bias_add_axis(X, b, axis))
    assert dropin.ref_device_elementwise(1, p(X), None, 0, p(out), i64(37), i64(52)) == 0
    np.testing.assert_array_equal(out, oracle.relu(X))
    assert dropin.ref_device_elementwise(2, p(X), None, 0, p(out), i64(37), i64(52)) == 0
    np.testing.assert_allclose(out, oracle.gelu(X), atol=1e-6)


@pytest.mark.parametrize("causal", [0, 1])
def test_sdpa_extension_slot(dropin, reference, oracle, causal):
    BH, S, dk = 6, 24, 16                                   # tests/test_attention.c:54-131 shape
    Q, K, V = oracle.normal((BH, S, dk), 41), oracle.normal((BH, S, dk), 43), oracle.normal((BH, S, dk), 47)
    O, L = np.zeros_like(Q), np.zeros((BH, S), np.float32)
    rc = dropin.ref_device_sdpa_fwd(p(Q), p(K), p(V), p(O), p(L), i64(BH), i64(S), i64(dk), ctypes.c_float(0.25), causal)
    assert rc == 0, dropin.ref_last_error()
    O_ref, L_ref = reference.sdpa_fwd(Q, K, V, 0.25, causal)
    assert np.abs(O - O_ref).max() < 1e-4 and np.abs(L - L_ref).max() < 1e-4


@pytest.mark.parametrize("case", [(2, 40, 2, 64, True), (3, 10, 2, 24, True), (1, 70, 3, 32, False), (1, 8, 2, 64, True)])
def test_qkv_head_gemm_slot(dropin, reference, oracle, case):
    """ax_compute_qkv_head_gemm dispatches into the qkv_head_gemm slot (the stock CUDA backend leaves it NULL)."""
    B, S, H, dk, with_bias = case
    D = H * dk
    X, W = oracle.uniform((B * S, D), 7), oracle.normal((D, 3 * D), 13, sigma=1.0 / np.sqrt(D))
    b = oracle.uniform((3 * D,), 29) if with_bias else None
    outs = [np.full((B * H, S, dk), np.nan, np.float32) for _ in range(3)]
    rc = dropin.ref_device_qkv_head_gemm(p(X), p(W), p(b), i64(B), i64(S), i64(H), i64(dk), *[p(t) for t in outs])
    assert rc == 0, (rc, dropin.ref_last_error())
    for got, want in zip(outs, reference.qkv_head_gemm(X, W, b, B, S, H, dk)):
        np.testing.assert_allclose(got, want, atol=1e-3, rtol=1e-4)
        assert nerr(got, want) <= 1e-5


@pytest.mark.parametrize("geom", [(8, 3, 12, 10, 3, 3, 1, 1, 1, 1), (16, 4, 9, 9, 3, 3, 2, 2, 0, 0), (12, 6, 14, 14, 5, 3, 2, 1, 2, 1)])
def test_conv_gemm_slot(dropin, reference, oracle, geom):
    """ax_compute_conv_gemm on device tensors made by the reference lands in the conv_gemm slot."""
    C_out, C_in, H, W, kh, kw, sh, sw, ph, pw = geom
    w, x = oracle.uniform((C_out, C_in * kh * kw), 7), oracle.uniform((C_in, H, W), 13)
    st, got = reference.conv_gemm(w, x, kh, kw, sh, sw, ph, pw, device=1)
    assert st == 0, (st, dropin.ref_last_error())
    st, want = reference.conv_gemm(w, x, kh, kw, sh, sw, ph, pw, device=0)
    assert st == 0
    np.testing.assert_allclose(got, want, atol=1e-3, rtol=1e-4)
    assert nerr(got, want) <= 1e-5


@pytest.mark.parametrize("shape", [(2, 64, 4, 32), (1, 40, 3, 16), (2, 128, 4, 64)])
def test_dattn_head_gemm_nt_slot(dropin, reference, oracle, shape):
    """ax_compute_dattn_head_gemm_nt on device tensors made by the reference lands in the dattn_head_gemm_nt slot (one
    tensor-core launch with a head-major epilogue for head dims that are multiples of 32, product + layout pass
    otherwise) and equals the reference's CPU implementation."""
    B, S, H, dk = shape
    D = H * dk
    dout, Wo = oracle.uniform((B * S, D), 7), oracle.normal((D, D), 13, sigma=1.0 / np.sqrt(D))
    got, want = np.full((B * H, S, dk), np.nan, np.float32), np.zeros((B * H, S, dk), np.float32)
    rc = dropin.ref_dattn_head_gemm_nt(p(dout), p(Wo), i64(B), i64(S), i64(H), i64(dk), p(got), 1)
    assert rc == 0, (rc, dropin.ref_last_error())
    assert dropin.ref_dattn_head_gemm_nt(p(dout), p(Wo), i64(B), i64(S), i64(H), i64(dk), p(want), 0) == 0
    np.testing.assert_allclose(got, want, atol=1e-3, rtol=1e-4)
    assert nerr(got, want) <= 1e-5


@pytest.mark.parametrize("shape", [(2, 64, 4, 32), (1, 40, 3, 16), (2, 128, 4, 64)])
@pytest.mark.parametrize("head_major", [0, 1])
def test_dwqkv_split_acc_slots(dropin, reference, oracle, shape, head_major):
    """ax_compute_dwqkv_split_acc[_hm] on device tensors made by the reference land in the two slots and accumulate
    into the three gradients what the reference's CPU implementation accumulates."""
    B, S, H, dk = shape
    D, rows = H * dk, B * S
    x, dqkv = oracle.uniform((rows, D), 7), oracle.normal((rows, 3 * D), 13, sigma=0.5)
    start = np.stack([oracle.uniform((D, D), 20 + i) for i in range(3)])
    if head_major:
        g = [np.ascontiguousarray(dqkv[:, i * D:(i + 1) * D].reshape(B, S, H, dk).transpose(0, 2, 1, 3)).reshape(B * H, S, dk)
             for i in range(3)]
    else:
        g = [dqkv, dqkv, dqkv]
    got, want = start.copy(), start.copy()
    rc = dropin.ref_dwqkv_split_acc(p(x), p(g[0]), p(g[1]), p(g[2]), head_major, i64(B), i64(S), i64(H), i64(dk), p(got), 1)
    assert rc == 0, (rc, dropin.ref_last_error())
    rc = dropin.ref_dwqkv_split_acc(p(x), p(g[0]), p(g[1]), p(g[2]), head_major, i64(B), i64(S), i64(H), i64(dk), p(want), 0)
    if rc and head_major:
        # the reference's CPU head-major form refuses widths that are not a multiple of its column panel
        # (src/compute/backends/cpu_opt.c:5841-5853); its flat form is the same sum
        want = start.copy()
        rc = dropin.ref_dwqkv_split_acc(p(x), p(dqkv), p(dqkv), p(dqkv), 0, i64(B), i64(S), i64(H), i64(dk), p(want), 0)
    assert rc == 0
    assert np.abs(want - start).max() > 0.1
    np.testing.assert_allclose(got, want, atol=1e-3, rtol=1e-4)
    assert nerr(got, want) <= 1e-5


@pytest.mark.parametrize("rows,D", [(128, 128), (40, 48), (256, 256)])
@pytest.mark.parametrize("forward", [1, 0])
def test_mha_output_proj_fused_slot(dropin, reference, oracle, rows, D, forward):
    """ax_compute_mha_output_proj_fused (and, with y and bo NULL, ax_compute_output_proj_bwd_fused's call) on device
    tensors made by the reference lands in the slot and equals the reference's CPU implementation."""
    attn, dout = oracle.uniform((rows, D), 7), oracle.normal((rows, D), 13, sigma=0.5)
    Wo, bo = oracle.normal((D, D), 17, sigma=1.0 / np.sqrt(D)), oracle.uniform((D,), 19)
    res = []
    for device in (1, 0):
        y, dattn = np.full((rows, D), np.nan, np.float32), np.full((rows, D), np.nan, np.float32)
        dWo, dbo = oracle.uniform((D, D), 23), oracle.uniform((D,), 29)
        rc = dropin.ref_mha_output_proj_fused(p(attn), p(Wo), p(bo) if forward else None, p(dout), p(y) if forward else None,
                                              p(dattn), p(dWo), p(dbo), i64(rows), i64(D), device)
        assert rc == 0, (device, rc, dropin.ref_last_error())
        res.append((y, dattn, dWo, dbo))
    for got, want in zip(res[0][0 if forward else 1:], res[1][0 if forward else 1:]):
        np.testing.assert_allclose(got, want, atol=1e-3, rtol=1e-4)
        assert nerr(got, want) <= 1e-5


@pytest.mark.parametrize("geom", [(3, 8, 4, 12, 12, 3, 3, 1, 1, 1, 1), (2, 16, 4, 9, 9, 3, 3, 2, 2, 0, 0), (4, 12, 6, 10, 16, 1, 1, 1, 1, 0, 0)])
def test_conv_gemm_batched_extension_slot(dropin, reference, oracle, geom):
    """The conv_gemm_batched slot, called as the reference's conv layer calls it on a device (N samples back to back,
    out [N, C_out, out_h*out_w]): every sample must match the reference's own CPU conv_gemm on that sample."""
    N, C_out, C_in, H, W, kh, kw, sh, sw, ph, pw = geom
    out_h, out_w = (H + 2 * ph - kh) // sh + 1, (W + 2 * pw - kw) // sw + 1
    w, x = oracle.uniform((C_out, C_in * kh * kw), 7), oracle.uniform((N, C_in, H, W), 13)
    got = np.full((N, C_out, out_h * out_w), np.nan, np.float32)
    rc = dropin.ref_device_conv_gemm_batched(p(w), p(x), i64(N), i64(C_out), i64(C_in), i64(H), i64(W), kh, kw, sh, sw, ph, pw,
                                             i64(out_h), i64(out_w), p(got))
    assert rc == 0, (rc, dropin.ref_last_error())
    for n in range(N):
        st, want = reference.conv_gemm(w, np.ascontiguousarray(x[n]), kh, kw, sh, sw, ph, pw, device=0)
        assert st == 0
        np.testing.assert_allclose(got[n], want, atol=1e-3, rtol=1e-4)
        assert nerr(got[n], want) <= 1e-5


@pytest.mark.parametrize("causal", [0, 1])
def test_sdpa_bwd_extension_slot(dropin, reference, oracle, causal):
    BH, S, dk = 6, 24, 16
    Q, K, V = oracle.normal((BH, S, dk), 41), oracle.normal((BH, S, dk), 43), oracle.normal((BH, S, dk), 47)
    dO = oracle.normal((BH, S, dk), 53)
    O, L = reference.sdpa_fwd(Q, K, V, 0.25, causal)
    grads = [np.full((BH, S, dk), np.nan, np.float32) for _ in range(3)]
    rc = dropin.ref_device_sdpa_bwd(p(Q), p(K), p(V), p(O), p(dO), p(L), *[p(t) for t in grads], i64(BH), i64(S), i64(dk),
                                    ctypes.c_float(0.25), causal)
    assert rc == 0, dropin.ref_last_error()
    for got, want in zip(grads, reference.sdpa_bwd(Q, K, V, O, dO, L, 0.25, causal)):
        assert np.abs(got - want).max() < 1e-4


def test_bias_add_axis0_is_per_row(dropin, oracle):
    """axis 0 broadcasts one value per ROW (the documented meaning of the slot), also for M != N."""
    M, N = 4, 6
    X, row_bias = oracle.uniform((M, N), 3), oracle.uniform((M,), 4)
    out = np.zeros((M, N), np.float32)
    assert dropin.ref_device_elementwise(0, p(X), p(row_bias), 0, p(out), i64(M), i64(N)) == 0
    np.testing.assert_array_equal(out, oracle.bias_add_axis(X, row_bias, 0))


# ---- the multi-head attention layer on the device -----------------------------------------------------------------

def mha_inputs(oracle, B, S, D, with_bias):
    x = oracle.uniform((B, S, D), 7)
    W = oracle.normal((4, D, D), 13, sigma=1.0 / np.sqrt(D))
    b = oracle.uniform((4, D), 29) if with_bias else None
    g = oracle.normal((B, S, D), 53)
    return x, W, b, g


@pytest.mark.parametrize("with_bias", [False, True])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(2, 128, 256, 4), (3, 50, 96, 4), (1, 16, 16, 2)])
def test_mha_layer_forward_on_device(dropin, reference, oracle, shape, causal, with_bias):
    """Inference forward of axiom's MHA layer, call by call through the dispatcher and the extension table on device
    tensors (fused-parameter builders, QKV GEMM on a mislabelled stack view, split, sdpa_fwd, merge, Wo GEMM, bias_add),
    against ax_layer_forward of the same layer on the reference's CPU backend; tests/test_attention.c tolerance 1e-4."""
    B, S, D, H = shape
    x, W, b, _ = mha_inputs(oracle, B, S, D, with_bias)
    from oracle_lib import mha_f64
    st, want = reference.mha_layer(x, W, b, H, causal)
    assert st == 0
    st, got = reference.mha_layer(x, W, b, H, causal, device=True)
    assert st == 0, (st, dropin.ref_last_error())
    assert np.abs(got["out"] - want["out"]).max() < 1e-4
    assert nerr(got["out"], want["out"]) <= 2e-5
    assert nerr(got["out"], mha_f64(x, W, b, H, causal)["out"]) <= 1e-5


@pytest.mark.parametrize("save_p", [False, True])
@pytest.mark.parametrize("with_bias", [False, True])
@pytest.mark.parametrize("causal", [False, True])
def test_mha_layer_training_step_on_device(dropin, reference, oracle, causal, with_bias, save_p):
    """Forward with L (and, when save_p, a P_save buffer handed on to sdpa_bwd as the layer does when P fits) and the
    layer's backward sequence (gemm_tn with skip_init, gemm_nt, head_interleave, sdpa_bwd, qkv_merge, gemm_tn, gemm_nt)
    on the device.  The forward is checked against ax_layer_forward of the reference's CPU backend and against the
    double-precision restatement of the layer; the gradients against the restatement only.  The reference's own CPU
    backward is not repeatable at this shape: its dX / dW change with the number of OpenMP threads and with the presence
    of (even all-zero) biases, and disagree with a float64 evaluation by 10 % and more (tests/test_mha_reference_defect.py
    records this on the CPU).  The pieces of the restatement's backward — the GEMMs and the attention backward — are
    each pinned against the reference separately (golden vectors of ax_compute_gemm* and ax_fused_attention_bwd)."""
    from oracle_lib import mha_f64
    B, S, D, H = 2, 128, 256, 4
    x, W, b, g = mha_inputs(oracle, B, S, D, with_bias)
    st, ref = reference.mha_layer(x, W, b, H, causal, dOut=g)
    assert st == 0
    want = mha_f64(x, W, b, H, causal, dOut=g)
    st, got = reference.mha_layer(x, W, b, H, causal, dOut=g, device=True, save_p=save_p)
    assert st == 0, (st, dropin.ref_last_error())
    assert np.abs(got["out"] - ref["out"]).max() < 1e-4
    for key in ("out", "dX", "dW") + (("db",) if with_bias else ()):
        assert nerr(got[key], want[key]) <= 1e-5, key
    if save_p:
        assert np.abs(got["P"] - want["P"]).max() < 1e-5
        if causal:
            assert np.all(got["P"][:, np.triu(np.ones((S, S), bool), 1)] == 0.0)


def test_sdpa_fwd_saved_probabilities(engine, oracle):
    """P_save != NULL: O and L are still produced (axiom's caller ignores the status) and P holds the soft-max
    probabilities, also on the FMA route (head dim 72) and without an L buffer."""
    import torch
    for (BH, S, dk, causal, with_L) in [(3, 200, 64, 1, True), (2, 130, 72, 0, True), (2, 64, 32, 1, False)]:
        Q, K, V = oracle.normal((BH, S, dk), 41), oracle.normal((BH, S, dk), 43), oracle.normal((BH, S, dk), 47)
        dev = lambda a: torch.from_numpy(a).cuda()
        O = torch.full((BH, S, dk), float("nan"), device="cuda")
        L = torch.full((BH, S), float("nan"), device="cuda") if with_L else None
        P = torch.full((BH, S, S), float("nan"), device="cuda")
        scale = 1.0 / np.sqrt(dk)
        engine.sdpa_fwd(dev(Q), dev(K), dev(V), O, L, scale, causal, P_save=P)
        O64, L64 = oracle.sdpa_fwd_f64(Q, K, V, scale, causal)
        assert np.abs(O.cpu().numpy() - O64).max() < 1e-5
        if with_L:
            assert np.abs(L.cpu().numpy() - L64).max() < 1e-5
        s = np.einsum("hid,hjd->hij", Q.astype(np.float64), K.astype(np.float64)) * scale
        if causal:
            s = np.where(np.triu(np.ones((S, S), bool), 1), -np.inf, s)
        P64 = np.exp(s - L64[:, :, None])
        assert np.abs(P.cpu().numpy() - P64).max() < 1e-5


@pytest.mark.parametrize("case", [(2, 40, 4, 64), (3, 7, 2, 24), (1, 130, 3, 5), (2, 1, 1, 16)])
def test_head_layout_slots_bit_exact(engine, reference, oracle, case):
    """The five layout slots against the CPU helpers of the reference's attention layer: pure moves, so every bit
    matches (the bias variant adds one fp32 value per element, in the same order)."""
    import torch
    B, S, H, dk = case
    D = H * dk
    dev = lambda a: torch.from_numpy(a).cuda()
    nan = lambda *sh: torch.full(sh, float("nan"), device="cuda")
    qkv, bias, flat = oracle.uniform((B * S, 3 * D), 3), oracle.uniform((3 * D,), 4), oracle.uniform((B * S, D), 5)
    heads = [oracle.uniform((B * H, S, dk), 11 + i) for i in range(3)]
    for bz in (None, bias):
        outs = [nan(B * H, S, dk) for _ in range(3)]
        engine.head_interleave_qkv_split(dev(qkv), None if bz is None else dev(bz), *outs, B, S, H, dk)
        for got, want in zip(outs, reference.head_layout("split", B, S, H, dk, flat=qkv, bias=bz)):
            np.testing.assert_array_equal(got.cpu().numpy(), want)
    o = nan(B * H, S, dk)
    engine.head_interleave(dev(flat), o, B, S, H, dk)
    np.testing.assert_array_equal(o.cpu().numpy(), reference.head_layout("interleave", B, S, H, dk, flat=flat))
    o = nan(B * S, D)
    engine.head_deinterleave(dev(heads[0]), o, B, S, H, dk)
    np.testing.assert_array_equal(o.cpu().numpy(), reference.head_layout("deinterleave", B, S, H, dk, heads=heads[0]))
    o = nan(B * S, 3 * D)
    engine.head_deinterleave_qkv_merge(*[dev(h) for h in heads], o, B, S, H, dk)
    np.testing.assert_array_equal(o.cpu().numpy(), reference.head_layout("merge", B, S, H, dk, heads=heads))
    # the fused-parameter builders
    w = [oracle.uniform((D, D), 21 + i) for i in range(3)]
    bq = [oracle.uniform((D,), 31 + i) for i in range(3)]
    Wc, bc = nan(D, 3 * D), nan(3 * D)
    engine.qkv_cache_build(Wc, *[dev(t) for t in w], D)
    engine.bias_cache_build(bc, *[dev(t) for t in bq], D)
    np.testing.assert_array_equal(Wc.cpu().numpy(), np.concatenate(w, axis=1))
    np.testing.assert_array_equal(bc.cpu().numpy(), np.concatenate(bq))


def test_device_label_is_checked_against_the_pointer(engine):
    """Host memory is never handed to a kernel, whatever a tensor's storage label says."""
    import torch
    h = np.zeros(16, np.float32)
    d = torch.zeros(16, device="cuda")
    assert engine.pointer_on_device(d.data_ptr()) and not engine.pointer_on_device(h.ctypes.data)
    assert not engine.pointer_on_device(0)


@pytest.mark.parametrize("shape", [(200, 384, 512), (64, 1024, 256), (1024, 1024, 1024)])
def test_dense_layer_weight_reuse_and_in_place_update(dropin, reference, oracle, shape):
    """The same device-resident weight tensor through the dispatcher again and again (the host layer keeps its operand
    planes from the second call on), then overwritten in place: every product must match the reference's CPU backend,
    the ones after the update with the NEW weights."""
    M, N, K = shape
    reps = 4
    As = np.stack([oracle.uniform((M, K), 7 + r) for r in range(reps)])
    B, B2, bias = oracle.uniform((K, N), 13), oracle.uniform((K, N), 113), oracle.uniform((N,), 29)
    out = np.full((reps + 1, M, N), np.nan, np.float32)
    rc = dropin.ref_device_dense_repeat(p(As), p(B), p(B2), p(bias), p(out), i64(M), i64(N), i64(K), reps)
    assert rc == 0, (rc, dropin.ref_last_error())
    for r in range(reps + 1):
        a = As[min(r, reps - 1)]
        w = B if r < reps else B2
        np.testing.assert_allclose(out[r], reference.gemm_relu(a, w, bias), atol=1e-3, rtol=1e-4)
        assert nerr(out[r], np.maximum(oracle.gemm_f64(a, w) + bias, 0)) <= 1e-5, r
