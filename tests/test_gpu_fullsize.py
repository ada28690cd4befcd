"""Full-size checks at the full benchmark configurations, through properties that do not need a full CPU
recomputation: sampled rows against the oracle (bit-exact for integers, normalised error for fp32),
linearity, and row-shard consistency (the multi-GPU row partition gives the same bits as the whole)."""
import numpy as np
import pytest
import torch

from oracle_lib import nerr

pytestmark = pytest.mark.gpu


def test_fp32_gemm_8192_sampled_rows_and_linearity(engine, oracle):
    n = 8192
    g = torch.Generator(device="cuda").manual_seed(7)
    A = torch.rand((n, n), device="cuda", generator=g) * 2 - 1
    B = torch.rand((n, n), device="cuda", generator=g) * 2 - 1
    C = torch.empty((n, n), device="cuda")
    engine.gemm(A, B, C)
    rows = np.array([0, 1, 127, 128, 255, 256, 4095, 4096, 8190, 8191])
    ref = oracle.gemm_f64(np.ascontiguousarray(A[rows].cpu().numpy()), B.cpu().numpy())
    got = C[rows].cpu().numpy()
    assert np.isfinite(got).all()
    assert nerr(got, ref) <= 1e-5, nerr(got, ref)                      # 3xTF32 tolerance at K = 8192
    # linearity: (2A).B == 2 (A.B) exactly (scaling by 2 commutes with every rounding in the split and the sums)
    C2 = torch.empty((n, n), device="cuda")
    engine.gemm(A * 2, B, C2)
    assert torch.equal(C2, C * 2)
    # row shards reproduce the whole bit for bit (what bench.py --gpus N relies on)
    half = torch.empty((n // 2, n), device="cuda")
    engine.gemm(A[n // 2:].contiguous(), B, half)
    assert torch.equal(half, C[n // 2:])
    # bf16 mode at full size stays inside its own tolerance
    engine.set_fp32_mode("bf16")
    try:
        engine.gemm(A, B, C2)
    finally:
        engine.set_fp32_mode("3xtf32")
    assert nerr(C2[rows].cpu().numpy(), ref) <= 5e-3


def test_int8_gemm_16384_sampled_rows_bit_exact(engine, oracle):
    n = 16384
    a = torch.randint(-127, 128, (n, n), device="cuda", dtype=torch.int8)
    b = torch.randint(-127, 128, (n, n), device="cuda", dtype=torch.int8)
    bs = (torch.rand((n,), device="cuda") * 0.019 + 0.001)
    q = torch.empty((n, n), device="cuda", dtype=torch.int8)
    a_scale, out_scale = 0.02, 0.02 * 0.0105 * 5373.0 * 128.0 / 50.0
    engine.qgemm_w8a8(a, a_scale, b, bs, out_scale, q, None)
    rows = np.array([0, 255, 256, 8191, 8192, 16383])
    acc_ref, q_ref = oracle.qgemm_w8a8(np.ascontiguousarray(a[rows].cpu().numpy()), a_scale, b.cpu().numpy(),
                                       bs.cpu().numpy(), out_scale)
    np.testing.assert_array_equal(q[rows].cpu().numpy(), q_ref)
    # a checksum of checksums over the whole output against the same kernel run on row shards
    total = int(q.to(torch.int64).sum().item())
    parts = 0
    for r0 in range(0, n, n // 4):
        qs = torch.empty((n // 4, n), device="cuda", dtype=torch.int8)
        engine.qgemm_w8a8(a[r0:r0 + n // 4], a_scale, b, bs, out_scale, qs, None)
        assert torch.equal(qs, q[r0:r0 + n // 4])
        parts += int(qs.to(torch.int64).sum().item())
    assert parts == total
    # s32 accumulators on a slab, exact
    acc = torch.empty((256, n), device="cuda", dtype=torch.int32)
    engine.qgemm_w8a8(a[:256], a_scale, b, None, 1.0, None, acc)
    np.testing.assert_array_equal(acc[rows[:2]].cpu().numpy(), acc_ref[:2])


def test_sdpa_config4_full(engine, oracle):
    BH, S, dk = 128, 1024, 64
    g = torch.Generator(device="cuda").manual_seed(41)
    Q, K, V = (torch.randn((BH, S, dk), device="cuda", generator=g) for _ in range(3))
    O = torch.empty_like(Q)
    L = torch.empty((BH, S), device="cuda")
    engine.sdpa_fwd(Q, K, V, O, L, 0.125, True)
    heads = [0, 63, 127]
    O64, L64 = oracle.sdpa_fwd_f64(Q[heads].cpu().numpy(), K[heads].cpu().numpy(), V[heads].cpu().numpy(), 0.125, 1)
    assert np.abs(O[heads].cpu().numpy() - O64).max() < 1e-5
    assert np.abs(L[heads].cpu().numpy() - L64).max() < 1e-5
    # causality: changing keys/values after position t must not change outputs up to t
    K2, V2 = K.clone(), V.clone()
    K2[:, 512:] = 0
    V2[:, 512:] = 7
    O2 = torch.empty_like(Q)
    engine.sdpa_fwd(Q, K2, V2, O2, None, 0.125, True)
    assert torch.equal(O2[:, :512], O[:, :512])


def test_mlp_chain_rows_vs_columns_single_gpu(engine, oracle):
    """The two sharding schemes on one GPU (world emulated by looping over ranks) against the oracle."""
    from axiom_b200.multi_gpu import ColumnShardedMLP, RowShardedMLP, gathered_to_full, shard_bounds
    dims, batch, world = [256, 512, 384, 128], 192, 2
    Ws = [oracle.normal((dims[i], dims[i + 1]), 10 + i, sigma=1 / np.sqrt(dims[i])) for i in range(3)]
    bs = [oracle.uniform((dims[i + 1],), 20 + i) for i in range(3)]
    x = oracle.uniform((batch, dims[0]), 3)
    h = x
    for W, b in zip(Ws, bs):
        h = oracle.bias_act(oracle.gemm(h, W), b, "gelu")
    new_empty = lambda shape: torch.empty(shape, device="cuda", dtype=torch.float32)
    dW, db, dx = [torch.from_numpy(W).cuda() for W in Ws], [torch.from_numpy(b).cuda() for b in bs], torch.from_numpy(x).cuda()
    y = RowShardedMLP(engine, dW, db).forward(dx, new_empty)
    assert nerr(y.cpu().numpy(), h) <= 1e-5
    # columns: run rank 0 and rank 1 in turn; the "all-gather" copies both slabs computed so far
    slabs = [[W[:, slice(*shard_bounds(W.shape[1], world, r))].contiguous() for W in dW] for r in range(world)]
    bslabs = [[b[slice(*shard_bounds(b.shape[0], world, r))].contiguous() for b in db] for r in range(world)]
    # layer by layer, emulating the collective
    chunks = [dx]
    for l in range(3):
        outs = []
        for r in range(world):
            M, n = chunks[0].shape[0], slabs[r][l].shape[1]
            slab = new_empty((M, n))
            k0 = 0
            for c, xc in enumerate(chunks):
                kc = xc.shape[1]
                last = c == len(chunks) - 1
                engine.gemm_bias_act(xc, slabs[r][l][k0:k0 + kc], bslabs[r][l] if last else None, slab, M, n, kc,
                                     beta=0.0 if c == 0 else 1.0, act="gelu" if last else "none")
                k0 += kc
            outs.append(slab)
        gathered = torch.stack(outs)
        chunks = [gathered[r] for r in range(world)]
    assert nerr(gathered_to_full(gathered).cpu().numpy(), h) <= 1e-5


def test_scatter_epilogue_writes_every_destination(engine, oracle):
    """axb_gemm_bias_act_scatter on one GPU: the extra destinations (stand-ins for peers' gather buffers)
    receive exactly what C receives, for an accumulating call with bias and activation, ragged shape included."""
    for (M, N, K) in [(512, 768, 320), (300, 520, 200)]:
        A, B, bias, C0 = oracle.uniform((M, K), 7), oracle.uniform((K, N), 13), oracle.uniform((N,), 29), oracle.uniform((M, N), 5)
        dA, dB, db = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), torch.from_numpy(bias).cuda()
        C = torch.from_numpy(C0).cuda()
        extras = [torch.full((M, N), float("nan"), device="cuda") for _ in range(3)]
        engine.gemm_bias_act_scatter(dA, dB, db, C, extras, M, N, K, beta=1.0, act="gelu")
        want = torch.from_numpy(C0).cuda()
        engine.gemm_bias_act(dA, dB, db, want, M, N, K, beta=1.0, act="gelu")
        assert torch.equal(C, want)
        for e in extras:
            assert torch.equal(e, want)
        ref = oracle.gelu(np.ascontiguousarray((oracle.gemm_f64(A, B) + C0 + bias).astype(np.float32)))
        assert nerr(C.cpu().numpy(), ref) <= 1e-5


def test_gathered_operand_gemm(engine, oracle):
    """axb_gemm_gathered_scatter reads a [g][M][kc] gather buffer in place as the [M, g*kc] operand."""
    g, M, kc, N = 4, 300, 96, 200
    A = oracle.uniform((M, g * kc), 7)
    B, bias = oracle.uniform((g * kc, N), 13), oracle.uniform((N,), 29)
    gathered = np.ascontiguousarray(A.reshape(M, g, kc).transpose(1, 0, 2))     # [g][M][kc]
    out = torch.full((M, N), float("nan"), device="cuda")
    extra = torch.full((M, N), float("nan"), device="cuda")
    engine.gemm_gathered_scatter(torch.from_numpy(gathered).cuda(), g, kc, torch.from_numpy(B).cuda(),
                                 torch.from_numpy(bias).cuda(), out, [extra], M, N, act="relu")
    want = torch.empty((M, N), device="cuda")
    engine.gemm_bias_act(torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), torch.from_numpy(bias).cuda(), want, M, N, g * kc,
                         act="relu")
    assert torch.equal(out, want) and torch.equal(extra, want)
    assert nerr(out.cpu().numpy(), np.maximum(oracle.gemm_f64(A, B) + bias, 0)) <= 1e-5


@pytest.mark.parametrize("shape", [(300, 200, 4, 96), (1024, 1024, 8, 128), (2560, 2560, 2, 256)])
def test_prepared_weight_scatter(engine, oracle, shape):
    """axb_gemm_prepared_scatter (the weight's operand planes made once) gives the bits of axb_gemm_bias_act on the same
    operands, from a plain left operand and from a [g][M][kc] gather buffer, in C and in every extra destination."""
    M, N, g, kc = shape
    K = g * kc
    A, B, bias = oracle.uniform((M, K), 7), oracle.uniform((K, N), 13), oracle.uniform((N,), 29)
    Ad, Bd, bd = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), torch.from_numpy(bias).cuda()
    want = torch.empty((M, N), device="cuda")
    engine.gemm_bias_act(Ad, Bd, bd, want, M, N, K, act="gelu")
    w = engine.weight_prepare(Bd)
    try:
        out, extra = torch.full((M, N), float("nan"), device="cuda"), torch.full((M, N), float("nan"), device="cuda")
        engine.gemm_prepared_scatter(Ad, 0, 0, w, bd, out, [extra], M, act="gelu")
        assert torch.equal(out, want) and torch.equal(extra, want)
        gathered = torch.from_numpy(np.ascontiguousarray(A.reshape(M, g, kc).transpose(1, 0, 2))).cuda()
        out2, extra2 = torch.full((M, N), float("nan"), device="cuda"), torch.full((M, N), float("nan"), device="cuda")
        engine.gemm_prepared_scatter(gathered, g, kc, w, bd, out2, [extra2], M, act="gelu")
        assert torch.equal(out2, want) and torch.equal(extra2, want)
        from axiom_b200.engine import EngineError
        with pytest.raises(EngineError):
            engine.gemm_prepared_scatter(gathered, g, kc + 4, w, bd, out2, [], M)      # chunks * chunk_k != K
    finally:
        engine.weight_release(w)
    assert engine.device_error() == 0
