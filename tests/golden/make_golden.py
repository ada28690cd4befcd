"""Regenerates tests/golden/axiom_ref_vectors.npz from the UNMODIFIED axiom reference.

Run where the reference was compiled (`make -C oracle ref`):

    python tests/golden/make_golden.py

Every case stores only (a) the seeds/shapes that rebuild its inputs through the
oracle's xorshift32 generators and (b) the OUTPUT the reference produced on
them, so the file stays a few hundred KB and travels to machines that have no
reference tree.  The known-answer entries (`kat_*`) are the literal expected
values written in the reference's own tests (tests/test_compute.c:162-199,
tests/test_cuda.c:169-191), read as text.  The `w8a8_*` entries have no reference
counterpart (the reference has no int8 x int8 kernel): they are computed here
with numpy int64 arithmetic, independently of the C oracle they pin.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from oracle_lib import Oracle, Reference  # noqa: E402

GEMM_CASES = [  # name, M, N, K
    ("g_small", 5, 7, 3), ("g_cuda_test", 64, 32, 128), ("g_odd", 33, 17, 65),
    ("g_96", 96, 96, 96), ("g_k1", 9, 11, 1), ("g_skinny1", 1, 192, 160), ("g_skinny8", 8, 130, 257),
]
SDPA_CASES = [("s_test", 6, 24, 16, 0.25), ("s_c4like", 3, 80, 64, 0.125)]
# (name, C_out, C_in, H, W, kh, kw, sh, sw, ph, pw)
CONV_CASES = [("conv_3x3_same", 8, 3, 12, 10, 3, 3, 1, 1, 1, 1), ("conv_3x3_s2", 16, 4, 9, 9, 3, 3, 2, 2, 0, 0),
              ("conv_1x1", 5, 2, 7, 8, 1, 1, 1, 1, 0, 0), ("conv_5x3_mixed", 12, 6, 14, 14, 5, 3, 2, 1, 2, 1)]
# (name, B, S, H, dk, bias): the fast-path shape class (dk = 64), a head dim off the fast path, no bias
QKV_CASES = [("qkv_64", 2, 40, 2, 64, 1), ("qkv_24", 3, 10, 2, 24, 1), ("qkv_32_nobias", 1, 70, 3, 32, 0)]
# (name, BH, max_seq, cur_len, dk): the reference test's shape, a ragged one, a longer cache at the config-4 head dim
KV_CASES = [("kv_test", 2, 16, 5, 8), ("kv_ragged", 3, 50, 37, 20), ("kv_c4like", 4, 512, 300, 64)]


def main():
    o, r = Oracle(), Reference()
    out = {}
    # -- literal known answers from the reference's tests
    out["kat_gemm_2x3x2_a"] = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    out["kat_gemm_2x3x2_b"] = np.array([[7, 8], [9, 10], [11, 12]], np.float32)
    out["kat_gemm_2x3x2_c"] = np.array([[58, 64], [139, 154]], np.float32)
    out["kat_gemm_2x2_a"] = np.array([[1, 2], [3, 4]], np.float32)
    out["kat_gemm_2x2_b"] = np.array([[5, 6], [7, 8]], np.float32)
    out["kat_gemm_2x2_c"] = np.array([[19, 22], [43, 50]], np.float32)

    for name, M, N, K in GEMM_CASES:
        A, B = o.uniform((M, K), 7), o.uniform((K, N), 13)
        bias = o.uniform((N,), 29)
        Cin = o.uniform((M, N), 5)
        out[name + "_shape"] = np.array([M, N, K], np.int64)
        out[name + "_nn"] = r.gemm(A, B)
        out[name + "_nn_naive"] = r.gemm(A, B, backend="naive")
        out[name + "_nt"] = r.gemm(A, np.ascontiguousarray(B.T), "nt")
        out[name + "_tn"] = r.gemm(np.ascontiguousarray(A.T), B, "tn")
        out[name + "_relu"] = r.gemm_relu(A, B, bias)
        out[name + "_gelu"] = r.dense_gelu(A, B, bias)
        out[name + "_ex"] = r.gemm_ex(A, B, 0.5, 2.0, Cin)

    # activations on a fixed grid (ax_gelu's SIMD tanh differs from libm by ~1e-6)
    x = np.linspace(-6, 6, 1537).astype(np.float32)
    out["gelu_x"] = x
    out["gelu_y"] = r.gelu(x)

    # quantiser + W8A32 at the shapes tests/test_quantize.c:133-137 uses (seeds 7 / 13)
    for M, N, K in [(1, 8, 8), (4, 16, 32), (8, 64, 128), (32, 128, 512), (16, 256, 1024)]:
        a, w = o.uniform((M, K), 7), o.uniform((N, K), 13)
        q, s = r.quantize(w)
        tag = f"q_{M}_{N}_{K}"
        if N * K <= 64 * 128:
            out[tag + "_q"] = q
        out[tag + "_qsum"] = np.array([int(q.astype(np.int64).sum()), int(np.abs(q.astype(np.int64)).sum())], np.int64)
        out[tag + "_scales"] = s
        out[tag + "_out"] = r.qgemm_w8a32(a, q, s)

    for name, BH, S, dk, scale in SDPA_CASES:
        Q, K_, V = o.normal((BH, S, dk), 41), o.normal((BH, S, dk), 43), o.normal((BH, S, dk), 47)
        out[name + "_shape"] = np.array([BH, S, dk], np.int64)
        out[name + "_scale"] = np.array([scale], np.float32)
        for causal in (0, 1):
            O, L = r.sdpa_fwd(Q, K_, V, scale, causal)
            out[f"{name}_c{causal}_O"] = O
            out[f"{name}_c{causal}_L"] = L
            dO = o.normal((BH, S, dk), 53)
            dq, dk_, dv = r.sdpa_bwd(Q, K_, V, O, dO, L, scale, causal)   # ax_fused_attention_bwd[_causal]
            out[f"{name}_c{causal}_dQ"], out[f"{name}_c{causal}_dK"], out[f"{name}_c{causal}_dV"] = dq, dk_, dv

    # KV-cache single-token attention (tests/test_attention.c:268-330 shape first, then longer caches)
    for name, BH, max_seq, cur_len, dk in KV_CASES:
        Kc, Vc = o.normal((BH, max_seq, dk), 43), o.normal((BH, max_seq, dk), 47)
        Qn = o.normal((BH, dk), 41)
        scale = np.float32(1.0 / np.sqrt(dk))
        out[name + "_shape"] = np.array([BH, max_seq, cur_len, dk], np.int64)
        out[name + "_out"] = r.kv_cache_attend(Kc, Vc, Qn, cur_len, scale)

    # fused QKV projection + head-major split (ax_compute_qkv_head_gemm)
    for name, B, S, H, dk, with_bias in QKV_CASES:
        D = H * dk
        X, W = o.uniform((B * S, D), 7), o.normal((D, 3 * D), 13, sigma=1.0 / np.sqrt(D))
        b = o.uniform((3 * D,), 29) if with_bias else None
        out[name + "_shape"] = np.array([B, S, H, dk, int(with_bias)], np.int64)
        q, k, v = r.qkv_head_gemm(X, W, b, B, S, H, dk)
        out[name + "_q"], out[name + "_k"], out[name + "_v"] = q, k, v

    # implicit-im2col convolution GEMM of one sample (ax_compute_conv_gemm on the CPU backend)
    for name, C_out, C_in, H, W, kh, kw, sh, sw, ph, pw in CONV_CASES:
        w, x = o.uniform((C_out, C_in * kh * kw), 7), o.uniform((C_in, H, W), 13)
        st, y = r.conv_gemm(w, x, kh, kw, sh, sw, ph, pw)
        assert st == 0, st
        out[name + "_geom"] = np.array([C_out, C_in, H, W, kh, kw, sh, sw, ph, pw], np.int64)
        out[name + "_out"] = y

    # -- W8A8 known answers (numpy, independent of the C oracle)
    rng = np.random.RandomState(1234)
    for i, (M, N, K) in enumerate([(4, 8, 16), (3, 5, 33), (16, 24, 128)]):
        a = rng.randint(-127, 128, size=(M, K)).astype(np.int8)
        b = rng.randint(-127, 128, size=(N, K)).astype(np.int8)
        bs = rng.uniform(0.001, 0.02, size=(N,)).astype(np.float32)
        a_scale, out_scale = np.float32(0.031), np.float32(0.9 + 0.3 * i)
        acc = (a.astype(np.int64) @ b.T.astype(np.int64)).astype(np.int32)
        mult = ((a_scale * bs).astype(np.float32) / out_scale).astype(np.float32)
        y = (acc.astype(np.float32) * mult[None, :]).astype(np.float32)
        qv = np.clip(np.rint(y), -127, 127).astype(np.int8)   # np.rint = round-half-even
        out[f"w8a8_{i}_a"], out[f"w8a8_{i}_b"], out[f"w8a8_{i}_bs"] = a, b, bs
        out[f"w8a8_{i}_scales"] = np.array([a_scale, out_scale], np.float32)
        out[f"w8a8_{i}_acc"], out[f"w8a8_{i}_q"] = acc, qv
    # hand-checkable: ones x ones with K=16 -> acc 16 everywhere; ties round to even
    out["w8a8_tie_acc"] = np.array([[1, 3, 5, -1, -3, 250, -250]], np.int32)   # * 0.5 -> .5 ties
    out["w8a8_tie_q"] = np.array([[0, 2, 2, 0, -2, 125, -125]], np.int8)

    path = os.path.join(HERE, "axiom_ref_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
