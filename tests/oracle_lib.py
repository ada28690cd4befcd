"""ctypes doors to the two CPU checkers (test infrastructure only).

``Oracle``  wraps ``oracle/liboracle.so`` — the plain-C restatement.
``Reference`` wraps ``oracle/_ref/libaxiom_ref.so`` — the unmodified axiom
reference compiled from its own sources (present only where that tree was
available at build time; tests that need it skip otherwise).

Only tests, the smoke check and the bench's CPU-baseline leg import this.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_SO = os.path.join(ORACLE_DIR, "liboracle.so")
REF_SO = os.path.join(ORACLE_DIR, "_ref", "libaxiom_ref.so")

_f32p = C.POINTER(C.c_float)
_f64p = C.POINTER(C.c_double)
_i8p = C.POINTER(C.c_int8)
_i32p = C.POINTER(C.c_int32)
_i64 = C.c_int64


def _p(a, typ):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(typ)


def build_oracle():
    """Compile oracle/liboracle.so (and oracle/_ref when the axiom tree exists)."""
    subprocess.run(["make", "-C", ORACLE_DIR, "-j8", "all"], check=True,
                   stdout=subprocess.DEVNULL)


class Oracle:
    def __init__(self):
        if not os.path.exists(ORACLE_SO):
            build_oracle()
        self.lib = C.CDLL(ORACLE_SO)
        L = self.lib
        L.orc_num_threads.restype = C.c_int

    # ---- seeded inputs -------------------------------------------------
    def uniform(self, shape, seed):
        out = np.empty(shape, np.float32)
        self.lib.orc_fill_uniform(_p(out, _f32p), _i64(out.size), C.c_uint32(seed))
        return out

    def normal(self, shape, seed, sigma=1.0):
        out = np.empty(shape, np.float32)
        self.lib.orc_fill_normal(_p(out, _f32p), _i64(out.size), C.c_uint32(seed), C.c_float(sigma))
        return out

    def int8(self, shape, seed):
        out = np.empty(shape, np.int8)
        self.lib.orc_fill_int8(_p(out, _i8p), _i64(out.size), C.c_uint32(seed))
        return out

    def frange(self, shape, seed, lo, hi):
        out = np.empty(shape, np.float32)
        self.lib.orc_fill_range(_p(out, _f32p), _i64(out.size), C.c_uint32(seed),
                                C.c_float(lo), C.c_float(hi))
        return out

    # ---- GEMM family ---------------------------------------------------
    def gemm(self, A, B, ta=False, tb=False):
        M = A.shape[1] if ta else A.shape[0]
        K = A.shape[0] if ta else A.shape[1]
        N = B.shape[0] if tb else B.shape[1]
        out = np.empty((M, N), np.float32)
        self.lib.orc_gemm_f32(_p(A, _f32p), _p(B, _f32p), _p(out, _f32p),
                              _i64(M), _i64(N), _i64(K), int(ta), int(tb))
        return out

    def gemm_f64(self, A, B, ta=False, tb=False):
        M = A.shape[1] if ta else A.shape[0]
        K = A.shape[0] if ta else A.shape[1]
        N = B.shape[0] if tb else B.shape[1]
        out = np.empty((M, N), np.float64)
        self.lib.orc_gemm_f64(_p(A, _f32p), _p(B, _f32p), _p(out, _f64p),
                              _i64(M), _i64(N), _i64(K), int(ta), int(tb))
        return out

    def gemm_ex(self, A, B, alpha, beta, Cin):
        M, K = A.shape
        N = B.shape[1]
        out = np.array(Cin, dtype=np.float32, copy=True)
        self.lib.orc_gemm_ex_f32(_p(A, _f32p), _p(B, _f32p), C.c_float(alpha), C.c_float(beta),
                                 _p(out, _f32p), _i64(M), _i64(N), _i64(K))
        return out

    def bias_act(self, X, bias, act):
        M, N = X.shape
        out = np.empty_like(X)
        self.lib.orc_bias_act(_p(X, _f32p), _p(bias, _f32p), _p(out, _f32p),
                              _i64(M), _i64(N), {"none": 0, "relu": 1, "gelu": 2}[act])
        return out

    def bias_add_axis(self, X, bias, axis):
        M, N = X.shape
        out = np.empty_like(X)
        self.lib.orc_bias_add_axis(_p(X, _f32p), _p(bias, _f32p), int(axis), _p(out, _f32p),
                                   _i64(M), _i64(N))
        return out

    def gelu(self, X):
        out = np.empty_like(X)
        self.lib.orc_gelu(_p(X, _f32p), _p(out, _f32p), _i64(X.size))
        return out

    def relu(self, X):
        out = np.empty_like(X)
        self.lib.orc_relu(_p(X, _f32p), _p(out, _f32p), _i64(X.size))
        return out

    # ---- quantised -----------------------------------------------------
    def quantize_rows(self, W):
        N, K = W.shape
        q = np.empty((N, K), np.int8)
        s = np.empty((N,), np.float32)
        self.lib.orc_quantize_rows(_p(W, _f32p), _i64(N), _i64(K), _p(q, _i8p), _p(s, _f32p))
        return q, s

    def dequantize_rows(self, q, s):
        N, K = q.shape
        out = np.empty((N, K), np.float32)
        self.lib.orc_dequantize_rows(_p(q, _i8p), _p(s, _f32p), _i64(N), _i64(K), _p(out, _f32p))
        return out

    def qgemm_w8a32(self, a, q, s):
        M, K = a.shape
        N = q.shape[0]
        out = np.empty((M, N), np.float32)
        self.lib.orc_qgemm_w8a32(_p(a, _f32p), _p(q, _i8p), _p(s, _f32p), _p(out, _f32p),
                                 _i64(M), _i64(N), _i64(K))
        return out

    def qgemm_w8a32_f64(self, a, q, s):
        M, K = a.shape
        N = q.shape[0]
        out = np.empty((M, N), np.float64)
        self.lib.orc_qgemm_w8a32_f64(_p(a, _f32p), _p(q, _i8p), _p(s, _f32p), _p(out, _f64p),
                                     _i64(M), _i64(N), _i64(K))
        return out

    def qgemm_w8a8(self, a_q, a_scale, b_q, b_scales, out_scale):
        M, K = a_q.shape
        N = b_q.shape[0]
        acc = np.empty((M, N), np.int32)
        out = np.empty((M, N), np.int8)
        self.lib.orc_qgemm_w8a8(_p(a_q, _i8p), C.c_float(a_scale), _p(b_q, _i8p),
                                _p(b_scales, _f32p), C.c_float(out_scale),
                                _p(acc, _i32p), _p(out, _i8p), _i64(M), _i64(N), _i64(K))
        return acc, out

    # ---- attention -----------------------------------------------------
    def sdpa_fwd(self, Q, K, V, scale, causal):
        BH, S, dk = Q.shape
        O = np.empty_like(Q)
        L = np.empty((BH, S), np.float32)
        self.lib.orc_sdpa_fwd(_p(Q, _f32p), _p(K, _f32p), _p(V, _f32p), _p(O, _f32p), _p(L, _f32p),
                              _i64(BH), _i64(S), _i64(dk), C.c_float(scale), int(causal))
        return O, L

    def sdpa_fwd_f64(self, Q, K, V, scale, causal):
        BH, S, dk = Q.shape
        O = np.empty(Q.shape, np.float64)
        L = np.empty((BH, S), np.float64)
        self.lib.orc_sdpa_fwd_f64(_p(Q, _f32p), _p(K, _f32p), _p(V, _f32p), _p(O, _f64p), _p(L, _f64p),
                                  _i64(BH), _i64(S), _i64(dk), C.c_float(scale), int(causal))
        return O, L

    def conv_gemm(self, weight, inp, kh, kw, sh, sw, ph, pw):
        C_in, H, W = inp.shape
        C_out = weight.shape[0]
        out_h, out_w = (H + 2 * ph - kh) // sh + 1, (W + 2 * pw - kw) // sw + 1
        out = np.empty((C_out, out_h * out_w), np.float32)
        self.lib.orc_conv_gemm(_p(weight, _f32p), _p(inp, _f32p), _i64(C_out), _i64(C_in), _i64(H), _i64(W), kh, kw, sh, sw,
                               ph, pw, _i64(out_h), _i64(out_w), _p(out, _f32p))
        return out

    def sdpa_bwd_f64(self, Q, K, V, O, dO, scale, causal):
        BH, S, dk = Q.shape
        outs = [np.empty(Q.shape, np.float64) for _ in range(3)]
        self.lib.orc_sdpa_bwd_f64(_p(Q, _f32p), _p(K, _f32p), _p(V, _f32p), _p(O, _f32p), _p(dO, _f32p),
                                  *[_p(t, _f64p) for t in outs], _i64(BH), _i64(S), _i64(dk), C.c_float(scale), int(causal))
        return outs

    def qkv_head_gemm(self, X, W, b, B, S, H, dk):
        outs = [np.empty((B * H, S, dk), np.float32) for _ in range(3)]
        self.lib.orc_qkv_head_gemm(_p(X, _f32p), _p(W, _f32p), _p(b, _f32p) if b is not None else None, _i64(B), _i64(S),
                                   _i64(H), _i64(dk), *[_p(t, _f32p) for t in outs])
        return outs

    def kv_cache_attend(self, Kc, Vc, Qn, cur_len, scale):
        BH, max_seq, dk = Kc.shape
        out = np.empty((BH, dk), np.float32)
        self.lib.orc_kv_cache_attend(_p(Kc, _f32p), _p(Vc, _f32p), _p(Qn, _f32p), _p(out, _f32p),
                                     _i64(BH), _i64(cur_len), _i64(max_seq), _i64(dk), C.c_float(scale))
        return out

    def kv_cache_attend_f64(self, Kc, Vc, Qn, cur_len, scale):
        BH, max_seq, dk = Kc.shape
        out = np.empty((BH, dk), np.float64)
        self.lib.orc_kv_cache_attend_f64(_p(Kc, _f32p), _p(Vc, _f32p), _p(Qn, _f32p), _p(out, _f64p),
                                         _i64(BH), _i64(cur_len), _i64(max_seq), _i64(dk), C.c_float(scale))
        return out

    def num_threads(self):
        return int(self.lib.orc_num_threads())


class Reference:
    """The compiled axiom reference behind oracle/ref_shim.c."""

    @staticmethod
    def available():
        return os.path.exists(REF_SO)

    def __init__(self, autotune=False):
        self.lib = C.CDLL(REF_SO)
        st = self.lib.ref_init(int(autotune))
        if st != 0:
            raise RuntimeError(f"ax_init failed with status {st}")

    def num_threads(self):
        return int(self.lib.ref_num_threads())

    def gemm(self, A, B, variant="nn", backend="opt"):
        v = {"nn": 0, "nt": 1, "tn": 2}[variant]
        M = A.shape[1] if v == 2 else A.shape[0]
        K = A.shape[0] if v == 2 else A.shape[1]
        N = B.shape[0] if v == 1 else B.shape[1]
        out = np.empty((M, N), np.float32)
        st = self.lib.ref_gemm(_p(A, _f32p), _p(B, _f32p), _p(out, _f32p), _i64(M), _i64(N), _i64(K),
                               v, 1 if backend == "opt" else 0)
        assert st == 0, st
        return out

    def gemm_ex(self, A, B, alpha, beta, Cin):
        M, K = A.shape
        N = B.shape[1]
        out = np.array(Cin, dtype=np.float32, copy=True)
        st = self.lib.ref_gemm_ex(_p(A, _f32p), _p(B, _f32p), C.c_float(alpha), C.c_float(beta),
                                  _p(out, _f32p), _i64(M), _i64(N), _i64(K))
        assert st == 0, st
        return out

    def gemm_relu(self, A, B, bias):
        M, K = A.shape
        N = B.shape[1]
        out = np.empty((M, N), np.float32)
        st = self.lib.ref_gemm_relu(_p(A, _f32p), _p(B, _f32p), _p(bias, _f32p), _p(out, _f32p),
                                    _i64(M), _i64(N), _i64(K))
        assert st == 0, st
        return out

    def matmul_bias_relu(self, A, B, bias):
        M, K = A.shape
        N = B.shape[1]
        out = np.empty((M, N), np.float32)
        st = self.lib.ref_matmul_bias_relu(_p(A, _f32p), _p(B, _f32p), _p(bias, _f32p), _p(out, _f32p),
                                           _i64(M), _i64(N), _i64(K))
        assert st == 0, st
        return out

    def gelu(self, X):
        out = np.empty_like(X)
        st = self.lib.ref_gelu(_p(X, _f32p), _p(out, _f32p), _i64(X.size))
        assert st == 0, st
        return out

    def dense_gelu(self, X, W, bias):
        M, K = X.shape
        N = W.shape[1]
        out = np.empty((M, N), np.float32)
        st = self.lib.ref_dense_gelu(_p(X, _f32p), _p(W, _f32p), _p(bias, _f32p), _p(out, _f32p),
                                     _i64(M), _i64(N), _i64(K))
        assert st == 0, st
        return out

    def bias_add(self, X, bias, axis):
        M, N = X.shape
        out = np.zeros_like(X)
        st = self.lib.ref_bias_add(_p(X, _f32p), _p(bias, _f32p), int(axis), _p(out, _f32p),
                                   _i64(M), _i64(N))
        return st, out

    def quantize(self, W):
        N, K = W.shape
        q = np.empty((N, K), np.int8)
        s = np.empty((N,), np.float32)
        st = self.lib.ref_quantize(_p(W, _f32p), _i64(N), _i64(K), _p(q, _i8p), _p(s, _f32p))
        assert st == 0, st
        return q, s

    def qgemm_w8a32(self, a, q, s):
        M, K = a.shape
        N = q.shape[0]
        out = np.zeros((M, N), np.float32)
        st = self.lib.ref_qgemm_w8a32(_p(a, _f32p), _p(q, _i8p), _p(s, _f32p), _p(out, _f32p),
                                      _i64(M), _i64(N), _i64(K))
        assert st == 0, st
        return out

    def sdpa_fwd(self, Q, K, V, scale, causal):
        BH, S, dk = Q.shape
        O = np.zeros_like(Q)
        L = np.zeros((BH, S), np.float32)
        self.lib.ref_sdpa_fwd(_p(Q, _f32p), _p(K, _f32p), _p(V, _f32p), _p(O, _f32p), _p(L, _f32p),
                              _i64(BH), _i64(S), _i64(dk), C.c_float(scale), int(causal))
        return O, L


    def conv_gemm(self, weight, inp, kh, kw, sh, sw, ph, pw, device=0):
        C_in, H, W = inp.shape
        C_out = weight.shape[0]
        out_h, out_w = (H + 2 * ph - kh) // sh + 1, (W + 2 * pw - kw) // sw + 1
        out = np.zeros((C_out, out_h * out_w), np.float32)
        st = self.lib.ref_conv_gemm(_p(weight, _f32p), _p(inp, _f32p), _i64(C_out), _i64(C_in), _i64(H), _i64(W), kh, kw,
                                    sh, sw, ph, pw, _i64(out_h), _i64(out_w), _p(out, _f32p), int(device))
        return st, out

    def sdpa_bwd(self, Q, K, V, O, dO, L, scale, causal):
        BH, S, dk = Q.shape
        outs = [np.zeros(Q.shape, np.float32) for _ in range(3)]
        self.lib.ref_sdpa_bwd(_p(Q, _f32p), _p(K, _f32p), _p(V, _f32p), _p(O, _f32p), _p(dO, _f32p), _p(L, _f32p),
                              *[_p(t, _f32p) for t in outs], _i64(BH), _i64(S), _i64(dk), C.c_float(scale), int(causal))
        return outs

    def qkv_head_gemm(self, X, W, b, B, S, H, dk):
        outs = [np.zeros((B * H, S, dk), np.float32) for _ in range(3)]
        st = self.lib.ref_qkv_head_gemm(_p(X, _f32p), _p(W, _f32p), _p(b, _f32p) if b is not None else None, _i64(B),
                                        _i64(S), _i64(H), _i64(dk), *[_p(t, _f32p) for t in outs])
        assert st == 0, st
        return outs

    def kv_cache_attend(self, Kc, Vc, Qn, cur_len, scale):
        """Kc, Vc: cache-layout [BH, max_seq, dk]; the rows are appended token by token through the reference API."""
        BH, max_seq, dk = Kc.shape
        Kseq = np.ascontiguousarray(Kc[:, :cur_len].transpose(1, 0, 2))
        Vseq = np.ascontiguousarray(Vc[:, :cur_len].transpose(1, 0, 2))
        out = np.zeros((BH, dk), np.float32)
        st = self.lib.ref_kv_cache_attend(_p(Kseq, _f32p), _p(Vseq, _f32p), _p(Qn, _f32p), _p(out, _f32p),
                                          _i64(BH), _i64(cur_len), _i64(max_seq), _i64(dk), C.c_float(scale))
        assert st == 0, st
        return out


def nerr(x, ref):
    """Normalised error max|x - ref| / max|ref| (the metric the fp32 tolerance is stated in)."""
    ref = np.asarray(ref, np.float64)
    d = np.abs(np.asarray(x, np.float64) - ref).max() if ref.size else 0.0
    m = np.abs(ref).max() if ref.size else 0.0
    return float(d / m) if m > 0 else float(d)
