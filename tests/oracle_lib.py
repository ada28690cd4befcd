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


def axiom_source_tree():
    """Root of the axiom source tree the compiled reference is built from: $AXIOM_SRC, else a checkout named
    `reference` beside this repository; None when neither exists (the prebuilt oracle/_ref is then used as it is)."""
    for cand in (os.environ.get("AXIOM_SRC"), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.exists(os.path.join(cand, "src", "compute", "dispatch.c")):
            return cand
    return None


def build_oracle():
    """Compile oracle/liboracle.so (and oracle/_ref when the axiom tree exists)."""
    src = axiom_source_tree()
    subprocess.run(["make", "-C", ORACLE_DIR, "-j8", "all"] + ([f"AXIOM_SRC={src}"] if src else []), check=True,
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

    # ---- timing doors (bench CPU baselines): operands built once, only the entry point is timed -------------
    def _timed(self, fn, args, warmup, iters):
        secs = (C.c_double * iters)()
        st = fn(*args, int(warmup), int(iters), secs)
        assert st == 0, st
        return list(secs)

    def time_gemm(self, A, B, out, warmup, iters):
        M, K = A.shape
        N = B.shape[1]
        return self._timed(self.lib.ref_time_gemm, [_p(A, _f32p), _p(B, _f32p), _p(out, _f32p), _i64(M), _i64(N), _i64(K)],
                           warmup, iters)

    def time_matmul_bias_relu(self, A, B, bias, out, warmup, iters):
        M, K = A.shape
        N = B.shape[1]
        return self._timed(self.lib.ref_time_matmul_bias_relu,
                           [_p(A, _f32p), _p(B, _f32p), _p(bias, _f32p), _p(out, _f32p), _i64(M), _i64(N), _i64(K)], warmup, iters)

    def time_dense_gelu(self, X, W, bias, out, warmup, iters):
        M, K = X.shape
        N = W.shape[1]
        return self._timed(self.lib.ref_time_dense_gelu,
                           [_p(X, _f32p), _p(W, _f32p), _p(bias, _f32p), _p(out, _f32p), _i64(M), _i64(N), _i64(K)], warmup, iters)

    def time_qgemm_w8a32(self, a, q, s, out, warmup, iters):
        M, K = a.shape
        N = q.shape[0]
        return self._timed(self.lib.ref_time_qgemm_w8a32,
                           [_p(a, _f32p), _p(q, _i8p), _p(s, _f32p), _p(out, _f32p), _i64(M), _i64(N), _i64(K)], warmup, iters)

    def time_sdpa_causal(self, Q, K, V, O, L, scale, warmup, iters):
        BH, S, dk = Q.shape
        return self._timed(self.lib.ref_time_sdpa_causal,
                           [_p(Q, _f32p), _p(K, _f32p), _p(V, _f32p), _p(O, _f32p), _p(L, _f32p), _i64(BH), _i64(S), _i64(dk),
                            C.c_float(scale)], warmup, iters)

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

    def mha_layer(self, x, W, b, H, causal, dOut=None, device=False, save_p=False):
        """The reference's multi-head attention layer: x [B,S,D], W [4,D,D] = Wq,Wk,Wv,Wo, b [4,D] or None.
        device=False: ax_mha_create + ax_layer_forward (+ ax_backward of sum(out*dOut)) on the CPU backend.
        device=True: the layer's device call sequence through the dispatcher and the registered extension table.
        Returns dict(out, dX, dW, db, P) with the gradients only when dOut is given."""
        B, S, D = x.shape
        out = np.zeros((B, S, D), np.float32)
        dX = np.zeros((B, S, D), np.float32) if dOut is not None else None
        dW = np.zeros((4, D, D), np.float32) if dOut is not None else None
        db = np.zeros((4, D), np.float32) if dOut is not None and b is not None else None
        P = np.zeros((B * H, S, S), np.float32) if device and save_p else None
        args = [_p(x, _f32p), _p(W, _f32p), _p(b, _f32p), _i64(B), _i64(S), _i64(D), int(H), int(causal)]
        if device:
            st = self.lib.ref_device_mha_sequence(*args, int(save_p), _p(dOut, _f32p), _p(out, _f32p), _p(dX, _f32p),
                                                  _p(dW, _f32p), _p(db, _f32p), _p(P, _f32p))
        else:
            st = self.lib.ref_mha_layer(*args, _p(dOut, _f32p), _p(out, _f32p), _p(dX, _f32p), _p(dW, _f32p), _p(db, _f32p))
        return st, dict(out=out, dX=dX, dW=dW, db=db, P=P)

    def head_layout(self, op, B, S, H, dk, flat=None, heads=None, bias=None):
        """CPU layout helpers of the reference's attention layer. op: 'split' (flat [B*S,3D] -> 3 heads), 'interleave'
        (flat [B*S,D] -> head), 'deinterleave' (head -> flat), 'merge' (3 heads -> flat [B*S,3D])."""
        D = H * dk
        hs = [np.zeros((B * H, S, dk), np.float32) for _ in range(3)]
        code = {"split": 0, "interleave": 1, "deinterleave": 2, "merge": 3}[op]
        if op in ("split", "interleave"):
            self.lib.ref_head_layout(code, _p(flat, _f32p), _p(bias, _f32p), *[_p(h, _f32p) for h in hs], None,
                                     _i64(B), _i64(S), _i64(H), _i64(dk))
            return hs if op == "split" else hs[0]
        out = np.zeros((B * S, D if op == "deinterleave" else 3 * D), np.float32)
        if op == "deinterleave":
            self.lib.ref_head_layout(code, _p(heads, _f32p), None, None, None, None, _p(out, _f32p), _i64(B), _i64(S), _i64(H), _i64(dk))
        else:
            self.lib.ref_head_layout(code, None, None, *[_p(h, _f32p) for h in heads], _p(out, _f32p), _i64(B), _i64(S), _i64(H), _i64(dk))
        return out

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


def mha_f64(x, W, b, H, causal, dOut=None):
    """Double-precision restatement of axiom's multi-head attention layer, forward and backward
    (src/core/attention.c:121-464 and :560-900): x [B,S,D]; W [4,D,D] = Wq,Wk,Wv,Wo; b [4,D] or None.
    Returns dict(out, dX, dW [4,D,D], db [4,D]); the gradients are those of sum(out * dOut)."""
    B, S, D = x.shape
    dk = D // H
    X = x.reshape(B * S, D).astype(np.float64)
    W = W.astype(np.float64)
    bb = b.astype(np.float64) if b is not None else np.zeros((4, D))
    heads = lambda t: t.reshape(B, S, H, dk).transpose(0, 2, 1, 3)
    flat = lambda t: t.transpose(0, 2, 1, 3).reshape(B * S, D)
    qh, kh, vh = (heads(X @ W[i] + bb[i]) for i in range(3))
    s = qh @ kh.transpose(0, 1, 3, 2) / np.sqrt(dk)
    if causal:
        s = np.where(np.triu(np.ones((S, S), bool), 1), -np.inf, s)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    attn = flat(p @ vh)
    res = dict(out=(attn @ W[3] + bb[3]).reshape(B, S, D), dX=None, dW=None, db=None, P=p.reshape(B * H, S, S))
    if dOut is None:
        return res
    G = dOut.reshape(B * S, D).astype(np.float64)
    doh = heads(G @ W[3].T)
    dv = p.transpose(0, 1, 3, 2) @ doh
    dp = doh @ vh.transpose(0, 1, 3, 2)
    ds = p * (dp - (dp * p).sum(-1, keepdims=True)) / np.sqrt(dk)
    dq, dkk, dv = flat(ds @ kh), flat(ds.transpose(0, 1, 3, 2) @ qh), flat(dv)
    res["dX"] = (dq @ W[0].T + dkk @ W[1].T + dv @ W[2].T).reshape(B, S, D)
    res["dW"] = np.stack([X.T @ dq, X.T @ dkk, X.T @ dv, attn.T @ G])
    res["db"] = np.stack([dq.sum(0), dkk.sum(0), dv.sum(0), G.sum(0)])
    return res


def nerr(x, ref):
    """Normalised error max|x - ref| / max|ref| (the metric the fp32 tolerance is stated in)."""
    ref = np.asarray(ref, np.float64)
    d = np.abs(np.asarray(x, np.float64) - ref).max() if ref.size else 0.0
    m = np.abs(ref).max() if ref.size else 0.0
    return float(d / m) if m > 0 else float(d)
