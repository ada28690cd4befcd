"""ctypes binding of libaxiom_b200.so for Python callers (tests, bench, multi-GPU drivers).

The functions mirror the C ABI in include/axiom_b200.h one to one and take
torch CUDA tensors (or raw device pointers as ints) for the buffers.  torch is
used only to own device memory; every computation is a kernel of the library.
There is no fallback: if the shared library is missing, loading raises.
"""
from __future__ import annotations

import ctypes as C
import math
import os

PKG = os.path.dirname(os.path.abspath(__file__))
ENGINE_SO = os.path.join(PKG, "lib", "libaxiom_b200.so")

ACT = {"none": 0, None: 0, "relu": 1, "gelu": 2}
FP32_MODES = {"3xtf32": 0, "bf16x3": 1, "bf16": 2}

# every symbol include/axiom_b200.h declares
EXPORTS = [
    "axb_init", "axb_shutdown", "axb_device_count", "axb_synchronize", "axb_storage_alloc",
    "axb_storage_free", "axb_memcpy_h2d", "axb_memcpy_d2h", "axb_memcpy_d2d", "axb_set_stream",
    "axb_set_fp32_mode", "axb_get_fp32_mode", "axb_last_error", "axb_device_error", "axb_launch_count",
    "axb_set_profiling", "axb_timing_summary", "axb_timing_samples",
    "axb_gemm", "axb_gemm_host", "axb_gemm_nt", "axb_gemm_tn", "axb_gemm_ex", "axb_gemm_relu", "axb_gemm_bias_act",
    "axb_skinny_gemm_static", "axb_skinny_gemm_static_error", "axb_gemm_bias_act_scatter", "axb_gemm_gathered_scatter", "axb_ipc_get_handle", "axb_ipc_open_handle",
    "axb_ipc_close_handle",
    "axb_bias_add", "axb_relu", "axb_gelu", "axb_qgemm_w8a32", "axb_qgemm_w8a8", "axb_quantize_rows",
    "axb_sdpa_fwd", "axb_kv_cache_append", "axb_kv_cache_attend", "axb_qkv_head_gemm", "axb_sdpa_bwd", "axb_conv_gemm", "axb_conv_gemm_batched", "axb_gemm_prepared_scatter", "axb_dattn_head_gemm_nt", "axb_dwqkv_split_acc", "axb_dwqkv_split_acc_hm", "axb_mha_output_proj_fused", "axb_qdense_w8a32",
    "axb_qgemm_w8a32_qw", "axb_bias_add_nd", "axb_head_interleave_qkv_split", "axb_head_interleave", "axb_head_deinterleave",
    "axb_head_deinterleave_qkv_merge", "axb_qkv_cache_build", "axb_bias_cache_build", "axb_pointer_on_device",
    "axb_weight_prepare", "axb_weight_release", "axb_gemm_prepared",
    "axb_mgpu_create", "axb_mgpu_destroy", "axb_mgpu_size", "axb_mgpu_device", "axb_mgpu_alloc", "axb_mgpu_free", "axb_mgpu_h2d",
    "axb_mgpu_d2h", "axb_mgpu_synchronize", "axb_mgpu_gemm_rows", "axb_mgpu_qgemm_w8a8_rows", "axb_mgpu_gemm_cols_allgather",
]


class QWeight(C.Structure):
    """Host struct with axiom's ax_qweight_t layout (include/axiom/quantize.h:50-55); data and scales are device pointers."""
    _fields_ = [("data", C.c_void_p), ("scales", C.c_void_p), ("N", C.c_int64), ("K", C.c_int64)]


class EngineError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"axiom_b200 status {status}: {message}")
        self.status = status


def _ptr(t):
    if t is None:
        return None
    if isinstance(t, int):
        return C.c_void_p(t)
    return C.c_void_p(t.data_ptr())


_i64 = C.c_int64
_f = C.c_float


class Engine:
    """One engine per process (one process per GPU)."""

    def __init__(self, device: int | None = None, so_path: str = ENGINE_SO):
        if not os.path.exists(so_path):
            raise FileNotFoundError(
                f"{so_path} is missing: build it with `python -m axiom_b200.build` (no CPU fallback exists)")
        self.lib = C.CDLL(so_path)
        self.stream_ptr = 0          # the stream the engine enqueues on (0 = legacy default stream)
        L = self.lib
        L.axb_last_error.restype = C.c_char_p
        L.axb_storage_alloc.restype = C.c_void_p
        L.axb_storage_alloc.argtypes = [C.c_size_t]
        L.axb_storage_free.argtypes = [C.c_void_p]
        L.axb_launch_count.restype = C.c_int64
        L.axb_set_stream.argtypes = [C.c_void_p]
        L.axb_weight_release.argtypes = [C.c_void_p]
        L.axb_gemm_prepared.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_float, C.c_int]
        for name in ("axb_memcpy_h2d", "axb_memcpy_d2h", "axb_memcpy_d2d"):
            getattr(L, name).argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        if device is not None:
            self._check(L.axb_init(int(device)))

    # ---- plumbing ------------------------------------------------------
    def _check(self, status):
        if status != 0:
            raise EngineError(status, self.lib.axb_last_error().decode())

    def init(self, device=-1):
        self._check(self.lib.axb_init(int(device)))

    def synchronize(self):
        self.lib.axb_synchronize()

    def device_error(self):
        return int(self.lib.axb_device_error())

    def launch_count(self, reset=False):
        return int(self.lib.axb_launch_count(int(reset)))

    def set_profiling(self, on=True):
        self.lib.axb_set_profiling(int(bool(on)))

    def timing_summary(self):
        """(calls, prepass_ms_total, core_ms_total) since profiling was switched on or last summarised."""
        n, a, b = C.c_int(0), C.c_float(0), C.c_float(0)
        self._check(self.lib.axb_timing_summary(C.byref(n), C.byref(a), C.byref(b)))
        return n.value, a.value, b.value

    def timing_samples(self, cap=256):
        """Per-call (prepass_ms, core_ms) lists of the current profiling window, oldest first."""
        pre, core, n = (C.c_float * cap)(), (C.c_float * cap)(), C.c_int(0)
        self._check(self.lib.axb_timing_samples(pre, core, cap, C.byref(n)))
        return list(pre[:n.value]), list(core[:n.value])

    def set_fp32_mode(self, mode):
        self._check(self.lib.axb_set_fp32_mode(FP32_MODES[mode] if isinstance(mode, str) else int(mode)))

    def set_stream(self, stream_ptr):
        self.lib.axb_set_stream(C.c_void_p(stream_ptr))
        self.stream_ptr = int(stream_ptr or 0)

    def last_error(self):
        return self.lib.axb_last_error().decode()

    def memcpy_h2d(self, dst, src_host_ptr, nbytes):
        self._check(self.lib.axb_memcpy_h2d(_ptr(dst), C.c_void_p(src_host_ptr), nbytes))

    def memcpy_d2h(self, dst_host_ptr, src, nbytes):
        self._check(self.lib.axb_memcpy_d2h(C.c_void_p(dst_host_ptr), _ptr(src), nbytes))

    # ---- GEMM family (out is caller-allocated, as in the reference) -----
    def gemm_host(self, A_host, B_host, C_host, row_chunk=0):
        """C_host = A_host . B_host on host tensors (pinned for full speed); transfers overlap the GEMM."""
        M, K = A_host.shape
        N = B_host.shape[1]
        assert not A_host.is_cuda and not B_host.is_cuda and not C_host.is_cuda
        assert A_host.is_contiguous() and B_host.is_contiguous() and C_host.is_contiguous()
        self._check(self.lib.axb_gemm_host(C.c_void_p(A_host.data_ptr()), C.c_void_p(B_host.data_ptr()),
                                           C.c_void_p(C_host.data_ptr()), _i64(M), _i64(N), _i64(K), _i64(row_chunk)))
        return C_host

    def gemm(self, A, B, out, variant="nn"):
        if variant == "nn":
            M, K = A.shape; N = B.shape[1]
            self._check(self.lib.axb_gemm(_ptr(A), _ptr(B), _ptr(out), _i64(M), _i64(N), _i64(K)))
        elif variant == "nt":
            M, K = A.shape; N = B.shape[0]
            self._check(self.lib.axb_gemm_nt(_ptr(A), _ptr(B), _ptr(out), _i64(M), _i64(N), _i64(K)))
        else:
            K, M = A.shape; N = B.shape[1]
            self._check(self.lib.axb_gemm_tn(_ptr(A), _ptr(B), _ptr(out), _i64(M), _i64(N), _i64(K)))
        return out

    def gemm_ex(self, A, B, alpha, beta, out):
        M, K = A.shape; N = B.shape[1]
        self._check(self.lib.axb_gemm_ex(_ptr(A), _ptr(B), _f(alpha), _f(beta), _ptr(out), _i64(M), _i64(N), _i64(K)))
        return out

    def gemm_relu(self, A, B, bias, out):
        M, K = A.shape; N = B.shape[1]
        self._check(self.lib.axb_gemm_relu(_ptr(A), _ptr(B), _ptr(bias), _ptr(out), _i64(M), _i64(N), _i64(K)))
        return out

    def gemm_bias_act(self, A, B, bias, out, M, N, K, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, act="none"):
        self._check(self.lib.axb_gemm_bias_act(_ptr(A), _ptr(B), _ptr(bias), _ptr(out), _i64(M), _i64(N), _i64(K),
                                               int(trans_a), int(trans_b), _f(alpha), _f(beta), ACT[act]))
        return out

    def weight_prepare(self, B, trans_b=False):
        """Operand planes of a weight matrix, made once (axb_weight_prepare); B must outlive the handle."""
        K, N = (B.shape[1], B.shape[0]) if trans_b else (B.shape[0], B.shape[1])
        h = C.c_void_p(0)
        self._check(self.lib.axb_weight_prepare(_ptr(B), _i64(K), _i64(N), int(trans_b), C.byref(h)))
        return h

    def weight_release(self, h):
        self.lib.axb_weight_release(h)

    def gemm_prepared(self, A, W, bias, out, M, trans_a=False, alpha=1.0, beta=0.0, act="none"):
        self._check(self.lib.axb_gemm_prepared(_ptr(A), W, _ptr(bias), _ptr(out), _i64(M), int(trans_a), _f(alpha), _f(beta),
                                               ACT[act]))
        return out

    def gemm_bias_act_scatter(self, A, B, bias, out, more, M, N, K, trans_a=False, trans_b=False, alpha=1.0, beta=0.0,
                              act="none"):
        """GEMM whose epilogue also stores the result to every buffer in `more` (tensors or raw device pointers)."""
        arr = (C.c_void_p * max(len(more), 1))(*[(_ptr(m).value if m is not None else None) for m in more])
        self._check(self.lib.axb_gemm_bias_act_scatter(_ptr(A), _ptr(B), _ptr(bias), _ptr(out), arr, len(more), _i64(M), _i64(N),
                                                       _i64(K), int(trans_a), int(trans_b), _f(alpha), _f(beta), ACT[act]))
        return out

    def gemm_gathered_scatter(self, A_gathered, chunks, chunk_k, B, bias, out, more, M, N, alpha=1.0, beta=0.0, act="none"):
        """GEMM whose left operand is a [chunks][M][chunk_k] gather buffer; result to `out` and every buffer in `more`."""
        arr = (C.c_void_p * max(len(more), 1))(*[(_ptr(m).value if m is not None else None) for m in more])
        self._check(self.lib.axb_gemm_gathered_scatter(_ptr(A_gathered), int(chunks), _i64(chunk_k), _ptr(B), _ptr(bias), _ptr(out),
                                                       arr, len(more), _i64(M), _i64(N), _f(alpha), _f(beta), ACT[act]))
        return out

    def gemm_prepared_scatter(self, A, chunks, chunk_k, weight, bias, out, more, M, alpha=1.0, beta=0.0, act="none"):
        """gemm_bias_act_scatter (chunks = 0, A a plain [M, K] matrix) or gemm_gathered_scatter (A a [chunks][M][chunk_k]
        gather buffer) with a weight prepared by weight_prepare."""
        arr = (C.c_void_p * max(len(more), 1))(*[(_ptr(m).value if m is not None else None) for m in more])
        self._check(self.lib.axb_gemm_prepared_scatter(_ptr(A), int(chunks), _i64(chunk_k), weight, _ptr(bias), _ptr(out), arr,
                                                       len(more), _i64(M), _f(alpha), _f(beta), ACT[act]))
        return out

    def storage_alloc(self, nbytes):
        p = self.lib.axb_storage_alloc(nbytes)
        if not p:
            raise EngineError(2, self.last_error())
        return int(p)

    def storage_free(self, ptr):
        self.lib.axb_storage_free(C.c_void_p(ptr))

    def ipc_get_handle(self, ptr):
        buf = C.create_string_buffer(64)
        self._check(self.lib.axb_ipc_get_handle(C.c_void_p(ptr), buf))
        return buf.raw

    def ipc_open_handle(self, handle):
        out = C.c_void_p(0)
        self._check(self.lib.axb_ipc_open_handle(C.create_string_buffer(handle, 64), C.byref(out)))
        return int(out.value)

    def ipc_close_handle(self, ptr):
        self._check(self.lib.axb_ipc_close_handle(C.c_void_p(ptr)))

    def skinny_gemm_static(self, X, W, bias, out, M, N, K, alpha=1.0, beta=0.0, act="none", stream_ptr=None):
        """Allocation-free skinny GEMM (axb_skinny_gemm_static): scratch lives inside the library."""
        self._check(self.lib.axb_skinny_gemm_static(_ptr(X), _ptr(W), _ptr(bias), _ptr(out), _i64(M), _i64(N), _i64(K),
                                                    _f(alpha), _f(beta), ACT[act], C.c_void_p(stream_ptr)))
        return out

    def skinny_gemm_static_error(self):
        return int(self.lib.axb_skinny_gemm_static_error())

    # ---- elementwise ---------------------------------------------------
    def bias_add(self, X, bias, axis, out):
        M, N = X.shape
        self._check(self.lib.axb_bias_add(_ptr(X), _ptr(bias), int(axis), _ptr(out), _i64(M), _i64(N)))
        return out

    def bias_add_nd(self, X, bias, axis, out):
        """out = X + bias broadcast along `axis` of a tensor of any rank."""
        shape = list(X.shape)
        outer = math.prod(shape[:axis])
        inner = math.prod(shape[axis + 1:])
        self._check(self.lib.axb_bias_add_nd(_ptr(X), _ptr(bias), _ptr(out), _i64(outer), _i64(shape[axis]), _i64(inner)))
        return out

    def relu(self, X, out):
        self._check(self.lib.axb_relu(_ptr(X), _ptr(out), _i64(X.numel())))
        return out

    def gelu(self, X, out):
        self._check(self.lib.axb_gelu(_ptr(X), _ptr(out), _i64(X.numel())))
        return out

    # ---- quantised -----------------------------------------------------
    def qgemm_w8a32(self, a, q, scales, out):
        M, K = a.shape; N = q.shape[0]
        self._check(self.lib.axb_qgemm_w8a32(_ptr(a), _ptr(q), _ptr(scales), _ptr(out), _i64(M), _i64(N), _i64(K)))
        return out

    def qgemm_w8a32_qw(self, a, q, scales, out):
        """axiom's own argument list: a host ax_qweight_t-layout struct whose members are device pointers."""
        M, K = a.shape; N = q.shape[0]
        qw = QWeight(q.data_ptr(), scales.data_ptr(), N, K)
        self._check(self.lib.axb_qgemm_w8a32_qw(_ptr(a), C.byref(qw), _ptr(out), _i64(M)))
        return out

    def qdense_w8a32(self, a, q, scales, bias, out, act="none"):
        M, K = a.shape; N = q.shape[0]
        self._check(self.lib.axb_qdense_w8a32(_ptr(a), _ptr(q), _ptr(scales), _ptr(bias), ACT[act], _ptr(out), _i64(M),
                                              _i64(N), _i64(K)))
        return out

    def qgemm_w8a8(self, a_q, a_scale, b_q, b_scales, out_scale, out_q=None, acc_out=None):
        M, K = a_q.shape; N = b_q.shape[0]
        self._check(self.lib.axb_qgemm_w8a8(_ptr(a_q), _f(a_scale), _ptr(b_q), _ptr(b_scales), _f(out_scale),
                                            _ptr(out_q), _ptr(acc_out), _i64(M), _i64(N), _i64(K)))
        return out_q, acc_out

    def quantize_rows(self, W, q, scales):
        N, K = W.shape
        self._check(self.lib.axb_quantize_rows(_ptr(W), _i64(N), _i64(K), _ptr(q), _ptr(scales)))
        return q, scales

    # ---- attention -----------------------------------------------------
    def sdpa_fwd(self, Q, K, V, out, L, scale, causal, P_save=None):
        BH, S, dk = Q.shape
        self._check(self.lib.axb_sdpa_fwd(_ptr(Q), _ptr(K), _ptr(V), _ptr(out), _ptr(L), _i64(BH), _i64(S), _i64(dk),
                                          _f(scale), int(bool(causal)), _ptr(P_save)))
        return out, L

    # ---- attention layout passes (flat = [B*S, H*dk], head-major = [B*H, S, dk]) ----
    def head_interleave_qkv_split(self, qkv, bqkv, Qh, Kh, Vh, B, S, H, dk):
        self._check(self.lib.axb_head_interleave_qkv_split(_ptr(qkv), _ptr(bqkv), _ptr(Qh), _ptr(Kh), _ptr(Vh), _i64(B), _i64(S),
                                                           _i64(H), _i64(dk)))

    def head_interleave(self, src, dst, B, S, H, dk):
        self._check(self.lib.axb_head_interleave(_ptr(src), _ptr(dst), _i64(B), _i64(S), _i64(H), _i64(dk)))

    def head_deinterleave(self, src, dst, B, S, H, dk):
        self._check(self.lib.axb_head_deinterleave(_ptr(src), _ptr(dst), _i64(B), _i64(S), _i64(H), _i64(dk)))

    def head_deinterleave_qkv_merge(self, dQ, dK, dV, dst, B, S, H, dk):
        self._check(self.lib.axb_head_deinterleave_qkv_merge(_ptr(dQ), _ptr(dK), _ptr(dV), _ptr(dst), _i64(B), _i64(S), _i64(H),
                                                             _i64(dk)))

    def qkv_cache_build(self, dst, wq, wk, wv, D):
        self._check(self.lib.axb_qkv_cache_build(_ptr(dst), _ptr(wq), _ptr(wk), _ptr(wv), _i64(D)))

    def bias_cache_build(self, dst, bq, bk, bv, D):
        self._check(self.lib.axb_bias_cache_build(_ptr(dst), _ptr(bq), _ptr(bk), _ptr(bv), _i64(D)))

    def pointer_on_device(self, ptr):
        return bool(self.lib.axb_pointer_on_device(C.c_void_p(ptr)))

    def conv_gemm(self, weight, inp, kh, kw, sh, sw, ph, pw, out):
        """weight [C_out, C_in*kh*kw], inp [C_in, H, W], out [C_out, out_h*out_w] with the usual output size."""
        C_in, H, W = inp.shape
        C_out = weight.shape[0]
        out_h, out_w = (H + 2 * ph - kh) // sh + 1, (W + 2 * pw - kw) // sw + 1
        assert tuple(out.shape) == (C_out, out_h * out_w)
        self._check(self.lib.axb_conv_gemm(_ptr(weight), _ptr(inp), _i64(C_out), _i64(C_in), _i64(H), _i64(W), kh, kw, sh, sw,
                                           ph, pw, _i64(out_h), _i64(out_w), _ptr(out)))
        return out

    def dattn_head_gemm_nt(self, dout, Wo, B, S, H, dk, dO_head):
        """dO_head[B*H, S, dk] = head-major(dout[B*S, D] . Wo[D, D]^T)."""
        self._check(self.lib.axb_dattn_head_gemm_nt(_ptr(dout), _ptr(Wo), _i64(B), _i64(S), _i64(H), _i64(dk), _ptr(dO_head)))
        return dO_head

    def dwqkv_split_acc(self, x_flat, dQKV, dWq, dWk, dWv):
        """dW{q,k,v}[D, D] += x_flat[rows, D]^T . the three D-wide column blocks of dQKV[rows, 3D]."""
        rows, D = x_flat.shape
        self._check(self.lib.axb_dwqkv_split_acc(_ptr(x_flat), _ptr(dQKV), _i64(rows), _i64(D), _ptr(dWq), _ptr(dWk), _ptr(dWv)))

    def dwqkv_split_acc_hm(self, x_flat, dQh, dKh, dVh, B, S, H, dk, dWq, dWk, dWv):
        """The same with the three gradients head-major [B*H, S, dk]."""
        self._check(self.lib.axb_dwqkv_split_acc_hm(_ptr(x_flat), _ptr(dQh), _ptr(dKh), _ptr(dVh), _i64(B), _i64(S), _i64(H),
                                                    _i64(dk), _ptr(dWq), _ptr(dWk), _ptr(dWv)))

    def mha_output_proj_fused(self, attn_flat, Wo, bo, dout, y, dattn, dWo_acc, dbo_acc):
        """y = attn.Wo + bo (y None: skipped); dattn = dout.Wo^T; dWo_acc += attn^T.dout; dbo_acc += column sums of dout."""
        rows, D = attn_flat.shape
        opt = lambda t: _ptr(t) if t is not None else None
        self._check(self.lib.axb_mha_output_proj_fused(_ptr(attn_flat), _ptr(Wo), opt(bo), _ptr(dout), opt(y), _ptr(dattn),
                                                       _ptr(dWo_acc), opt(dbo_acc), _i64(rows), _i64(D)))

    def conv_gemm_batched(self, weight, inp, kh, kw, sh, sw, ph, pw, out):
        """weight [C_out, C_in*kh*kw], inp [N, C_in, H, W], out [N, C_out, out_h*out_w]."""
        N, C_in, H, W = inp.shape
        C_out = weight.shape[0]
        out_h, out_w = (H + 2 * ph - kh) // sh + 1, (W + 2 * pw - kw) // sw + 1
        assert tuple(out.shape) == (N, C_out, out_h * out_w)
        self._check(self.lib.axb_conv_gemm_batched(_ptr(weight), _ptr(inp), _i64(N), _i64(C_out), _i64(C_in), _i64(H), _i64(W), kh, kw,
                                                   sh, sw, ph, pw, _i64(out_h), _i64(out_w), _ptr(out)))
        return out

    def sdpa_bwd(self, Q, K, V, O, dO, L, dQ, dK, dV, scale, causal):
        BH, S, dk = Q.shape
        self._check(self.lib.axb_sdpa_bwd(_ptr(Q), _ptr(K), _ptr(V), _ptr(O), _ptr(dO), _ptr(L), _ptr(dQ), _ptr(dK), _ptr(dV),
                                          _i64(BH), _i64(S), _i64(dk), _f(scale), int(bool(causal)), None))
        return dQ, dK, dV

    def qkv_head_gemm(self, X, Wqkv, bqkv, B, S, H, dk, Qh, Kh, Vh):
        self._check(self.lib.axb_qkv_head_gemm(_ptr(X), _ptr(Wqkv), _ptr(bqkv), _i64(B), _i64(S), _i64(H), _i64(dk),
                                               _ptr(Qh), _ptr(Kh), _ptr(Vh)))
        return Qh, Kh, Vh

    def kv_cache_append(self, K_cache, V_cache, new_K, new_V, cur_len):
        BH, max_seq, dk = K_cache.shape
        self._check(self.lib.axb_kv_cache_append(_ptr(K_cache), _ptr(V_cache), _ptr(new_K), _ptr(new_V), _i64(BH),
                                                 _i64(cur_len), _i64(max_seq), _i64(dk)))
        return cur_len + 1

    def kv_cache_attend(self, K_cache, V_cache, Q_new, out, cur_len, scale):
        BH, max_seq, dk = K_cache.shape
        self._check(self.lib.axb_kv_cache_attend(_ptr(K_cache), _ptr(V_cache), _ptr(Q_new), _ptr(out), _i64(BH),
                                                 _i64(cur_len), _i64(max_seq), _i64(dk), _f(scale)))
        return out


class MultiGpu:
    """The C multi-GPU entry points (axb_mgpu_*): one host thread, n devices.  Buffers are raw device pointers owned by
    this object (allocated through the library, no torch involved)."""

    def __init__(self, engine: Engine, n_devices: int, devices=None):
        self.eng, self.lib = engine, engine.lib
        L = self.lib
        L.axb_mgpu_alloc.restype = C.c_void_p
        L.axb_mgpu_alloc.argtypes = [C.c_void_p, C.c_int, C.c_size_t]
        L.axb_mgpu_free.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.axb_mgpu_h2d.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_size_t]
        L.axb_mgpu_d2h.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_size_t]
        L.axb_mgpu_destroy.argtypes = [C.c_void_p]
        L.axb_mgpu_synchronize.argtypes = [C.c_void_p]
        h = C.c_void_p(0)
        devs = (C.c_int * n_devices)(*devices) if devices is not None else None
        engine._check(L.axb_mgpu_create(int(n_devices), devs, C.byref(h)))
        self.h, self.n = h, n_devices
        self._owned = []

    def alloc(self, rank, nbytes):
        p = self.lib.axb_mgpu_alloc(self.h, rank, nbytes)
        if not p:
            raise EngineError(2, self.eng.last_error())
        self._owned.append((rank, p))
        return int(p)

    def upload(self, rank, array):
        """numpy array -> a new device buffer on `rank`; returns the device pointer."""
        import numpy as np
        a = np.ascontiguousarray(array)
        p = self.alloc(rank, max(a.nbytes, 4))
        self.eng._check(self.lib.axb_mgpu_h2d(self.h, rank, C.c_void_p(p), a.ctypes.data_as(C.c_void_p), a.nbytes))
        return p

    def download(self, rank, ptr, shape, dtype):
        import numpy as np
        out = np.empty(shape, dtype)
        self.eng._check(self.lib.axb_mgpu_d2h(self.h, rank, out.ctypes.data_as(C.c_void_p), C.c_void_p(ptr), out.nbytes))
        return out

    def _ptrs(self, ptrs):
        return (C.c_void_p * self.n)(*[None if p is None else C.c_void_p(p) for p in ptrs]) if ptrs is not None else None

    def gemm_rows(self, A, B, bias, Cout, rows, N, K, act="none"):
        r = (C.c_int64 * self.n)(*rows)
        self.eng._check(self.lib.axb_mgpu_gemm_rows(self.h, self._ptrs(A), self._ptrs(B), self._ptrs(bias), self._ptrs(Cout), r,
                                                    _i64(N), _i64(K), ACT[act]))

    def qgemm_w8a8_rows(self, a_q, a_scale, b_q, b_scales, out_scale, out_q, rows, N, K):
        r = (C.c_int64 * self.n)(*rows)
        self.eng._check(self.lib.axb_mgpu_qgemm_w8a8_rows(self.h, self._ptrs(a_q), _f(a_scale), self._ptrs(b_q), self._ptrs(b_scales),
                                                          _f(out_scale), self._ptrs(out_q), r, _i64(N), _i64(K)))

    def gemm_cols_allgather(self, X, x_chunks, W, bias, slab, gathered, M, n, K, act="none"):
        self.eng._check(self.lib.axb_mgpu_gemm_cols_allgather(self.h, self._ptrs(X), int(x_chunks), self._ptrs(W), self._ptrs(bias),
                                                              self._ptrs(slab), self._ptrs(gathered), _i64(M), _i64(n), _i64(K),
                                                              ACT[act]))

    def synchronize(self):
        self.eng._check(self.lib.axb_mgpu_synchronize(self.h))

    def close(self):
        if self.h:
            for rank, p in self._owned:
                self.lib.axb_mgpu_free(self.h, rank, C.c_void_p(p))
            self._owned = []
            self.lib.axb_mgpu_destroy(self.h)
            self.h = None


_engine = None


def get_engine(device: int | None = None) -> Engine:
    """Process-wide engine, initialised on `device` (default: torch's current device)."""
    global _engine
    if _engine is None:
        if device is None:
            import torch
            device = torch.cuda.current_device()
        _engine = Engine(device)
    return _engine
