"""The C host layer (libaxiom_b200_backend.so): table layout against the reference headers,
registration with the reference's own dispatcher, and host-side error behaviour.  CPU only."""
import ctypes
import os
import subprocess
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
from oracle_lib import axiom_source_tree

AXIOM_INCLUDE = os.path.join(axiom_source_tree() or "", "include")

LAYOUT_CHECK = r"""
#include <stddef.h>
#include "axiom/tensor.h"
#include "axiom/internal/backend_ops.h"
#include "axiom/internal/cuda_extension.h"
#include "axiom_b200_backend.h"
#define SAME(T1, T2, f) _Static_assert(offsetof(T1, f) == offsetof(T2, f), "offset of " #f)
_Static_assert(sizeof(ax_storage_t) == sizeof(axb_ax_storage_t), "storage size");
SAME(ax_storage_t, axb_ax_storage_t, data); SAME(ax_storage_t, axb_ax_storage_t, size_bytes);
SAME(ax_storage_t, axb_ax_storage_t, device); SAME(ax_storage_t, axb_ax_storage_t, generation);
_Static_assert(sizeof(ax_tensor_t) == sizeof(axb_ax_tensor_t), "tensor size");
SAME(ax_tensor_t, axb_ax_tensor_t, storage); SAME(ax_tensor_t, axb_ax_tensor_t, shape);
SAME(ax_tensor_t, axb_ax_tensor_t, strides); SAME(ax_tensor_t, axb_ax_tensor_t, ndim);
SAME(ax_tensor_t, axb_ax_tensor_t, dtype); SAME(ax_tensor_t, axb_ax_tensor_t, offset);
SAME(ax_tensor_t, axb_ax_tensor_t, layout);
_Static_assert(sizeof(struct ax_backend_ops) == sizeof(axb_ax_backend_ops_t), "vtable size");
#define SLOT(f) SAME(struct ax_backend_ops, axb_ax_backend_ops_t, f)
SLOT(name); SLOT(add); SLOT(mul_scalar); SLOT(gemm); SLOT(gemm_nt); SLOT(gemm_tn); SLOT(dwqkv_split_acc); SLOT(dwqkv_split_acc_hm); SLOT(qkv_head_gemm); SLOT(dattn_head_gemm_nt);
SLOT(mha_output_proj_fused); SLOT(gemm_relu); SLOT(gemm_ex); SLOT(add_relu); SLOT(softmax_rowwise); SLOT(bias_add);
SLOT(conv_gemm); SLOT(sum); SLOT(argmax); SLOT(equal); SLOT(fill); SLOT(copy); SLOT(relu); SLOT(sigmoid);
SLOT(leaky_relu); SLOT(gelu_op); SLOT(swish_op); SLOT(adam_update); SLOT(sgd_update); SLOT(device); SLOT(init);
SLOT(shutdown); SLOT(synchronize); SLOT(device_count); SLOT(storage_alloc); SLOT(storage_free); SLOT(memcpy_h2d);
SLOT(memcpy_d2h); SLOT(memcpy_d2d);
_Static_assert(sizeof(ax_cuda_extension_t) == sizeof(axb_ax_cuda_extension_t), "extension size");
#define EXT(f) SAME(ax_cuda_extension_t, axb_ax_cuda_extension_t, f)
EXT(head_interleave_qkv_split); EXT(head_interleave_qkv_split_bias); EXT(head_interleave); EXT(head_deinterleave);
EXT(head_deinterleave_qkv_merge); EXT(qkv_cache_build); EXT(bias_cache_build); EXT(conv_gemm_batched);
/* the slots are called through the reference's own prototypes: they must be assignable both ways */
static void same_signatures(ax_cuda_extension_t *r, const axb_ax_cuda_extension_t *m)
{
    r->head_interleave_qkv_split = m->head_interleave_qkv_split;
    r->head_interleave_qkv_split_bias = m->head_interleave_qkv_split_bias;
    r->head_interleave = m->head_interleave;
    r->head_deinterleave = m->head_deinterleave;
    r->head_deinterleave_qkv_merge = m->head_deinterleave_qkv_merge;
    r->qkv_cache_build = (ax_status_t (*)(float *, const float *, const float *, const float *, int64_t))m->qkv_cache_build;
    r->bias_cache_build = (ax_status_t (*)(float *, const float *, const float *, const float *, int64_t))m->bias_cache_build;
}
SAME(ax_cuda_extension_t, axb_ax_cuda_extension_t, sdpa_fwd); SAME(ax_cuda_extension_t, axb_ax_cuda_extension_t, sdpa_bwd);
SAME(ax_cuda_extension_t, axb_ax_cuda_extension_t, winograd_f23_prefer);
_Static_assert(AX_FLOAT32 == AXB_AX_FLOAT32 && AX_DEVICE_CUDA == AXB_AX_DEVICE_CUDA && AX_BACKEND_CUDA == AXB_AX_BACKEND_CUDA, "enums");
int main(void) { return 0; }
"""


@pytest.fixture(scope="module")
def backend():
    from axiom_b200 import build
    build.build()
    return ctypes.CDLL(build.BACKEND_SO)


def test_table_layout_matches_reference_headers(tmp_path):
    if not os.path.exists(os.path.join(AXIOM_INCLUDE, "axiom", "internal", "backend_ops.h")):
        pytest.skip("axiom headers not present on this machine")
    src = tmp_path / "layout.c"
    src.write_text(LAYOUT_CHECK)
    subprocess.run(["gcc", "-std=c11", "-Werror=incompatible-pointer-types", "-I", AXIOM_INCLUDE, "-I", os.path.join(ROOT, "include"), "-c", str(src),
                    "-o", str(tmp_path / "layout.o")], check=True)


def test_tables_are_filled(backend):
    backend.axb_backend_ops.restype = ctypes.c_void_p
    backend.axb_cuda_extension.restype = ctypes.c_void_p
    ops = backend.axb_backend_ops()
    slots = (ctypes.c_void_p * 58).from_address(ops)
    name = ctypes.cast(slots[0], ctypes.c_char_p).value
    assert name == b"b200_tcgen05"
    # 0 name, 1-4 binops, 5-10 unops, 11-12 scalar, 13 gemm, 14 gemm_nt, 15 gemm_tn
    assert all(slots[i] for i in (13, 14, 15))
    assert not any(slots[i] for i in range(1, 13))
    ext = (ctypes.c_void_p * 12).from_address(backend.axb_cuda_extension())
    assert ext[7] and ext[8] and ext[9] and not ext[10] and not ext[11]   # sdpa_fwd, sdpa_bwd, conv_gemm_batched set; Winograd NULL
    assert slots[16] and slots[17]                     # dwqkv_split_acc, dwqkv_split_acc_hm
    assert slots[18] and slots[19] and slots[20]       # qkv_head_gemm, dattn_head_gemm_nt, mha_output_proj_fused
    assert not slots[23]                               # add_relu (gemm_relu 21 and gemm_ex 22 are set)


def test_registers_with_the_reference_dispatcher(backend, reference):
    """ax_compute_register_backend accepts the table; without a GPU the init hook reports AX_ERR_BACKEND
    through ax_err_set and tensors cannot move to the device — nothing is computed on the host."""
    import numpy as np
    import torch
    lib = reference.lib
    backend.axb_backend_ops.restype = ctypes.c_void_p
    backend.axb_cuda_extension.restype = ctypes.c_void_p
    SKIP = ctypes.CFUNCTYPE(ctypes.c_int)
    ERR = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_char_p)
    skip_cb = SKIP(lambda: lib.ref_skip_init_flag())
    err_cb = ERR(lambda st, msg: lib.ref_err_set(st, msg))
    backend._keep = (skip_cb, err_cb)
    backend.axb_backend_set_hooks(skip_cb, err_cb)
    st = lib.ref_register_cuda_backend(ctypes.c_void_p(backend.axb_backend_ops()),
                                       ctypes.c_void_p(backend.axb_cuda_extension()))
    assert st == 0
    if torch.cuda.is_available():
        pytest.skip("GPU present: the device path is covered by the gpu-marked test")
    A = np.ones((2, 2), np.float32)
    C = np.zeros((2, 2), np.float32)
    f32p = ctypes.POINTER(ctypes.c_float)
    rc = lib.ref_device_gemm_op(0, A.ctypes.data_as(f32p), A.ctypes.data_as(f32p), None, C.ctypes.data_as(f32p),
                                ctypes.c_int64(2), ctypes.c_int64(2), ctypes.c_int64(2), ctypes.c_float(1), ctypes.c_float(0))
    assert rc != 0 and not C.any()


class _Storage(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("size_bytes", ctypes.c_size_t), ("refcount", ctypes.c_int),
                ("device", ctypes.c_int), ("is_arena_temp", ctypes.c_bool), ("generation", ctypes.c_uint64)]


class _Tensor(ctypes.Structure):
    pass


_Tensor._fields_ = [("storage", ctypes.POINTER(_Storage)), ("shape", ctypes.c_int64 * 8), ("strides", ctypes.c_int64 * 8),
                    ("ndim", ctypes.c_int), ("dtype", ctypes.c_int), ("offset", ctypes.c_int64),
                    ("requires_grad", ctypes.c_bool), ("grad", ctypes.POINTER(_Tensor)), ("grad_fn", ctypes.c_void_p),
                    ("layout", ctypes.c_int)]


def _tensor(buf, shape, device=0, dtype=0, strides=None):
    st = _Storage(ctypes.cast(buf, ctypes.c_void_p), ctypes.sizeof(buf), 1, device, False, 1)
    t = _Tensor()
    t.storage = ctypes.pointer(st)
    t.ndim, t.dtype, t.offset = len(shape), dtype, 0
    acc = 1
    for i in range(len(shape) - 1, -1, -1):
        t.shape[i] = shape[i]
        t.strides[i] = acc if strides is None else strides[i]
        acc *= shape[i]
    t._keep = st
    return t


def test_host_validation_of_the_gemm_slot(backend):
    """Failures are injected on the host: NULL, wrong rank, wrong dtype, strided and CPU-resident tensors are
    refused by the vtable slot with axiom's status codes and the message goes to the error hook; no kernel runs."""
    backend.axb_backend_ops.restype = ctypes.c_void_p
    slots = (ctypes.c_void_p * 58).from_address(backend.axb_backend_ops())
    GEMM = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(_Tensor), ctypes.POINTER(_Tensor), ctypes.POINTER(_Tensor))
    gemm = GEMM(slots[13])
    seen = []
    ERR = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_char_p)
    cb = ERR(lambda st, msg: seen.append((st, msg)))
    backend.axb_backend_set_hooks(None, cb)
    buf = (ctypes.c_float * 64)()
    ok = _tensor(buf, (4, 4), device=1)
    assert gemm(None, ctypes.byref(ok), ctypes.byref(ok)) == 1                                   # AX_ERR_NULL_ARG
    assert gemm(ctypes.byref(_tensor(buf, (4, 4, 1), device=1)), ctypes.byref(ok), ctypes.byref(ok)) == 3   # rank
    assert gemm(ctypes.byref(_tensor(buf, (4, 4), device=1, dtype=1)), ctypes.byref(ok), ctypes.byref(ok)) == 4  # dtype
    assert gemm(ctypes.byref(_tensor(buf, (4, 4), device=1, strides=(1, 4))), ctypes.byref(ok), ctypes.byref(ok)) == 6
    assert gemm(ctypes.byref(_tensor(buf, (4, 4), device=0)), ctypes.byref(ok), ctypes.byref(ok)) == 9       # on the CPU
    assert gemm(ctypes.byref(_tensor(buf, (4, 3), device=1)), ctypes.byref(ok), ctypes.byref(ok)) == 3       # K mismatch
    assert len(seen) == 6 and all(m for _, m in seen)
    backend.axb_backend_set_hooks(None, None)


def test_host_validation_of_the_attention_projection_slots(backend):
    """The attention-projection slots refuse wrong shapes, ranks, dtypes and host-resident tensors with axiom's status
    codes before anything reaches a kernel (shape rules of src/compute/backends/cpu_opt.c:6062-6119, 6527-6560, 6825-6857)."""
    backend.axb_backend_ops.restype = ctypes.c_void_p
    slots = (ctypes.c_void_p * 58).from_address(backend.axb_backend_ops())
    T, I64 = ctypes.POINTER(_Tensor), ctypes.c_int64
    dwqkv = ctypes.CFUNCTYPE(ctypes.c_int, T, T, T, T, T)(slots[16])
    dwqkv_hm = ctypes.CFUNCTYPE(ctypes.c_int, T, T, T, T, I64, I64, I64, I64, T, T, T)(slots[17])
    dattn = ctypes.CFUNCTYPE(ctypes.c_int, T, T, I64, I64, I64, I64, T)(slots[19])
    outproj = ctypes.CFUNCTYPE(ctypes.c_int, T, T, T, T, T, T, T, T)(slots[20])
    seen = []
    cb = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_char_p)(lambda st, msg: seen.append((st, msg)))
    backend.axb_backend_set_hooks(None, cb)
    buf = (ctypes.c_float * 4096)()
    t = lambda *shape, **kw: ctypes.byref(_tensor(buf, shape, device=kw.get("device", 1), dtype=kw.get("dtype", 0)))
    B, S, H, dk, D, rows = 2, 4, 2, 4, 8, 8
    # dwqkv_split_acc(x_flat [rows, D], dQKV [rows, 3D], dWq, dWk, dWv [D, D])
    assert dwqkv(None, t(rows, 3 * D), t(D, D), t(D, D), t(D, D)) == 1
    assert dwqkv(t(rows, D), t(rows, 2 * D), t(D, D), t(D, D), t(D, D)) == 3          # dQKV is not [rows, 3D]
    assert dwqkv(t(rows, D), t(rows, 3 * D), t(D, D), t(D, D + 1), t(D, D)) == 3      # a gradient is not [D, D]
    assert dwqkv(t(rows, D), t(rows, 3 * D, dtype=1), t(D, D), t(D, D), t(D, D)) == 4
    assert dwqkv(t(rows, D, device=0), t(rows, 3 * D), t(D, D), t(D, D), t(D, D)) == 9  # on the host
    # the head-major form: dQh, dKh, dVh [B*H, S, dk]
    assert dwqkv_hm(t(rows, D), t(B * H, S, dk), t(B * H, S, dk), t(B * H, S + 1, dk), B, S, H, dk, t(D, D), t(D, D), t(D, D)) == 3
    assert dwqkv_hm(t(rows + 1, D), t(B * H, S, dk), t(B * H, S, dk), t(B * H, S, dk), B, S, H, dk, t(D, D), t(D, D), t(D, D)) == 3
    assert dwqkv_hm(t(rows, D), t(B * H * S, dk), t(B * H, S, dk), t(B * H, S, dk), B, S, H, dk, t(D, D), t(D, D), t(D, D)) == 3  # rank
    # dattn_head_gemm_nt(dout [B*S, D], Wo [D, D], dO_head [B*H, S, dk])
    assert dattn(t(rows, D), t(D, D + 1), B, S, H, dk, t(B * H, S, dk)) == 3
    assert dattn(t(rows, D), t(D, D), B, S, H, dk, t(B * H, S, dk + 1)) == 3
    # mha_output_proj_fused(attn, Wo, bo?, dout, y?, dattn, dWo, dbo?)
    assert outproj(t(rows, D), t(D, D), None, t(rows, D), None, None, t(D, D), None) == 1       # dattn is required
    assert outproj(t(rows, D), t(D, D), t(D + 1), t(rows, D), t(rows, D), t(rows, D), t(D, D), None) == 3   # bo length
    assert outproj(t(rows, D), t(D, D), None, t(rows + 1, D), None, t(rows, D), t(D, D), None) == 3          # dout rows
    assert outproj(t(rows, D), t(D, D), None, t(rows, D), None, t(rows, D), t(D, D), t(D, device=0)) == 9   # dbo on the host
    assert len(seen) == 14 and all(m for _, m in seen)
    backend.axb_backend_set_hooks(None, None)

