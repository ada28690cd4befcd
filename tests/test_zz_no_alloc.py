"""The allocation-free skinny GEMM (axb_skinny_gemm_static) against the regular entry point.

Some users of this library are not allowed to allocate device memory while they
run — an engine that gave the whole GPU to its own arena at start-up, a serving
loop that must not hit the stall an allocation can cause.  For them the library
carries one entry point whose scratch is a fixed array inside the library
itself.  This test calls it through the C ABI twice in a row, with different
operands, and requires the same numbers as axb_gemm_bias_act (same kernel, so
the results must agree to the bit; the check also states the fp32 tolerance the
other tests use).  The file sorts last so a failure here cannot hide another.
"""
import numpy as np
import pytest
import torch

from oracle_lib import nerr

pytestmark = pytest.mark.gpu


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


@pytest.mark.parametrize("shape", [(1, 4096, 4096), (8, 4096, 4096), (5, 1000, 777), (2, 512, 8192), (16, 4096, 4096),
                                   (32, 4096, 4096), (9, 1000, 1028), (20, 1001, 777)])
def test_static_scratch_matches_regular_entry_point(engine, oracle, shape):
    M, N, K = shape
    W = dev(oracle.normal((K, N), 13, sigma=1.0 / np.sqrt(K)))
    bias = dev(oracle.uniform((N,), 29))
    for call, seed in enumerate((31, 37)):                      # two calls in a row share the built-in scratch
        x_host = oracle.normal((M, K), seed)
        x = dev(x_host)
        want = torch.empty((M, N), device="cuda")
        engine.gemm_bias_act(x, W, bias, want, M, N, K, act="gelu")
        got = torch.full((M, N), float("nan"), device="cuda")
        if call == 1:
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
        engine.skinny_gemm_static(x, W, bias, got, M, N, K, act="gelu")
        torch.cuda.synchronize()
        if call == 1:   # the kernel variant was loaded by the first call: the second changes nothing on the device
            assert torch.cuda.mem_get_info()[0] == free_before
        assert engine.skinny_gemm_static_error() == 0
        g, w = got.cpu().numpy(), want.cpu().numpy()
        assert nerr(g, w) <= 1e-5, (call, nerr(g, w))
        np.testing.assert_array_equal(g, w)
        ref = oracle.bias_act(oracle.gemm(x_host, W.cpu().numpy()), bias.cpu().numpy(), "gelu")
        assert nerr(g, ref) <= 1e-5


def test_static_scratch_refuses_oversized_shapes(engine):
    from axiom_b200.engine import EngineError
    M, N, K = 32, 8192, 16386                # K % 4 != 0 keeps it off the tensor-core kernel: split-K scratch beyond the 4 MiB array
    x = torch.zeros((M, K), device="cuda")
    W = torch.zeros((K, N), device="cuda")
    y = torch.zeros((M, N), device="cuda")
    with pytest.raises(EngineError) as e:
        engine.skinny_gemm_static(x, W, None, y, M, N, K)
    assert e.value.status == 6 and "scratch" in str(e.value)
    with pytest.raises(EngineError):
        engine.skinny_gemm_static(torch.zeros((33, 8), device="cuda"), torch.zeros((8, 8), device="cuda"), None,
                                  torch.zeros((33, 8), device="cuda"), 33, 8, 8)
