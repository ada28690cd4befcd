"""CPU-only checks of the attention-layer oracle.

The double-precision restatement (oracle_lib.mha_f64) is pinned against the reference's own layer
(ax_mha_create + ax_layer_forward + ax_backward, compiled unmodified into oracle/_ref): forward for every
configuration, gradients for layers without biases.  With biases the reference's CPU backward is not usable as
an oracle: at some shapes it returns different dX / dW than the same layer without biases even when every bias
is zero.  That defect is recorded here so the GPU tests may rely on the restatement for that case.
"""
import numpy as np
import pytest

from oracle_lib import mha_f64, nerr


def inputs(oracle, B, S, D, with_bias):
    x = oracle.uniform((B, S, D), 7)
    W = oracle.normal((4, D, D), 13, sigma=1.0 / np.sqrt(D))
    b = oracle.uniform((4, D), 29) if with_bias else None
    return x, W, b, oracle.normal((B, S, D), 53)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(2, 4, 16, 2), (2, 128, 256, 4), (3, 50, 96, 4)])
def test_restatement_matches_reference_layer(reference, oracle, shape, causal):
    B, S, D, H = shape
    x, W, b, g = inputs(oracle, B, S, D, True)
    for bias in (None, b):
        st, ref = reference.mha_layer(x, W, bias, H, causal)
        assert st == 0
        assert nerr(ref["out"], mha_f64(x, W, bias, H, causal)["out"]) <= 1e-5   # tests/test_attention.c uses 1e-4 abs
    st, ref = reference.mha_layer(x, W, None, H, causal, dOut=g)
    assert st == 0
    want = mha_f64(x, W, None, H, causal, dOut=g)
    for key in ("out", "dX", "dW"):
        assert nerr(ref[key], want[key]) <= 5e-5, key


def test_reference_backward_with_biases_is_not_an_oracle(reference, oracle):
    """All-zero biases must give the gradients of the bias-free layer.  The reference does so at small shapes; where it
    does not, the restatement is right (it agrees with the reference's own bias-free run) and the GPU tests use it."""
    B, S, D, H = 1, 128, 256, 4
    x, W, b, g = inputs(oracle, B, S, D, True)
    st, without = reference.mha_layer(x, W, None, H, False, dOut=g)
    assert st == 0
    st, zeros = reference.mha_layer(x, W, b * 0, H, False, dOut=g)
    assert st == 0
    want = mha_f64(x, W, None, H, False, dOut=g)
    assert nerr(without["dX"], want["dX"]) <= 5e-5
    assert nerr(mha_f64(x, W, b * 0, H, False, dOut=g)["dX"], want["dX"]) == 0.0
    if nerr(zeros["dX"], without["dX"]) > 1e-4:
        pytest.xfail("reference defect: MHA backward with (zero) biases differs from the bias-free layer")
