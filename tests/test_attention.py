"""Scaled dot-product attention around BatchMatrixMultiplication: the oracle pinned on the reference's
golden predictions (Tests/NonReg/TestNetworkPropagation.cs:500-575), then the CUDA path against the oracle."""
import numpy as np
import pytest

from oracle import sharpnet_oracle as orc


def _golden_network(golden, key, causal, sdpa):
    """Conv1D(kernel 1) projections of X[b] ([4 channels, 5 steps]) to Q, K, V ([2, 5] each: 2 time steps of
    embedding 5), attention, Flatten, Linear(10 -> 3, [in, out] weights), Softmax."""
    X = np.asarray(golden["X_3_4_5"], np.float32).reshape(3, 4, 5)
    wq, wk, wv = (np.asarray(golden[f"{key}_w{n}"], np.float32).reshape(4, 2) for n in "qkv")
    Q, K, V = (np.stack([w.T @ X[b] for b in range(3)]).astype(np.float32) for w in (wq, wk, wv))
    y = sdpa(Q, K, V, False, causal)
    z = y.reshape(3, 10).astype(np.float64) @ np.asarray(golden[f"{key}_wlinear"], np.float64).reshape(10, 3)
    e = np.exp(z - z.max(1, keepdims=True))
    return e / e.sum(1, keepdims=True)


def test_oracle_attention_matches_reference_goldens(golden):
    for key, causal in (("sdpa", False), ("sdpa_causal", True)):
        p = _golden_network(golden, key, causal, lambda Q, K, V, s, c: orc.sdpa_forward(Q, K, V, s, c)[1])
        np.testing.assert_allclose(p.ravel(), golden[f"{key}_pred"], rtol=0, atol=1e-6)


def test_oracle_attention_backward_by_finite_differences():
    # the backward restates cuDNN's softmax Jacobian, which the reference's CPU code does not hold: check it numerically
    rng = np.random.default_rng(3)
    B, Tq, Tk, E = 2, 3, 4, 5
    Q, K, V = (rng.normal(size=s).astype(np.float32) for s in ((B, Tq, E), (B, Tk, E), (B, Tk, E)))
    dy = rng.normal(size=(B, Tq, E)).astype(np.float32)
    for causal in (False, True):
        w, _ = orc.sdpa_forward(Q, K, V, True, causal, f64=True)
        dQ, dK, dV = orc.sdpa_backward(Q, K, V, dy, w, True)

        def loss(q, k, v):
            return float((orc.sdpa_forward(q, k, v, True, causal, f64=True)[1] * dy).sum())
        eps = 1e-5
        for arr, grad, which in ((Q, dQ, 0), (K, dK, 1), (V, dV, 2)):
            for idx in ((0, 0, 0), (1, 2, 3), (1, 1, 4)):
                hi, lo = arr.astype(np.float64).copy(), arr.astype(np.float64).copy()
                hi[idx] += eps
                lo[idx] -= eps
                args_hi = [Q, K, V]; args_lo = [Q, K, V]
                args_hi[which], args_lo[which] = hi, lo
                num = (loss(*args_hi) - loss(*args_lo)) / (2 * eps)
                assert abs(num - grad[idx]) < 1e-6 * max(1.0, abs(num))


def test_oracle_softmax_rows():
    x = orc.uniform((7, 33), -3, 3, 1)
    y = orc.softmax_last_dimension(x)
    np.testing.assert_allclose(y.sum(1), 1.0, atol=1e-6)
    e = np.exp(x.astype(np.float64) - x.max(1, keepdims=True))
    np.testing.assert_allclose(y, e / e.sum(1, keepdims=True), atol=1e-7)


# ------------------------------------------------------------------------------------------ GPU
def _gpu_sdpa(wrapper):
    from sharpnet_b200.attention import ScaledDotProductAttentionForwardPropagation
    from sharpnet_b200.tensor import GPUTensor

    def run(Q, K, V, use_scale, causal):
        Qg, Kg, Vg = (GPUTensor(a.shape, a, wrapper) for a in (Q, K, V))
        y = GPUTensor(Q.shape, None, wrapper)
        ScaledDotProductAttentionForwardPropagation(Qg, Kg, Vg, y, False, None, use_scale, causal)
        return y.ContentAsFloatArray()
    return run


@pytest.mark.gpu
def test_gpu_attention_matches_reference_goldens(wrapper, golden):
    for key, causal in (("sdpa", False), ("sdpa_causal", True)):
        p = _golden_network(golden, key, causal, _gpu_sdpa(wrapper))
        np.testing.assert_allclose(p.ravel(), golden[f"{key}_pred"], rtol=0, atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(3, 12, 12, 7), (2, 5, 9, 4), (8, 128, 128, 64), (4, 96, 200, 32), (2, 64, 1500, 16)])
def test_gpu_attention_forward_backward_against_oracle(wrapper, shape, causal):
    from sharpnet_b200.attention import (ScaledDotProductAttentionBackwardPropagation,
                                         ScaledDotProductAttentionForwardPropagation)
    from sharpnet_b200.tensor import GPUTensor
    B, Tq, Tk, E = shape
    rng = np.random.default_rng(B * Tq + Tk)
    Q, K, V = (rng.uniform(-1.5, 1.5, s).astype(np.float32) for s in ((B, Tq, E), (B, Tk, E), (B, Tk, E)))
    dy = rng.uniform(-1.5, 1.5, (B, Tq, E)).astype(np.float32)
    Qg, Kg, Vg, DY = (GPUTensor(a.shape, a, wrapper) for a in (Q, K, V, dy))
    y = GPUTensor((B, Tq, E), None, wrapper)
    W = ScaledDotProductAttentionForwardPropagation(Qg, Kg, Vg, y, True, None, True, causal)
    wrapper.check_device_status()
    w64, y64 = orc.sdpa_forward(Q, K, V, True, causal, f64=True)
    w = W.ContentAsFloatArray()
    # the scores carry the 1e-5 * sqrt(E) GEMM bound (times |q||k| <= 2.25, over sqrt(E)); softmax has slope <= 1/4
    assert np.abs(w - w64).max() <= 1e-5 * 2.25 + 1e-6
    np.testing.assert_allclose(w.sum(-1), 1.0, atol=1e-5)
    if causal:
        r, c = np.triu_indices(Tq, 1, Tk)
        assert not w[:, r, c].any()                  # exp(-1e12 - max) is exactly 0
    assert np.abs(y.ContentAsFloatArray() - y64).max() <= 1e-5 * np.sqrt(Tk) * 1.5 + 1e-5
    if B * Tq * Tk <= 200000:
        wm, ym = orc.sdpa_forward(Q, K, V, True, causal)          # the reference's CPU arithmetic
        assert np.abs(w - wm).max() <= 1e-5 * 2.25 + 1e-6
        assert np.abs(y.ContentAsFloatArray() - ym).max() <= 1e-5 * np.sqrt(Tk) * 1.5 + 1e-5
    dQ, dK, dV = (GPUTensor(s, None, wrapper) for s in ((B, Tq, E), (B, Tk, E), (B, Tk, E)))
    ScaledDotProductAttentionBackwardPropagation(dQ, dK, dV, Qg, Kg, Vg, DY, W, True)
    wrapper.check_device_status()
    dQ64, dK64, dV64 = orc.sdpa_backward(Q, K, V, dy, w, True)
    assert np.abs(dV.ContentAsFloatArray() - dV64).max() <= 1e-5 * np.sqrt(Tq) * 1.5 + 1e-5
    assert np.abs(dQ.ContentAsFloatArray() - dQ64).max() <= 1e-4
    assert np.abs(dK.ContentAsFloatArray() - dK64).max() <= 1e-4


@pytest.mark.gpu
def test_gpu_softmax_alone(wrapper):
    from sharpnet_b200.tensor import GPUTensor
    for shape in ((1, 1), (5, 3), (2, 3, 130), (7, 1024), (3, 1025), (2, 5000)):
        x = orc.uniform(shape, -4, 4, 5)
        dy = orc.uniform(shape, -1.5, 1.5, 6)
        X, DY = GPUTensor(shape, x, wrapper), GPUTensor(shape, dy, wrapper)
        Y, DX = GPUTensor(shape, None, wrapper), GPUTensor(shape, None, wrapper)
        X.SoftmaxLastDimension(Y)
        y = Y.ContentAsFloatArray()
        np.testing.assert_allclose(y, orc.softmax_last_dimension(x), rtol=2e-6, atol=1e-8)
        DX.SoftmaxGradientLastDimension(DY, Y)
        np.testing.assert_allclose(DX.ContentAsFloatArray(), orc.softmax_gradient_last_dimension(dy, y, f64=True),
                                   rtol=0, atol=2e-6)
        DY.SoftmaxGradientLastDimension(DY, Y)       # in place, as the attention layer calls it
        np.testing.assert_array_equal(DY.ContentAsFloatArray(), DX.ContentAsFloatArray())
