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
@pytest.mark.parametrize("shape", [(3, 12, 12, 7), (2, 5, 9, 4), (8, 128, 128, 64), (4, 96, 200, 32), (2, 64, 1500, 16),
                                   (5, 100, 72, 24), (3, 300, 128, 128), (6, 40, 32, 64), (2, 130, 60, 36),
                                   (80, 128, 128, 6)])
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
    # a score row that fits one tile (up to 128 keys, head width up to 128 and a multiple of 4, 16 queries or more):
    # one kernel for the forward pass, three for the backward pass (dV; dScores + dQ; dK)
    fused = Tk <= 128 and E <= 128 and E % 4 == 0 and Tk % 4 == 0 and Tq >= 16
    n0 = wrapper.launch_count()
    W = ScaledDotProductAttentionForwardPropagation(Qg, Kg, Vg, y, True, None, True, causal)
    wrapper.check_device_status()
    if fused:
        assert wrapper.launch_count() - n0 == 1 and wrapper.last_kernel().startswith("attention_fwd")
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
    n0 = wrapper.launch_count()
    ScaledDotProductAttentionBackwardPropagation(dQ, dK, dV, Qg, Kg, Vg, DY, W, True)
    wrapper.check_device_status()
    if fused:      # two launches (dScores + dQ; dV and dK as one grouped product) instead of four, the same gradients
        assert wrapper.last_kernel().endswith("_grouped"), wrapper.last_kernel()
        from sharpnet_b200._capi import TUNE_NO_FUSED_ATTN
        n_fused = wrapper.launch_count() - n0
        dQ2, dK2, dV2 = (GPUTensor(s, None, wrapper) for s in ((B, Tq, E), (B, Tk, E), (B, Tk, E)))
        wrapper.set_tuning(TUNE_NO_FUSED_ATTN, 1)
        try:
            n0 = wrapper.launch_count()
            ScaledDotProductAttentionBackwardPropagation(dQ2, dK2, dV2, Qg, Kg, Vg, DY, W, True)
            assert n_fused == 2 and wrapper.launch_count() - n0 >= 4
        finally:
            wrapper.set_tuning(TUNE_NO_FUSED_ATTN, 0)
        for a, b2 in ((dQ, dQ2), (dK, dK2), (dV, dV2)):
            assert np.abs(a.ContentAsFloatArray() - b2.ContentAsFloatArray()).max() <= 2e-5
    dQ64, dK64, dV64 = orc.sdpa_backward(Q, K, V, dy, w, True)
    assert np.abs(dV.ContentAsFloatArray() - dV64).max() <= 1e-5 * np.sqrt(Tq) * 1.5 + 1e-5
    assert np.abs(dQ.ContentAsFloatArray() - dQ64).max() <= 1e-4
    assert np.abs(dK.ContentAsFloatArray() - dK64).max() <= 1e-4


@pytest.mark.gpu
def test_gpu_attention_seeded_sweep(wrapper):
    """A seeded draw of batch, query / key lengths, head widths, scaling and masking: every tile shape of the fused
    kernels (and the paths beside them) against the float64 oracle, forward and backward."""
    from sharpnet_b200.attention import (ScaledDotProductAttentionBackwardPropagation,
                                         ScaledDotProductAttentionForwardPropagation)
    from sharpnet_b200.tensor import GPUTensor
    rng = np.random.default_rng(7)
    kernels = set()
    for it in range(90):
        B = int(rng.choice([1, 2, 3, 7, 12]))
        Tq = int(rng.choice([16, 17, 40, 64, 100, 128, 129, 200, 300]))
        Tk = int(rng.choice([8, 12, 32, 36, 60, 64, 72, 100, 128, 132, 200]))
        E = int(rng.choice([4, 8, 20, 32, 36, 64, 68, 100, 128, 132]))
        causal = False
        if rng.integers(3) == 0 and Tq <= 128:
            Tk, causal = Tq, bool(rng.integers(2))
        use_scale = bool(rng.integers(2))
        g = np.random.default_rng(100 + it)
        Q, K, V = (g.uniform(-1.5, 1.5, s).astype(np.float32) for s in ((B, Tq, E), (B, Tk, E), (B, Tk, E)))
        dy = g.uniform(-1.5, 1.5, (B, Tq, E)).astype(np.float32)
        Qg, Kg, Vg, DY = (GPUTensor(a.shape, a, wrapper) for a in (Q, K, V, dy))
        y = GPUTensor((B, Tq, E), None, wrapper)
        W = ScaledDotProductAttentionForwardPropagation(Qg, Kg, Vg, y, True, None, use_scale, causal)
        kernels.add(wrapper.last_kernel())
        wrapper.check_device_status()
        w64, y64 = orc.sdpa_forward(Q, K, V, use_scale, causal, f64=True)
        wt = W.ContentAsFloatArray()
        slack = 4.0 * (1.0 if use_scale else np.sqrt(E))     # unscaled scores are sqrt(E) times larger
        case = (it, B, Tq, Tk, E, causal, use_scale)
        assert np.abs(wt - w64).max() <= (1e-5 * 2.25 + 1e-6) * slack, case
        assert np.abs(y.ContentAsFloatArray() - y64).max() <= (1e-5 * np.sqrt(Tk) * 1.5 + 1e-5) * slack, case
        dQ, dK, dV = (GPUTensor(s, None, wrapper) for s in ((B, Tq, E), (B, Tk, E), (B, Tk, E)))
        ScaledDotProductAttentionBackwardPropagation(dQ, dK, dV, Qg, Kg, Vg, DY, W, use_scale)
        kernels.add(wrapper.last_kernel())
        wrapper.check_device_status()
        dQ64, dK64, dV64 = orc.sdpa_backward(Q, K, V, dy, wt, use_scale)
        assert np.abs(dV.ContentAsFloatArray() - dV64).max() <= 1e-5 * np.sqrt(Tq) * 1.5 + 1e-5, case
        assert np.abs(dQ.ContentAsFloatArray() - dQ64).max() <= 5e-5 * slack, case
        assert np.abs(dK.ContentAsFloatArray() - dK64).max() <= 5e-5 * slack, case
    assert sum(k.startswith("attention_fwd") for k in kernels) >= 6 and any(k.endswith("_grouped") for k in kernels), kernels


@pytest.mark.gpu
def test_gpu_softmax_alone(wrapper):
    from sharpnet_b200.tensor import GPUTensor
    # (the last three: enough short rows for the kernel that takes several rows per warp, 4 and 2 at a time)
    for shape in ((1, 1), (5, 3), (2, 3, 130), (7, 1024), (3, 1025), (2, 5000), (20001, 100), (3, 4001, 32), (12001, 200)):
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


# ------------------------------------------------------------------------------------------ multi-head attention
from sharpnet_b200._capi import W_IN_OUT, W_OUT_IN  # noqa: E402


def _softmax64(z):
    e = np.exp(z - z.max(1, keepdims=True))
    return e / e.sum(1, keepdims=True)


def _mha_tf_network(golden, case, mha):
    """Tests/NonReg/TestNetworkPropagation.cs:580-623: X [3, 7 channels, 15] -> three Conv1D(kernel 1, 2 filters)
    -> MultiHeadAttention(3 heads x 5) on Q, K, V [3, 2 steps, 15] -> Flatten -> Linear(30 -> 3) -> Softmax, all
    weights [in, out].  ``mha(Q, K, V, weights, biases, heads, key_dim, value_dim, causal, layout)`` -> y."""
    g = golden["mha_tf"]
    X = orc.numpy_array_for_tests(3, 7, 15)
    Q, K, V = (np.stack([np.asarray(g[k], np.float32).reshape(7, 2).T @ X[b] for b in range(3)]).astype(np.float32)
               for k in ("conv_q", "conv_k", "conv_v"))
    weights = [np.asarray(g[k], np.float32).reshape(15, 15) for k in ("w_q", "w_k", "w_v", "w_o")]
    biases = [np.zeros(15, np.float32)] * 4 if case["use_bias"] else None       # biases start at zero (:300)
    y = mha(Q, K, V, weights, biases, 3, 5, 5, case["causal"], W_IN_OUT)
    return _softmax64(y.reshape(3, 30).astype(np.float64) @ np.asarray(g["w_linear"], np.float64).reshape(30, 3))


def _mha_pt_loss(golden, name, case, mha):
    """Tests/NonReg/ParallelRunWithPyTorch.cs:1013-1129: X [10, 2 channels, 6] -> three Conv1D(kernel 1, 2 filters,
    [out, in, 1]) -> MultiHeadAttention(3 heads x 2, in_proj_weight [18, 6]) -> Flatten -> Linear(12 -> 3) -> Softmax,
    all weights [out, in]; returns the CategoricalCrossentropy loss on Y = y_numpy_array_for_tests(10, 3)."""
    g = golden["mha_pt_" + name]
    X = orc.numpy_array_for_tests(10, 2, 6)
    Y = orc.y_numpy_array_for_tests(10, 3)
    Q, K, V = (np.stack([np.asarray(g[k], np.float32).reshape(2, 2) @ X[b] for b in range(10)]).astype(np.float32)
               for k in ("conv_q", "conv_k", "conv_v"))
    inw = np.asarray(g["in_proj_weight"], np.float32).reshape(18, 6)
    weights = [inw[:6].copy(), inw[6:12].copy(), inw[12:].copy(), np.asarray(g["out_proj_weight"], np.float32).reshape(6, 6)]
    biases = [np.zeros(6, np.float32)] * 4 if name == "with_bias" else None
    y = mha(Q, K, V, weights, biases, 3, 2, 2, case["causal"], W_OUT_IN)
    p = _softmax64(y.reshape(10, 12).astype(np.float64) @ np.asarray(g["w_linear"], np.float64).reshape(3, 12).T)
    return float(-(Y * np.log(p)).sum(1).mean())


def _oracle_mha(f64):
    return lambda Q, K, V, w, b, H, kd, vd, causal, layout: orc.multihead_attention_forward(
        Q, K, V, w, b, H, kd, vd, causal, layout, f64=f64)[0]


@pytest.mark.parametrize("f64", [False, True])
def test_oracle_multihead_attention_matches_reference_goldens(golden, f64):
    for case in golden["mha_tf"]["cases"]:
        p = _mha_tf_network(golden, case, _oracle_mha(f64))
        np.testing.assert_allclose(p.ravel(), case["pred_before"], rtol=0, atol=1e-6)
    for name in ("no_bias", "with_bias"):
        for case in golden["mha_pt_" + name]["cases"]:
            assert abs(_mha_pt_loss(golden, name, case, _oracle_mha(f64)) - case["loss_before"]) <= 1e-6


def _mha_random(B, Tq, Tk, H, kd, seed, bias):
    rng = np.random.default_rng(seed)
    E = H * kd
    Q, K, V = (rng.normal(size=s).astype(np.float32) for s in ((B, Tq, E), (B, Tk, E), (B, Tk, E)))
    lim = np.sqrt(6.0 / (2 * E))
    weights = [rng.uniform(-lim, lim, (E, E)).astype(np.float32) for _ in range(4)]
    biases = [rng.uniform(-0.2, 0.2, E).astype(np.float32) for _ in range(4)] if bias else None
    dy = rng.normal(size=(B, Tq, E)).astype(np.float32)
    return Q, K, V, weights, biases, dy


@pytest.mark.parametrize("layout", [W_OUT_IN, W_IN_OUT])
def test_oracle_multihead_attention_backward_by_finite_differences(layout):
    B, Tq, Tk, H, kd = 2, 3, 3, 2, 2
    Q, K, V, weights, biases, dy = _mha_random(B, Tq, Tk, H, kd, 5, True)
    y, cache = orc.multihead_attention_forward(Q, K, V, weights, biases, H, kd, kd, True, layout, f64=True)
    dQ, dK, dV, dws, dbs = orc.multihead_attention_backward(Q, K, V, dy, weights, cache, H, kd, kd, 1.0, layout)

    def loss(Q_, K_, V_, w_, b_):
        return float((orc.multihead_attention_forward(Q_, K_, V_, w_, b_, H, kd, kd, True, layout, f64=True)[0] * dy).sum())
    eps = 1e-6
    checks = [("Q", dQ, (1, 2, 3)), ("K", dK, (0, 1, 2)), ("V", dV, (1, 0, 0))]
    checks += [(("w", i), dws[i], (1, 3)) for i in range(4)] + [(("b", i), dbs[i], (2,)) for i in range(4)]
    for which, grad, idx in checks:
        vals = {"Q": Q.astype(np.float64), "K": K.astype(np.float64), "V": V.astype(np.float64),
                "w": [w.astype(np.float64) for w in weights], "b": [b.astype(np.float64) for b in biases]}
        num = []
        for sign in (1, -1):
            v = {k: ([a.copy() for a in x] if isinstance(x, list) else x.copy()) for k, x in vals.items()}
            target = v[which] if isinstance(which, str) else v[which[0]][which[1]]
            target[idx] += sign * eps
            num.append(loss(v["Q"], v["K"], v["V"], v["w"], v["b"]))
        num = (num[0] - num[1]) / (2 * eps)
        assert abs(num - grad[idx]) < 2e-6 * max(1.0, abs(num)), (which, num, grad[idx])


def _gpu_mha(wrapper, keep=None):
    from sharpnet_b200.attention import MultiheadAttention
    from sharpnet_b200.tensor import GPUTensor

    def run(Q, K, V, weights, biases, H, kd, vd, causal, layout):
        layer = MultiheadAttention(H, kd, vd, biases is not None, biases is not None, causal, Q.shape[2], wrapper, layout)
        flat_w = np.concatenate([w.ravel() for w in weights])
        layer.Weights.storage[: flat_w.size].copy_(GPUTensor((flat_w.size,), flat_w, wrapper).storage)
        if biases is not None:
            flat_b = np.concatenate(biases)
            layer.Bias.storage[: flat_b.size].copy_(GPUTensor((flat_b.size,), flat_b, wrapper).storage)
        Qg, Kg, Vg = (GPUTensor(a.shape, a, wrapper) for a in (Q, K, V))
        y = GPUTensor(Q.shape, None, wrapper)
        layer.ForwardPropagation([Qg, Kg, Vg], y, True)
        wrapper.check_device_status()
        if keep is not None:
            keep.update(layer=layer, X=[Qg, Kg, Vg])
        return y.ContentAsFloatArray()
    return run


@pytest.mark.gpu
def test_gpu_multihead_attention_matches_reference_goldens(wrapper, golden):
    for case in golden["mha_tf"]["cases"]:
        p = _mha_tf_network(golden, case, _gpu_mha(wrapper))
        np.testing.assert_allclose(p.ravel(), case["pred_before"], rtol=0, atol=1e-6)
    for name in ("no_bias", "with_bias"):
        for case in golden["mha_pt_" + name]["cases"]:
            assert abs(_mha_pt_loss(golden, name, case, _gpu_mha(wrapper)) - case["loss_before"]) <= 1e-6


@pytest.mark.gpu
@pytest.mark.parametrize("layout", [W_OUT_IN, W_IN_OUT])
@pytest.mark.parametrize("shape,causal,bias", [((2, 3, 3, 2, 2), True, True), ((3, 7, 7, 3, 5), False, False),
                                               ((4, 64, 64, 8, 32), True, True), ((2, 128, 128, 4, 64), False, True),
                                               ((2, 48, 80, 4, 16), False, True)])
def test_gpu_multihead_attention_forward_backward_against_oracle(wrapper, layout, shape, causal, bias):
    from sharpnet_b200.tensor import GPUTensor
    B, Tq, Tk, H, kd = shape
    E = H * kd
    Q, K, V, weights, biases, dy = _mha_random(B, Tq, Tk, H, kd, 11 + B + Tq, bias)
    keep = {}
    y = _gpu_mha(wrapper, keep)(Q, K, V, weights, biases, H, kd, kd, causal, layout)
    y64, cache = orc.multihead_attention_forward(Q, K, V, weights, biases, H, kd, kd, causal, layout, f64=True)
    # four chained products of O(1) values over K = E or T terms each: the 1e-5 * sqrt(K) bound, with head room
    tol = 1e-5 * np.sqrt(max(E, Tk)) * 4 + 2e-5
    assert np.abs(y - y64).max() <= tol
    if B * Tq * E <= 40000:
        ym = orc.multihead_attention_forward(Q, K, V, weights, biases, H, kd, kd, causal, layout)[0]
        assert np.abs(y - ym).max() <= tol
    layer = keep["layer"]
    dX = [GPUTensor(a.shape, None, wrapper) for a in (Q, K, V)]
    layer.BackwardPropagation(keep["X"], GPUTensor(dy.shape, dy, wrapper), dX, 1.0)
    wrapper.check_device_status()
    dQ, dK, dV, dws, dbs = orc.multihead_attention_backward(Q, K, V, dy, weights, cache, H, kd, kd, 1.0, layout)
    gtol = 1e-5 * np.sqrt(max(E, Tk, B * max(Tq, Tk))) * 16 + 1e-4
    for got, ref in zip(dX, (dQ, dK, dV)):
        assert np.abs(got.ContentAsFloatArray() - ref).max() <= gtol
    gws, gbs = layer.gradients()
    for got, ref in zip(gws, dws):
        assert np.abs(got.ContentAsFloatArray() - ref).max() <= gtol
    if bias:
        for got, ref in zip(gbs, dbs):
            assert np.abs(got.ContentAsFloatArray() - ref).max() <= gtol


@pytest.mark.gpu
@pytest.mark.parametrize("layout", [W_OUT_IN, W_IN_OUT])
def test_gpu_multihead_attention_head_width_not_a_multiple_of_four(wrapper, layout):
    """Heads 6 wide with embed_dim a multiple of 4: the projections run on the tensor cores and store their result
    split by head through runs of 6 floats, which a group of four columns straddles.  K of the last wave is cut on
    purpose (tuning key 8) so that the reduction pass does that store."""
    from sharpnet_b200 import _capi
    from sharpnet_b200.tensor import GPUTensor
    B, T, H, kd = 4, 128, 128, 6
    E = H * kd
    Q, K, V, weights, biases, dy = _mha_random(B, T, T, H, kd, 77, True)
    y64, cache = orc.multihead_attention_forward(Q, K, V, weights, biases, H, kd, kd, True, layout, f64=True)
    dQ, dK, dV, dws, dbs = orc.multihead_attention_backward(Q, K, V, dy, weights, cache, H, kd, kd, 1.0, layout)
    tol = 1e-5 * np.sqrt(E) * 4 + 2e-5
    gtol = 1e-5 * np.sqrt(B * T) * 16 + 1e-4
    for splits in (0, 3):
        wrapper.set_tuning(_capi.TUNE_FORCE_SPLITS, splits)
        try:
            if splits:      # the chooser does cut this projection's K when told to
                x2, w2, y2 = GPUTensor((B * T, E), Q, wrapper), GPUTensor((E, E), weights[0], wrapper), GPUTensor((B * T, E), None, wrapper)
                assert wrapper.lib.snb200_dense_fwd(wrapper.handle, layout, B * T, E, E, x2.Pointer, w2.Pointer, None, 5,
                                                    None, y2.Pointer) == 0
                assert "splitk" in wrapper.last_kernel()
            keep = {}
            y = _gpu_mha(wrapper, keep)(Q, K, V, weights, biases, H, kd, kd, True, layout)
            assert np.abs(y - y64).max() <= tol
            dX = [GPUTensor(a.shape, None, wrapper) for a in (Q, K, V)]
            keep["layer"].BackwardPropagation(keep["X"], GPUTensor(dy.shape, dy, wrapper), dX, 1.0)
            wrapper.check_device_status()
        finally:
            wrapper.set_tuning(_capi.TUNE_FORCE_SPLITS, 0)
        for got, ref in zip(dX, (dQ, dK, dV)):
            assert np.abs(got.ContentAsFloatArray() - ref).max() <= gtol
        gws, gbs = keep["layer"].gradients()
        for got, ref in zip(gws, dws):
            assert np.abs(got.ContentAsFloatArray() - ref).max() <= gtol
        for got, ref in zip(gbs, dbs):
            assert np.abs(got.ContentAsFloatArray() - ref).max() <= gtol


@pytest.mark.gpu
def test_gpu_transpose_second_and_third_dimension(wrapper):
    from sharpnet_b200.tensor import GPUTensor
    for shape in ((1, 1, 1, 1), (2, 3, 4, 5), (3, 7, 2, 8), (4, 16, 33, 64), (2, 5, 3), (6, 128, 8, 32), (3, 2, 1000, 3)):
        x = orc.uniform(shape, -1, 1, sum(shape))
        src = GPUTensor(shape, x, wrapper)
        dst = GPUTensor(shape, None, wrapper)
        src.TransposeSecondAndThirdDimension(dst)
        assert dst.Shape == [shape[0], shape[2], shape[1]] + list(shape[3:])
        np.testing.assert_array_equal(dst.ContentAsFloatArray(), orc.transpose_second_third(x))
        back = GPUTensor(shape, None, wrapper)
        dst.TransposeSecondAndThirdDimension(back)                    # the permutation is its own inverse
        np.testing.assert_array_equal(back.ContentAsFloatArray(), x)


@pytest.mark.gpu
def test_gpu_multihead_attention_argument_errors(wrapper):
    from sharpnet_b200 import _capi
    from sharpnet_b200.attention import MultiheadAttention
    from sharpnet_b200.tensor import GPUTensor
    with pytest.raises(ValueError):
        MultiheadAttention(3, 2, 2, False, False, False, 8, wrapper)          # heads * value_dim != embed
    layer = MultiheadAttention(2, 4, 4, True, True, False, 8, wrapper)
    Q, K = GPUTensor((2, 3, 8), None, wrapper), GPUTensor((2, 5, 8), None, wrapper)
    with pytest.raises(ValueError):
        layer.ForwardPropagation([Q, K, GPUTensor((2, 4, 8), None, wrapper)], GPUTensor((2, 3, 8), None, wrapper))
    lib, h = wrapper.lib, wrapper.handle
    desc = _capi.MhaDesc(0, 2, 3, 5, 8, 2, 4, 4, 0)
    # nothing for the forward pass; the backward pass: d_attention_heads, the three projection-output gradients, the
    # gradient of the scores, each rounded up to 64 floats
    assert lib.snb200_mha_scratch_floats(desc, 0) == 0
    assert lib.snb200_mha_scratch_floats(desc, 1) == 64 + 64 + 128 + 128 + 64
    bad = _capi.MhaDesc(0, 2, 3, 5, 8, 3, 4, 4, 0)
    assert lib.snb200_mha_fwd(h, bad, _capi.MhaWeights(), None, None, None, _capi.MhaState(), None, None) == 7
    assert "embed_dim" in lib.snb200_last_error_string(h).decode()
    assert lib.snb200_mha_fwd(h, desc, _capi.MhaWeights(), None, None, None, _capi.MhaState(), None, None) == 7
    assert lib.snb200_mha_fwd(h, None, None, None, None, None, None, None, None) == 7


# ------------------------------------------------------------------------------------------ training replays
# The reference's multi-head goldens after training pin the backward pass (dQ, dK, dV, weight and bias gradients)
# and the momentum update: Tests/NonReg/TestNetworkPropagation.cs:580-623 (Keras layout, one batch of 3, SGD lr 0.01,
# momentum 0.9, 10 epochs, predictions at 1e-6) and Tests/NonReg/ParallelRunWithPyTorch.cs:1013-1129 (PyTorch layout,
# batches of 2 in order, lr 0.1, momentum 0.9, 10 epochs, CategoricalCrossentropy loss at 1e-6).
# Network: X -> three Conv1D(kernel 1, 2 filters, with bias) -> MultiHeadAttention -> Flatten -> Linear(3, with
# bias) -> Softmax.  The convolutions are not on the path: they run on the host in float64 in both replays.
class _MhaNet:
    def __init__(self, golden, key, case, use_bias):
        g = golden[key]
        self.tf = key == "mha_tf"
        self.causal, self.use_bias = case["causal"], use_bias
        if self.tf:
            self.B, self.C, self.L, self.H, self.kd, self.batch, self.lr = 3, 7, 15, 3, 5, 3, 0.01
            self.layout = W_IN_OUT
            self.conv_w = [np.asarray(g[k], np.float64).reshape(7, 2).T.copy() for k in ("conv_q", "conv_k", "conv_v")]
            self.mha_w = [np.asarray(g[k], np.float64).reshape(15, 15) for k in ("w_q", "w_k", "w_v", "w_o")]
            self.lin_w = np.asarray(g["w_linear"], np.float64).reshape(30, 3)            # [in, out]
        else:
            self.B, self.C, self.L, self.H, self.kd, self.batch, self.lr = 10, 2, 6, 3, 2, 2, 0.1
            self.layout = W_OUT_IN
            self.conv_w = [np.asarray(g[k], np.float64).reshape(2, 2) for k in ("conv_q", "conv_k", "conv_v")]
            inw = np.asarray(g["in_proj_weight"], np.float64).reshape(18, 6)
            self.mha_w = [inw[:6].copy(), inw[6:12].copy(), inw[12:].copy(),
                          np.asarray(g["out_proj_weight"], np.float64).reshape(6, 6)]
            self.lin_w = np.asarray(g["w_linear"], np.float64).reshape(3, 12)            # [out, in]
        self.E = self.H * self.kd
        self.conv_b = [np.zeros(2) for _ in range(3)]
        self.mha_b = [np.zeros(self.E) for _ in range(4)] if use_bias else None
        self.lin_b = np.zeros(3)
        self.X = orc.numpy_array_for_tests(self.B, self.C, self.L).astype(np.float64)
        self.Y = orc.y_numpy_array_for_tests(self.B, 3).astype(np.float64)
        self.momentum = 0.9

    def conv_forward(self, Xb):
        return [np.stack([w @ x + b[:, None] for x in Xb]) for w, b in zip(self.conv_w, self.conv_b)]   # [n, 2, L] each

    def conv_gradients(self, Xb, dQKV):
        return ([sum(d[i] @ Xb[i].T for i in range(len(Xb))) for d in dQKV], [d.sum((0, 2)) for d in dQKV])

    def linear(self, flat):
        return flat @ (self.lin_w if self.tf else self.lin_w.T) + self.lin_b

    def batches(self):
        return [slice(s, s + self.batch) for s in range(0, self.B, self.batch)]


class _SdpaPtNet:
    """Tests/NonReg/ParallelRunWithPyTorch.cs:963-1010: X [6, 4 channels, 5] -> three Conv1D(kernel 1, 2 filters,
    [out, in, 1], with bias) -> ScaledDotProductAttention(no scaling) on Q, K, V [n, 2 steps, 5] -> Flatten ->
    Linear(10 -> 3, [out, in]) -> Softmax; CategoricalCrossentropy; SGD lr 0.1, momentum 0.9, weight decay 0.07 in the
    PyTorch compatibility mode (every gradient, biases included, gets + batch * wd * parameter:
    Prod/Layers/Linear.cs:167-181, ConvolutionLayer.cs:210-220); batches of 2."""
    lr, momentum, wd, batch = 0.1, 0.9, 0.07, 2

    def __init__(self, golden, case):
        g = golden["sdpa_pt"]
        self.causal = case["causal"]
        self.conv_w = [np.asarray(g[k], np.float64).reshape(2, 4) for k in ("conv_q", "conv_k", "conv_v")]
        self.conv_b = [np.zeros(2) for _ in range(3)]
        self.lin_w, self.lin_b = np.asarray(g["w_linear"], np.float64).reshape(3, 10), np.zeros(3)
        self.X = orc.numpy_array_for_tests(6, 4, 5).astype(np.float64)
        self.Y = orc.y_numpy_array_for_tests(6, 3).astype(np.float64)

    def params(self):
        return self.conv_w + self.conv_b + [self.lin_w, self.lin_b]

    def conv_forward(self, Xb):
        return [np.stack([w @ x + b[:, None] for x in Xb]) for w, b in zip(self.conv_w, self.conv_b)]   # [n, 2, 5] each

    def conv_gradients(self, Xb, dQKV):
        return ([sum(d[i] @ Xb[i].T for i in range(len(Xb))) for d in dQKV], [d.sum((0, 2)) for d in dQKV])

    def batches(self):
        return [slice(s, s + self.batch) for s in range(0, 6, self.batch)]

    def loss(self, p):
        return float(-(self.Y * np.log(p)).sum(1).mean())

    def step(self, grads, vel, n):
        params = self.params()
        for p, g in zip(params, grads):
            g += n * self.wd * p
        _sgd_momentum(params, grads, vel, self.lr / n, self.momentum)


def _sdpa_pt_train_with_oracle(net, epochs=10):
    vel = [np.zeros_like(p) for p in net.params()]

    def forward(Xb):
        Q, K, V = net.conv_forward(Xb)
        w, y = orc.sdpa_forward(Q, K, V, False, net.causal, f64=True)
        flat = y.reshape(len(Xb), -1)
        return (Q, K, V), w, flat, _softmax64(flat @ net.lin_w.T + net.lin_b)
    for _ in range(epochs):
        for sl in net.batches():
            Xb, Yb = net.X[sl], net.Y[sl]
            (Q, K, V), w, flat, p = forward(Xb)
            dz = p - Yb
            dflat = dz @ net.lin_w
            dQ, dK, dV = orc.sdpa_backward(Q, K, V, dflat.reshape(len(Xb), 2, 5), w, False)
            d_conv_w, d_conv_b = net.conv_gradients(Xb, (dQ, dK, dV))
            net.step(d_conv_w + d_conv_b + [dz.T @ flat, dz.sum(0)], vel, len(Xb))
    return forward(net.X)[3]


def test_oracle_attention_training_matches_reference_goldens_pytorch_layout(golden):
    for case in golden["sdpa_pt"]["cases"]:
        net = _SdpaPtNet(golden, case)
        assert abs(net.loss(_sdpa_pt_train_with_oracle(net, 0)) - case["loss_before"]) <= 1e-6
        assert abs(net.loss(_sdpa_pt_train_with_oracle(net)) - case["loss_after"]) <= 1e-6


@pytest.mark.gpu
def test_gpu_attention_training_matches_reference_goldens_pytorch_layout(wrapper, golden):
    # the same replay with the attention core (snb200_sdpa_fwd / _bwd), the output Dense layer, the loss gradient, the
    # weight decay and the momentum updates on the device
    from sharpnet_b200._capi import ACT_SOFTMAX, LOSS_CATEGORICAL_CROSSENTROPY
    from sharpnet_b200.attention import (ScaledDotProductAttentionBackwardPropagation,
                                         ScaledDotProductAttentionForwardPropagation)
    from sharpnet_b200.linear import FusedDenseBackwardFromLoss, FusedDenseForward
    from sharpnet_b200.tensor import GPUTensor
    T = lambda a: GPUTensor(np.shape(a), np.asarray(a, np.float32), wrapper)  # noqa: E731
    for case in golden["sdpa_pt"]["cases"]:
        net = _SdpaPtNet(golden, case)
        lin_w, lin_b = T(net.lin_w), T(net.lin_b)
        d_lin_w, d_lin_b = GPUTensor((3, 10), None, wrapper), GPUTensor((3,), None, wrapper)
        v_w, v_b = GPUTensor((3, 10), None, wrapper), GPUTensor((3,), None, wrapper)
        conv_params = net.conv_w + net.conv_b
        conv_vel = [np.zeros_like(p) for p in conv_params]

        def forward(Xb):
            n = len(Xb)
            Q, K, V = (T(a) for a in net.conv_forward(Xb))
            y = GPUTensor((n, 2, 5), None, wrapper)
            W = ScaledDotProductAttentionForwardPropagation(Q, K, V, y, True, None, False, net.causal)
            p = GPUTensor((n, 3), None, wrapper)
            FusedDenseForward(p, y.Reshape(n, 10), lin_w, lin_b, ACT_SOFTMAX, None, W_OUT_IN)
            return (Q, K, V), W, y, p
        assert abs(net.loss(forward(net.X)[3].ContentAsFloatArray().astype(np.float64)) - case["loss_before"]) <= 1e-6
        for _ in range(10):
            for sl in net.batches():
                Xb, n = net.X[sl], net.batch
                (Q, K, V), W, y, p = forward(Xb)
                dflat, dz = GPUTensor((n, 10), None, wrapper), GPUTensor((n, 3), None, wrapper)
                FusedDenseBackwardFromLoss(dflat, d_lin_w, d_lin_b, y.Reshape(n, 10), T(net.Y[sl]), p, lin_w,
                                           LOSS_CATEGORICAL_CROSSENTROPY, 1.0, dz, W_OUT_IN)
                dQ, dK, dV = (GPUTensor((n, 2, 5), None, wrapper) for _ in range(3))
                ScaledDotProductAttentionBackwardPropagation(dQ, dK, dV, Q, K, V, dflat.Reshape(n, 2, 5), W, False)
                d_conv_w, d_conv_b = net.conv_gradients(Xb, [t.ContentAsFloatArray().astype(np.float64) for t in (dQ, dK, dV)])
                grads = d_conv_w + d_conv_b
                for prm, g in zip(conv_params, grads):
                    g += n * net.wd * prm
                _sgd_momentum(conv_params, grads, conv_vel, net.lr / n, net.momentum)
                d_lin_w.Update_Adding_Alpha_X(n * net.wd, lin_w)
                d_lin_b.Update_Adding_Alpha_X(n * net.wd, lin_b)
                lin_w.UpdateSGDOptimizer(net.lr / n, net.momentum, False, d_lin_w, v_w)
                lin_b.UpdateSGDOptimizer(net.lr / n, net.momentum, False, d_lin_b, v_b)
        wrapper.check_device_status()
        assert abs(net.loss(forward(net.X)[3].ContentAsFloatArray().astype(np.float64)) - case["loss_after"]) <= 1e-6


def _sgd_momentum(params, grads, velocities, lr, momentum):
    for p, g, v in zip(params, grads, velocities):
        v[...] = momentum * v - lr * g            # Prod/Optimizers/Sgd.cs:43-52, Prod/CPU/CpuTensor.cs:470-489
        p += v


def _train_with_oracle(net):
    params = net.conv_w + net.conv_b + net.mha_w + (net.mha_b or []) + [net.lin_w, net.lin_b]
    vel = [np.zeros_like(p) for p in params]

    def forward(Xb):
        Q, K, V = net.conv_forward(Xb)
        y, cache = orc.multihead_attention_forward(Q, K, V, net.mha_w, net.mha_b, net.H, net.kd, net.kd, net.causal,
                                                   net.layout, f64=True)
        flat = y.reshape(len(Xb), -1)
        return (Q, K, V), cache, flat, _softmax64(net.linear(flat))
    for _ in range(10):
        for sl in net.batches():
            Xb, Yb = net.X[sl], net.Y[sl]
            (Q, K, V), cache, flat, p = forward(Xb)
            dz = p - Yb                                                       # softmax + CategoricalCrossentropy
            d_lin_w = flat.T @ dz if net.tf else dz.T @ flat
            dflat = dz @ (net.lin_w.T if net.tf else net.lin_w)
            dQ, dK, dV, dws, dbs = orc.multihead_attention_backward(Q, K, V, dflat.reshape(len(Xb), 2, net.E), net.mha_w,
                                                                    cache, net.H, net.kd, net.kd, 1.0, net.layout)
            d_conv_w, d_conv_b = net.conv_gradients(Xb, (dQ, dK, dV))
            grads = d_conv_w + d_conv_b + dws + (dbs if net.use_bias else []) + [d_lin_w, dz.sum(0)]
            _sgd_momentum(params, grads, vel, net.lr / len(Xb), net.momentum)   # PonderedLearning, Optimizer.cs:26-29
    return forward(net.X)[3]


def _all_training_cases(golden):
    for case in golden["mha_tf"]["cases"]:
        yield "mha_tf", case, case["use_bias"]
    for name in ("no_bias", "with_bias"):
        for case in golden["mha_pt_" + name]["cases"]:
            yield "mha_pt_" + name, case, name == "with_bias"


def _check_after_training(net, case, p):
    if net.tf:
        np.testing.assert_allclose(p.ravel(), case["pred_after"], rtol=0, atol=1e-6)
    else:
        assert abs(float(-(net.Y * np.log(p)).sum(1).mean()) - case["loss_after"]) <= 1e-6


def test_oracle_multihead_attention_training_matches_reference_goldens(golden):
    for key, case, use_bias in _all_training_cases(golden):
        net = _MhaNet(golden, key, case, use_bias)
        _check_after_training(net, case, _train_with_oracle(net))


@pytest.mark.gpu
def test_gpu_multihead_attention_training_matches_reference_goldens(wrapper, golden):
    # the same replays with the attention layer, the output Dense layer, the loss gradient and the momentum updates on
    # the device through the C ABI (snb200_mha_fwd / _bwd, snb200_dense_fwd, snb200_softmax_fwd,
    # snb200_dense_bwd_from_loss, snb200_sgd_update)
    from sharpnet_b200._capi import ACT_SOFTMAX, LOSS_CATEGORICAL_CROSSENTROPY
    from sharpnet_b200.attention import MultiheadAttention
    from sharpnet_b200.linear import FusedDenseBackwardFromLoss, FusedDenseForward
    from sharpnet_b200.tensor import GPUTensor
    T = lambda a: GPUTensor(np.shape(a), np.asarray(a, np.float32), wrapper)  # noqa: E731
    for key, case, use_bias in _all_training_cases(golden):
        net = _MhaNet(golden, key, case, use_bias)
        layer = MultiheadAttention(net.H, net.kd, net.kd, use_bias, use_bias, net.causal, net.E, wrapper, net.layout)
        flat_w = np.concatenate([w.ravel() for w in net.mha_w]).astype(np.float32)
        layer.Weights.storage[: flat_w.size].copy_(T(flat_w).storage)
        lin_w, lin_b = T(net.lin_w), T(net.lin_b)
        vel = {id(t): GPUTensor(t.Shape, None, wrapper) for t in (layer.Weights, layer.Bias, lin_w, lin_b) if t is not None}
        d_lin_w, d_lin_b = GPUTensor(lin_w.Shape, None, wrapper), GPUTensor((3,), None, wrapper)
        conv_params = net.conv_w + net.conv_b
        conv_vel = [np.zeros_like(p) for p in conv_params]

        def forward(Xb, keep):
            n = len(Xb)
            Q, K, V = (T(a) for a in net.conv_forward(Xb))
            y = GPUTensor((n, 2, net.E), None, wrapper)
            layer.ForwardPropagation([Q, K, V], y, keep)
            flat = y.Reshape(n, 2 * net.E)
            p = GPUTensor((n, 3), None, wrapper)
            FusedDenseForward(p, flat, lin_w, lin_b, ACT_SOFTMAX, None, net.layout)      # Linear + Softmax output layer
            return (Q, K, V), flat, p
        for _ in range(10):
            for sl in net.batches():
                Xb, n = net.X[sl], net.batch
                (Q, K, V), flat, p = forward(Xb, True)
                dflat, dz = GPUTensor((n, 2 * net.E), None, wrapper), GPUTensor((n, 3), None, wrapper)
                FusedDenseBackwardFromLoss(dflat, d_lin_w, d_lin_b, flat, T(net.Y[sl]), p, lin_w, LOSS_CATEGORICAL_CROSSENTROPY,
                                           1.0, dz, net.layout)
                dX = [GPUTensor((n, 2, net.E), None, wrapper) for _ in range(3)]
                layer.BackwardPropagation([Q, K, V], dflat.Reshape(n, 2, net.E), dX, 1.0)
                d_conv_w, d_conv_b = net.conv_gradients(Xb, [t.ContentAsFloatArray().astype(np.float64) for t in dX])
                _sgd_momentum(conv_params, d_conv_w + d_conv_b, conv_vel, net.lr / n, net.momentum)
                for W, dW in ((layer.Weights, layer.WeightGradients), (layer.Bias, layer.BiasGradients), (lin_w, d_lin_w),
                              (lin_b, d_lin_b)):
                    if W is not None:
                        W.UpdateSGDOptimizer(net.lr / n, net.momentum, False, dW, vel[id(W)])
        wrapper.check_device_status()
        p = forward(net.X, False)[2].ContentAsFloatArray().astype(np.float64)
        _check_after_training(net, case, p)
