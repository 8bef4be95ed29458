"""Pins the CPU oracle on the known-answer vectors SharpNet's own tests hold for the path
(extracted by tests/golden/make_golden.py)."""
import numpy as np

from oracle import sharpnet_oracle as orc


def _dot(a, a_shape, b, b_shape, tA=False, tB=False, alpha=1.0, beta=0.0, c=None):
    aH, aW = a_shape[0], int(np.prod(a_shape[1:]))
    bH, bW = b_shape[0], int(np.prod(b_shape[1:]))
    M, N, _, _, _, _ = orc.gemm_dims(aH, aW, tA, bH, bW, tB)
    out = np.zeros(M * N, dtype=np.float32) if c is None else c.astype(np.float32).ravel().copy()
    return orc.dot_mkl(np.asarray(a, np.float32), aH, aW, tA, np.asarray(b, np.float32), bH, bW, tB, out, alpha, beta)


def test_exact_dot_cases(golden):
    # Tests/GPU/TestGpuTensor.cs:50-120, tolerance 1e-9
    assert len(golden["dot_exact"]) == 5
    for case in golden["dot_exact"]:
        got = _dot(case["a"], case["a_shape"], case["b"], case["b_shape"])
        np.testing.assert_allclose(got.ravel(), case["expected"], rtol=0, atol=1e-9)
        f64 = orc.dot_f64(case["a"], case["a_shape"][0], int(np.prod(case["a_shape"][1:])), False, case["b"],
                          case["b_shape"][0], int(np.prod(case["b_shape"][1:])), False, None, 1.0, 0.0)
        np.testing.assert_allclose(f64.ravel(), case["expected"], rtol=0, atol=1e-12)
    for case in golden["dot_exact_zero_cases"]:
        a = np.zeros(case["a_shape"], np.float32)
        b = np.zeros(case["b_shape"], np.float32)
        got = _dot(a.ravel(), case["a_shape"], b.ravel(), case["b_shape"])
        assert got.size == int(np.prod(case["expected_shape"])) and not got.any()


def test_keras_layout_sigmoid_predictions(golden):
    # Tests/NonReg/TestNetworkPropagation.cs:80-132: Linear(3, bias=0) + Sigmoid, weights [in, out], tol 1e-6
    W = np.asarray(golden["W_N_1_4_4"], np.float32).reshape(16, 3)
    for key, rows in (("1_1_4_4", 1), ("2_1_4_4", 2)):
        x = np.asarray(golden["X_" + key], np.float32).reshape(rows, 16)
        _, y = orc.dense_forward(x, W, np.zeros(3, np.float32), orc.ACT_SIGMOID, orc.W_IN_OUT)
        np.testing.assert_allclose(y.ravel(), golden[f"sigmoid_{key}_pred"], rtol=0, atol=1e-6)
    y_true = np.asarray([[1, 0, 0]], np.float32)
    x = np.asarray(golden["X_1_1_4_4"], np.float32).reshape(1, 16)
    _, y = orc.dense_forward(x, W, None, orc.ACT_SIGMOID, orc.W_IN_OUT)
    assert abs(orc.binary_crossentropy(y_true, y) - golden["sigmoid_1_1_4_4_loss"]) < 1e-5
    # 1x1x1x1 input, Linear(2): both layouts coincide
    w = np.asarray(golden["sigmoid_1_1_1_1_w"], np.float32).reshape(1, 2)
    _, y = orc.dense_forward(np.ones((1, 1), np.float32), w, None, orc.ACT_SIGMOID, orc.W_IN_OUT)
    np.testing.assert_allclose(y.ravel(), golden["sigmoid_1_1_1_1_pred"], rtol=0, atol=1e-6)


def test_pytorch_layout_relu_network_loss(golden):
    # Tests/NonReg/ParallelRunWithPyTorch.cs:179-214: Linear(16->3)+ReLU+Linear(3->3)+Sigmoid, BCE, [out, in]
    x = orc.numpy_array_for_tests(2, 1, 4, 4).reshape(2, 16)
    y_true = orc.y_numpy_array_for_tests(2, 3)
    w1 = np.asarray(golden["pt_relu_w1"], np.float32).reshape(3, 16)
    w2 = np.asarray(golden["pt_relu_w2"], np.float32).reshape(3, 3)
    _, h = orc.dense_forward(x, w1, np.zeros(3, np.float32), orc.ACT_RELU, orc.W_OUT_IN)
    _, p = orc.dense_forward(h, w2, np.zeros(3, np.float32), orc.ACT_SIGMOID, orc.W_OUT_IN)
    assert abs(orc.binary_crossentropy(y_true, p) - golden["pt_relu_loss_before"]) < 1e-6


def test_pytorch_layout_last_dim_flatten_mse(golden):
    # Tests/NonReg/ParallelRunWithPyTorch.cs:102-138: Linear(5->3 on the last dim)+ReLU+Flatten+Linear(36->3), Mse
    x = orc.numpy_array_for_tests(2, 3, 4, 5)
    y_true = orc.y_numpy_array_for_tests(2, 3)
    w1 = np.asarray(golden["pt_mse_w1"], np.float32).reshape(3, 5)
    w2 = np.asarray(golden["pt_mse_w2"], np.float32).reshape(3, 36)
    _, h = orc.dense_forward(x.reshape(-1, 5), w1, np.zeros(3, np.float32), orc.ACT_RELU, orc.W_OUT_IN)
    _, p = orc.dense_forward(h.reshape(2, 36), w2, np.zeros(3, np.float32), orc.ACT_IDENTITY, orc.W_OUT_IN)
    assert abs(orc.mse(y_true, p) - golden["pt_mse_loss_before"]) < 1e-6


def test_mkl_agrees_with_float64_on_all_transposes():
    rng = np.random.default_rng(3)
    M, N, K = 37, 29, 53
    for tA in (False, True):
        for tB in (False, True):
            a = rng.uniform(-1.5, 1.5, (K, M) if tA else (M, K)).astype(np.float32)
            b = rng.uniform(-1.5, 1.5, (N, K) if tB else (K, N)).astype(np.float32)
            c = rng.uniform(-1.5, 1.5, (M, N)).astype(np.float32)
            got = _dot(a.ravel(), a.shape, b.ravel(), b.shape, tA, tB, 0.25, 1.0, c)
            ref = orc.dot_f64(a.ravel(), a.shape[0], a.shape[1], tA, b.ravel(), b.shape[0], b.shape[1], tB,
                              c.ravel(), 0.25, 1.0)
            assert orc.scaled_error(got, ref, K, 1.5, 1.5) < 1e-6


def test_gradient_check_dense_backward():
    # Tests/TestGradient.cs:20-36: central differences vs analytic dW/db, relative error <= 1e-3
    rng = np.random.default_rng(5)
    M, K, N = 6, 7, 4
    x = rng.normal(size=(M, K)).astype(np.float32)
    W = rng.normal(size=(N, K)).astype(np.float32) * 0.5
    b = rng.normal(size=N).astype(np.float32) * 0.1
    dy = rng.normal(size=(M, N)).astype(np.float32)
    for act in (orc.ACT_TANH, orc.ACT_SIGMOID, orc.ACT_SWISH):
        z, y = orc.dense_forward(x, W, b, act, orc.W_OUT_IN)
        _, dW, db, dx = orc.dense_backward(x, W, dy, act, y, z, 1.0, orc.W_OUT_IN)

        def loss(Wp, bp):
            _, yy = orc.dense_forward(x, Wp, bp, act, orc.W_OUT_IN, f64=True)
            return float((yy * dy).sum())
        eps = 1e-3
        for (i, j) in ((0, 0), (1, 3), (3, 6)):
            Wp, Wm = W.astype(np.float64).copy(), W.astype(np.float64).copy()
            Wp[i, j] += eps
            Wm[i, j] -= eps
            num = (loss(Wp, b) - loss(Wm, b)) / (2 * eps)
            assert abs(num - dW[i, j]) <= 1e-3 * max(1.0, abs(num))
        bp, bm = b.astype(np.float64).copy(), b.astype(np.float64).copy()
        bp[2] += eps
        bm[2] -= eps
        num = (loss(W, bp) - loss(W, bm)) / (2 * eps)
        assert abs(num - db[2]) <= 1e-3 * max(1.0, abs(num))


def test_bias_gradient_and_bias_add():
    rng = np.random.default_rng(7)
    dy = rng.uniform(-1.5, 1.5, (9, 1632)).astype(np.float32)   # shape of TestCompute_BiasGradient_from_dy
    db = orc.compute_bias_gradient_from_dy(dy)
    np.testing.assert_allclose(db, dy.astype(np.float64).sum(0), rtol=0, atol=1e-5)
    y = rng.uniform(-1.5, 1.5, (9, 1632)).astype(np.float32)
    bias = rng.uniform(-1.5, 1.5, 1632).astype(np.float32)
    ref = y + bias[None, :]
    orc.broadcast_add_vector_to_output(bias, y)
    np.testing.assert_array_equal(y, ref)


def _train_10_epochs(x, y_true, W, lr=0.1):
    # TensorFlow compatibility mode (dW multiplier 1), VanillaSGD with lr / batchSize, sigmoid output layer whose
    # gradient is folded into the loss gradient (1/numClass)(p - y): Tests/NonReg/TestNetworkPropagation.cs:80-132
    W, b = W.copy(), np.zeros(W.shape[1], np.float32)
    for _ in range(10):
        _, p = orc.dense_forward(x, W, b, orc.ACT_SIGMOID, orc.W_IN_OUT)
        dy = ((p - y_true) / y_true.shape[1]).astype(np.float32)
        _, dW, db, _ = orc.dense_backward(x, W, dy, orc.ACT_IDENTITY, None, None, 1.0, orc.W_IN_OUT, need_dx=False)
        orc.update_sgd_optimizer(W, lr / x.shape[0], 0.0, False, dW, None)
        orc.update_sgd_optimizer(b, lr / x.shape[0], 0.0, False, db, None)
    return orc.dense_forward(x, W, b, orc.ACT_SIGMOID, orc.W_IN_OUT)[1]


def test_predictions_after_ten_epochs_of_sgd(golden):
    # pins the backward pass (dW, db) and the VanillaSGD update on the reference's after-training goldens
    W = np.asarray(golden["W_N_1_4_4"], np.float32).reshape(16, 3)
    for key, rows, y_true in (("1_1_4_4", 1, [[1, 0, 0]]), ("2_1_4_4", 2, [[1, 0, 0], [0, 0, 1]])):
        x = np.asarray(golden["X_" + key], np.float32).reshape(rows, 16)
        y_true = np.asarray(y_true, np.float32)
        p = _train_10_epochs(x, y_true, W)
        np.testing.assert_allclose(p.ravel(), golden[f"sigmoid_{key}_pred_after"], rtol=0, atol=1e-6)
        assert abs(orc.binary_crossentropy(y_true, p) - golden[f"sigmoid_{key}_loss_after"]) < 1e-5


def test_optimizer_updates_against_closed_forms():
    rng = np.random.default_rng(11)
    W, dW, v = (rng.uniform(-1.5, 1.5, (32, 17)).astype(np.float32) for _ in range(3))
    W0, v0 = W.copy(), v.copy()
    orc.update_sgd_optimizer(W, 0.1, 0.9, True, dW, v)
    v_want = 0.9 * v0.astype(np.float64) - 0.1 * dW
    np.testing.assert_allclose(v, v_want, rtol=0, atol=1e-6)
    np.testing.assert_allclose(W, W0 + 0.9 * v_want - 0.1 * dW, rtol=0, atol=1e-6)
    W = W0.copy()
    m, s = np.zeros_like(W), np.zeros_like(W)
    orc.update_adam_optimizer(W, 0.001, 0.9, 0.999, 1e-8, 0.0, dW, m, s, 1)
    # first Adam step moves every weight by lr * sign(dW) (bias-corrected moments cancel)
    np.testing.assert_allclose(W0 - W, 0.001 * np.sign(dW), rtol=0, atol=1e-6)


# ---- the other Dense networks of Tests/NonReg/TestNetworkPropagation.cs, before and after 10 epochs -------------
def _mlp_forward(x, Ws, bs, acts, alphas, first_on_last_dim):
    """Forward of a stack of Linear layers with [in, out] weights; returns the per-layer (input, z, y).  The first
    layer may act on the last dimension (flattenInputTensorOnLastDimension), later layers flatten per row."""
    cache, h = [], x
    for i, (W, b, act, alpha) in enumerate(zip(Ws, bs, acts, alphas)):
        h2 = h.reshape(-1, W.shape[0]) if (i == 0 and first_on_last_dim) else h.reshape(x.shape[0], -1)
        out_act = orc.ACT_IDENTITY if act in (orc.ACT_SIGMOID, orc.ACT_SOFTMAX) and i == len(Ws) - 1 else act
        z, y = orc.dense_forward(h2, W, b, act, orc.W_IN_OUT, alpha=alpha)
        cache.append((h2, z, y, out_act))
        h = y
    return cache


def _train_mlp(g, acts, loss, lr, momentum=0.0, weight_decay=0.0, alphas=None, x=None, first_on_last_dim=False,
               epochs=10):
    """TensorFlow compatibility mode as the reference's tests set it: dW multiplier 1 (Prod/Layers/Linear.cs:150-155),
    learning rate / batch size (Prod/Optimizers/Optimizer.cs:26-29), the output layer's Sigmoid / Softmax folded into
    the loss gradient (Prod/Layers/ActivationLayer.cs:59-62), weight decay as dW += 2 * batch * wd * W (Linear.cs:167-176),
    biases from zero.  Returns predictions before and after training."""
    n = len(acts)
    Ws = [np.asarray(w, np.float32) for w in g["weights"][:n]]
    y_true = np.asarray([[1, 0, 0], [0, 0, 1]], np.float32)
    alphas = alphas or [0.0] * n
    widths = []
    fan_in = (x.shape[-1] if first_on_last_dim else x[0].size)
    for i, w in enumerate(Ws):
        out = 3
        Ws[i] = w.reshape(fan_in, out)
        widths.append(out)
        fan_in = (x[0].size // x.shape[-1]) * out if (i == 0 and first_on_last_dim) else out
    bs = [np.zeros(w.shape[1], np.float32) for w in Ws]
    vW = [np.zeros_like(w) for w in Ws] if momentum else [None] * n
    vb = [np.zeros_like(b) for b in bs] if momentum else [None] * n
    batch = x.shape[0]
    predict = lambda: _mlp_forward(x, Ws, bs, acts, alphas, first_on_last_dim)[-1][2].reshape(batch, -1)  # noqa: E731
    before = predict()
    for _ in range(epochs):
        cache = _mlp_forward(x, Ws, bs, acts, alphas, first_on_last_dim)
        grad = orc.loss_gradient(loss, y_true, cache[-1][2].reshape(batch, -1))
        for i in reversed(range(n)):
            h2, z, y, act = cache[i]
            dz, dW, db, dx = orc.dense_backward(h2, Ws[i], grad.reshape(z.shape), act, y, z, 1.0, orc.W_IN_OUT,
                                                need_dx=i > 0, alpha=alphas[i])
            if weight_decay:
                orc.update_adding_alpha_x(dW, 2 * batch * np.float32(weight_decay), Ws[i])
            grad = dx
            orc.update_sgd_optimizer(Ws[i], lr / batch, momentum, False, dW, vW[i])
            orc.update_sgd_optimizer(bs[i], lr / batch, momentum, False, db, vb[i])
    return before, predict()


def _x_2_1_4_4(golden):
    return np.asarray(golden["X_2_1_4_4"], np.float32).reshape(2, 16)


def test_softmax_relu_and_leaky_relu_networks_before_and_after_training(golden):
    x = _x_2_1_4_4(golden)
    y_true = np.asarray(golden["Y_2_3"], np.float32).reshape(2, 3)
    cases = (
        # :135-160 Linear + Softmax, CategoricalCrossentropy, VanillaSGD 0.1
        ("softmax_2_1_4_4", (orc.ACT_SOFTMAX,), orc.LOSS_CATEGORICAL_CROSSENTROPY, dict(lr=0.1), 1e-6),
        # :216-244 Linear + ReLU + Linear + Sigmoid, BinaryCrossentropy, VanillaSGD 0.1
        ("relu_2_1_4_4", (orc.ACT_RELU, orc.ACT_SIGMOID), orc.LOSS_BINARY_CROSSENTROPY, dict(lr=0.1), 1e-6),
        # :330-358 Linear + LeakyRelu(0.1) + Linear + Sigmoid, BinaryCrossentropy, SGD 0.1 with momentum 0.9
        ("leaky_relu_2_1_4_4", (orc.ACT_LEAKY_RELU, orc.ACT_SIGMOID), orc.LOSS_BINARY_CROSSENTROPY,
         dict(lr=0.1, momentum=0.9, alphas=[0.1, 0.0]), 1e-6),
        # :725-747 Linear + Softmax with weight decay 0.05, VanillaSGD 0.12
        ("weight_decay_vanilla_2_1_4_4", (orc.ACT_SOFTMAX,), orc.LOSS_CATEGORICAL_CROSSENTROPY,
         dict(lr=0.12, weight_decay=0.05), 1e-6),
        # :749-770 the same with SGD 0.12, momentum 0.9, weight decay 0.5
        ("weight_decay_momentum_2_1_4_4", (orc.ACT_SOFTMAX,), orc.LOSS_CATEGORICAL_CROSSENTROPY,
         dict(lr=0.12, momentum=0.9, weight_decay=0.5), 1e-6),
    )
    for key, acts, loss, kw, tol in cases:
        g = golden[key]
        before, after = _train_mlp(g, acts, loss, x=x, **kw)
        np.testing.assert_allclose(before.ravel(), g["pred_before"], rtol=0, atol=tol, err_msg=key)
        np.testing.assert_allclose(after.ravel(), g["pred_after"], rtol=0, atol=tol, err_msg=key)
        if loss == orc.LOSS_BINARY_CROSSENTROPY:
            assert abs(orc.binary_crossentropy(y_true, before) - g["loss_before"]) < 1e-5, key
            assert abs(orc.binary_crossentropy(y_true, after) - g["loss_after"]) < 1e-5, key
        elif not kw.get("weight_decay"):
            cce = lambda p: float(-(y_true * np.log(p.astype(np.float64))).sum(1).mean())  # noqa: E731
            assert abs(cce(before) - g["loss_before"]) < 1e-5 and abs(cce(after) - g["loss_after"]) < 1e-5, key


def test_mse_network_on_the_last_dimension_before_and_after_training(golden):
    # :1161-1192 Linear(5 -> 3 on the last dimension) + ReLU + Linear(36 -> 3), Mse, SGD 0.1 with momentum 0.9; the
    # reference states these predictions to 1e-3
    x = np.asarray(golden["X_2_3_4_5"], np.float32).reshape(2, 3, 4, 5)
    g = golden["mse_2_3_4_5"]
    before, after = _train_mlp(g, (orc.ACT_RELU, orc.ACT_IDENTITY), orc.LOSS_MSE, lr=0.1, momentum=0.9, x=x,
                               first_on_last_dim=True)
    np.testing.assert_allclose(before.ravel(), g["pred_before"], rtol=0, atol=1e-3)
    np.testing.assert_allclose(after.ravel(), g["pred_after"], rtol=0, atol=1e-3)


# ---- PyTorch compatibility mode: [out, in] weights, weight decay dW += batch * wd * W and likewise for the bias
#      (Prod/Layers/Linear.cs:167-181), after 10 epochs (Tests/NonReg/ParallelRunWithPyTorch.cs) ------------------
def _train_pytorch_mlp(x, y_true, W1, W2, act1, alpha1, out_act, loss, lr, momentum, weight_decay, nesterov,
                       batch_size, first_on_last_dim=False, epochs=10):
    Ws, bs = [W1.copy(), W2.copy()], [np.zeros(W1.shape[0], np.float32), np.zeros(W2.shape[0], np.float32)]
    vW, vb = [np.zeros_like(w) for w in Ws], [np.zeros_like(b) for b in bs]

    def forward(xb):
        h0 = xb.reshape(-1, W1.shape[1]) if first_on_last_dim else xb.reshape(xb.shape[0], -1)
        z1, y1 = orc.dense_forward(h0, Ws[0], bs[0], act1, orc.W_OUT_IN, alpha=alpha1)
        h1 = y1.reshape(xb.shape[0], -1)
        z2, y2 = orc.dense_forward(h1, Ws[1], bs[1], out_act, orc.W_OUT_IN)
        return h0, z1, y1, h1, y2
    for _ in range(epochs):
        for r0 in range(0, x.shape[0], batch_size):
            xb, tb = x[r0:r0 + batch_size], y_true[r0:r0 + batch_size]
            n = xb.shape[0]
            h0, z1, y1, h1, p = forward(xb)
            dy = orc.loss_gradient(loss, tb, p)
            _, dW2, db2, dx = orc.dense_backward(h1, Ws[1], dy, orc.ACT_IDENTITY, None, None, 1.0, orc.W_OUT_IN)
            _, dW1, db1, _ = orc.dense_backward(h0, Ws[0], dx.reshape(z1.shape), act1, y1, z1, 1.0, orc.W_OUT_IN,
                                                need_dx=False, alpha=alpha1)
            for W, b, dW, db, v, u in ((Ws[0], bs[0], dW1, db1, vW[0], vb[0]), (Ws[1], bs[1], dW2, db2, vW[1], vb[1])):
                if weight_decay:
                    orc.update_adding_alpha_x(dW, n * np.float32(weight_decay), W)
                    orc.update_adding_alpha_x(db, n * np.float32(weight_decay), b)
                orc.update_sgd_optimizer(W, lr / n, momentum, nesterov, dW, v)
                orc.update_sgd_optimizer(b, lr / n, momentum, nesterov, db, u)
    return lambda xb: forward(xb)[-1]


def test_pytorch_layout_networks_after_training(golden):
    cce = lambda t, p: float(-(t * np.log(p.astype(np.float64))).sum(1).mean())  # noqa: E731
    # :179-214 Linear(16->3) + ReLU + Linear(3->3) + Sigmoid, BCE, SGD 0.1 momentum 0.9 weight decay 0.03
    x, t = orc.numpy_array_for_tests(2, 1, 4, 4), orc.y_numpy_array_for_tests(2, 3)
    w1 = np.asarray(golden["pt_relu_w1"], np.float32).reshape(3, 16)
    w2 = np.asarray(golden["pt_relu_w2"], np.float32).reshape(3, 3)
    predict = _train_pytorch_mlp(x, t, w1, w2, orc.ACT_RELU, 0.0, orc.ACT_SIGMOID, orc.LOSS_BINARY_CROSSENTROPY, 0.1, 0.9,
                                 0.03, False, 2)
    assert abs(orc.binary_crossentropy(t, predict(x)) - golden["pt_relu_loss_after"]) < 1e-6
    # :102-138 Linear(5->3 on the last dimension) + ReLU + Flatten + Linear(36->3), Mse, SGD 0.1 momentum 0.9
    x = orc.numpy_array_for_tests(2, 3, 4, 5)
    w1 = np.asarray(golden["pt_mse_w1"], np.float32).reshape(3, 5)
    w2 = np.asarray(golden["pt_mse_w2"], np.float32).reshape(3, 36)
    predict = _train_pytorch_mlp(x, t, w1, w2, orc.ACT_RELU, 0.0, orc.ACT_IDENTITY, orc.LOSS_MSE, 0.1, 0.9, 0.0, False, 2,
                                 first_on_last_dim=True)
    assert abs(orc.mse(t, predict(x)) - golden["pt_mse_loss_after"]) < 1e-6
    # :813-850 Linear(16->3) + LeakyRelu(0.1) + Linear(3->3) + Softmax on 10 rows in batches of 2,
    # CategoricalCrossentropy, SGD 0.1 momentum 0.66 weight decay 0.17 with Nesterov
    x, t = orc.numpy_array_for_tests(10, 1, 4, 4), orc.y_numpy_array_for_tests(10, 3)
    w1 = np.asarray(golden["pt_leaky_w1"], np.float32).reshape(3, 16)
    w2 = np.asarray(golden["pt_leaky_w2"], np.float32).reshape(3, 3)
    before = _train_pytorch_mlp(x, t, w1, w2, orc.ACT_LEAKY_RELU, 0.1, orc.ACT_SOFTMAX, orc.LOSS_CATEGORICAL_CROSSENTROPY,
                                0.1, 0.66, 0.17, True, 2, epochs=0)
    assert abs(cce(t, before(x)) - golden["pt_leaky_loss_before"]) < 1e-6
    predict = _train_pytorch_mlp(x, t, w1, w2, orc.ACT_LEAKY_RELU, 0.1, orc.ACT_SOFTMAX, orc.LOSS_CATEGORICAL_CROSSENTROPY,
                                 0.1, 0.66, 0.17, True, 2)
    assert abs(cce(t, predict(x)) - golden["pt_leaky_loss_after"]) < 1e-6


def test_transposition_and_causal_mask_goldens_of_the_reference():
    """Tests/CPU/TestCpuTensor.cs:104-112 (TransposeSecondAndThirdDimension of arange(2*3*4*5), expected values as
    written there) and :162-196 (SetAllElementsAboveMainDiagonal with -666 on 1x1, 1x6, 6x1, 2x3, 3x2 and 3x3)."""
    x = np.arange(2 * 3 * 4 * 5, dtype=np.float32).reshape(2, 3, 4, 5)
    expected = np.array(
        [[[[0, 1, 2, 3, 4], [20, 21, 22, 23, 24], [40, 41, 42, 43, 44]], [[5, 6, 7, 8, 9], [25, 26, 27, 28, 29], [45, 46, 47, 48, 49]],
          [[10, 11, 12, 13, 14], [30, 31, 32, 33, 34], [50, 51, 52, 53, 54]], [[15, 16, 17, 18, 19], [35, 36, 37, 38, 39], [55, 56, 57, 58, 59]]],
         [[[60, 61, 62, 63, 64], [80, 81, 82, 83, 84], [100, 101, 102, 103, 104]], [[65, 66, 67, 68, 69], [85, 86, 87, 88, 89], [105, 106, 107, 108, 109]],
          [[70, 71, 72, 73, 74], [90, 91, 92, 93, 94], [110, 111, 112, 113, 114]], [[75, 76, 77, 78, 79], [95, 96, 97, 98, 99], [115, 116, 117, 118, 119]]]],
        dtype=np.float32)
    np.testing.assert_array_equal(orc.transpose_second_third(x), expected)
    v = -666.0
    data = [0.5, 1, 2, 3, 4, 5]
    cases = [((1, 1), [1.0], [1.0]),
             ((1, 6), data, [0.5, v, v, v, v, v]),
             ((6, 1), data, data),
             ((2, 3), data, [0.5, v, v, 3, 4, v]),
             ((3, 2), data, [0.5, v, 2, 3, 4, 5]),
             ((3, 3), [0.5, 1, 2, 3, 4, 5, 6, 7, 8], [0.5, v, v, 3, 4, v, 6, 7, 8])]
    for shape, src, want in cases:
        got = orc.set_all_elements_above_main_diagonal(np.asarray(src, np.float32).reshape(shape), v)
        np.testing.assert_array_equal(got.ravel(), np.asarray(want, np.float32))
    # a batch of matrices is masked matrix by matrix (Prod/CPU/CpuTensor.cs:3040-3043)
    batch = np.arange(2 * 3 * 3, dtype=np.float32).reshape(2, 3, 3)
    got = orc.set_all_elements_above_main_diagonal(batch.copy(), v)
    for b in range(2):
        np.testing.assert_array_equal(got[b], orc.set_all_elements_above_main_diagonal(batch[b].copy(), v))
