"""Parity of the Dense-layer entry points (snb200_dense_fwd / snb200_dense_bwd and the companions
behind BroadcastAddVectorToOutput, Compute_BiasGradient_from_dy, ActivationForward/Backward,
Update_Adding_Alpha_X) against the CPU oracle, on a B200."""
import numpy as np
import pytest

from oracle import sharpnet_oracle as orc
from sharpnet_b200 import (ACT_ELU, ACT_IDENTITY, ACT_LEAKY_RELU, ACT_RELU, ACT_SIGMOID, ACT_SWISH, ACT_TANH, MATH_3XTF32,
                           MATH_TF32, W_IN_OUT, W_OUT_IN)
from sharpnet_b200._capi import ACT_CLIPPED_RELU, ACT_LN, TUNE_CLUSTER, TUNE_FORCE_PATH
from sharpnet_b200._capi import LOSS_BINARY_CROSSENTROPY, LOSS_CATEGORICAL_CROSSENTROPY, LOSS_MSE
from sharpnet_b200.linear import (DenseBackwardPropagation, DenseForwardPropagation, FusedDenseBackward,
                                  FusedDenseBackwardFromLoss, FusedDenseForward)
from sharpnet_b200.tensor import GPUTensor

from gpu_util import TOL_3XTF32, TOL_TF32

pytestmark = pytest.mark.gpu
ACTS = [ACT_IDENTITY, ACT_RELU, ACT_SWISH, ACT_TANH, ACT_SIGMOID, ACT_ELU, ACT_LEAKY_RELU, ACT_CLIPPED_RELU]
ALPHA = {ACT_ELU: 0.7, ACT_LEAKY_RELU: 0.3}      # the coefficient the parametric activations are tested with


@pytest.fixture(autouse=True)
def _reset(wrapper):
    wrapper.set_math_mode(MATH_3XTF32)
    wrapper.set_tuning(TUNE_FORCE_PATH, 0)
    yield
    wrapper.set_math_mode(MATH_3XTF32)
    wrapper.set_tuning(TUNE_FORCE_PATH, 0)


def _t(w, arr):
    return GPUTensor(arr.shape, arr, w)


def test_golden_keras_layout_predictions(wrapper, golden):
    # Tests/NonReg/TestNetworkPropagation.cs:80-132: Linear(3) + Sigmoid, weights [in, out], 1e-6
    W = np.asarray(golden["W_N_1_4_4"], np.float32).reshape(16, 3)
    for key, rows in (("1_1_4_4", 1), ("2_1_4_4", 2)):
        x = np.asarray(golden["X_" + key], np.float32).reshape(rows, 1, 4, 4)
        y = GPUTensor((rows, 3), None, wrapper)
        FusedDenseForward(y, _t(wrapper, x), _t(wrapper, W), _t(wrapper, np.zeros(3, np.float32)), ACT_SIGMOID,
                          w_layout=W_IN_OUT)
        np.testing.assert_allclose(y.ContentAsFloatArray().ravel(), golden[f"sigmoid_{key}_pred"], rtol=0, atol=1e-6)


def test_golden_pytorch_layout_networks(wrapper, golden):
    # Tests/NonReg/ParallelRunWithPyTorch.cs:179-214 (BCE 0.67267912...) through the unfused call
    # sequence of Linear.cs + ActivationLayer.cs, and :102-138 (Mse 0.29795372...) through the fused one.
    x = _t(wrapper, orc.numpy_array_for_tests(2, 1, 4, 4))
    w1 = _t(wrapper, np.asarray(golden["pt_relu_w1"], np.float32).reshape(3, 16))
    w2 = _t(wrapper, np.asarray(golden["pt_relu_w2"], np.float32).reshape(3, 3))
    zeros = _t(wrapper, np.zeros(3, np.float32))
    h, ha = GPUTensor((2, 3), None, wrapper), GPUTensor((2, 3), None, wrapper)
    p, pa = GPUTensor((2, 3), None, wrapper), GPUTensor((2, 3), None, wrapper)
    DenseForwardPropagation(h, x, w1, zeros)
    h.ActivationForward(ACT_RELU, None, ha)
    DenseForwardPropagation(p, ha, w2, zeros)
    p.ActivationForward(ACT_SIGMOID, None, pa)
    loss = orc.binary_crossentropy(orc.y_numpy_array_for_tests(2, 3), pa.ContentAsFloatArray())
    assert abs(loss - golden["pt_relu_loss_before"]) < 1e-6

    x = _t(wrapper, orc.numpy_array_for_tests(2, 3, 4, 5))
    w1 = _t(wrapper, np.asarray(golden["pt_mse_w1"], np.float32).reshape(3, 5))
    w2 = _t(wrapper, np.asarray(golden["pt_mse_w2"], np.float32).reshape(3, 36))
    h = GPUTensor((2, 3, 4, 3), None, wrapper)
    FusedDenseForward(h, x, w1, zeros, ACT_RELU, flattenInputTensorOnLastDimension=True)
    p = GPUTensor((2, 3), None, wrapper)
    FusedDenseForward(p, h.Reshape(2, 36), w2, zeros, ACT_IDENTITY)
    loss = orc.mse(orc.y_numpy_array_for_tests(2, 3), p.ContentAsFloatArray())
    assert abs(loss - golden["pt_mse_loss_before"]) < 1e-6


def _dense_case(wrapper, M, K, N, act, layout, seed, tol, with_bias=True, need_dx=True, mult=1.0):
    x = orc.normal((M, K), 0, 1, seed)
    Wl = orc.glorot_uniform((N, K) if layout == W_OUT_IN else (K, N), seed + 1)
    b = orc.uniform((N,), -0.5, 0.5, seed + 2) if with_bias else None
    dy = orc.normal((M, N), 0, 1, seed + 3)
    wmax = float(np.abs(Wl).max())
    X, W, DY = _t(wrapper, x), _t(wrapper, Wl), _t(wrapper, dy)
    B = _t(wrapper, b) if with_bias else None
    Y, Z = GPUTensor((M, N), None, wrapper), GPUTensor((M, N), None, wrapper)
    alpha = ALPHA.get(act, 0.0)
    FusedDenseForward(Y, X, W, B, act, z=Z, w_layout=layout, activationParameter=alpha)
    wrapper.check_device_status()
    z64, y64 = orc.dense_forward(x, Wl, b, act, layout, f64=True, alpha=alpha)
    zm, ym = orc.dense_forward(x, Wl, b, act, layout, alpha=alpha)
    y, z = Y.ContentAsFloatArray(), Z.ContentAsFloatArray()
    for got, r64, rm in ((z, z64, zm), (y, y64, ym)):
        assert orc.scaled_error(got, r64, K, 4.0, wmax) <= tol
        assert orc.scaled_error(got, rm, K, 4.0, wmax) <= tol
    # backward, from the GPU's own y / z (what the layer would have kept)
    DZ = GPUTensor((M, N), None, wrapper)
    DX = GPUTensor((M, K), None, wrapper) if need_dx else None
    DW = GPUTensor(Wl.shape, None, wrapper)
    DB = GPUTensor((N,), None, wrapper) if with_bias else None
    FusedDenseBackward(DX, DW, DB, X, DY, W, act, y=Y, z=Z, multiplier=mult, dz_scratch=DZ, w_layout=layout)
    wrapper.check_device_status()
    dz64, dW64, db64, dx64 = orc.dense_backward(x, Wl, dy, act, y, z, mult, layout, need_dx, f64=True, alpha=alpha)
    dzm, dWm, dbm, dxm = orc.dense_backward(x, Wl, dy, act, y, z, mult, layout, need_dx, alpha=alpha)
    if act != ACT_IDENTITY:
        np.testing.assert_allclose(DZ.ContentAsFloatArray(), dzm, rtol=2e-6, atol=1e-6)
    gmax = 4.0 * 1.2  # |dz| <= |dy| * max|act'| (1.1 for Swish)
    assert orc.scaled_error(DW.ContentAsFloatArray(), dW64, M, 4.0, gmax) <= tol * max(1.0, abs(mult))
    assert orc.scaled_error(DW.ContentAsFloatArray(), dWm, M, 4.0, gmax) <= tol * max(1.0, abs(mult))
    if with_bias:
        assert orc.scaled_error(DB.ContentAsFloatArray(), db64, M, 1.0, gmax) <= TOL_3XTF32
        assert orc.scaled_error(DB.ContentAsFloatArray(), dbm, M, 1.0, gmax) <= TOL_3XTF32
    if need_dx:
        assert orc.scaled_error(DX.ContentAsFloatArray(), dx64, N, gmax, wmax) <= tol
        assert orc.scaled_error(DX.ContentAsFloatArray(), dxm, N, gmax, wmax) <= tol


@pytest.mark.parametrize("act", ACTS)
@pytest.mark.parametrize("layout", [W_OUT_IN, W_IN_OUT])
def test_dense_fwd_bwd_small_simt(wrapper, act, layout):
    _dense_case(wrapper, 9, 21, 5, act, layout, 40 + act, TOL_3XTF32)
    _dense_case(wrapper, 33, 7, 3, act, layout, 60 + act, TOL_3XTF32, with_bias=False, need_dx=False, mult=1.0 / 33)


@pytest.mark.parametrize("act", ACTS)
@pytest.mark.parametrize("layout", [W_OUT_IN, W_IN_OUT])
@pytest.mark.parametrize("mode,tol", [(MATH_3XTF32, TOL_3XTF32), (MATH_TF32, TOL_TF32)])
def test_dense_fwd_bwd_tensor_core(wrapper, act, layout, mode, tol):
    wrapper.set_math_mode(mode)
    _dense_case(wrapper, 512, 384, 256, act, layout, 80 + act, tol)
    assert wrapper.last_kernel().startswith("umma")
    _dense_case(wrapper, 300, 200, 136, act, layout, 90 + act, tol, mult=1.0 / 300)


@pytest.mark.parametrize("act", [ACT_RELU, ACT_SWISH])
@pytest.mark.parametrize("layout", [W_IN_OUT, W_OUT_IN])
@pytest.mark.parametrize("clusters", [0, 1])
def test_dense_small_batch_takes_the_split_k_plans(wrapper, act, layout, clusters):
    # inference-sized batches: forward runs with swapped operands, the gradients with K cut in pieces;
    # bias, activation and the pre-activation output then come from the CTAs of a cluster that store the
    # transposed tile, or (clusters switched off) from the reduction kernel
    wrapper.set_tuning(TUNE_CLUSTER, clusters)
    try:
        _dense_case(wrapper, 32, 2048, 512, act, layout, 300 + act, TOL_3XTF32)
        _dense_case(wrapper, 8, 1024, 260, act, layout, 320 + act, TOL_3XTF32, mult=0.125)
    finally:
        wrapper.set_tuning(TUNE_CLUSTER, 0)


@pytest.mark.parametrize("act", [ACT_RELU, ACT_SWISH, ACT_TANH])
@pytest.mark.parametrize("layout", [W_IN_OUT, W_OUT_IN])
def test_dense_with_a_cut_last_wave(wrapper, act, layout):
    # 9 x 9 pair tiles on 74 SM pairs: the last 7 tiles are cut along K, so bias, activation and the
    # pre-activation copy of those tiles come from the tile reduction kernel, the rest from the GEMM epilogue
    _dense_case(wrapper, 2300, 1032, 2292, act, layout, 340 + act, TOL_3XTF32)


@pytest.mark.parametrize("act", [ACT_RELU, ACT_SWISH])
@pytest.mark.parametrize("layout", [W_IN_OUT, W_OUT_IN])
def test_config_3_dense_4096x3072x1024(wrapper, act, layout):
    # benchmark config 3: x[4096x3072] N(0,1), W Glorot, dy N(0,1); bias drawn non-zero to exercise the add
    _dense_case(wrapper, 4096, 3072, 1024, act, layout, 6, TOL_3XTF32)


def test_unfused_sequence_matches_fused(wrapper):
    # Linear.cs call sequence (Dot, bias add, activation; activation backward, Dot, bias gradient, Dot)
    # against the fused entry points on the same inputs
    M, K, N = 256, 192, 128
    x, Wl = orc.normal((M, K), 0, 1, 1), orc.glorot_uniform((N, K), 2)
    b, dy = orc.uniform((N,), -0.5, 0.5, 3), orc.normal((M, N), 0, 1, 4)
    X, W, B, DY = (_t(wrapper, v) for v in (x, Wl, b, dy))
    for act in ACTS:
        z1, y1 = GPUTensor((M, N), None, wrapper), GPUTensor((M, N), None, wrapper)
        DenseForwardPropagation(z1, X, W, B)
        z1.ActivationForward(act, None, y1)
        z2, y2 = GPUTensor((M, N), None, wrapper), GPUTensor((M, N), None, wrapper)
        FusedDenseForward(y2, X, W, B, act, z=z2)
        np.testing.assert_array_equal(z1.ContentAsFloatArray(), z2.ContentAsFloatArray())
        np.testing.assert_array_equal(y1.ContentAsFloatArray(), y2.ContentAsFloatArray())
        dz1 = GPUTensor((M, N), None, wrapper)
        dz1.ActivationBackward(act, None, DY, z1, y1)
        dx1, dW1, db1 = GPUTensor((M, K), None, wrapper), GPUTensor((N, K), None, wrapper), GPUTensor((N,), None, wrapper)
        DenseBackwardPropagation(dx1, dW1, db1, X, dz1, W, multiplier=0.5)
        dz2 = GPUTensor((M, N), None, wrapper)
        dx2, dW2, db2 = GPUTensor((M, K), None, wrapper), GPUTensor((N, K), None, wrapper), GPUTensor((N,), None, wrapper)
        FusedDenseBackward(dx2, dW2, db2, X, DY, W, act, y=y2, z=z2, multiplier=0.5, dz_scratch=dz2)
        np.testing.assert_array_equal(dW1.ContentAsFloatArray(), dW2.ContentAsFloatArray())
        np.testing.assert_array_equal(dx1.ContentAsFloatArray(), dx2.ContentAsFloatArray())
        np.testing.assert_allclose(db1.ContentAsFloatArray(), db2.ContentAsFloatArray(), rtol=0, atol=1e-4)


def test_bias_add_and_bias_gradient(wrapper):
    # Tests/TestParallelRunCpuVersusGpu.cs:730-736 (9 x 1632) and :938-944, plus odd and tall shapes
    for (M, N) in ((9, 1632), (1, 1), (3, 7), (4096, 1024), (1000, 333), (70000, 8)):
        dy = orc.uniform((M, N), -1.5, 1.5, M + N)
        bias = orc.uniform((N,), -1.5, 1.5, M)
        DB = GPUTensor((N,), None, wrapper)
        _t(wrapper, dy).Compute_BiasGradient_from_dy(DB)
        ref64 = dy.astype(np.float64).sum(0)
        assert np.max(np.abs(DB.ContentAsFloatArray() - ref64)) <= 1e-5 * np.sqrt(M) * 1.5 + 1e-6
        if M <= 4096:
            assert np.max(np.abs(DB.ContentAsFloatArray() - orc.compute_bias_gradient_from_dy(dy))) <= 1e-2
        Y = _t(wrapper, dy)
        _t(wrapper, bias).BroadcastAddVectorToOutput(Y)
        np.testing.assert_array_equal(Y.ContentAsFloatArray(), orc.broadcast_add_vector_to_output(bias, dy.copy()))


def test_activations_and_axpy(wrapper):
    # Tests/TestParallelRunCpuVersusGpu.cs:759-835 shapes; fp32 device math vs the double-precision host formulas
    for shape in ((1, 1), (5, 3), (2, 3, 4, 5), (1000, 257)):
        x = orc.uniform(shape, -1.5, 1.5, 7)
        x.ravel()[0] = 5e-5   # inside the |x| < 1e-4 branch of the Swish gradient
        dy = orc.uniform(shape, -1.5, 1.5, 8)
        X, DY = _t(wrapper, x), _t(wrapper, dy)
        for act in ACTS:
            Y, DX = GPUTensor(shape, None, wrapper), GPUTensor(shape, None, wrapper)
            alpha = ALPHA.get(act)
            ref_alpha = 1.0 if act == ACT_ELU else alpha or 0.0   # Elu runs with 1 whatever the parameter (CpuTensor.cs:954)
            X.ActivationForward(act, alpha, Y)
            y = Y.ContentAsFloatArray()
            np.testing.assert_allclose(y, orc.activation_forward(act, x, ref_alpha), rtol=1e-6, atol=1e-7)
            DX.ActivationBackward(act, alpha, DY, X, Y)
            np.testing.assert_allclose(DX.ContentAsFloatArray(), orc.activation_backward(act, dy, x, y, ref_alpha),
                                       rtol=2e-6, atol=1e-6)
        # the coefficients the reference's own CPU-versus-GPU cases use (Tests/TestParallelRunCpuVersusGpu.cs:761-763,811-813)
        for act, alpha in ((ACT_LEAKY_RELU, 0.1), (ACT_LEAKY_RELU, 0.3), (ACT_ELU, 0.0), (ACT_ELU, 1.0), (ACT_LN, None)):
            Y, DX = GPUTensor(shape, None, wrapper), GPUTensor(shape, None, wrapper)
            ref_alpha = 1.0 if act == ACT_ELU else alpha or 0.0
            X.ActivationForward(act, alpha, Y)
            y = Y.ContentAsFloatArray()
            np.testing.assert_allclose(y, orc.activation_forward(act, x, ref_alpha), rtol=1e-6, atol=1e-7)
            DX.ActivationBackward(act, alpha, DY, X, Y)
            np.testing.assert_allclose(DX.ContentAsFloatArray(), orc.activation_backward(act, dy, x, y, ref_alpha), rtol=2e-6,
                                       atol=1e-6)
            # the C entry points themselves take any coefficient
            for coefficient in ((0.7, 0.25) if act in (ACT_ELU, ACT_LEAKY_RELU) else ()):
                wrapper.set_activation_parameter(coefficient)
                lib, h = wrapper.lib, wrapper.handle
                assert lib.snb200_activation_fwd(h, act, X.Count, X.Pointer, Y.Pointer) == 0
                y = Y.ContentAsFloatArray()
                np.testing.assert_allclose(y, orc.activation_forward(act, x, coefficient), rtol=1e-6, atol=1e-7)
                assert lib.snb200_activation_bwd(h, act, X.Count, DY.Pointer, X.Pointer, Y.Pointer, DX.Pointer) == 0
                np.testing.assert_allclose(DX.ContentAsFloatArray(), orc.activation_backward(act, dy, x, y, coefficient),
                                           rtol=2e-6, atol=1e-6)
        Yv = _t(wrapper, dy)
        Yv.Update_Adding_Alpha_X(0.25, X)
        np.testing.assert_allclose(Yv.ContentAsFloatArray(), orc.update_adding_alpha_x(dy.copy(), 0.25, x), rtol=0,
                                   atol=1e-7)


def test_dense_argument_errors(wrapper):
    lib, h = wrapper.lib, wrapper.handle
    T = GPUTensor((4, 4), None, wrapper)
    assert lib.snb200_dense_fwd(h, 2, 4, 4, 4, T.Pointer, T.Pointer, None, ACT_RELU, None, T.Pointer) == 7
    assert lib.snb200_dense_fwd(h, 0, 4, 4, 4, T.Pointer, T.Pointer, None, 7, None, T.Pointer) == 15   # not an activation of the reference
    # Swish backward without the pre-activation
    assert lib.snb200_dense_bwd(h, 0, 4, 4, 4, T.Pointer, T.Pointer, T.Pointer, ACT_SWISH, T.Pointer, None, 1.0,
                                T.Pointer, None, T.Pointer, None) == 7
    assert b"pre-activation" in lib.snb200_last_error_string(h)


def test_optimizer_updates(wrapper):
    # Tests/TestParallelRunCpuVersusGpu.cs:944-977: Adam, AdamW (timestep 5) and the four SGD cases on a 32 x 17 tensor
    rng = np.random.default_rng(21)
    shape = (32, 17)
    W0, dW = (rng.uniform(-1.5, 1.5, shape).astype(np.float32) for _ in range(2))
    for wd in (0.0, 0.0005):
        vW, sW = rng.uniform(-1.5, 1.5, shape).astype(np.float32), rng.uniform(0, 1.5, shape).astype(np.float32)
        sW[0, 0] = -0.5            # a negative second moment gives NaN on both sides, as in the reference's random test
        Wg, dWg, vg, sg = (_t(wrapper, a) for a in (W0, dW, vW, sW))
        Wg.UpdateAdamOptimizer(0.001, 0.9, 0.999, 1e-8, wd, dWg, vg, sg, 5)
        Wc, vc, sc = W0.copy(), vW.copy(), sW.copy()
        orc.update_adam_optimizer(Wc, 0.001, 0.9, 0.999, 1e-8, wd, dW, vc, sc, 5)
        np.testing.assert_allclose(vg.ContentAsFloatArray(), vc, rtol=2e-6, atol=1e-7)
        np.testing.assert_allclose(sg.ContentAsFloatArray(), sc, rtol=2e-6, atol=1e-7)
        np.testing.assert_allclose(Wg.ContentAsFloatArray(), Wc, rtol=2e-6, atol=1e-6, equal_nan=True)
        assert np.isnan(Wg.ContentAsFloatArray()[0, 0])
    for nesterov in (True, False):
        v = rng.uniform(-1.5, 1.5, shape).astype(np.float32)
        Wg, dWg, vg = (_t(wrapper, a) for a in (W0, dW, v))
        Wg.UpdateSGDOptimizer(0.1, 0.9, nesterov, dWg, vg)
        Wc, vc = W0.copy(), v.copy()
        orc.update_sgd_optimizer(Wc, 0.1, 0.9, nesterov, dW, vc)
        np.testing.assert_allclose(vg.ContentAsFloatArray(), vc, rtol=1e-6, atol=1e-7)
        np.testing.assert_allclose(Wg.ContentAsFloatArray(), Wc, rtol=1e-6, atol=1e-6)
    big = rng.uniform(-1, 1, 1 << 20).astype(np.float32)       # grid-stride path
    Wg, dWg = _t(wrapper, big), _t(wrapper, big)
    Wg.UpdateSGDOptimizer(0.5, 0.0, False, dWg, None)
    np.testing.assert_allclose(Wg.ContentAsFloatArray(), big * np.float32(0.5), rtol=0, atol=1e-7)


def test_golden_ten_epochs_of_training(wrapper, golden):
    # Tests/NonReg/TestNetworkPropagation.cs:80-132: forward, backward and VanillaSGD for 10 epochs through the C ABI;
    # predictions after training at 1e-6
    from sharpnet_b200.optimizers import VanillaSgd
    for key, rows, y_true in (("1_1_4_4", 1, [[1, 0, 0]]), ("2_1_4_4", 2, [[1, 0, 0], [0, 0, 1]])):
        x = _t(wrapper, np.asarray(golden["X_" + key], np.float32).reshape(rows, 16))
        W = _t(wrapper, np.asarray(golden["W_N_1_4_4"], np.float32).reshape(16, 3))
        b = GPUTensor((3,), None, wrapper)
        y_true = np.asarray(y_true, np.float32)
        p, dW, db = GPUTensor((rows, 3), None, wrapper), GPUTensor((16, 3), None, wrapper), GPUTensor((3,), None, wrapper)
        opt = VanillaSgd()
        for _ in range(10):
            FusedDenseForward(p, x, W, b, ACT_SIGMOID, w_layout=W_IN_OUT)
            dy = _t(wrapper, ((p.ContentAsFloatArray() - y_true) / 3).astype(np.float32))   # loss gradient (host side: out of scope)
            FusedDenseBackward(None, dW, db, x, dy, W, ACT_IDENTITY, multiplier=1.0, w_layout=W_IN_OUT)
            opt.UpdateWeights(0.1, 0.1, rows, W, dW, b, db)
        FusedDenseForward(p, x, W, b, ACT_SIGMOID, w_layout=W_IN_OUT)
        np.testing.assert_allclose(p.ContentAsFloatArray().ravel(), golden[f"sigmoid_{key}_pred_after"], rtol=0, atol=1e-6)


def test_loss_gradients_alone_and_fused_into_the_output_layer(wrapper):
    # dy = scale (p - t) for BCE / CCE / Mse against the reference's operation order, then the fused
    # "loss gradient + bias gradient + dW + dx" call against the three-step sequence on the same inputs
    rng = np.random.default_rng(31)
    for (M, K, N) in ((2, 16, 3), (37, 20, 10), (512, 256, 128)):
        x = orc.normal((M, K), 0, 1, M)
        Wl = orc.glorot_uniform((N, K), M + 1)
        p = rng.uniform(0.01, 0.99, (M, N)).astype(np.float32)
        t = (rng.uniform(0, 1, (M, N)) > 0.7).astype(np.float32)
        X, W, P, T = (_t(wrapper, a) for a in (x, Wl, p, t))
        for loss in (LOSS_BINARY_CROSSENTROPY, LOSS_CATEGORICAL_CROSSENTROPY, LOSS_MSE):
            DY = GPUTensor((M, N), None, wrapper)
            DY.ComputeGradientForEvaluationMetric(T, P, loss)
            want = orc.loss_gradient(loss, t, p)
            np.testing.assert_allclose(DY.ContentAsFloatArray(), want, rtol=1e-6, atol=1e-7)
            dx1, dW1, db1 = GPUTensor((M, K), None, wrapper), GPUTensor((N, K), None, wrapper), GPUTensor((N,), None, wrapper)
            DenseBackwardPropagation(dx1, dW1, db1, X, DY, W, multiplier=1.0)
            dz, dx2 = GPUTensor((M, N), None, wrapper), GPUTensor((M, K), None, wrapper)
            dW2, db2 = GPUTensor((N, K), None, wrapper), GPUTensor((N,), None, wrapper)
            FusedDenseBackwardFromLoss(dx2, dW2, db2, X, T, P, W, loss, multiplier=1.0, dz_scratch=dz)
            np.testing.assert_array_equal(dz.ContentAsFloatArray(), DY.ContentAsFloatArray())
            np.testing.assert_array_equal(dW1.ContentAsFloatArray(), dW2.ContentAsFloatArray())
            np.testing.assert_array_equal(dx1.ContentAsFloatArray(), dx2.ContentAsFloatArray())
            np.testing.assert_allclose(db1.ContentAsFloatArray(), db2.ContentAsFloatArray(), rtol=0, atol=1e-5)
            _, dW64, db64, _ = orc.dense_backward(x, Wl, want, orc.ACT_IDENTITY, None, None, 1.0, orc.W_OUT_IN, f64=True)
            assert orc.scaled_error(dW2.ContentAsFloatArray(), dW64, M, 4.0, 2.0) <= TOL_3XTF32
            assert orc.scaled_error(db2.ContentAsFloatArray(), db64, M, 1.0, 2.0) <= TOL_3XTF32


def test_golden_ten_epochs_entirely_on_the_device(wrapper, golden):
    # the same golden as above with nothing on the host between the steps: fused forward, fused
    # "loss gradient + backward" and the SGD update, all through the C ABI
    from sharpnet_b200.optimizers import VanillaSgd
    for key, rows, y_true in (("1_1_4_4", 1, [[1, 0, 0]]), ("2_1_4_4", 2, [[1, 0, 0], [0, 0, 1]])):
        x = _t(wrapper, np.asarray(golden["X_" + key], np.float32).reshape(rows, 16))
        W = _t(wrapper, np.asarray(golden["W_N_1_4_4"], np.float32).reshape(16, 3))
        T = _t(wrapper, np.asarray(y_true, np.float32))
        b, p = GPUTensor((3,), None, wrapper), GPUTensor((rows, 3), None, wrapper)
        dz, dW, db = GPUTensor((rows, 3), None, wrapper), GPUTensor((16, 3), None, wrapper), GPUTensor((3,), None, wrapper)
        opt = VanillaSgd()
        for _ in range(10):
            FusedDenseForward(p, x, W, b, ACT_SIGMOID, w_layout=W_IN_OUT)
            FusedDenseBackwardFromLoss(None, dW, db, x, T, p, W, LOSS_BINARY_CROSSENTROPY, 1.0, dz, W_IN_OUT)
            opt.UpdateWeights(0.1, 0.1, rows, W, dW, b, db)
        FusedDenseForward(p, x, W, b, ACT_SIGMOID, w_layout=W_IN_OUT)
        np.testing.assert_allclose(p.ContentAsFloatArray().ravel(), golden[f"sigmoid_{key}_pred_after"], rtol=0, atol=1e-6)


@pytest.mark.parametrize("layout", [W_OUT_IN, W_IN_OUT])
@pytest.mark.parametrize("mode,tol", [(MATH_3XTF32, TOL_3XTF32), (MATH_TF32, TOL_TF32)])
def test_dense_followed_by_softmax(wrapper, layout, mode, tol):
    # Linear + ActivationLayer(CUDNN_ACTIVATION_SOFTMAX), the output layer of a classifier: softmax applied where the
    # logits are stored (class counts that are multiples of 4, up to 256), or as a pass after the product (10 classes,
    # 1000 classes, tiny batches, a kept pre-activation)
    from sharpnet_b200._capi import ACT_SOFTMAX
    wrapper.set_math_mode(mode)
    for (M, K, N, with_z) in ((512, 384, 100, False), (300, 256, 256, False), (512, 384, 100, True), (64, 128, 10, False),
                              (256, 512, 1000, False), (3, 30, 3, False)):
        x = orc.normal((M, K), 0, 1, 50 + N)
        Wl = orc.glorot_uniform((N, K) if layout == W_OUT_IN else (K, N), 51 + N)
        b = orc.uniform((N,), -0.5, 0.5, 52 + N)
        Y = GPUTensor((M, N), None, wrapper)
        Z = GPUTensor((M, N), None, wrapper) if with_z else None
        FusedDenseForward(Y, _t(wrapper, x), _t(wrapper, Wl), _t(wrapper, b), ACT_SOFTMAX, z=Z, w_layout=layout)
        wrapper.check_device_status()
        z64, y64 = orc.dense_forward(x, Wl, b, ACT_SOFTMAX, layout, f64=True)
        y = Y.ContentAsFloatArray()
        np.testing.assert_allclose(y.sum(1), 1.0, atol=2e-6)
        # softmax has slope <= 1/4: the logits' bound carries over
        wmax = float(np.abs(Wl).max())
        assert np.abs(y - y64).max() <= tol * np.sqrt(K) * 4.0 * wmax
        if with_z:
            assert orc.scaled_error(Z.ContentAsFloatArray(), z64, K, 4.0, wmax) <= tol
        if mode == MATH_3XTF32:
            ym = orc.dense_forward(x, Wl, b, ACT_SOFTMAX, layout)[1]
            assert np.abs(y - ym).max() <= tol * np.sqrt(K) * 4.0 * wmax


def test_dense_backward_rejects_softmax(wrapper):
    from sharpnet_b200._capi import ACT_SOFTMAX, SharpNetB200Error
    t = GPUTensor((4, 4), None, wrapper)
    with pytest.raises(SharpNetB200Error):
        FusedDenseBackward(t, t, None, t, t, t, ACT_SOFTMAX, y=t)


def test_dense_seeded_sweep(wrapper):
    """A seeded draw of batch sizes (down to single rows, which run with swapped operands), widths, activations, weight
    layouts, bias on / off, dx on / off, math modes and K cuts inside clusters: forward and backward against the
    oracle, whatever kernels the shapes end up on."""
    rng = np.random.default_rng(11)
    try:
        for it in range(90):
            M = int(rng.choice([1, 8, 17, 32, 64, 100, 300, 512, 1024]))
            K = int(rng.choice([64, 260, 1024, 2048, 516]))
            N = int(rng.choice([8, 40, 128, 260, 512, 1000]))
            act, layout = int(rng.choice(ACTS)), int(rng.choice([W_IN_OUT, W_OUT_IN]))
            bias, need_dx = bool(rng.integers(4)), bool(rng.integers(4))
            wrapper.set_tuning(TUNE_CLUSTER, int(rng.choice([0, 0, 1, 2, 4])))
            mode, tol = ((MATH_3XTF32, TOL_3XTF32), (MATH_TF32, TOL_TF32))[it % 6 == 5]
            wrapper.set_math_mode(mode)
            _dense_case(wrapper, M, K, N, act, layout, 5000 + it, tol, with_bias=bias, need_dx=need_dx,
                        mult=float(rng.choice([1.0, 0.25])))
    finally:
        wrapper.set_tuning(TUNE_CLUSTER, 0)


def _golden_mlp_on_device(wrapper, g, acts, loss, lr, momentum=0.0, weight_decay=0.0, alphas=None, x=None,
                          first_on_last_dim=False, epochs=10):
    """The reference's small Dense networks (Tests/NonReg/TestNetworkPropagation.cs) trained for 10 epochs entirely
    through the C ABI: fused forward, loss gradient fused into the output layer's backward, hidden layers through
    snb200_dense_bwd, weight decay as dW += 2 * batch * wd * W (Update_Adding_Alpha_X), SGD with or without momentum.
    TensorFlow compatibility mode (dW multiplier 1, [in, out] weights).  Returns predictions before and after."""
    from sharpnet_b200._capi import LOSS_BINARY_CROSSENTROPY, LOSS_CATEGORICAL_CROSSENTROPY, LOSS_MSE  # noqa: F401
    from sharpnet_b200 import ACT_SOFTMAX
    from sharpnet_b200.optimizers import Sgd, VanillaSgd
    n = len(acts)
    alphas = alphas or [None] * n
    batch = x.shape[0]
    y_true = _t(wrapper, np.asarray([[1, 0, 0], [0, 0, 1]], np.float32))
    shapes, fan_in = [], (x.shape[-1] if first_on_last_dim else x[0].size)
    for i in range(n):
        shapes.append((fan_in, 3))
        fan_in = (x[0].size // x.shape[-1]) * 3 if (i == 0 and first_on_last_dim) else 3
    Ws = [_t(wrapper, np.asarray(g["weights"][i], np.float32).reshape(shapes[i])) for i in range(n)]
    bs = [GPUTensor((3,), None, wrapper) for _ in range(n)]
    dWs = [GPUTensor(shapes[i], None, wrapper) for i in range(n)]
    dbs = [GPUTensor((3,), None, wrapper) for _ in range(n)]
    opts = [Sgd(wrapper, momentum, False, shapes[i], (3,)) if momentum else VanillaSgd() for i in range(n)]
    rows = [x.size // shapes[0][0] if first_on_last_dim else batch] + [batch] * (n - 1)
    ins = [_t(wrapper, x.reshape(rows[0], shapes[0][0]))]
    zs = [GPUTensor((rows[i], 3), None, wrapper) for i in range(n)]
    ys = [GPUTensor((rows[i], 3), None, wrapper) for i in range(n)]
    dzs = [GPUTensor((rows[i], 3), None, wrapper) for i in range(n)]
    dxs = [None] + [GPUTensor((rows[i], shapes[i][0]), None, wrapper) for i in range(1, n)]

    def forward():
        h = ins[0]
        for i in range(n):
            if i > 0:
                h = GPUTensor((rows[i], shapes[i][0]), None, wrapper, storage=ys[i - 1].storage)   # Flatten: a view
            FusedDenseForward(ys[i], h, Ws[i], bs[i], acts[i], z=None if acts[i] == ACT_SOFTMAX else zs[i],
                              w_layout=W_IN_OUT, activationParameter=alphas[i])
            ins[i:i + 1] = [h]
        return ys[-1].ContentAsFloatArray().reshape(batch, -1).copy()
    before = forward()
    for _ in range(epochs):
        forward()
        last = n - 1
        FusedDenseBackwardFromLoss(dxs[last], dWs[last], dbs[last], ins[last], y_true, ys[last], Ws[last], loss, 1.0,
                                   dzs[last], W_IN_OUT)
        for i in reversed(range(n - 1)):
            dy = GPUTensor((rows[i], 3), None, wrapper, storage=dxs[i + 1].storage)
            FusedDenseBackward(dxs[i], dWs[i], dbs[i], ins[i], dy, Ws[i], acts[i], y=ys[i], z=zs[i], multiplier=1.0,
                               dz_scratch=dzs[i], w_layout=W_IN_OUT, activationParameter=alphas[i])
        for i in range(n):
            if weight_decay:
                dWs[i].Update_Adding_Alpha_X(2 * batch * weight_decay, Ws[i])
            opts[i].UpdateWeights(lr, lr, batch, Ws[i], dWs[i], bs[i], dbs[i])
        wrapper.check_device_status()
    return before, forward()


def test_golden_softmax_relu_leaky_relu_weight_decay_and_mse_networks(wrapper, golden):
    # Tests/NonReg/TestNetworkPropagation.cs:135-160, 216-244, 330-358, 725-770 at 1e-6 and :1161-1192 at 1e-3:
    # predictions before training and after 10 epochs, nothing on the host between the steps
    from sharpnet_b200 import ACT_SOFTMAX
    from sharpnet_b200._capi import LOSS_BINARY_CROSSENTROPY, LOSS_CATEGORICAL_CROSSENTROPY, LOSS_MSE
    x = np.asarray(golden["X_2_1_4_4"], np.float32).reshape(2, 16)
    cases = (
        ("softmax_2_1_4_4", (ACT_SOFTMAX,), LOSS_CATEGORICAL_CROSSENTROPY, dict(lr=0.1), x, 1e-6),
        ("relu_2_1_4_4", (ACT_RELU, ACT_SIGMOID), LOSS_BINARY_CROSSENTROPY, dict(lr=0.1), x, 1e-6),
        ("leaky_relu_2_1_4_4", (ACT_LEAKY_RELU, ACT_SIGMOID), LOSS_BINARY_CROSSENTROPY,
         dict(lr=0.1, momentum=0.9, alphas=[0.1, None]), x, 1e-6),
        ("weight_decay_vanilla_2_1_4_4", (ACT_SOFTMAX,), LOSS_CATEGORICAL_CROSSENTROPY, dict(lr=0.12, weight_decay=0.05), x, 1e-6),
        ("weight_decay_momentum_2_1_4_4", (ACT_SOFTMAX,), LOSS_CATEGORICAL_CROSSENTROPY,
         dict(lr=0.12, momentum=0.9, weight_decay=0.5), x, 1e-6),
        ("mse_2_3_4_5", (ACT_RELU, ACT_IDENTITY), LOSS_MSE, dict(lr=0.1, momentum=0.9, first_on_last_dim=True),
         np.asarray(golden["X_2_3_4_5"], np.float32).reshape(2, 3, 4, 5), 1e-3),
    )
    for key, acts, loss, kw, xin, tol in cases:
        before, after = _golden_mlp_on_device(wrapper, golden[key], acts, loss, x=xin, **kw)
        np.testing.assert_allclose(before.ravel(), golden[key]["pred_before"], rtol=0, atol=tol, err_msg=key)
        np.testing.assert_allclose(after.ravel(), golden[key]["pred_after"], rtol=0, atol=tol, err_msg=key)


def _pytorch_mlp_on_device(wrapper, x, t, w1, w2, act1, alpha1, out_act, loss, lr, momentum, weight_decay, nesterov,
                           batch_size, first_on_last_dim=False, epochs=10):
    """Two Linear layers with [out, in] weights in the reference's PyTorch compatibility mode (weight decay
    dW += batch * wd * W and db += batch * wd * b, Prod/Layers/Linear.cs:167-181), trained in mini-batches entirely
    through the C ABI.  Returns the predictions on all of x after training."""
    from sharpnet_b200 import ACT_SOFTMAX
    from sharpnet_b200.optimizers import Sgd
    rows = x.shape[0]
    X, T = _t(wrapper, x), _t(wrapper, t)
    Ws, bs = [_t(wrapper, w1), _t(wrapper, w2)], [GPUTensor((w1.shape[0],), None, wrapper), GPUTensor((w2.shape[0],), None, wrapper)]
    dWs = [GPUTensor(w1.shape, None, wrapper), GPUTensor(w2.shape, None, wrapper)]
    dbs = [GPUTensor((w1.shape[0],), None, wrapper), GPUTensor((w2.shape[0],), None, wrapper)]
    opts = [Sgd(wrapper, momentum, nesterov, w.shape, (w.shape[0],)) for w in (w1, w2)]
    per_row_in = x[0].size
    inner = per_row_in // w1.shape[1] if first_on_last_dim else 1      # rows of the first product per sample
    h_per_row = inner * w1.shape[0]
    view = lambda t_, r0, n, width: GPUTensor((n, width), None, wrapper, storage=t_.storage[r0 * width:(r0 + n) * width])  # noqa: E731

    def forward(r0, n, bufs):
        h0 = GPUTensor((n * inner, w1.shape[1]), None, wrapper, storage=X.storage[r0 * per_row_in:(r0 + n) * per_row_in])
        z1, y1, p = bufs
        FusedDenseForward(y1, h0, Ws[0], bs[0], act1, z=z1, w_layout=W_OUT_IN, activationParameter=alpha1)
        h1 = GPUTensor((n, h_per_row), None, wrapper, storage=y1.storage)
        FusedDenseForward(p, h1, Ws[1], bs[1], out_act, z=None, w_layout=W_OUT_IN)
        return h0, h1
    for _ in range(epochs):
        for r0 in range(0, rows, batch_size):
            n = min(batch_size, rows - r0)
            z1, y1 = GPUTensor((n * inner, w1.shape[0]), None, wrapper), GPUTensor((n * inner, w1.shape[0]), None, wrapper)
            p, dz2, dz1 = GPUTensor((n, w2.shape[0]), None, wrapper), GPUTensor((n, w2.shape[0]), None, wrapper), GPUTensor(
                (n * inner, w1.shape[0]), None, wrapper)
            dx = GPUTensor((n, h_per_row), None, wrapper)
            h0, h1 = forward(r0, n, (z1, y1, p))
            FusedDenseBackwardFromLoss(dx, dWs[1], dbs[1], h1, view(T, r0, n, t.shape[1]), p, Ws[1], loss, 1.0, dz2, W_OUT_IN)
            dy1 = GPUTensor((n * inner, w1.shape[0]), None, wrapper, storage=dx.storage)
            FusedDenseBackward(None, dWs[0], dbs[0], h0, dy1, Ws[0], act1, y=y1, z=z1, multiplier=1.0, dz_scratch=dz1,
                               w_layout=W_OUT_IN, activationParameter=alpha1)
            for i in range(2):
                if weight_decay:
                    dWs[i].Update_Adding_Alpha_X(n * weight_decay, Ws[i])
                    dbs[i].Update_Adding_Alpha_X(n * weight_decay, bs[i])
                opts[i].UpdateWeights(lr, lr, n, Ws[i], dWs[i], bs[i], dbs[i])
            wrapper.check_device_status()
    z1, y1 = GPUTensor((rows * inner, w1.shape[0]), None, wrapper), GPUTensor((rows * inner, w1.shape[0]), None, wrapper)
    p = GPUTensor((rows, w2.shape[0]), None, wrapper)
    forward(0, rows, (z1, y1, p))
    return p.ContentAsFloatArray()


def test_golden_pytorch_layout_networks_after_training(wrapper, golden):
    # Tests/NonReg/ParallelRunWithPyTorch.cs:179-214, :102-138 and :813-850: the loss after 10 epochs (1e-6) with SGD
    # momentum, weight decay on weights and biases, Nesterov and mini-batches, all through the C ABI
    from sharpnet_b200 import ACT_SOFTMAX
    from sharpnet_b200._capi import LOSS_BINARY_CROSSENTROPY, LOSS_CATEGORICAL_CROSSENTROPY, LOSS_MSE
    x, t = orc.numpy_array_for_tests(2, 1, 4, 4), orc.y_numpy_array_for_tests(2, 3)
    w1 = np.asarray(golden["pt_relu_w1"], np.float32).reshape(3, 16)
    w2 = np.asarray(golden["pt_relu_w2"], np.float32).reshape(3, 3)
    p = _pytorch_mlp_on_device(wrapper, x, t, w1, w2, ACT_RELU, None, ACT_SIGMOID, LOSS_BINARY_CROSSENTROPY, 0.1, 0.9, 0.03,
                               False, 2)
    assert abs(orc.binary_crossentropy(t, p) - golden["pt_relu_loss_after"]) < 1e-6
    x = orc.numpy_array_for_tests(2, 3, 4, 5)
    w1 = np.asarray(golden["pt_mse_w1"], np.float32).reshape(3, 5)
    w2 = np.asarray(golden["pt_mse_w2"], np.float32).reshape(3, 36)
    p = _pytorch_mlp_on_device(wrapper, x, t, w1, w2, ACT_RELU, None, ACT_IDENTITY, LOSS_MSE, 0.1, 0.9, 0.0, False, 2,
                               first_on_last_dim=True)
    assert abs(orc.mse(t, p) - golden["pt_mse_loss_after"]) < 1e-6
    x, t = orc.numpy_array_for_tests(10, 1, 4, 4), orc.y_numpy_array_for_tests(10, 3)
    w1 = np.asarray(golden["pt_leaky_w1"], np.float32).reshape(3, 16)
    w2 = np.asarray(golden["pt_leaky_w2"], np.float32).reshape(3, 3)
    cce = lambda p_: float(-(t * np.log(p_.astype(np.float64))).sum(1).mean())  # noqa: E731
    p = _pytorch_mlp_on_device(wrapper, x, t, w1, w2, ACT_LEAKY_RELU, 0.1, ACT_SOFTMAX, LOSS_CATEGORICAL_CROSSENTROPY, 0.1,
                               0.66, 0.17, True, 2, epochs=0)
    assert abs(cce(p) - golden["pt_leaky_loss_before"]) < 1e-6
    p = _pytorch_mlp_on_device(wrapper, x, t, w1, w2, ACT_LEAKY_RELU, 0.1, ACT_SOFTMAX, LOSS_CATEGORICAL_CROSSENTROPY, 0.1,
                               0.66, 0.17, True, 2)
    assert abs(cce(p) - golden["pt_leaky_loss_after"]) < 1e-6
