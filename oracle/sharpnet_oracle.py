"""CPU oracle for the Tensor.Dot / Dense path of SharpNet.

THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  It restates on the CPU what SharpNet's CPU
backend computes for the path, so that the CUDA kernels can be checked against it.  Only the test
suite, the smoke check and the ``cpu_baseline`` / ``--impl reference`` legs of the benchmark may
import it; nothing under ``sharpnet_b200/`` does.

Where the arithmetic lives.  SharpNet's CPU path hands every matrix product to Intel MKL
(``cblas_sgemm`` in ``mkl_rt``; no version is pinned: Prod/Data/BlasServices.cs:44-45 imports it
by bare name).  MKL's source is not part of the reference; the stand-in here is the oneAPI MKL
2024.2 that PyTorch links statically (``torch.addmm`` on CPU fp32 tensors calls its ``sgemm``).
Everything around the product -- dimension rules, the batched loop, the Dense call sequence,
bias add, bias gradient, activations and their gradients -- follows the reference's own C# code,
cited per function.  The float64 functions are the ground truth error is measured against.

Parity is pinned on the reference's own vectors: the exact ``Dot`` cases of
Tests/GPU/TestGpuTensor.cs:50-120 and the network goldens of
Tests/NonReg/TestNetworkPropagation.cs:80-132 and Tests/NonReg/ParallelRunWithPyTorch.cs:102-214
(committed under tests/golden/ and checked by tests/test_oracle_golden.py).
"""
import math

import numpy as np
import torch

# cudnnActivationMode_t values (Prod/GPU/CudnnWrapper.cs:267-281)
ACT_SIGMOID, ACT_RELU, ACT_TANH, ACT_IDENTITY, ACT_SWISH = 0, 1, 2, 5, 6
ACT_ELU, ACT_LEAKY_RELU = 4, 1002   # CUDNN_ACTIVATION_ELU / _LEAKY_RELU (Prod/GPU/CudnnWrapper.cs:273,277): take an alpha
ACT_LN = 1004                       # CUDNN_ACTIVATION_LN (:279)
ACT_CLIPPED_RELU = 3                # CUDNN_ACTIVATION_CLIPPED_RELU (:272); the reference has no CPU code for it:
                                    # cuDNN's definition min(max(x, 0), coef) with the coef 1.0 of Prod/GPU/GPUWrapper.cs:183
ACT_SOFTMAX = 1000          # CUDNN_ACTIVATION_SOFTMAX (Prod/GPU/CudnnWrapper.cs:276): softmax over every row
W_OUT_IN, W_IN_OUT = 0, 1
LOSS_BINARY_CROSSENTROPY, LOSS_CATEGORICAL_CROSSENTROPY, LOSS_MSE = 0, 1, 2


# --------------------------------------------------------------------------------------------
# Tensor.Dot
# --------------------------------------------------------------------------------------------
def gemm_dims(aH, aW, transposeA, bH, bW, transposeB):
    """M, N, K, lda, ldb, ldc as BlasServices.DotMkl derives them (Prod/Data/BlasServices.cs:14-19)."""
    M = aW if transposeA else aH
    N = bH if transposeB else bW
    K = aH if transposeA else aW
    return M, N, K, aW, bW, N


def dot_mkl(A, aH, aW, transposeA, B, bH, bW, transposeB, C, alpha, beta):
    """C = alpha * op(A) * op(B) + beta * C in fp32 through MKL sgemm, row-major, in place.

    Mirrors BlasServices.DotMkl (Prod/Data/BlasServices.cs:10-21) as called by CpuTensor.Dot
    (Prod/CPU/CpuTensor.cs:2991-3002).  A, B, C are flat float32 numpy arrays (C is updated and
    returned reshaped to [M, N])."""
    M, N, K, _, _, _ = gemm_dims(aH, aW, transposeA, bH, bW, transposeB)
    kB = bW if transposeB else bH
    if K != kB:
        raise ValueError("inner dimensions differ")
    a = torch.from_numpy(np.ascontiguousarray(A, dtype=np.float32).reshape(aH, aW))
    b = torch.from_numpy(np.ascontiguousarray(B, dtype=np.float32).reshape(bH, bW))
    c = torch.from_numpy(C.reshape(M, N))  # shares memory with C
    opa = a.t() if transposeA else a
    opb = b.t() if transposeB else b
    if K == 0:
        c.mul_(beta) if beta != 0 else c.zero_()
    else:
        torch.addmm(c, opa, opb, beta=float(beta), alpha=float(alpha), out=c)
    return C.reshape(M, N)


def dot_f64(A, aH, aW, transposeA, B, bH, bW, transposeB, C, alpha, beta):
    """Same contract in float64 (ground truth); returns a new [M, N] float64 array."""
    M, N, K, _, _, _ = gemm_dims(aH, aW, transposeA, bH, bW, transposeB)
    a = np.asarray(A, dtype=np.float64).reshape(aH, aW)
    b = np.asarray(B, dtype=np.float64).reshape(bH, bW)
    opa = a.T if transposeA else a
    opb = b.T if transposeB else b
    out = float(alpha) * (opa @ opb)
    if beta != 0:
        out = out + float(beta) * np.asarray(C, dtype=np.float64).reshape(M, N)
    return out


def batch_matrix_multiplication(a_3D, transposeA, b_3D, transposeB, c_3D, alpha, beta, f64=False):
    """c[i] = alpha * op(a[i]) * op(b[i]) + beta * c[i], one Dot per matrix in a serial loop, which
    is how CpuTensor.BatchMatrixMultiplication does it (Prod/CPU/CpuTensor.cs:3004-3025)."""
    nb = a_3D.shape[0]
    assert b_3D.shape[0] == nb and c_3D.shape[0] == nb
    out = np.empty(c_3D.shape, dtype=np.float64) if f64 else c_3D
    for i in range(nb):
        if f64:
            out[i] = dot_f64(a_3D[i].ravel(), a_3D.shape[1], a_3D.shape[2], transposeA, b_3D[i].ravel(),
                             b_3D.shape[1], b_3D.shape[2], transposeB, c_3D[i].ravel(), alpha, beta)
        else:
            dot_mkl(a_3D[i].ravel(), a_3D.shape[1], a_3D.shape[2], transposeA, b_3D[i].ravel(), b_3D.shape[1],
                    b_3D.shape[2], transposeB, c_3D[i].reshape(-1), alpha, beta)
    return out


# --------------------------------------------------------------------------------------------
# Dense companions
# --------------------------------------------------------------------------------------------
def broadcast_add_vector_to_output(bias, y):
    """y[n, col] += bias[col], fp32 (Prod/CPU/CpuTensor.cs:1468-1487).  In place."""
    y2 = y.reshape(y.shape[0], -1)
    y2 += np.asarray(bias, dtype=np.float32).reshape(1, -1)
    return y


def compute_bias_gradient_from_dy(dy):
    """db[col] = sum over rows of dy, accumulated row after row in fp32 exactly as
    CpuTensor.ComputeSumByColumn does (Prod/CPU/CpuTensor.cs:3343-3362)."""
    dy2 = np.asarray(dy, dtype=np.float32).reshape(dy.shape[0], -1)
    acc = np.zeros(dy2.shape[1], dtype=np.float32)
    for r in range(dy2.shape[0]):
        acc += dy2[r]
    return acc


def update_adding_alpha_x(y, alpha, x):
    """y += alpha * x via saxpy (Prod/CPU/CpuTensor.cs:1032-1038).  In place."""
    y += np.float32(alpha) * np.asarray(x, dtype=np.float32)
    return y


def activation_forward(act, x, alpha=0.0):
    """Element-wise activations with the precision SharpNet's CPU code uses
    (Prod/CPU/CpuTensorActivationFunctions.cs): Swish and Sigmoid go through double
    (:152-156, Prod/Utils.cs:888-891), Tanh is MathF.Tanh (:184-189), Relu is max(0, x) (:198-201),
    LeakyRelu is x or (float)alpha * x (:210-213), Elu is x or (float)(alpha * (exp(x) - 1)) through double (:223-226)."""
    x = np.asarray(x, dtype=np.float32)
    if act == ACT_LN:                                    # x <= 0 ? -100 : MathF.Log(x)  (:170-174)
        with np.errstate(divide="ignore", invalid="ignore"):
            return np.where(x <= 0, np.float32(-100), np.log(x)).astype(np.float32)
    if act == ACT_LEAKY_RELU:
        return np.where(x >= 0, x, np.float32(alpha) * x).astype(np.float32)
    if act == ACT_ELU:
        return np.where(x >= 0, x, (float(alpha) * (np.exp(x.astype(np.float64)) - 1.0)).astype(np.float32)).astype(np.float32)
    if act == ACT_RELU:
        return np.maximum(x, np.float32(0))
    if act == ACT_CLIPPED_RELU:
        return np.minimum(np.maximum(x, np.float32(0)), np.float32(1))
    if act == ACT_SWISH:
        xd = x.astype(np.float64)
        return (xd / (1.0 + np.exp(-xd))).astype(np.float32)
    if act == ACT_SIGMOID:
        xd = x.astype(np.float64)
        return (1.0 / (1.0 + np.exp(-xd))).astype(np.float32)
    if act == ACT_TANH:
        return np.tanh(x).astype(np.float32)
    if act == ACT_IDENTITY:
        return x.copy()
    if act == ACT_SOFTMAX:
        return softmax_last_dimension(x)
    raise ValueError(f"activation {act} is not on the path")


def activation_backward(act, dy, x, y, alpha=0.0):
    """dx from dy, the activation input x and output y, all in fp32
    (Prod/CPU/CpuTensorActivationFunctions.cs:158-167 Swish, :190-194 Tanh, :202-206 Relu,
    :240-244 Sigmoid, :214-219 LeakyRelu from y, :227-231 Elu from x and y)."""
    dy = np.asarray(dy, dtype=np.float32)
    one = np.float32(1)
    if act == ACT_LN:                                    # dy / x  (:176-180)
        return (dy / np.asarray(x, dtype=np.float32)).astype(np.float32)
    if act == ACT_LEAKY_RELU:
        return np.where(np.asarray(y) >= 0, dy, np.float32(alpha) * dy).astype(np.float32)
    if act == ACT_ELU:
        return np.where(np.asarray(x) >= 0, dy, dy * (np.asarray(y, dtype=np.float32) + np.float32(alpha))).astype(np.float32)
    if act == ACT_RELU:
        return np.where(y > 0, dy, np.float32(0)).astype(np.float32)
    if act == ACT_CLIPPED_RELU:
        y = np.asarray(y)
        return np.where((y > 0) & (y < 1), dy, np.float32(0)).astype(np.float32)
    if act == ACT_SWISH:
        x = np.asarray(x, dtype=np.float32)
        with np.errstate(divide="ignore", invalid="ignore"):
            s = np.where(np.abs(x) < np.float32(0.0001), np.float32(0.5), y / x).astype(np.float32)
        return (dy * (s + x * s * (one - s))).astype(np.float32)
    if act == ACT_TANH:
        return (dy * (one - y * y)).astype(np.float32)
    if act == ACT_SIGMOID:
        return (dy * y * (one - y)).astype(np.float32)
    if act == ACT_IDENTITY:
        return dy.copy()
    raise ValueError(f"activation {act} is not on the path")


def softmax_last_dimension(x):
    """Row softmax exactly as CpuTensorActivationFunctions.Softmax computes it
    (Prod/CPU/CpuTensorActivationFunctions.cs:19-46): row max, exp in double cast to float, fp32 running sum,
    fp32 division."""
    x2 = np.asarray(x, dtype=np.float32).reshape(-1, x.shape[-1])
    out = np.empty_like(x2)
    for r in range(x2.shape[0]):
        e = np.exp((x2[r] - x2[r].max()).astype(np.float64)).astype(np.float32)
        acc = np.float32(0)
        for v in e:
            acc = np.float32(acc + v)
        out[r] = e / acc
    return out.reshape(x.shape)


def softmax_gradient_last_dimension(dy, y, f64=False):
    """dx = y * (dy - sum_j dy_j y_j): the Jacobian product cudnnSoftmaxBackward(CUDNN_SOFTMAX_ACCURATE,
    MODE_INSTANCE) applies on SharpNet's GPU path (Prod/GPU/GpuTensor.cs:445-490).  cuDNN's source is not part
    of the reference; this restates its documented formula.  (SharpNet's CPU shortcut,
    CpuTensorActivationFunctions.cs:109-121, is a different, loss-specific approximation and is not followed.)"""
    t = np.float64 if f64 else np.float32
    g, p = np.asarray(dy, dtype=t), np.asarray(y, dtype=t)
    return (p * (g - (g * p).sum(axis=-1, keepdims=True))).astype(t)


def set_all_elements_above_main_diagonal(x, value):
    """In place: x[..., row, col] = value for col > row, on one matrix or a batch of matrices
    (Tensor.SetAllElementsAboveMainDiagonal, Prod/CPU/CpuTensor.cs:3037-3052): the causal mask of attention."""
    assert x.ndim in (2, 3)
    rows, cols = np.triu_indices(x.shape[-2], 1, x.shape[-1])
    x[..., rows, cols] = value
    return x


def sdpa_forward(Q, K, V, use_scale, is_causal, f64=False):
    """Returns (weights, y) of ScaledDotProductAttentionLayer.ScaledDotProductAttentionForwardPropagation
    (Prod/Layers/ScaledDotProductAttentionLayer.cs:46-91): scores = scaling * Q K^T per batch element,
    -1e12 above the main diagonal when causal (Prod/CPU/CpuTensor.cs:3037-3052), softmax over the last
    dimension, y = weights V."""
    B, Tq, E = Q.shape
    Tk = K.shape[1]
    scaling = (1.0 / math.sqrt(E)) if use_scale else 1.0
    if f64:
        s = scaling * np.einsum("bqe,bke->bqk", Q.astype(np.float64), K.astype(np.float64))
    else:
        s = np.zeros((B, Tq, Tk), dtype=np.float32)
        batch_matrix_multiplication(Q, False, K, True, s, np.float32(scaling), 0.0)
    if is_causal:
        s = set_all_elements_above_main_diagonal(s.copy(), -1e12)
    if f64:
        e = np.exp(s - s.max(-1, keepdims=True))
        w = e / e.sum(-1, keepdims=True)
        return w, np.einsum("bqk,bke->bqe", w, V.astype(np.float64))
    w = softmax_last_dimension(s)
    y = np.zeros((B, Tq, E), dtype=np.float32)
    batch_matrix_multiplication(w, False, V, False, y, 1.0, 0.0)
    return w, y


def sdpa_backward(Q, K, V, dy, weights, use_scale):
    """Returns (dQ, dK, dV) in float64 following ScaledDotProductAttentionBackwardPropagation
    (Prod/Layers/ScaledDotProductAttentionLayer.cs:108-129)."""
    E = Q.shape[2]
    scaling = (1.0 / math.sqrt(E)) if use_scale else 1.0
    Qd, Kd, Vd, g, w = (np.asarray(a, dtype=np.float64) for a in (Q, K, V, dy, weights))
    dV = np.einsum("bqk,bqe->bke", w, g)
    ds = softmax_gradient_last_dimension(scaling * np.einsum("bqe,bke->bqk", g, Vd), w, f64=True)
    return np.einsum("bqk,bke->bqe", ds, Kd), np.einsum("bqk,bqe->bke", ds, Qd), dV


def transpose_second_third(x):
    """target[a, c, b, :] = x[a, b, c, :]   (Tensor.TransposeSecondAndThirdDimension, Prod/CPU/CpuTensor.cs:301-322)."""
    return np.ascontiguousarray(np.swapaxes(x, 1, 2))


def multihead_attention_forward(Q, K, V, weights, biases, num_heads, key_dim, value_dim, is_causal,
                                w_layout=W_OUT_IN, f64=False):
    """MultiheadAttention.ForwardPropagation (Prod/Layers/MultiheadAttention.cs:178-238).

    Q [batch, q_steps, embed], K and V [batch, v_steps, embed]; ``weights`` = (w_Q, w_K, w_V, out_proj_weight),
    ``biases`` the four matching vectors or None each.  Every projection is Linear.DenseForwardPropagation on the
    last dimension, the heads are split with TransposeSecondAndThirdDimension ([b, t, h, d] -> [b, h, t, d]),
    attention always scales by 1/sqrt(key_dim) (use_scale is a constant of the layer, :32), the heads are merged by
    the inverse permutation and projected by out_proj_weight.  Returns (y, cache) with the tensors the backward pass
    reads: the per-head Q, K, V, the attention weights and the merged heads."""
    B, Tq, E = Q.shape
    Tk = V.shape[1]
    wq, wk, wv, wo = weights
    bq, bk, bv, bo = biases if biases is not None else (None, None, None, None)
    H = num_heads

    def project(x, W, b, d):
        y = dense_forward(x.reshape(-1, x.shape[-1]), W, b, ACT_IDENTITY, w_layout, f64)[1]
        return transpose_second_third(y.reshape(B, -1, H, d)).reshape(B * H, -1, d)
    dt = np.float64 if f64 else np.float32
    Qh, Kh, Vh = project(Q, wq, bq, key_dim), project(K, wk, bk, key_dim), project(V, wv, bv, value_dim)
    w, a = sdpa_forward(Qh.astype(dt), Kh.astype(dt), Vh.astype(dt), True, is_causal, f64)
    merged = transpose_second_third(a.reshape(B, H, Tq, value_dim)).reshape(B * Tq, H * value_dim)
    y = dense_forward(merged.astype(dt), wo, bo, ACT_IDENTITY, w_layout, f64)[1].reshape(B, Tq, -1)
    return y, {"Qh": Qh, "Kh": Kh, "Vh": Vh, "weights": w, "merged": merged}


def multihead_attention_backward(Q, K, V, dy, weights, cache, num_heads, key_dim, value_dim, multiplier=1.0,
                                 w_layout=W_OUT_IN):
    """MultiheadAttention.BackwardPropagation (Prod/Layers/MultiheadAttention.cs:240-295) in float64.
    Returns (dQ, dK, dV, [dw_Q, dw_K, dw_V, d_out_proj_weight], [db_Q, db_K, db_V, db_O])."""
    B, Tq, E = Q.shape
    Tk = V.shape[1]
    H = num_heads
    wq, wk, wv, wo = weights
    g2 = np.asarray(dy, np.float64).reshape(B * Tq, -1)
    _, dwo, dbo, dmerged = dense_backward(cache["merged"], wo, g2, ACT_IDENTITY, None, None, multiplier, w_layout, True,
                                          f64=True)
    da = transpose_second_third(dmerged.reshape(B, Tq, H, value_dim)).reshape(B * H, Tq, value_dim)
    dQh, dKh, dVh = sdpa_backward(cache["Qh"], cache["Kh"], cache["Vh"], da, cache["weights"], True)

    def unproject(dh, x, W, T, d):
        flat = transpose_second_third(dh.reshape(B, H, T, d)).reshape(B * T, H * d)
        _, dW, db, dx = dense_backward(x.reshape(-1, x.shape[-1]), W, flat, ACT_IDENTITY, None, None, multiplier,
                                       w_layout, True, f64=True)
        return dx.reshape(x.shape), dW, db
    dQ, dwq, dbq = unproject(dQh, Q, wq, Tq, key_dim)
    dK, dwk, dbk = unproject(dKh, K, wk, Tk, key_dim)
    dV, dwv, dbv = unproject(dVh, V, wv, Tk, value_dim)
    return dQ, dK, dV, [dwq, dwk, dwv, dwo], [dbq, dbk, dbv, dbo]


def loss_gradient(loss, y_expected, y_predicted):
    """dy of the loss w.r.t. the prediction, in fp32 with the reference's operation order:
    BinaryCrossentropy  m*p - m*y, m = 1/numClass   (Prod/Data/Tensor.cs:1379-1387, AddTensor(-m, y, m));
    CategoricalCrossentropy  p - y                  (:1389-1395);
    Mse  (2*(p - y)) / numClass                     (Prod/CPU/CpuTensor.cs:2466-2475)."""
    p = np.asarray(y_predicted, dtype=np.float32)
    t = np.asarray(y_expected, dtype=np.float32)
    n = np.float32(p.shape[-1])
    if loss == LOSS_BINARY_CROSSENTROPY:
        m = np.float32(1) / n
        return (-m) * t + m * p
    if loss == LOSS_CATEGORICAL_CROSSENTROPY:
        return p - t
    if loss == LOSS_MSE:
        return (np.float32(2) * (p - t)) / n
    raise ValueError(f"loss {loss} is not on the path")


def update_sgd_optimizer(W, learning_rate, momentum, nesterov, dW, velocity):
    """In place, fp32, element by element as CpuTensor.UpdateSGDOptimizer does
    (Prod/CPU/CpuTensor.cs:470-489).  velocity None: the VanillaSgd update (Prod/Optimizers/VanillaSgd.cs:18-20)."""
    lr, mom = np.float32(learning_rate), np.float32(momentum)
    if velocity is None:
        W += (-lr) * dW
        return W
    velocity[...] = (mom * velocity) - (dW * lr)
    if nesterov:
        W += mom * velocity - (dW * lr)
    else:
        W += velocity
    return W


def update_adam_optimizer(W, learning_rate, beta1, beta2, epsilon, weight_decay, dW, adam_vW, adam_sW, time_step):
    """In place; every expression in double then cast to float, as CpuTensor.UpdateAdamOptimizer does
    (Prod/CPU/CpuTensor.cs:1755-1769)."""
    b1p, b2p = beta1 ** time_step, beta2 ** time_step
    dw = dW.astype(np.float64)
    adam_vW[...] = (beta1 * adam_vW.astype(np.float64) + (1 - beta1) * dw).astype(np.float32)
    adam_sW[...] = (beta2 * adam_sW.astype(np.float64) + (1 - beta2) * dw * dw).astype(np.float32)
    factor = learning_rate * (math.sqrt(1.0 - b2p) / (1.0 - b1p))
    w = W.astype(np.float64)
    with np.errstate(invalid="ignore"):
        W[...] = (w - (factor * (adam_vW.astype(np.float64) / (np.sqrt(adam_sW.astype(np.float64)) + epsilon))
                       + weight_decay * w)).astype(np.float32)
    return W


# --------------------------------------------------------------------------------------------
# Dense layer
# --------------------------------------------------------------------------------------------
def dense_forward(x, W, bias, act=ACT_IDENTITY, w_layout=W_OUT_IN, f64=False, alpha=0.0):
    """Returns (z, y): z = x * op(W) + bias, y = act(z).

    OUT_IN follows Linear.DenseForwardPropagation (Prod/Layers/Linear.cs:125-132: Dot(x, false,
    W, true, 1, 0) then BroadcastAddVectorToOutput) and ActivationLayer.ForwardPropagation
    (Prod/Layers/ActivationLayer.cs:32-38).  IN_OUT is the same product with W stored
    [in, out] (the layout of the Keras goldens, Tests/NonReg/TestNetworkPropagation.cs:34,95)."""
    M, K = x.shape
    N = W.shape[0] if w_layout == W_OUT_IN else W.shape[1]
    tB = w_layout == W_OUT_IN
    if f64:
        z = dot_f64(x.ravel(), M, K, False, W.ravel(), W.shape[0], W.shape[1], tB, np.zeros(M * N), 1.0, 0.0)
        if bias is not None:
            z = z + np.asarray(bias, dtype=np.float64).reshape(1, -1)
        return z, _act_f64(act, z, alpha)
    z = np.zeros((M, N), dtype=np.float32)
    dot_mkl(x.ravel(), M, K, False, W.ravel(), W.shape[0], W.shape[1], tB, z.reshape(-1), 1.0, 0.0)
    if bias is not None:
        broadcast_add_vector_to_output(bias, z)
    return z, activation_forward(act, z, alpha)


def dense_backward(x, W, dy, act=ACT_IDENTITY, y=None, z=None, multiplier=1.0, w_layout=W_OUT_IN, need_dx=True,
                   f64=False, alpha=0.0):
    """Returns (dz, dW, db, dx).

    dz = ActivationBackward(dy, z, y) (Prod/Layers/ActivationLayer.cs:39-69), then
    Linear.DenseBackwardPropagation (Prod/Layers/Linear.cs:142-191): dW = multiplier * dz^T * x
    (:158), db = column sums of dz (:160-165), dx = dz * W (:190), skipped when the previous layer
    is the input (:184-187).  IN_OUT stores dW as [in, out] = x^T * dz and uses dx = dz * W^T."""
    M, K = x.shape
    N = dy.shape[1]
    if f64:
        dz = _act_bwd_f64(act, dy, z, y, alpha)
        xd, Wd = x.astype(np.float64), W.astype(np.float64)
        if w_layout == W_OUT_IN:
            dW = multiplier * (dz.T @ xd)
            dx = dz @ Wd if need_dx else None
        else:
            dW = multiplier * (xd.T @ dz)
            dx = dz @ Wd.T if need_dx else None
        return dz, dW, dz.sum(axis=0), dx
    dz = activation_backward(act, dy, z, y, alpha)
    if w_layout == W_OUT_IN:
        dW = np.zeros((N, K), dtype=np.float32)
        dot_mkl(dz.ravel(), M, N, True, x.ravel(), M, K, False, dW.reshape(-1), multiplier, 0.0)
    else:
        dW = np.zeros((K, N), dtype=np.float32)
        dot_mkl(x.ravel(), M, K, True, dz.ravel(), M, N, False, dW.reshape(-1), multiplier, 0.0)
    db = compute_bias_gradient_from_dy(dz)
    dx = None
    if need_dx:
        dx = np.zeros((M, K), dtype=np.float32)
        if w_layout == W_OUT_IN:
            dot_mkl(dz.ravel(), M, N, False, W.ravel(), N, K, False, dx.reshape(-1), 1.0, 0.0)
        else:
            dot_mkl(dz.ravel(), M, N, False, W.ravel(), K, N, True, dx.reshape(-1), 1.0, 0.0)
    return dz, dW, db, dx


def _act_f64(act, z, alpha=0.0):
    if act == ACT_LEAKY_RELU:
        return np.where(z >= 0, z, alpha * z)
    if act == ACT_ELU:
        return np.where(z >= 0, z, alpha * (np.exp(np.minimum(z, 0.0)) - 1.0))
    if act == ACT_RELU:
        return np.maximum(z, 0.0)
    if act == ACT_CLIPPED_RELU:
        return np.minimum(np.maximum(z, 0.0), 1.0)
    if act == ACT_LN:
        with np.errstate(divide="ignore", invalid="ignore"):
            return np.where(z <= 0, -100.0, np.log(z))
    if act == ACT_SWISH:
        return z / (1.0 + np.exp(-z))
    if act == ACT_SIGMOID:
        return 1.0 / (1.0 + np.exp(-z))
    if act == ACT_TANH:
        return np.tanh(z)
    if act == ACT_SOFTMAX:
        e = np.exp(z - z.max(-1, keepdims=True))
        return e / e.sum(-1, keepdims=True)
    return z.copy()


def _act_bwd_f64(act, dy, z, y, alpha=0.0):
    dy = np.asarray(dy, dtype=np.float64)
    if act == ACT_LEAKY_RELU:
        return np.where(np.asarray(y) >= 0, dy, alpha * dy)
    if act == ACT_ELU:
        return np.where(np.asarray(z) >= 0, dy, dy * (np.asarray(y, dtype=np.float64) + alpha))
    if act == ACT_RELU:
        return np.where(np.asarray(y) > 0, dy, 0.0)
    if act == ACT_CLIPPED_RELU:
        return np.where((np.asarray(y) > 0) & (np.asarray(y) < 1), dy, 0.0)
    if act == ACT_LN:
        return dy / np.asarray(z, dtype=np.float64)
    if act == ACT_SWISH:
        zd = np.asarray(z, dtype=np.float64)
        s = 1.0 / (1.0 + np.exp(-zd))
        return dy * (s + zd * s * (1.0 - s))
    if act == ACT_TANH:
        yd = np.asarray(y, dtype=np.float64)
        return dy * (1.0 - yd * yd)
    if act == ACT_SIGMOID:
        yd = np.asarray(y, dtype=np.float64)
        return dy * yd * (1.0 - yd)
    return dy.copy()


# --------------------------------------------------------------------------------------------
# Losses used by the reference's golden network tests (checker side only)
# --------------------------------------------------------------------------------------------
def binary_crossentropy(y_true, y_pred):
    """Mean over rows of the mean over columns of -(t*log(p) + (1-t)*log(1-p))
    (BinaryCrossentropyLossBuffer, Prod/GPU/Kernels/SinglePrecision.cu:773-791)."""
    p = np.asarray(y_pred, dtype=np.float64)
    t = np.asarray(y_true, dtype=np.float64)
    return float(np.mean(-(t * np.log(p) + (1.0 - t) * np.log(1.0 - p))))


def mse(y_true, y_pred):
    """Mean squared error over all elements (MseLossBuffer, SinglePrecision.cu:991-1006)."""
    d = np.asarray(y_pred, dtype=np.float64) - np.asarray(y_true, dtype=np.float64)
    return float(np.mean(d * d))


# --------------------------------------------------------------------------------------------
# Deterministic inputs
# --------------------------------------------------------------------------------------------
def numpy_array_for_tests(*shape):
    """data[i] = (float)(2*(i+1)/count * ((i % 2) - 0.5))
    (Tests/NonReg/TestNetworkPropagation.cs:167-176)."""
    count = int(np.prod(shape))
    i = np.arange(count, dtype=np.float64)
    return ((2.0 * (i + 1)) / count * ((i % 2) - 0.5)).astype(np.float32).reshape(shape)


def y_numpy_array_for_tests(rows, cols):
    """One-hot rows with the 1 in column row % cols (Tests/NonReg/TestNetworkPropagation.cs:178-186)."""
    out = np.zeros((rows, cols), dtype=np.float32)
    for r in range(rows):
        out[r, r % cols] = 1
    return out


def uniform(shape, lo, hi, seed):
    """U[lo, hi) float32 from a seeded generator (stands in for Utils.UniformDistribution,
    Prod/Utils.cs:411-417; .NET's Random stream itself is not reproducible without .NET)."""
    return np.random.default_rng(seed).uniform(lo, hi, size=shape).astype(np.float32)


def normal(shape, mean, std, seed):
    """N(mean, std) float32 (stands in for Utils.NormalDistribution, Prod/Utils.cs:425-431)."""
    return np.random.default_rng(seed).normal(mean, std, size=shape).astype(np.float32)


def glorot_uniform(shape, seed):
    """U[-limit, limit), limit = sqrt(6 / (Shape[0] + MultDim0)) (Prod/Data/Tensor.cs:1480-1486)."""
    fan = shape[0] + int(np.prod(shape[1:]))
    limit = math.sqrt(6.0 / fan)
    return uniform(shape, -limit, limit, seed)


def scaled_error(got, ref, K, a_max, b_max):
    """max |got - ref| / (sqrt(K) * a_max * b_max): the error measure the accuracy gates use
    (<= 1e-5 in 3xTF32 mode, <= 2e-3 in TF32 mode)."""
    d = np.max(np.abs(np.asarray(got, dtype=np.float64) - np.asarray(ref, dtype=np.float64)))
    return float(d / (math.sqrt(max(K, 1)) * a_max * b_max))
