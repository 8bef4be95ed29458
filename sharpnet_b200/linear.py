"""Host-side mirror of SharpNet's Dense layer (Prod/Layers/Linear.cs) on top of the C ABI.

``DenseForwardPropagation`` / ``DenseBackwardPropagation`` keep the reference's static-method
signatures and call sequence (Dot, bias add, bias gradient, Dot, Dot).  ``FusedDenseForward`` /
``FusedDenseBackward`` are what the same two methods call once the following ActivationLayer is
folded in: one ``snb200_dense_fwd`` / ``snb200_dense_bwd`` each.
"""
from ._capi import ACT_IDENTITY, W_IN_OUT, W_OUT_IN, check  # noqa: F401
from .tensor import GPUTensor


def DenseForwardPropagation(y, x, weights, biasIfAny_1D, flattenInputTensorOnLastDimension=False):
    """y = x * weights^T + bias   (Prod/Layers/Linear.cs:125-132; weights are [out, in])."""
    x2 = x.As2DTensor(flattenInputTensorOnLastDimension)
    y2 = y.As2DTensor(flattenInputTensorOnLastDimension)
    y2.Dot(x2, False, weights, True, 1, 0)
    if biasIfAny_1D is not None:
        biasIfAny_1D.BroadcastAddVectorToOutput(y2)


def DenseBackwardPropagation(dx, weightGradients, biasGradients_1D, x, dy, weights, bias_1D=None, multiplier=None,
                             weight_decay_alpha=0.0, prevLayerIsInputLayer=False,
                             flattenInputTensorOnLastDimension=False):
    """dW = multiplier * dy^T * x ; db = column sums of dy ; dW += alpha * W ; dx = dy * W
    (Prod/Layers/Linear.cs:142-191).  ``multiplier`` defaults to 1/batch as in SharpNet's own
    compatibility mode (:152-156); ``weight_decay_alpha`` is the already-combined factor of :174."""
    x2 = x.As2DTensor(flattenInputTensorOnLastDimension)
    dy2 = dy.As2DTensor(flattenInputTensorOnLastDimension)
    if multiplier is None:
        multiplier = 1.0 / x.Shape[0]
    weightGradients.Dot(dy2, True, x2, False, multiplier, 0)
    if biasGradients_1D is not None:
        dy2.Compute_BiasGradient_from_dy(biasGradients_1D)
    if weight_decay_alpha > 0:
        weightGradients.Update_Adding_Alpha_X(weight_decay_alpha, weights)
    if prevLayerIsInputLayer:
        return
    dx.As2DTensor(flattenInputTensorOnLastDimension).Dot(dy2, False, weights, False, 1, 0)


def FusedDenseForward(y, x, weights, biasIfAny_1D, activation=ACT_IDENTITY, z=None, w_layout=W_OUT_IN,
                      flattenInputTensorOnLastDimension=False, activationParameter=None):
    """y = act(x * op(W) + bias) in one kernel; ``z`` optionally receives the pre-activation;
    ``activationParameter`` is the coefficient of ELU / LeakyRelu."""
    x2 = x.As2DTensor(flattenInputTensorOnLastDimension)
    y2 = y.As2DTensor(flattenInputTensorOnLastDimension)
    M, K = x2.Shape
    N = y2.Shape[1]
    w = y.wrapper
    if activationParameter is not None:
        w.set_activation_parameter(activationParameter)
    st = w.lib.snb200_dense_fwd(w.handle, w_layout, M, K, N, x2.Pointer, weights.Pointer,
                                None if biasIfAny_1D is None else biasIfAny_1D.Pointer, int(activation),
                                None if z is None else z.Pointer, y2.Pointer)
    check(w.handle, st)


def FusedDenseBackward(dx, weightGradients, biasGradients_1D, x, dy, weights, activation=ACT_IDENTITY, y=None, z=None,
                       multiplier=1.0, dz_scratch=None, w_layout=W_OUT_IN, flattenInputTensorOnLastDimension=False,
                       activationParameter=None):
    """ActivationLayer backward + Dense backward through one ``snb200_dense_bwd`` call."""
    x2 = x.As2DTensor(flattenInputTensorOnLastDimension)
    dy2 = dy.As2DTensor(flattenInputTensorOnLastDimension)
    M, K = x2.Shape
    N = dy2.Shape[1]
    w = dy.wrapper
    if activationParameter is not None:
        w.set_activation_parameter(activationParameter)
    p = lambda t: None if t is None else t.Pointer  # noqa: E731
    st = w.lib.snb200_dense_bwd(w.handle, w_layout, M, K, N, x2.Pointer, weights.Pointer, dy2.Pointer, int(activation),
                                p(y), p(z), float(multiplier), p(dz_scratch), p(dx), weightGradients.Pointer,
                                p(biasGradients_1D))
    check(w.handle, st)


def FusedDenseBackwardFromLoss(dx, weightGradients, biasGradients_1D, x, yExpected, yPredicted, weights, loss,
                               multiplier=1.0, dz_scratch=None, w_layout=W_OUT_IN):
    """Backward of the output Dense layer from the labels: loss gradient + bias gradient in one pass, then dW, dx."""
    x2 = x.As2DTensor(False)
    M, K = x2.Shape
    N = yPredicted.MultDim0
    w = yPredicted.wrapper
    p = lambda t: None if t is None else t.Pointer  # noqa: E731
    st = w.lib.snb200_dense_bwd_from_loss(w.handle, w_layout, M, K, N, x2.Pointer, weights.Pointer, int(loss),
                                          yExpected.Pointer, yPredicted.Pointer, float(multiplier), p(dz_scratch), p(dx),
                                          weightGradients.Pointer, p(biasGradients_1D))
    check(w.handle, st)
