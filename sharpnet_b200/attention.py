"""Host-side mirror of SharpNet's scaled dot-product attention layer
(Prod/Layers/ScaledDotProductAttentionLayer.cs) on top of the C ABI: same static-method names and
argument meaning; each direction is one ``snb200_sdpa_*`` call (strided-batched GEMMs + one fused
mask/softmax pass)."""
from ._capi import check
from .tensor import GPUTensor


def ScaledDotProductAttentionForwardPropagation(Q, K, V, y, isTraining, weights_buffer, use_scale, is_causal):
    """weights = softmax(mask(scale * Q K^T)); y = weights V   (ScaledDotProductAttentionLayer.cs:46-91).
    ``weights_buffer`` is the [batch, q_steps, v_steps] tensor the layer keeps for the backward pass; it is
    returned (allocated here when None)."""
    if V.Shape != K.Shape:
        raise ValueError(f"V.Shape and K.Shape must be equal, but are {V.Shape} and {K.Shape}")
    if V.Shape[0] != Q.Shape[0] or Q.Shape[2] != V.Shape[2]:
        raise ValueError("queries and values must share the batch size and the embedding dim")
    batch, Tq, E = Q.Shape
    Tk = V.Shape[1]
    if y.Shape != [batch, Tq, E]:
        raise ValueError("y must be [batch, query_timeSteps, embedding_dim]")
    w = y.wrapper
    if weights_buffer is None:
        weights_buffer = GPUTensor((batch, Tq, Tk), None, w)
    st = w.lib.snb200_sdpa_fwd(w.handle, batch, Tq, Tk, E, int(bool(use_scale)), int(bool(is_causal)), Q.Pointer,
                               K.Pointer, V.Pointer, weights_buffer.Pointer, y.Pointer)
    check(w.handle, st)
    return weights_buffer


def ScaledDotProductAttentionBackwardPropagation(dQ, dK, dV, Q, K, V, dy, weights_buffer, use_scale,
                                                 scores_gradients_buffer=None):
    """dV, dQ, dK from dy and the weights kept by the forward pass   (ScaledDotProductAttentionLayer.cs:108-129)."""
    batch, Tq, E = Q.Shape
    Tk = V.Shape[1]
    w = dy.wrapper
    if scores_gradients_buffer is None:
        scores_gradients_buffer = GPUTensor((batch, Tq, Tk), None, w)
    st = w.lib.snb200_sdpa_bwd(w.handle, batch, Tq, Tk, E, int(bool(use_scale)), Q.Pointer, K.Pointer, V.Pointer,
                               dy.Pointer, weights_buffer.Pointer, scores_gradients_buffer.Pointer, dQ.Pointer,
                               dK.Pointer, dV.Pointer)
    check(w.handle, st)
