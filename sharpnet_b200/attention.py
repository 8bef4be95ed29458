"""Host-side mirror of SharpNet's attention layers on top of the C ABI.

``ScaledDotProductAttention*Propagation`` (Prod/Layers/ScaledDotProductAttentionLayer.cs): same static-method
names and argument meaning; each direction is one ``snb200_sdpa_*`` call (strided-batched GEMMs + one fused
mask/softmax pass).  ``MultiheadAttention`` (Prod/Layers/MultiheadAttention.cs): the four Dense projections,
the head split / merge permutations and the attention core, in the reference's call order, behind one
``snb200_mha_fwd`` / ``snb200_mha_bwd`` call each."""

from . import _capi
from ._capi import W_OUT_IN, check
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


class MultiheadAttention:
    """Multi-head attention over Q [batch, q_steps, embed] and K, V [batch, v_steps, embed]
    (Prod/Layers/MultiheadAttention.cs:24-295).

    Parameters live in one weights tensor [2*heads*key_dim + 2*heads*value_dim, embed] and one bias vector, sliced
    into w_Q, w_K, w_V, out_proj_weight and their biases as the layer does (:37-50,137-140).  ``w_layout`` selects
    [out, in] rows (the layer's own form, Linear.cs:125-132) or the [in, out] form of the Keras-derived goldens.
    Forward keeps the per-head Q, K, V, the attention weights and the merged heads for the backward pass."""

    def __init__(self, num_heads, key_dim, value_dim, use_bias_Q_K_V, use_bias_O, is_causal, embed_dim, wrapper,
                 w_layout=W_OUT_IN):
        if num_heads * value_dim != embed_dim:
            # out_proj_weight is declared [heads*value_dim, embed] and used as [embed, heads*value_dim] (:121-126,236)
            raise ValueError("num_heads * value_dim must equal the embedding dimension")
        self.num_heads, self.key_dim, self.value_dim = num_heads, key_dim, value_dim
        self.is_causal, self.embed_dim, self.layout, self.w = bool(is_causal), embed_dim, w_layout, wrapper
        outs = [num_heads * key_dim, num_heads * key_dim, num_heads * value_dim, embed_dim]
        ins = [embed_dim, embed_dim, embed_dim, num_heads * value_dim]
        self._w_shapes = [(o, i) if w_layout == W_OUT_IN else (i, o) for o, i in zip(outs, ins)]
        self._w_counts = [o * i for o, i in zip(outs, ins)]
        self._b_counts = [o if use else 0 for o, use in zip(outs, (use_bias_Q_K_V,) * 3 + (use_bias_O,))]
        self.Weights = GPUTensor((sum(self._w_counts) // embed_dim, embed_dim), None, wrapper)
        self.WeightGradients = GPUTensor(self.Weights.Shape, None, wrapper)
        nb = sum(self._b_counts)
        self.Bias = GPUTensor((nb,), None, wrapper) if nb else None
        self.BiasGradients = GPUTensor((nb,), None, wrapper) if nb else None
        self._cache = None

    # -- slices of the parameter tensors (Prod/Layers/MultiheadAttention.cs:344-376) -------------
    def _w(self, t, i):
        return t.Slice(sum(self._w_counts[:i]), self._w_shapes[i])

    def _b(self, t, i):
        if t is None or self._b_counts[i] == 0:
            return None
        return t.Slice(sum(self._b_counts[:i]), (self._b_counts[i],))

    w_Q = property(lambda self: self._w(self.Weights, 0))
    w_K = property(lambda self: self._w(self.Weights, 1))
    w_V = property(lambda self: self._w(self.Weights, 2))
    out_proj_weight = property(lambda self: self._w(self.Weights, 3))
    w_Q_bias = property(lambda self: self._b(self.Bias, 0))
    w_K_bias = property(lambda self: self._b(self.Bias, 1))
    w_V_bias = property(lambda self: self._b(self.Bias, 2))
    out_proj_bias = property(lambda self: self._b(self.Bias, 3))

    def gradients(self):
        """([dw_Q, dw_K, dw_V, d_out_proj_weight], [db_Q, db_K, db_V, db_O]) as views of the gradient tensors."""
        return ([self._w(self.WeightGradients, i) for i in range(4)],
                [self._b(self.BiasGradients, i) for i in range(4)])

    def _desc(self, B, Tq, Tk):
        return _capi.MhaDesc(self.layout, B, Tq, Tk, self.embed_dim, self.num_heads, self.key_dim, self.value_dim,
                             int(self.is_causal))

    @staticmethod
    def _ptrs(struct, tensors):
        return struct(*[None if t is None else t.Pointer for t in tensors])

    def ForwardPropagation(self, allX, y, isTraining=True):
        """One ``snb200_mha_fwd`` call: projections, head split, attention, head merge, output projection
        (Prod/Layers/MultiheadAttention.cs:178-238)."""
        Q, K, V = allX
        if V.Shape != K.Shape:
            raise ValueError(f"V.Shape and K.Shape must be equal, but are {V.Shape} and {K.Shape}")
        if Q.Shape[2] != V.Shape[2]:
            raise ValueError("queries.Shape[2] and values.Shape[2] must be equal (same embedding dim)")
        B, Tq, E = Q.Shape
        Tk = V.Shape[1]
        if y.Shape != [B, Tq, E]:
            raise ValueError("y must be [batch, query_timeSteps, embed_dim]")
        H, kd, vd = self.num_heads, self.key_dim, self.value_dim
        w = self.w
        desc = self._desc(B, Tq, Tk)
        state = [GPUTensor(s, None, w) for s in ((B * H, Tq, kd), (B * H, Tk, kd), (B * H, Tk, vd), (B, Tq, H * vd),
                                                 (B * H, Tq, Tk))]
        weights = self._ptrs(_capi.MhaWeights, [self._w(self.Weights, i) for i in range(4)] +
                             [self._b(self.Bias, i) for i in range(4)])
        check(w.handle, w.lib.snb200_mha_fwd(w.handle, desc, weights, Q.Pointer, K.Pointer, V.Pointer,
                                             self._ptrs(_capi.MhaState, state), None, y.Pointer))
        self._cache = state if isTraining else None

    def BackwardPropagation(self, allX, dy, allDx, multiplier=1.0):
        """One ``snb200_mha_bwd`` call (Prod/Layers/MultiheadAttention.cs:240-295); ``multiplier`` is the dW factor of
        Linear.cs:152-158."""
        Q, K, V = allX
        dQ, dK, dV = allDx
        B, Tq, _ = Q.Shape
        Tk = V.Shape[1]
        w = self.w
        desc = self._desc(B, Tq, Tk)
        scratch = GPUTensor((w.lib.snb200_mha_scratch_floats(desc, 1),), None, w)
        weights = self._ptrs(_capi.MhaWeights, [self._w(self.Weights, i) for i in range(4)] +
                             [self._b(self.Bias, i) for i in range(4)])
        dws, dbs = self.gradients()
        check(w.handle, w.lib.snb200_mha_bwd(w.handle, desc, weights, Q.Pointer, K.Pointer, V.Pointer, dy.Pointer,
                                             self._ptrs(_capi.MhaState, self._cache), float(multiplier), scratch.Pointer,
                                             self._ptrs(_capi.MhaWeights, dws + dbs), dQ.Pointer, dK.Pointer, dV.Pointer))
        self._cache = None
