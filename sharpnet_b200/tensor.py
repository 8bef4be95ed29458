"""Host-side mirror of SharpNet's GPU tensor for the matrix-multiply path.

``GPUTensor`` keeps the method names, argument order and meaning of ``SharpNet.GPU.GPUTensor<float>``
(Prod/GPU/GpuTensor.cs) for the members on the path -- ``Dot``, ``BatchMatrixMultiplication``,
``BroadcastAddVectorToOutput``, ``Compute_BiasGradient_from_dy``, ``ActivationForward``,
``ActivationBackward``, ``Update_Adding_Alpha_X`` -- and forwards each of them to the C ABI of
libsharpnet_b200.so exactly as the C# P/Invoke shim does.  PyTorch is used only to own device
memory; no arithmetic happens in PyTorch or on the host.
"""
import ctypes

import numpy as np
import torch

from . import _capi
from ._capi import (ACT_IDENTITY, ACT_RELU, ACT_SIGMOID, ACT_SWISH, ACT_TANH, MATH_3XTF32, MATH_FP32_SIMT,  # noqa: F401
                    MATH_TF32, SharpNetB200Error, check)


class GPUWrapper:
    """Per-device owner of the library handle (the role of Prod/GPU/GPUWrapper.cs:99-160:
    one cached wrapper per device id holding the cuBLAS/cuDNN handles)."""

    _cache = {}

    def __init__(self, device_id=0):
        if not torch.cuda.is_available():
            raise RuntimeError("sharpnet_b200 needs a CUDA device: there is no CPU path")
        self.lib = _capi.load()
        self.device_id = device_id
        self.device = torch.device("cuda", device_id)
        h = ctypes.c_void_p()
        st = self.lib.snb200_create(ctypes.byref(h), device_id)
        if st != 0:
            raise SharpNetB200Error(st, f"snb200_create(device {device_id}) failed")
        self.handle = h

    @classmethod
    def FromDeviceId(cls, device_id=0):
        if device_id not in cls._cache:
            cls._cache[device_id] = cls(device_id)
        return cls._cache[device_id]

    # -- knobs -------------------------------------------------------------------------------
    def set_math_mode(self, mode):
        check(self.handle, self.lib.snb200_set_math_mode(self.handle, mode))

    def set_activation_parameter(self, alpha):
        """Coefficient of the ELU / LeakyRelu calls that follow (the layer's activationParameter)."""
        check(self.handle, self.lib.snb200_set_activation_parameter(self.handle, float(alpha)))

    def get_math_mode(self):
        m = ctypes.c_int()
        check(self.handle, self.lib.snb200_get_math_mode(self.handle, ctypes.byref(m)))
        return m.value

    def set_tuning(self, key, value):
        check(self.handle, self.lib.snb200_set_tuning(self.handle, key, value))

    def set_stream(self, stream):
        ptr = None if stream is None else ctypes.c_void_p(stream.cuda_stream)
        check(self.handle, self.lib.snb200_set_stream(self.handle, ptr))

    def last_kernel(self):
        buf = ctypes.create_string_buffer(64)
        check(self.handle, self.lib.snb200_get_last_kernel(self.handle, buf, 64))
        return buf.value.decode()

    def launch_count(self):
        c = ctypes.c_longlong()
        check(self.handle, self.lib.snb200_get_launch_count(self.handle, ctypes.byref(c)))
        return c.value

    def check_device_status(self):
        check(self.handle, self.lib.snb200_check_device_status(self.handle))

    def gemm_timing_begin(self):
        """Starts recording a CUDA-event pair around every matrix product this handle launches."""
        check(self.handle, self.lib.snb200_gemm_timing_begin(self.handle))

    def gemm_timing_end(self):
        """Waits for the stream; returns (device milliseconds spent in matrix products, how many)."""
        ms, n = ctypes.c_double(), ctypes.c_int()
        check(self.handle, self.lib.snb200_gemm_timing_end(self.handle, ctypes.byref(ms), ctypes.byref(n)))
        return ms.value, n.value

    def Dispose(self):
        if self.handle is not None:
            self.lib.snb200_destroy(self.handle)
            self.handle = None
            if GPUWrapper._cache.get(self.device_id) is self:
                del GPUWrapper._cache[self.device_id]


def _reference_coefficient(activationType, activationParameter):
    """The coefficient SharpNet itself would run this activation with: 1 for ELU, the layer's parameter otherwise."""
    return 1.0 if int(activationType) == _capi.ACT_ELU else activationParameter


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


class GPUTensor:
    """fp32 tensor of up to 4 dimensions living in device memory (Prod/GPU/GpuTensor.cs)."""

    def __init__(self, shape, data=None, wrapper=None, storage=None):
        self.wrapper = wrapper or GPUWrapper.FromDeviceId(0)
        self.Shape = [int(s) for s in shape]
        count = int(np.prod(self.Shape)) if self.Shape else 1
        if storage is not None:
            assert storage.dtype == torch.float32 and storage.is_cuda and storage.is_contiguous()
            assert storage.numel() >= count
            self.storage = storage
        elif data is not None:
            host = np.ascontiguousarray(np.asarray(data, dtype=np.float32)).reshape(-1)
            assert host.size == count, "data does not match the shape"
            self.storage = torch.from_numpy(host).to(self.wrapper.device)
        else:
            self.storage = torch.zeros(max(count, 1), dtype=torch.float32, device=self.wrapper.device)

    # -- shape helpers (Prod/Data/Tensor.cs:189,1521-1526,1645-1654) --------------------------
    @property
    def Count(self):
        return int(np.prod(self.Shape)) if self.Shape else 1

    @property
    def MultDim0(self):
        return int(np.prod(self.Shape[1:])) if len(self.Shape) > 1 else 1

    @property
    def Dimension(self):
        return len(self.Shape)

    def Reshape(self, *shape):
        shape = list(shape)
        if -1 in shape:
            known = int(np.prod([s for s in shape if s != -1]))
            shape[shape.index(-1)] = self.Count // known
        assert int(np.prod(shape)) == self.Count
        return GPUTensor(shape, wrapper=self.wrapper, storage=self.storage)

    def As2DTensor(self, flattenInputTensorOnLastDimension=False):
        if len(self.Shape) == 2:
            return self
        if flattenInputTensorOnLastDimension:
            return self.Reshape(-1, self.Shape[-1])
        return self.Reshape(self.Shape[0], -1)

    def Slice(self, startIndex, sliceShape):
        """A view of ``Count(sliceShape)`` elements starting at element ``startIndex``, sharing this tensor's memory
        (Prod/GPU/GpuTensor.cs:606-620)."""
        count = int(np.prod(sliceShape))
        assert 0 <= startIndex and startIndex + count <= self.storage.numel()
        return GPUTensor(sliceShape, wrapper=self.wrapper, storage=self.storage[startIndex:startIndex + count])

    def TransposeSecondAndThirdDimension(self, target):
        """target[a, c, b, :] = this[a, b, c, :]; ``target`` takes the permuted shape
        (Prod/GPU/GpuTensor.cs:672-684, Prod/CPU/CpuTensor.cs:301-322)."""
        assert len(self.Shape) >= 3 and target.Count == self.Count
        A, B, C = self.Shape[:3]
        D = self.Count // (A * B * C) if A * B * C else 0
        target.Shape = [A, C, B] + self.Shape[3:]
        w = self.wrapper
        check(w.handle, w.lib.snb200_transpose_second_third(w.handle, A, B, C, D, self.Pointer, target.Pointer))

    def ZeroMemory(self):
        self.storage[: self.Count].zero_()

    def ContentAsFloatArray(self):
        return self.storage[: self.Count].cpu().numpy().reshape(self.Shape)

    @property
    def Pointer(self):
        return _ptr(self.storage)

    # -- the hot path -------------------------------------------------------------------------
    def Dot(self, a, transposeA=False, b=None, transposeB=False, alpha=1.0, beta=0.0):
        """this = alpha * op(a) * op(b) + beta * this   (Prod/Data/Tensor.cs:388-397;
        GPU: Prod/GPU/GpuTensor.cs:1196-1227).  ``Dot(a, b)`` is the convenience form of Tensor.cs:60."""
        if isinstance(transposeA, GPUTensor):   # Dot(a, b)
            b, transposeA = transposeA, False
        if b is None:
            raise TypeError("Dot needs two operands")
        w = self.wrapper
        st = w.lib.snb200_gemm(w.handle, int(bool(transposeA)), int(bool(transposeB)), a.Shape[0], a.MultDim0,
                               b.Shape[0], b.MultDim0, float(alpha), a.Pointer, b.Pointer, float(beta), self.Pointer)
        check(w.handle, st)

    def BatchMatrixMultiplication(self, a_3D, transposeA, b_3D, transposeB, alpha, beta):
        """this[i] = alpha * op(a[i]) * op(b[i]) + beta * this[i]   (Prod/Data/Tensor.cs:400-415;
        GPU: Prod/GPU/GpuTensor.cs:1163-1194)."""
        assert len(a_3D.Shape) == 3 and len(b_3D.Shape) == 3 and len(self.Shape) == 3
        assert a_3D.Shape[0] == b_3D.Shape[0] == self.Shape[0]
        w = self.wrapper
        st = w.lib.snb200_batched_gemm(
            w.handle, int(bool(transposeA)), int(bool(transposeB)), a_3D.Shape[1], a_3D.Shape[2], a_3D.MultDim0,
            b_3D.Shape[1], b_3D.Shape[2], b_3D.MultDim0, self.MultDim0, a_3D.Shape[0], float(alpha), a_3D.Pointer,
            b_3D.Pointer, float(beta), self.Pointer)
        check(w.handle, st)

    def BroadcastAddVectorToOutput(self, y):
        """y[m, :] += this  -- called on the bias (Prod/Data/Tensor.cs:495, Prod/GPU/GpuTensor.cs:633-644)."""
        assert y.MultDim0 == self.Count
        w = self.wrapper
        check(w.handle, w.lib.snb200_bias_add(w.handle, y.Shape[0], y.MultDim0, self.Pointer, y.Pointer))

    def Compute_BiasGradient_from_dy(self, biasGradient_1D):
        """biasGradient[n] = sum_m this[m, n]  -- called on dy (Prod/Data/Tensor.cs:710,
        Prod/GPU/GpuTensor.cs:686-701)."""
        assert biasGradient_1D.Count == self.MultDim0
        w = self.wrapper
        check(w.handle, w.lib.snb200_bias_grad(w.handle, self.Shape[0], self.MultDim0, self.Pointer,
                                               biasGradient_1D.Pointer))

    def ActivationForward(self, activationType, activationParameter, y):
        """y = act(this)   (Prod/Data/Tensor.cs:618, Prod/GPU/GpuTensor.cs:397-443).  ``activationParameter``: the
        coefficient of LeakyRelu (a number here, a one-element tensor in SharpNet).  ELU runs with coefficient 1
        whatever the parameter says, as in SharpNet (Prod/CPU/CpuTensor.cs:954; the cuDNN descriptor of
        Prod/GPU/GPUWrapper.cs:183)."""
        w = self.wrapper
        activationParameter = _reference_coefficient(activationType, activationParameter)
        if activationParameter is not None:
            w.set_activation_parameter(activationParameter)
        check(w.handle, w.lib.snb200_activation_fwd(w.handle, int(activationType), self.Count, self.Pointer, y.Pointer))

    def ActivationBackward(self, activationType, activationParameter, dy, x, y):
        """this = dx = act'(x, y) * dy   (Prod/Data/Tensor.cs:628, Prod/GPU/GpuTensor.cs:445-490)."""
        w = self.wrapper
        activationParameter = _reference_coefficient(activationType, activationParameter)   # ELU: 1 (CpuTensor.cs:1000)
        if activationParameter is not None:
            w.set_activation_parameter(activationParameter)
        check(w.handle, w.lib.snb200_activation_bwd(
            w.handle, int(activationType), self.Count, dy.Pointer, None if x is None else x.Pointer,
            None if y is None else y.Pointer, self.Pointer))

    def Update_Adding_Alpha_X(self, alpha, x):
        """this += alpha * x   (Prod/Data/Tensor.cs:555, Prod/GPU/GpuTensor.cs:1359-1362)."""
        assert x.Count == self.Count
        w = self.wrapper
        check(w.handle, w.lib.snb200_axpy(w.handle, self.Count, float(alpha), x.Pointer, self.Pointer))

    def UpdateSGDOptimizer(self, learningRate, momentum, nesterov, dW, velocity):
        """this = W: SGD with momentum   (Prod/GPU/GpuTensor.cs:1147-1161, Prod/CPU/CpuTensor.cs:470-489).
        ``velocity`` None gives the VanillaSgd update W -= learningRate * dW."""
        w = self.wrapper
        check(w.handle, w.lib.snb200_sgd_update(w.handle, self.Count, float(learningRate), float(momentum),
                                                int(bool(nesterov)), dW.Pointer, self.Pointer,
                                                None if velocity is None else velocity.Pointer))

    def UpdateAdamOptimizer(self, learningRate, beta1, beta2, epsilon, weight_decay, dW, adam_vW, adam_sW, timeStep):
        """this = W: Adam / AdamW   (Prod/GPU/GpuTensor.cs:1136-1145, Prod/CPU/CpuTensor.cs:1755-1769)."""
        w = self.wrapper
        check(w.handle, w.lib.snb200_adam_update(w.handle, self.Count, float(learningRate), float(beta1), float(beta2),
                                                 float(epsilon), float(weight_decay), int(timeStep), dW.Pointer,
                                                 self.Pointer, adam_vW.Pointer, adam_sW.Pointer))

    def ComputeGradientForEvaluationMetric(self, yExpected, yPredicted, loss):
        """this = dyPredicted = scale * (yPredicted - yExpected) for BinaryCrossentropy, CategoricalCrossentropy
        and Mse (Prod/Data/Tensor.cs:1182-1217); ``loss`` is one of the LOSS_* constants."""
        w = self.wrapper
        check(w.handle, w.lib.snb200_loss_gradient(w.handle, int(loss), self.Shape[0], self.MultDim0, yExpected.Pointer,
                                                   yPredicted.Pointer, self.Pointer))

    def SoftmaxLastDimension(self, y):
        """y = softmax(this) over the last dimension (ActivationForward with
        CUDNN_ACTIVATION_SOFTMAX_LAST_DIMENSION, Prod/GPU/GpuTensor.cs:411-413)."""
        w = self.wrapper
        cols = self.Shape[-1]
        check(w.handle, w.lib.snb200_softmax_fwd(w.handle, self.Count // cols, cols, self.Pointer, y.Pointer))

    def SoftmaxGradientLastDimension(self, dy, y):
        """this = dx = y * (dy - sum(dy * y)) over the last dimension (cudnnSoftmaxBackward, Prod/GPU/GpuTensor.cs:445-490)."""
        w = self.wrapper
        cols = self.Shape[-1]
        check(w.handle, w.lib.snb200_softmax_bwd(w.handle, self.Count // cols, cols, dy.Pointer, y.Pointer, self.Pointer))
