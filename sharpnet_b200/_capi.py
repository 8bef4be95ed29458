"""ctypes binding of libsharpnet_b200.so: one Python function per entry point of
include/sharpnet_b200.h, with the same argument order.  This is the Python twin of the C#
P/Invoke class a SharpNet maintainer adds (one ``[DllImport("sharpnet_b200")]`` per function).

There is no fallback: if the library has not been built, importing it raises.
"""
import ctypes
import os

from .build import LIB_PATH

STATUS_NAMES = {
    0: "SUCCESS", 1: "NOT_INITIALIZED", 3: "ALLOC_FAILED", 7: "INVALID_VALUE", 8: "ARCH_MISMATCH",
    13: "EXECUTION_FAILED", 14: "INTERNAL_ERROR", 15: "NOT_SUPPORTED",
}
MATH_3XTF32, MATH_TF32, MATH_FP32_SIMT, MATH_TF32_BF16X2 = 0, 1, 2, 3
ACT_SIGMOID, ACT_RELU, ACT_TANH, ACT_IDENTITY, ACT_SWISH = 0, 1, 2, 5, 6
ACT_ELU, ACT_LEAKY_RELU = 4, 1002   # take a coefficient: snb200_set_activation_parameter
ACT_LN = 1004
ACT_CLIPPED_RELU = 3                # ceiling 1.0, as the reference's cuDNN descriptors have it
ACT_SOFTMAX = 1000   # snb200_dense_fwd only
W_OUT_IN, W_IN_OUT = 0, 1
LOSS_BINARY_CROSSENTROPY, LOSS_CATEGORICAL_CROSSENTROPY, LOSS_MSE = 0, 1, 2
(TUNE_FORCE_PATH, TUNE_FORCE_BN, TUNE_REWRITE_HI, TUNE_CHUNK_K, TUNE_PAIR, TUNE_SPLITK, TUNE_VARIANT, TUNE_PDL,
 TUNE_FORCE_SPLITS, TUNE_NO_TS, TUNE_NO_FUSED_ATTN, TUNE_NO_SWLOAD, TUNE_SM_RESERVE, TUNE_CLUSTER) = range(14)

_c = ctypes
_H = _c.c_void_p
_F = _c.c_float
_I = _c.c_int
_L = _c.c_longlong
_P = _c.c_void_p



class MhaDesc(_c.Structure):        # snb200_mha_desc
    _fields_ = [(n, _I) for n in ("w_layout", "batch", "q_steps", "v_steps", "embed_dim", "num_heads", "key_dim",
                                  "value_dim", "is_causal")]


class MhaWeights(_c.Structure):     # snb200_mha_weights and snb200_mha_gradients (same field order)
    _fields_ = [(n, _P) for n in ("w_Q", "w_K", "w_V", "out_proj_weight", "w_Q_bias", "w_K_bias", "w_V_bias",
                                  "out_proj_bias")]


class MhaState(_c.Structure):       # snb200_mha_state
    _fields_ = [(n, _P) for n in ("Q_heads_T", "K_heads_T", "V_heads_T", "attention_heads_T", "weights_buffer")]


# name -> (restype, argtypes); every symbol include/sharpnet_b200.h declares.
SIGNATURES = {
    "snb200_create": (_I, [_c.POINTER(_H), _I]),
    "snb200_destroy": (_I, [_H]),
    "snb200_set_stream": (_I, [_H, _P]),
    "snb200_set_math_mode": (_I, [_H, _I]),
    "snb200_set_activation_parameter": (_I, [_H, _F]),
    "snb200_get_math_mode": (_I, [_H, _c.POINTER(_I)]),
    "snb200_set_tuning": (_I, [_H, _I, _I]),
    "snb200_last_error_string": (_c.c_char_p, [_H]),
    "snb200_check_device_status": (_I, [_H]),
    "snb200_get_launch_count": (_I, [_H, _c.POINTER(_L)]),
    "snb200_get_last_kernel": (_I, [_H, _c.c_char_p, _I]),
    "snb200_get_version": (_I, []),
    "snb200_gemm_timing_begin": (_I, [_H]),
    "snb200_gemm_timing_end": (_I, [_H, _c.POINTER(_c.c_double), _c.POINTER(_I)]),
    "snb200_gemm": (_I, [_H, _I, _I, _I, _I, _I, _I, _F, _P, _P, _F, _P]),
    "snb200_batched_gemm": (_I, [_H, _I, _I, _I, _I, _L, _I, _I, _L, _L, _I, _F, _P, _P, _F, _P]),
    "snb200_dense_fwd": (_I, [_H, _I, _I, _I, _I, _P, _P, _P, _I, _P, _P]),
    "snb200_dense_bwd": (_I, [_H, _I, _I, _I, _I, _P, _P, _P, _I, _P, _P, _F, _P, _P, _P, _P]),
    "snb200_dense_bwd_weight_rows": (_I, [_H, _I, _I, _I, _I, _P, _P, _F, _I, _I, _P]),
    "snb200_loss_gradient": (_I, [_H, _I, _I, _I, _P, _P, _P]),
    "snb200_dense_bwd_from_loss": (_I, [_H, _I, _I, _I, _I, _P, _P, _I, _P, _P, _F, _P, _P, _P, _P]),
    "snb200_bias_add": (_I, [_H, _I, _I, _P, _P]),
    "snb200_bias_grad": (_I, [_H, _I, _I, _P, _P]),
    "snb200_bias_grad_noalloc": (_I, [_I, _P, _I, _I, _P, _P, _c.c_char_p, _I]),
    "snb200_activation_fwd": (_I, [_H, _I, _L, _P, _P]),
    "snb200_activation_bwd": (_I, [_H, _I, _L, _P, _P, _P, _P]),
    "snb200_axpy": (_I, [_H, _L, _F, _P, _P]),
    "snb200_softmax_fwd": (_I, [_H, _L, _I, _P, _P]),
    "snb200_softmax_bwd": (_I, [_H, _L, _I, _P, _P, _P]),
    "snb200_sdpa_fwd": (_I, [_H, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P]),
    "snb200_sdpa_bwd": (_I, [_H, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "snb200_transpose_second_third": (_I, [_H, _I, _I, _I, _I, _P, _P]),
    "snb200_mha_scratch_floats": (_L, [_c.POINTER(MhaDesc), _I]),
    "snb200_mha_fwd": (_I, [_H, _c.POINTER(MhaDesc), _c.POINTER(MhaWeights), _P, _P, _P, _c.POINTER(MhaState), _P, _P]),
    "snb200_mha_bwd": (_I, [_H, _c.POINTER(MhaDesc), _c.POINTER(MhaWeights), _P, _P, _P, _P, _c.POINTER(MhaState), _F, _P,
                           _c.POINTER(MhaWeights), _P, _P, _P]),
    "snb200_sgd_update": (_I, [_H, _L, _F, _F, _I, _P, _P, _P]),
    "snb200_adam_update": (_I, [_H, _L, _c.c_double, _c.c_double, _c.c_double, _c.c_double, _c.c_double, _I, _P, _P, _P, _P]),
    "snb200_comm_get_unique_id": (_I, [_P]),
    "snb200_comm_init_rank": (_I, [_H, _I, _I, _P]),
    "snb200_comm_init_all": (_I, [_c.POINTER(_H), _I]),
    "snb200_allreduce_sum": (_I, [_H, _P, _L]),
    "snb200_allreduce_sum_group": (_I, [_H, _I, _c.POINTER(_P), _c.POINTER(_L)]),
    "snb200_comm_destroy": (_I, [_H]),
    "snb200_selftest_wait_timeout": (_I, [_H, _I]),
    "snb200_stager_create": (_I, [_H, _I, _c.POINTER(_P)]),
    "snb200_stager_destroy": (_I, [_P]),
    "snb200_stager_issue": (_I, [_P, _I, _I, _c.POINTER(_P), _c.POINTER(_P), _c.POINTER(_L)]),
    "snb200_stager_acquire": (_I, [_P, _I]),
    "snb200_stager_acquire_part": (_I, [_P, _I, _I]),
    "snb200_stager_release": (_I, [_P, _I]),
    "snb200_host_pin": (_I, [_P, _L]),
    "snb200_host_unpin": (_I, [_P]),
}

_lib = None


def load():
    """Loads the shared library (once) and declares the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m sharpnet_b200.build` "
            "(there is no CPU or PyTorch fallback for this library)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class SharpNetB200Error(Exception):
    """Raised when an entry point returns a non-zero status, like GPUWrapper.CheckStatus
    (Prod/GPU/GPUWrapper.cs:662-668) throws on a cuBLAS status."""

    def __init__(self, status, message):
        self.status = status
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")


def check(handle, status):
    if status != 0:
        msg = load().snb200_last_error_string(handle)
        raise SharpNetB200Error(status, msg.decode() if msg else "")
