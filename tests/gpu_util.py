"""Helpers shared by the GPU parity tests: run one call through the C ABI (via the GPUTensor
mirror) and the same call through the CPU oracle on identical seeded inputs."""
import numpy as np

from oracle import sharpnet_oracle as orc
from sharpnet_b200.tensor import GPUTensor

TOL_3XTF32 = 1e-5   # max |err| / (sqrt(K) * a_max * b_max), 3xTF32 and SIMT fp32 modes
TOL_TF32 = 2e-3     # same measure, TF32 mode


def stored_shape(rows, cols, transposed):
    return (cols, rows) if transposed else (rows, cols)


def run_dot(w, M, N, K, tA, tB, alpha, beta, seed, lo=-1.0, hi=1.0, batch=None):
    """Returns (gpu_result, mkl_result, f64_result) for one Dot / BatchMatrixMultiplication."""
    rng = np.random.default_rng(seed)
    nb = batch or 1
    a = rng.uniform(lo, hi, (nb,) + stored_shape(M, K, tA)).astype(np.float32)
    b = rng.uniform(lo, hi, (nb,) + stored_shape(K, N, tB)).astype(np.float32)
    c = rng.uniform(lo, hi, (nb, M, N)).astype(np.float32)
    if batch is None:
        A, B, C = GPUTensor(a.shape[1:], a, w), GPUTensor(b.shape[1:], b, w), GPUTensor((M, N), c, w)
        C.Dot(A, tA, B, tB, alpha, beta)
    else:
        A, B, C = GPUTensor(a.shape, a, w), GPUTensor(b.shape, b, w), GPUTensor(c.shape, c, w)
        C.BatchMatrixMultiplication(A, tA, B, tB, alpha, beta)
    w.check_device_status()
    got = C.ContentAsFloatArray().reshape(nb, M, N)
    f64 = orc.batch_matrix_multiplication(a, tA, b, tB, c, alpha, beta, f64=True)
    mkl = orc.batch_matrix_multiplication(a, tA, b, tB, c.copy(), alpha, beta)
    return got, mkl, f64
