"""Parity of snb200_gemm / snb200_batched_gemm (through the GPUTensor mirror of Tensor.Dot and
Tensor.BatchMatrixMultiplication) against the CPU oracle, on a B200."""
import numpy as np
import pytest

from oracle import sharpnet_oracle as orc
from sharpnet_b200 import MATH_3XTF32, MATH_FP32_SIMT, MATH_TF32
from sharpnet_b200._capi import TUNE_CLUSTER, TUNE_FORCE_BN, TUNE_FORCE_PATH, TUNE_PAIR, SharpNetB200Error
from sharpnet_b200.tensor import GPUTensor

from gpu_util import TOL_3XTF32, TOL_TF32, run_dot

pytestmark = pytest.mark.gpu

MODES = [(MATH_3XTF32, TOL_3XTF32), (MATH_TF32, TOL_TF32), (MATH_FP32_SIMT, TOL_3XTF32)]


@pytest.fixture(autouse=True)
def _reset(wrapper):
    wrapper.set_math_mode(MATH_3XTF32)
    wrapper.set_tuning(TUNE_FORCE_PATH, 0)
    wrapper.set_tuning(TUNE_FORCE_BN, 0)
    wrapper.set_tuning(TUNE_PAIR, 0)
    wrapper.set_tuning(TUNE_CLUSTER, 0)
    yield
    wrapper.set_math_mode(MATH_3XTF32)
    wrapper.set_tuning(TUNE_FORCE_PATH, 0)
    wrapper.set_tuning(TUNE_FORCE_BN, 0)
    wrapper.set_tuning(TUNE_PAIR, 0)
    wrapper.set_tuning(TUNE_CLUSTER, 0)


def _check(w, M, N, K, tA, tB, alpha, beta, seed, tol, lo=-1.0, hi=1.0, batch=None):
    got, mkl, f64 = run_dot(w, M, N, K, tA, tB, alpha, beta, seed, lo, hi, batch)
    amax = max(abs(lo), abs(hi))
    scale = abs(alpha) if alpha != 0 else 1.0
    e64 = orc.scaled_error(got, f64, K, amax, amax) / scale
    emkl = orc.scaled_error(got, mkl, K, amax, amax) / scale
    assert e64 <= tol and emkl <= tol, (w.last_kernel(), M, N, K, tA, tB, e64, emkl)
    return e64


def test_reference_exact_cases(wrapper, golden):
    # Tests/GPU/TestGpuTensor.cs:50-120 -- small integer matrices, tolerance 1e-9, every math mode
    for mode, _ in MODES:
        wrapper.set_math_mode(mode)
        for case in golden["dot_exact"]:
            a = GPUTensor(case["a_shape"], case["a"], wrapper)
            b = GPUTensor(case["b_shape"], case["b"], wrapper)
            r = GPUTensor(case["expected_shape"], None, wrapper)
            r.Dot(a, False, b, False, 1, 0)
            np.testing.assert_allclose(r.ContentAsFloatArray().ravel(), case["expected"], rtol=0, atol=1e-9)
        for case in golden["dot_exact_zero_cases"]:
            a = GPUTensor(case["a_shape"], None, wrapper)
            b = GPUTensor(case["b_shape"], None, wrapper)
            r = GPUTensor(case["expected_shape"], np.ones(case["expected_shape"], np.float32), wrapper)
            r.Dot(a, False, b, False, 1, 0)
            assert not r.ContentAsFloatArray().any()


def test_integer_matrices_are_exact_on_tensor_cores(wrapper):
    # Small integers are exactly representable in TF32: the tensor-core paths must be bit exact.
    rng = np.random.default_rng(0)
    a = rng.integers(-8, 9, (128, 64)).astype(np.float32)
    b = rng.integers(-8, 9, (64, 96)).astype(np.float32)
    want = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)
    wrapper.set_tuning(TUNE_FORCE_PATH, 1)
    for mode in (MATH_3XTF32, MATH_TF32):
        wrapper.set_math_mode(mode)
        A, B, C = GPUTensor(a.shape, a, wrapper), GPUTensor(b.shape, b, wrapper), GPUTensor((128, 96), None, wrapper)
        C.Dot(A, B)
        assert wrapper.last_kernel().startswith("umma")
        np.testing.assert_array_equal(C.ContentAsFloatArray(), want)


def test_differential_cases_of_the_reference(wrapper):
    # Tests/TestParallelRunCpuVersusGpu.cs:368-375,436-456: 8x10 * 10x12 and 2x20000 * 20000x2,
    # U[-1.5, 1.5); the reference accepts an absolute error of 1e-2, we hold the scaled bound.
    for mode, tol in MODES:
        wrapper.set_math_mode(mode)
        _check(wrapper, 8, 12, 10, False, False, 1, 0, 1, tol, -1.5, 1.5)
        _check(wrapper, 2, 2, 20000, False, False, 1, 0, 2, tol, -1.5, 1.5)
        got, mkl, _ = run_dot(wrapper, 2, 2, 20000, False, False, 1, 0, 2, -1.5, 1.5)
        if mode != MATH_TF32:
            assert np.max(np.abs(got - mkl)) < 1e-2


def test_batched_cases_of_the_reference(wrapper):
    # Tests/TestParallelRunCpuVersusGpu.cs:377-401: batch 3, 12x12 / 12x7, (N,T) alpha 0.25, (N,N), (T,N)
    for mode, tol in MODES:
        wrapper.set_math_mode(mode)
        _check(wrapper, 12, 12, 7, False, True, 0.25, 0, 3, tol, -1.5, 1.5, batch=3)
        _check(wrapper, 12, 7, 12, False, False, 1, 0, 4, tol, -1.5, 1.5, batch=3)
        _check(wrapper, 12, 7, 12, True, False, 1, 0, 5, tol, -1.5, 1.5, batch=3)


@pytest.mark.parametrize("tA", [False, True])
@pytest.mark.parametrize("tB", [False, True])
def test_small_shape_sweep_simt(wrapper, tA, tB):
    # every (M, N, K) in a small grid, beta in {0, 1}; these shapes take the SIMT kernel
    wrapper.set_math_mode(MATH_3XTF32)
    seed = 100
    for M in (1, 2, 3, 5, 17, 40):
        for N in (1, 2, 7, 33, 40):
            for K in (1, 2, 9, 31, 40):
                for beta in (0.0, 1.0):
                    seed += 1
                    _check(wrapper, M, N, K, tA, tB, 1.0, beta, seed, TOL_3XTF32, -1.5, 1.5)
    assert wrapper.last_kernel().startswith("simt")


@pytest.mark.parametrize("pair", [2, 1])
@pytest.mark.parametrize("mode,tol", [(MATH_3XTF32, TOL_3XTF32), (MATH_TF32, TOL_TF32)])
@pytest.mark.parametrize("tA", [False, True])
@pytest.mark.parametrize("tB", [False, True])
def test_tensor_core_ragged_shapes(wrapper, mode, tol, tA, tB, pair):
    # sizes that are not multiples of the tile, every tile width, alpha/beta accumulate;
    # pair = 2: one CTA per 128-row tile, pair = 1: CTA pairs on 256-row tiles
    wrapper.set_math_mode(mode)
    wrapper.set_tuning(TUNE_FORCE_PATH, 1)
    wrapper.set_tuning(TUNE_PAIR, pair)
    seed = 500
    for bn in ((32, 64, 128, 256) if pair == 2 else (64, 128, 192, 256)):
        wrapper.set_tuning(TUNE_FORCE_BN, bn)
        for (M, N, K) in ((128, 256, 64), (132, 260, 36), (200, 328, 100), (4, 8, 4), (260, 516, 20), (96, 40, 520)):
            seed += 1
            _check(wrapper, M, N, K, tA, tB, 0.5, 1.0, seed, tol)
            assert wrapper.last_kernel().startswith("umma2" if pair == 1 else "umma_"), wrapper.last_kernel()
    wrapper.set_tuning(TUNE_FORCE_BN, 0)
    _check(wrapper, 300, 200, 72, tA, tB, -2.0, 0.0, 999, tol)


def test_beta_zero_ignores_nan_in_c(wrapper):
    # BLAS semantics: with beta = 0 the old content of C is not read
    rng = np.random.default_rng(9)
    for force, (M, N, K) in ((2, (9, 11, 13)), (1, (256, 256, 64))):
        wrapper.set_tuning(TUNE_FORCE_PATH, force)
        a = rng.uniform(-1, 1, (M, K)).astype(np.float32)
        b = rng.uniform(-1, 1, (K, N)).astype(np.float32)
        C = GPUTensor((M, N), np.full((M, N), np.nan, np.float32), wrapper)
        C.Dot(GPUTensor(a.shape, a, wrapper), False, GPUTensor(b.shape, b, wrapper), False, 1, 0)
        assert np.isfinite(C.ContentAsFloatArray()).all()


@pytest.mark.parametrize("mode,tol", [(MATH_3XTF32, TOL_3XTF32), (MATH_TF32, TOL_TF32)])
@pytest.mark.parametrize("tA", [False, True])
@pytest.mark.parametrize("tB", [False, True])
def test_unaligned_operands_run_on_the_tensor_cores(wrapper, mode, tol, tA, tB):
    """Views that start 4 bytes into an allocation and widths that are not multiples of 4 floats (SharpNet slices
    tensors at float granularity, Prod/GPU/GpuTensor.cs:1518-1521): TMA cannot load them, loader warps do, and the
    product still runs on the tensor cores."""
    import torch
    wrapper.set_math_mode(mode)
    rng = np.random.default_rng(21)
    for (M, N, K, off_a, off_b, beta, batch) in ((512, 384, 768, 1, 0, 0.0, 1), (517, 389, 771, 0, 0, 1.0, 1),
                                                 (517, 389, 771, 3, 2, 0.0, 1), (130, 70, 203, 1, 1, 1.0, 3),
                                                 (128, 33, 64, 1, 0, 0.0, 1)):
        sa = (batch,) + ((K, M) if tA else (M, K))
        sb = (batch,) + ((N, K) if tB else (K, N))
        a = rng.uniform(-1, 1, sa).astype(np.float32)
        b = rng.uniform(-1, 1, sb).astype(np.float32)
        c = rng.uniform(-1, 1, (batch, M, N)).astype(np.float32)
        base_a = torch.zeros(a.size + off_a, dtype=torch.float32, device=wrapper.device)
        base_b = torch.zeros(b.size + off_b, dtype=torch.float32, device=wrapper.device)
        base_a[off_a:] = torch.from_numpy(a.ravel()).to(wrapper.device)
        base_b[off_b:] = torch.from_numpy(b.ravel()).to(wrapper.device)
        A = GPUTensor(sa, wrapper=wrapper, storage=base_a[off_a:])
        B = GPUTensor(sb, wrapper=wrapper, storage=base_b[off_b:])
        C = GPUTensor((batch, M, N), c, wrapper)
        C.BatchMatrixMultiplication(A, tA, B, tB, 1.0, beta)
        wrapper.check_device_status()
        # large products run on the TMA kernels after one realignment pass over their operands, a batch of
        # smaller ones on the tensor-core kernel with loader warps, and what cannot fill 128-row tiles on SIMT
        name = wrapper.last_kernel()
        if M * N * K * batch < 128 ** 3:
            assert name.startswith("simt"), name
        elif batch == 1:
            assert name.endswith("_realigned") and name.startswith("umma"), name
        else:
            assert "swload" in name, name
        f64 = orc.batch_matrix_multiplication(a, tA, b, tB, c, 1.0, beta, f64=True)
        mkl = orc.batch_matrix_multiplication(a, tA, b, tB, c.copy(), 1.0, beta)
        got = C.ContentAsFloatArray()
        e64, emkl = orc.scaled_error(got, f64, K, 1, 1), orc.scaled_error(got, mkl, K, 1, 1)
        assert e64 <= tol and emkl <= tol, (M, N, K, tA, tB, off_a, off_b, e64, emkl)


def test_unaligned_views_fall_back_to_simt(wrapper):
    # SharpNet slices tensors at 4-byte granularity: a pointer that is not 16-byte aligned must work
    import torch
    rng = np.random.default_rng(11)
    M, N, K = 128, 128, 64
    a = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    b = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    base = torch.zeros(M * K + 1, dtype=torch.float32, device=wrapper.device)
    base[1:] = torch.from_numpy(a.ravel()).to(wrapper.device)
    A = GPUTensor((M, K), wrapper=wrapper, storage=base[1:])
    B = GPUTensor((K, N), b, wrapper)
    C = GPUTensor((M, N), None, wrapper)
    wrapper.set_tuning(11, 1)        # loader-warp kernel off: the SIMT kernel is the net under it
    try:
        C.Dot(A, False, B, False, 1, 0)
    finally:
        wrapper.set_tuning(11, 0)
    assert wrapper.last_kernel().startswith("simt")
    ref = orc.dot_f64(a.ravel(), M, K, False, b.ravel(), K, N, False, None, 1.0, 0.0)
    assert orc.scaled_error(C.ContentAsFloatArray(), ref, K, 1, 1) <= TOL_3XTF32


def test_empty_and_invalid_arguments(wrapper):
    C = GPUTensor((4, 4), np.ones((4, 4), np.float32), wrapper)
    A = GPUTensor((4, 3), None, wrapper)
    B = GPUTensor((5, 4), None, wrapper)
    with pytest.raises(SharpNetB200Error) as e:
        C.Dot(A, False, B, False, 1, 0)          # inner dimensions 3 vs 5
    assert e.value.status == 7
    lib, h = wrapper.lib, wrapper.handle
    assert lib.snb200_gemm(h, 0, 0, 0, 3, 3, 4, 1.0, None, None, 0.0, None) == 0       # M = 0: nothing to do
    assert lib.snb200_gemm(h, 0, 0, -1, 3, 3, 4, 1.0, None, None, 0.0, None) == 7
    assert lib.snb200_gemm(h, 0, 0, 4, 3, 3, 4, 1.0, None, B.Pointer, 0.0, C.Pointer) == 7  # null A
    # K = 0: C = beta * C
    A0 = GPUTensor((4, 0), None, wrapper)
    B0 = GPUTensor((0, 4), None, wrapper)
    C.Dot(A0, False, B0, False, 1, 2.0)
    np.testing.assert_array_equal(C.ContentAsFloatArray(), np.full((4, 4), 2.0, np.float32))


def test_inputs_may_alias(wrapper):
    # VanillaSgdOrtho computes Dot(W, false, W, true, ...) (Prod/Optimizers/VanillaSgdOrtho.cs:83)
    rng = np.random.default_rng(13)
    w_ = rng.uniform(-1, 1, (256, 128)).astype(np.float32)
    W = GPUTensor(w_.shape, w_, wrapper)
    C = GPUTensor((256, 256), None, wrapper)
    C.Dot(W, False, W, True, 1, 0)
    ref = w_.astype(np.float64) @ w_.astype(np.float64).T
    # every product on the diagonal is positive, so the sum grows like K, not sqrt(K): bound the relative error
    assert np.max(np.abs(C.ContentAsFloatArray() - ref)) / np.max(np.abs(ref)) <= TOL_3XTF32


@pytest.mark.parametrize("mode,tol", MODES)
def test_config_1_square_1024(wrapper, mode, tol):
    wrapper.set_math_mode(mode)
    _check(wrapper, 1024, 1024, 1024, False, False, 1, 0, 0, tol)


@pytest.mark.parametrize("mode,tol", [(MATH_3XTF32, TOL_3XTF32), (MATH_TF32, TOL_TF32)])
def test_config_2_four_transposes_beta_one(wrapper, mode, tol):
    wrapper.set_math_mode(mode)
    seed = 1
    for tA in (False, True):
        for tB in (False, True):
            _check(wrapper, 2048, 1536, 768, tA, tB, 1, 1, seed, tol)
            # 8 x 8 tiles of 256 x 192 fill 64 of the 74 SM pairs where 8 x 6 tiles of 256 x 256 fill 48
            assert wrapper.last_kernel().startswith("umma2") and "256x192" in wrapper.last_kernel(), wrapper.last_kernel()
            _check(wrapper, 32, 4096, 4096, tA, tB, 1, 1, 5, tol)
            seed += 1


@pytest.mark.parametrize("mode,tol", [(MATH_3XTF32, TOL_3XTF32), (MATH_TF32, TOL_TF32)])
def test_config_4_batched_and_lstm_gate(wrapper, mode, tol):
    wrapper.set_math_mode(mode)
    # 64 x [256x64] * [256x64]^T, U[-0.1, 0.1), alpha = 1 and 1/sqrt(64)
    _check(wrapper, 256, 256, 64, False, True, 1.0, 0, 9, tol, -0.1, 0.1, batch=64)
    _check(wrapper, 256, 256, 64, False, True, 0.125, 0, 9, tol, -0.1, 0.1, batch=64)
    # LSTM gate GEMM [256 x 2048] * [2048 x 4096] as Dot and as a batch of one
    _check(wrapper, 256, 4096, 2048, False, False, 1, 0, 11, tol, -0.1, 0.1)
    _check(wrapper, 256, 4096, 2048, False, False, 1, 0, 11, tol, -0.1, 0.1, batch=1)


@pytest.mark.parametrize("mode,tol", [(MATH_3XTF32, TOL_3XTF32), (MATH_TF32, TOL_TF32)])
def test_cta_pair_kernel_batched_and_many_tiles(wrapper, mode, tol):
    # the CTA-pair kernel on batches, on more tiles than there are SM pairs, and on an odd number of row tiles
    wrapper.set_math_mode(mode)
    wrapper.set_tuning(TUNE_FORCE_PATH, 1)
    wrapper.set_tuning(TUNE_PAIR, 1)
    _check(wrapper, 300, 200, 96, False, True, 1.0, 0.0, 41, tol, batch=5)
    _check(wrapper, 300, 200, 96, True, False, 0.5, 1.0, 42, tol, batch=3)
    wrapper.set_tuning(TUNE_FORCE_BN, 64)
    _check(wrapper, 1920, 1984, 80, False, False, 1.0, 1.0, 43, tol)      # 8 x 31 = 248 pair tiles > 74 pairs
    _check(wrapper, 384, 512, 4096, False, True, 1.0, 0.0, 44, tol)       # 3 row tiles: the odd CTA's rows are all padding
    assert wrapper.last_kernel().startswith("umma2")


@pytest.mark.parametrize("mode,tol", [(MATH_3XTF32, TOL_3XTF32), (MATH_TF32, TOL_TF32)])
@pytest.mark.parametrize("tA", [False, True])
@pytest.mark.parametrize("tB", [False, True])
def test_few_tiles_split_k_and_swapped_operands(wrapper, mode, tol, tA, tB):
    # problems with fewer tiles than SMs: K is cut into partial sums (workspace + reduction kernel), and
    # with few rows the operands are swapped so that N fills the 128-row tile
    wrapper.set_math_mode(mode)
    wrapper.set_tuning(TUNE_CLUSTER, 1)       # this test: the workspace plans (clusters have their own test below)
    seed = 700
    for (M, N, K) in ((256, 512, 4096), (132, 300, 2052), (512, 128, 8192)):
        seed += 1
        _check(wrapper, M, N, K, tA, tB, 0.5, 1.0, seed, tol)
        assert "splitk" in wrapper.last_kernel(), wrapper.last_kernel()
    for (M, N, K) in ((32, 4096, 4096), (1, 512, 1024), (5, 1000, 516), (64, 260, 256), (17, 256, 300)):
        for beta in (0.0, 1.0):
            seed += 1
            _check(wrapper, M, N, K, tA, tB, 1.0, beta, seed, tol)
            tma_ok = (not tA or M % 4 == 0)      # a transposed A is stored [K x M]: its pitch M must be a 16-byte multiple
            assert ("swapAB" in wrapper.last_kernel()) == tma_ok, wrapper.last_kernel()
    _check(wrapper, 8, 512, 1024, tA, tB, 1.0, 0.0, 777, tol, batch=6)       # batched, swapped


@pytest.mark.parametrize("mode,tol", [(MATH_3XTF32, TOL_3XTF32), (MATH_TF32, TOL_TF32)])
@pytest.mark.parametrize("tA,tB", [(False, False), (False, True), (True, False), (True, True)])
def test_k_cut_inside_clusters(wrapper, mode, tol, tA, tB):
    # K parts computed by the CTAs of a thread-block cluster and summed through distributed shared memory: every
    # tile width, clusters of 2 and 4, ragged edges, beta = 1 (read by the CTA that stores the rows), a batch, a
    # grid of more clusters than the GPU holds at once, and the swapped-operand form that stores the transpose
    wrapper.set_math_mode(mode)
    seed = 900
    for cs in (2, 4):
        wrapper.set_tuning(TUNE_CLUSTER, cs)
        for bn in (32, 64, 128, 256):
            wrapper.set_tuning(TUNE_FORCE_BN, bn)
            seed += 1
            _check(wrapper, 260, 300, 2052, tA, tB, 0.5, 1.0, seed, tol)
            assert wrapper.last_kernel() == "umma_%s_128x%d_clusterk%d" % (
                "3xtf32" if mode == MATH_3XTF32 else "tf32", bn, cs), wrapper.last_kernel()
        wrapper.set_tuning(TUNE_FORCE_BN, 128)
        _check(wrapper, 1024, 1024, 1024, tA, tB, 1.0, 0.0, seed + 50, tol)
        _check(wrapper, 132, 200, 1280, tA, tB, 1.0, 1.0, seed + 51, tol, batch=5)
        _check(wrapper, 2048, 2304, 512, tA, tB, 1.0, 0.0, seed + 52, tol)      # 288 tiles: several waves of clusters
        assert "clusterk%d" % cs in wrapper.last_kernel(), wrapper.last_kernel()
        wrapper.set_tuning(TUNE_FORCE_BN, 0)
        for (M, N, K) in ((32, 4096, 4096), (5, 1000, 2052), (64, 260, 2048)):
            for beta in (0.0, 1.0):
                seed += 1
                _check(wrapper, M, N, K, tA, tB, 0.5, beta, seed, tol)
                if not tA or M % 4 == 0:
                    assert "swapAB_clusterk%d" % cs in wrapper.last_kernel(), wrapper.last_kernel()
        _check(wrapper, 8, 512, 1024, tA, tB, 1.0, 1.0, seed + 60, tol, batch=6)
    # left to itself the library takes clusters where one wave of tiles leaves SMs idle
    wrapper.set_tuning(TUNE_CLUSTER, 0)
    _check(wrapper, 1024, 1024, 1024, tA, tB, 1.0, 0.0, 990, tol)
    _check(wrapper, 32, 4096, 4096, tA, tB, 1.0, 1.0, 991, tol)
    assert "swapAB_clusterk4" in wrapper.last_kernel(), wrapper.last_kernel()


@pytest.mark.parametrize("mode,tol", [(MATH_3XTF32, TOL_3XTF32), (MATH_TF32, TOL_TF32)])
@pytest.mark.parametrize("tA,tB", [(False, False), (False, True), (True, False), (True, True)])
def test_partly_filled_last_wave_is_cut_along_k(wrapper, mode, tol, tA, tB):
    # more tiles than SM pairs, with a last wave that would leave most SMs idle: the first waves run whole
    # tiles, the tiles of the last wave are cut along K (tile-shaped partial sums + reduction kernel).
    # Ragged right and bottom edges, beta = 1, and a batch whose tiles straddle the whole / cut boundary.
    wrapper.set_math_mode(mode)
    _check(wrapper, 2308, 2300, 1028, tA, tB, 0.5, 1.0, 811, tol)
    _check(wrapper, 772, 1000, 1536, tA, tB, 1.0, 0.0, 812, tol, batch=7)
    wrapper.set_tuning(TUNE_FORCE_BN, 256)
    for pair in (1, 2):                       # the same on the CTA-pair and on the single-CTA kernel
        wrapper.set_tuning(TUNE_PAIR, pair)
        _check(wrapper, 2308, 2300, 1028, tA, tB, 1.0, 1.0, 813 + pair, tol)
        assert wrapper.last_kernel().startswith("umma2" if pair == 1 else "umma_"), wrapper.last_kernel()
        if mode == MATH_3XTF32:               # 81 (171) tiles on 74 (148) slots: the model must cut the 7 (23) left over
            assert "splitk" in wrapper.last_kernel(), wrapper.last_kernel()
        _check(wrapper, 772, 1000, 1536, tA, tB, 1.0, 1.0, 815 + pair, tol, batch=7)
    # the 192-wide pair tile with its tail cut: 10 x 8 = 80 tiles on 74 pairs, the 6 left over cut along K
    wrapper.set_tuning(TUNE_FORCE_BN, 192)
    wrapper.set_tuning(TUNE_PAIR, 1)
    _check(wrapper, 2308, 1530, 1028, tA, tB, 1.0, 1.0, 819, tol)
    assert wrapper.last_kernel().startswith("umma2") and "256x192" in wrapper.last_kernel(), wrapper.last_kernel()
    if mode == MATH_3XTF32:
        assert "splitk" in wrapper.last_kernel(), wrapper.last_kernel()


def test_long_k_keeps_fp32_accuracy(wrapper):
    # the tensor-core accumulator truncates; the kernel must not let that grow with K
    wrapper.set_math_mode(MATH_3XTF32)
    e = _check(wrapper, 256, 256, 16384, False, True, 1, 0, 21, TOL_3XTF32)
    assert e < 5e-6


def test_linearity_at_full_size(wrapper):
    # size-independent property at a size the CPU oracle would take minutes for (4096^3 per product):
    # (A1 + A2) * B == A1 * B + A2 * B up to rounding, and C == C^T for A * A^T
    import torch
    n = 4096
    g = torch.Generator(device="cpu").manual_seed(31)
    a1 = torch.rand(n, n, generator=g) * 2 - 1
    a2 = torch.rand(n, n, generator=g) * 2 - 1
    b = torch.rand(n, n, generator=g) * 2 - 1
    T = lambda t: GPUTensor((n, n), wrapper=wrapper, storage=t.to(wrapper.device).contiguous().view(-1))  # noqa: E731
    A1, A2, A12, B = T(a1), T(a2), T(a1 + a2), T(b)
    C1, C2 = GPUTensor((n, n), None, wrapper), GPUTensor((n, n), None, wrapper)
    C1.Dot(A1, False, B, False, 1, 0)
    C1.Dot(A2, False, B, False, 1, 1)          # accumulate with beta = 1
    C2.Dot(A12, False, B, False, 1, 0)
    wrapper.check_device_status()
    d = (C1.storage - C2.storage).abs().max().item()
    assert d / (np.sqrt(n) * 2.0) <= 2 * TOL_3XTF32
    C1.Dot(A1, False, A1, True, 1, 0)
    sym = (C1.storage.view(n, n) - C1.storage.view(n, n).t()).abs().max().item()
    assert sym / np.sqrt(n) <= 2 * TOL_3XTF32


def test_gemm_timing_entry_points(wrapper):
    # event pairs around every product between _begin and _end; nothing is recorded outside
    import ctypes
    a = GPUTensor((512, 256), orc.uniform((512, 256), -1, 1, 1), wrapper)
    b = GPUTensor((256, 384), orc.uniform((256, 384), -1, 1, 2), wrapper)
    c = GPUTensor((512, 384), None, wrapper)
    ms, n = ctypes.c_double(), ctypes.c_int()
    assert wrapper.lib.snb200_gemm_timing_end(wrapper.handle, ctypes.byref(ms), ctypes.byref(n)) == 7   # not begun
    c.Dot(a, b)
    wrapper.gemm_timing_begin()
    for _ in range(3):
        c.Dot(a, b)
    total, calls = wrapper.gemm_timing_end()
    assert calls == 3 and 0.0 < total < 50.0
    c.Dot(a, b)
    wrapper.gemm_timing_begin()
    total, calls = wrapper.gemm_timing_end()
    assert calls == 0 and total == 0.0


@pytest.mark.parametrize("mode,tol", [(MATH_3XTF32, TOL_3XTF32), (MATH_TF32, TOL_TF32)])
def test_dependent_launch_on_and_off_give_the_same_bits(wrapper, mode, tol):
    # a chain of products, each reading what the previous one wrote, with the kernels' set-up overlapping the
    # previous kernel's tail (default) and without: identical results
    from sharpnet_b200._capi import TUNE_PDL
    wrapper.set_math_mode(mode)
    x = orc.uniform((384, 384), -1, 1, 5)
    W = orc.uniform((384, 384), -0.08, 0.08, 6)
    outs = []
    for off in (0, 1):
        wrapper.set_tuning(TUNE_PDL, off)
        bufs = [GPUTensor(x.shape, x, wrapper), GPUTensor(x.shape, None, wrapper)]
        Wg = GPUTensor(W.shape, W, wrapper)
        for i in range(12):
            bufs[(i + 1) % 2].Dot(bufs[i % 2], False, Wg, i % 2 == 1, 1.0, 0.0)
        wrapper.check_device_status()
        outs.append(bufs[0].ContentAsFloatArray())
    wrapper.set_tuning(TUNE_PDL, 0)
    np.testing.assert_array_equal(outs[0], outs[1])
    ref = x.astype(np.float64)
    for i in range(12):
        ref = ref @ (W.T if i % 2 == 1 else W).astype(np.float64)
    assert np.abs(outs[0] - ref).max() <= 12 * tol * np.sqrt(384) * np.abs(ref).max() + 1e-12


def test_tf32_bf16x2_mode(wrapper):
    # opt-in math mode 3: hi * hi in TF32, both cross terms as one bf16 instruction.  Same 1e-5 bound as 3xTF32 on the
    # shapes that reach its kernel (A not transposed, B transposed, M > 128), 3xTF32 itself on everything else.
    from sharpnet_b200._capi import MATH_TF32_BF16X2
    wrapper.set_math_mode(MATH_TF32_BF16X2)
    assert wrapper.get_math_mode() == MATH_TF32_BF16X2
    for (M, N, K) in ((512, 512, 512), (1000, 3108, 1028), (2304, 2300, 1028), (256, 256, 16384), (4096, 1024, 3072)):
        e = _check(wrapper, M, N, K, False, True, 1.0, 0.0, 900 + M, TOL_3XTF32)
        if M >= 1000:        # wide pair tiles; the smaller problems may be given narrower (3xTF32) kernels
            assert "tf32bf16x2" in wrapper.last_kernel(), wrapper.last_kernel()
        assert e < 5e-6
    _check(wrapper, 2304, 2300, 1028, False, True, 0.5, 1.0, 950, TOL_3XTF32)            # beta, cut last wave
    _check(wrapper, 772, 1000, 1536, False, True, 1.0, 0.0, 951, TOL_3XTF32, batch=3)
    for tA, tB in ((False, False), (True, False), (True, True)):                            # other layouts: 3xTF32
        _check(wrapper, 512, 384, 640, tA, tB, 1.0, 0.0, 960, TOL_3XTF32)
        assert "3xtf32" in wrapper.last_kernel(), wrapper.last_kernel()
    _check(wrapper, 64, 64, 64, False, True, 1.0, 0.0, 970, TOL_3XTF32)                   # small: single-CTA 3xTF32
    # small integers are exact in TF32 and their low parts are zero: bit exact
    rng = np.random.default_rng(5)
    a = rng.integers(-8, 9, (300, 160)).astype(np.float32)
    b = rng.integers(-8, 9, (280, 160)).astype(np.float32)
    A, B, C = GPUTensor(a.shape, a, wrapper), GPUTensor(b.shape, b, wrapper), GPUTensor((300, 280), None, wrapper)
    C.Dot(A, False, B, True, 1, 0)
    np.testing.assert_array_equal(C.ContentAsFloatArray(), a @ b.T)


@pytest.mark.parametrize("mode,tol", [(MATH_3XTF32, TOL_3XTF32), (MATH_TF32, TOL_TF32)])
def test_config_5_square_16384_on_row_samples(wrapper, mode, tol):
    """benchmark config 5a at full size (16384^3, U[-1, 1), seed 13): the whole product runs on the device; three
    blocks of 64 rows of it -- the first rows, rows from the middle of a tile band, the last rows -- are compared
    with MKL sgemm and with float64 on the same operands (the full product on the host would take minutes)."""
    import torch
    n = 16384
    wrapper.set_math_mode(mode)
    rng = np.random.default_rng(13)
    a = rng.uniform(-1, 1, (n, n)).astype(np.float32)
    b = rng.uniform(-1, 1, (n, n)).astype(np.float32)
    A, B, C = GPUTensor((n, n), a, wrapper), GPUTensor((n, n), b, wrapper), GPUTensor((n, n), None, wrapper)
    C.Dot(A, False, B, False, 1.0, 0.0)
    wrapper.check_device_status()
    assert wrapper.last_kernel().startswith("umma2_")
    b64 = b.astype(np.float64)
    for r0 in (0, 8000, n - 64):
        got = C.storage[r0 * n:(r0 + 64) * n].view(64, n).cpu().numpy()
        rows = np.ascontiguousarray(a[r0:r0 + 64])
        f64 = rows.astype(np.float64) @ b64
        mkl = np.zeros((64, n), np.float32)
        orc.dot_mkl(rows.ravel(), 64, n, False, b.ravel(), n, n, False, mkl.reshape(-1), 1.0, 0.0)
        e64, emkl = orc.scaled_error(got, f64, n, 1.0, 1.0), orc.scaled_error(got, mkl, n, 1.0, 1.0)
        assert e64 <= tol and emkl <= tol, (r0, e64, emkl)
    del A, B, C
    torch.cuda.empty_cache()


def test_seeded_sweep_over_shapes_and_plans(wrapper):
    """A seeded draw of shapes, transposes, alpha / beta, batches, math modes and forced kernel plans (tile width,
    CTA pair on or off, K cut inside clusters of 2 or 4 or never): whatever kernel the library ends up with, the
    result stays within the mode's bound of the float64 product."""
    rng = np.random.default_rng(2026)
    kernels = set()
    try:
        for it in range(160):
            mode, tol = ((MATH_3XTF32, TOL_3XTF32), (MATH_TF32, TOL_TF32))[it % 5 == 4]
            M = int(rng.choice([1, 5, 17, 32, 33, 64, 100, 128, 129, 200, 256, 300, 513, 700]))
            N = int(rng.choice([8, 12, 32, 40, 64, 100, 128, 132, 256, 260, 384, 512, 640]))
            K = int(rng.choice([64, 100, 128, 256, 300, 512, 516, 1000, 1024, 2052, 3000]))
            tA, tB = bool(rng.integers(2)), bool(rng.integers(2))
            beta, alpha = float(rng.choice([0.0, 1.0, -0.5])), float(rng.choice([1.0, 0.5]))
            batch = None if rng.integers(4) else int(rng.choice([2, 5]))
            wrapper.set_math_mode(mode)
            wrapper.set_tuning(TUNE_CLUSTER, int(rng.choice([0, 0, 2, 4, 1])))
            wrapper.set_tuning(TUNE_FORCE_BN, int(rng.choice([0, 0, 32, 64, 128, 192, 256])))
            wrapper.set_tuning(TUNE_PAIR, int(rng.choice([0, 0, 2])))
            _check(wrapper, M, N, K, tA, tB, alpha, beta, 1000 + it, tol, batch=batch)
            kernels.add(wrapper.last_kernel().split("_p")[0])
    finally:
        wrapper.set_tuning(TUNE_CLUSTER, 0)
    # the draw reaches every family of plans
    for family in ("clusterk2", "clusterk4", "swapAB", "splitk", "swload", "realigned", "umma2_", "256x192", "simt"):
        assert any(family in k for k in kernels), (family, sorted(kernels))


def test_two_handles_on_two_host_threads(built_library):
    """Handles are independent of one another: each owns its workspace, its tensor-map cache, its error word and its
    stream, and SharpNet drives every device from a thread of its own (Prod/GPU/GPUWrapper.cs:782-832,
    Prod/Networks/Network.cs:71-83).  Two host threads drive one handle each on the same GPU at the same time,
    through products that take the workspace, clusters, swapped operands and the FMA kernel; small integer operands
    make every result exact, so one wrong tile or one torn workspace shows."""
    import threading
    import torch
    from sharpnet_b200.tensor import GPUWrapper
    shapes = [(1024, 1024, 1024), (256, 4096, 2048), (32, 4096, 4096), (2048, 1536, 768), (9, 5, 21), (300, 136, 200)]
    rng = np.random.default_rng(5)
    cases = []
    for M, N, K in shapes:
        a = rng.integers(-2, 3, (M, K)).astype(np.float32)
        b = rng.integers(-2, 3, (K, N)).astype(np.float32)
        cases.append((a, b, (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)))
    errors = []

    def drive(tid):
        w = GPUWrapper(0)      # a handle of this thread's own, not the cached one
        try:
            stream = torch.cuda.Stream(device=0)
            w.set_stream(stream)
            with torch.cuda.stream(stream):
                tensors = [(GPUTensor(a.shape, a, w), GPUTensor(b.shape, b, w), GPUTensor(c.shape, None, w), c)
                           for a, b, c in cases]
                for it in range(6):
                    order = range(len(tensors)) if tid == 0 else reversed(range(len(tensors)))
                    for i in order:
                        A, B, C, _ = tensors[i]
                        C.Dot(A, False, B, False, 1.0, 0.0)
                    for i, (_, _, C, want) in enumerate(tensors):
                        if not np.array_equal(C.ContentAsFloatArray(), want):
                            errors.append((tid, it, shapes[i]))
                    w.check_device_status()
        except Exception as e:   # noqa: BLE001 -- reported by the assertion below
            errors.append((tid, repr(e)))
        finally:
            torch.cuda.synchronize()
            w.Dispose()

    threads = [threading.Thread(target=drive, args=(t,)) for t in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors


def test_tensors_beyond_four_gigabytes(wrapper):
    """SharpNet's tensors hold up to 2^31 - 1 floats (Prod/Data/Tensor.cs:189), 8.6 GB: element offsets beyond 2^30
    and byte offsets beyond 2^32 are inside the contract.  A 1 114 112 x 1024 tensor (4.56 GB) as the result of a
    product, as the transposed operand of a weight-gradient product whose K is its 1.1 M rows, as the input of a bias
    gradient and of an activation pass; small integers, so every result is exact."""
    import torch
    from sharpnet_b200 import ACT_RELU
    dev = wrapper.device
    block, reps, N, k = 65536, 17, 1024, 32
    M = block * reps
    rng = np.random.default_rng(21)
    a_block = rng.integers(-1, 2, (block, N)).astype(np.float32)          # the big tensor is this block 17 times over
    big = torch.from_numpy(a_block).to(dev).repeat(reps, 1).contiguous()
    assert big.numel() * 4 > 2 ** 32
    BIG = GPUTensor((M, N), wrapper=wrapper, storage=big.view(-1))
    try:
        # dW = big^T * dy, K = M                                       (Prod/Layers/Linear.cs:158)
        dy = rng.integers(-1, 2, (M, k)).astype(np.float32)
        DY, DW = GPUTensor(dy.shape, dy, wrapper), GPUTensor((N, k), None, wrapper)
        DW.Dot(BIG, True, DY, False, 1.0, 0.0)
        want = sum(a_block.T @ dy[r * block:(r + 1) * block] for r in range(reps))
        np.testing.assert_array_equal(DW.ContentAsFloatArray(), want)
        # db = column sums of big                                      (Prod/GPU/GpuTensor.cs:686-701)
        DB = GPUTensor((N,), None, wrapper)
        BIG.Compute_BiasGradient_from_dy(DB)
        np.testing.assert_array_equal(DB.ContentAsFloatArray(), reps * a_block.sum(0, dtype=np.float64).astype(np.float32))
        # y = relu(big), a second 4.56 GB tensor, then overwritten as the result of a product with K = 32
        out = torch.empty_like(big)
        OUT = GPUTensor((M, N), wrapper=wrapper, storage=out.view(-1))
        BIG.ActivationForward(ACT_RELU, None, OUT)
        assert torch.equal(out, torch.clamp_min(big, 0))
        x = rng.integers(-2, 3, (M, k)).astype(np.float32)
        wgt = rng.integers(-2, 3, (k, N)).astype(np.float32)
        X, W = GPUTensor(x.shape, x, wrapper), GPUTensor(wgt.shape, wgt, wrapper)
        OUT.Dot(X, False, W, False, 1.0, 0.0)
        wrapper.check_device_status()
        for r0 in (0, 2 ** 20 - 64, M - 128):        # the start, across byte offset 2^32, the end
            np.testing.assert_array_equal(out[r0:r0 + 128].cpu().numpy(), x[r0:r0 + 128] @ wgt)
        assert torch.equal(out.sum(1, dtype=torch.float64).cpu(), torch.from_numpy((x @ wgt.sum(1)).astype(np.float64)))
    finally:
        del big, BIG
        torch.cuda.empty_cache()


def test_create_and_destroy_release_what_they_took(built_library):
    """A handle owns its workspace, its error word and its timing events and nothing else (SharpNet creates one
    wrapper per device and disposes it with the process, Prod/GPU/GPUWrapper.cs:99-160,737-777): creating a handle,
    working through it and destroying it, over and over, leaves the device's free memory where it was."""
    import torch
    from sharpnet_b200.tensor import GPUWrapper
    a = np.arange(64 * 48, dtype=np.float32).reshape(64, 48) % 5 - 2
    b = np.arange(48 * 40, dtype=np.float32).reshape(48, 40) % 3 - 1

    def cycle():
        w = GPUWrapper(0)
        try:
            A, B, C = GPUTensor(a.shape, a, w), GPUTensor(b.shape, b, w), GPUTensor((64, 40), None, w)
            w.gemm_timing_begin()
            C.Dot(A, False, B, False, 1.0, 0.0)
            w.gemm_timing_end()
            np.testing.assert_array_equal(C.ContentAsFloatArray(), a @ b)
        finally:
            w.Dispose()

    cycle()                                   # first use: module load, function attributes
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(0)
    for _ in range(20):
        cycle()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(0)
    assert free_before - free_after < (8 << 20), (free_before, free_after)   # a leaked 128 MB workspace would show
    lib = GPUWrapper.FromDeviceId(0).lib
    assert lib.snb200_destroy(None) == 1      # CUBLAS_STATUS_NOT_INITIALIZED's number: no handle
