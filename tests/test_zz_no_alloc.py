"""snb200_bias_grad_noalloc: the handle-free, allocation-free bias gradient, for hosts that cannot call
cudaMalloc while they run (their own pool holds the device memory, or they cannot take the
device-wide synchronisation an allocation implies).  Checked through the C ABI against the
handle-based snb200_bias_grad on the same inputs, on two calls in a row that share the library's
fixed scratch array.  This file sorts last on purpose, so a run that stops at the first failure has
already been through every other test."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _noalloc(lib, dy_t, M, N, device=0, stream=None):
    import torch
    db = torch.full((max(N, 1),), float("nan"), dtype=torch.float32, device=dy_t.device)
    err = ctypes.create_string_buffer(256)
    st = lib.snb200_bias_grad_noalloc(device, None if stream is None else ctypes.c_void_p(stream.cuda_stream), M, N,
                                      ctypes.c_void_p(dy_t.data_ptr()), ctypes.c_void_p(db.data_ptr()), err, 256)
    return st, db, err.value.decode()


def test_noalloc_bias_gradient_matches_the_handle_entry_point(wrapper):
    import torch
    lib, h = wrapper.lib, wrapper.handle
    rng = np.random.default_rng(42)
    # first call: many slabs in the scratch array; second call: a different, smaller problem right after,
    # so stale partial sums of the first call would show up; then odd sizes that take the scalar kernel
    # (4096, 65536): the widest matrix allowed, where the slab count is cut down to what the array holds
    side = torch.cuda.Stream(device=wrapper.device)
    for (M, N) in ((4096, 1024), (300, 64), (1000, 333), (9, 1632), (5, 65536), (4096, 65536)):
        dy = rng.uniform(-1.5, 1.5, (M, N)).astype(np.float32)
        dy_t = torch.from_numpy(dy).to(wrapper.device)
        ref = torch.empty(N, dtype=torch.float32, device=wrapper.device)
        assert lib.snb200_bias_grad(h, M, N, ctypes.c_void_p(dy_t.data_ptr()), ctypes.c_void_p(ref.data_ptr())) == 0
        torch.cuda.synchronize()
        for stream in (None, side):   # two calls in a row on the shared scratch: default stream, then a stream of the caller's
            st, db, msg = _noalloc(lib, dy_t, M, N, stream=stream)
            assert st == 0, msg
            torch.cuda.synchronize()
            tol = 1e-5 * np.sqrt(M) * 1.5 + 1e-6          # the bound test_dense_gpu.py uses for column sums
            assert float((db - ref).abs().max()) <= tol
            assert float(np.abs(db.cpu().numpy() - dy.astype(np.float64).sum(0)).max()) <= tol


def test_noalloc_rejects_what_does_not_fit(wrapper):
    import torch
    lib = wrapper.lib
    dy_t = torch.zeros(8, dtype=torch.float32, device=wrapper.device)
    st, _, msg = _noalloc(lib, dy_t, 1, 65537)
    assert st == 15 and "65536" in msg                     # NOT_SUPPORTED, with the limit in the text
    st, _, msg = _noalloc(lib, dy_t, -1, 4)
    assert st == 7 and msg
    st, db, _ = _noalloc(lib, dy_t, 0, 4)                  # no rows: the sums are zero
    torch.cuda.synchronize()
    assert st == 0 and not db.cpu().numpy().any()
