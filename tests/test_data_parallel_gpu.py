"""The data-parallel Dense step on the device: this library's DenseStack / training_step / SgdUpdate host logic,
its NCCL binding (snb200_comm_*, snb200_allreduce_sum[_group]) and the mini-batch stager, checked against the CPU
oracle on the full batch.  SharpNet sums the replicas' gradients on the master
(Prod/Networks/NetworkMultiGPUSupport.cs:161-173) after slicing the mini-batch by rows
(Prod/Networks/Network.cs:1229-1258); every replica here must end the step holding exactly that sum.

The two-rank cases run one child process per GPU and are skipped on a single-GPU machine."""
import ctypes
import os
import socket
import subprocess
import sys
import threading

import numpy as np
import pytest

from oracle import sharpnet_oracle as orc

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = 1e-5     # max |err| / (sqrt(K) * a_max * b_max), the bound of the 3xTF32 products


def _oracle_forward(x, Ws, bs, acts):
    """Activations of every layer over the whole batch (float64 products, stored as float32 like the device does)."""
    a = [x]
    for W, b, act in zip(Ws, bs, acts):
        a.append(orc.dense_forward(a[-1], W, b, act, orc.W_OUT_IN, f64=True)[1].astype(np.float32))
    return a


def _oracle_backward(a, dy, Ws, acts):
    """(dW, db) of every layer in float64 from the activations ``a`` and the upstream gradient.  ``a`` are the
    activations the device produced: a pre-activation within rounding of zero may fall on either side of the ReLU
    on the two machines, and the gradient mask has to be taken from the same values on both."""
    g, grads, gmax = dy, [None] * len(Ws), [None] * len(Ws)
    for i in reversed(range(len(Ws))):
        dz, dW, db, g = orc.dense_backward(a[i], Ws[i], g, acts[i], a[i + 1], None, 1.0, orc.W_OUT_IN, need_dx=i > 0,
                                           f64=True)
        grads[i] = (dW, db)
        gmax[i] = float(np.abs(dz).max())
        if g is not None:
            g = g.astype(np.float32)
    return grads, gmax


def _problem(batch, dims, seed):
    x = orc.normal((batch, dims[0]), 0, 1, seed)
    dy = orc.normal((batch, dims[-1]), 0, 1, seed + 1)
    Ws = [orc.glorot_uniform((dims[i + 1], dims[i]), seed + 2 + i) for i in range(len(dims) - 1)]
    bs = [orc.uniform((dims[i + 1],), -0.1, 0.1, seed + 10 + i) for i in range(len(dims) - 1)]
    return x, dy, Ws, bs


def _load(stack, x, dy, bs):
    import torch
    stack.x.storage.copy_(torch.from_numpy(x).view(-1))
    stack.dy.storage.copy_(torch.from_numpy(dy).view(-1))
    for t, b in zip(stack.b, bs):
        t.storage.copy_(torch.from_numpy(b))


def _activations(stack):
    return [stack.x.ContentAsFloatArray()] + [t.ContentAsFloatArray() for t in stack.y]


def _check_gradients(stack, grads, gmax, a, batch):
    """dW[i] = dz_i^T a_i and db[i] = column sums of dz_i are sums over the ``batch`` rows."""
    for i, (dW, db) in enumerate(grads):
        e = orc.scaled_error(stack.dW[i].ContentAsFloatArray(), dW, batch, float(np.abs(a[i]).max()), gmax[i])
        assert e <= TOL, (i, "dW", e)
        e = orc.scaled_error(stack.db[i].ContentAsFloatArray(), db, batch, 1.0, gmax[i])
        assert e <= TOL, (i, "db", e)


@pytest.mark.parametrize("batch,dims,defer,dw_panels", [(384, (256, 192, 128, 40), False, 1), (384, (256, 192, 128, 40), True, 1),
                                                        (4096, (4096, 4096, 4096, 1000), True, 1),
                                                        (384, (256, 600, 128, 40), True, 2), (4096, (4096, 4096, 4096, 1000), True, 4)])
def test_training_step_and_update_on_one_gpu(wrapper, batch, dims, defer, dw_panels):
    """DenseStack + training_step + SgdUpdate against the oracle: activations, every dW / db, and the weights after
    the update; the second shape is benchmark config 5's network on 4096 of its 65536 rows."""
    from sharpnet_b200 import ACT_IDENTITY, ACT_RELU, MATH_3XTF32
    from sharpnet_b200.data_parallel import DenseStack, SgdUpdate, training_step
    wrapper.set_math_mode(MATH_3XTF32)
    acts = (ACT_RELU, ACT_RELU, ACT_IDENTITY)
    x, dy, Ws, bs = _problem(batch, dims, 100 + batch)
    stack = DenseStack(wrapper, batch, dims, acts, Ws)
    _load(stack, x, dy, bs)
    oacts = (orc.ACT_RELU, orc.ACT_RELU, orc.ACT_IDENTITY)
    a = _oracle_forward(x, Ws, bs, oacts)
    if defer and dw_panels > 1:
        # layer 0's weight gradient as row panels (snb200_dense_bwd_weight_rows), a hook behind each
        stack.forward()
        stack.dw_row_panels = dw_panels
        order = []
        stack.backward(after_gradients=order.append, defer_smallest=True,
                       after_gradient_rows=lambda i, r0, n, last: order.append((i, r0, n, last)))
        rows = dims[1]
        per = -(-(-(-rows // dw_panels)) // 256) * 256
        want = [(0, r0, min(per, rows - r0), r0 + per >= rows) for r0 in range(0, rows, per)]
        assert order == [1] + want + [2], order
    elif defer:
        stack.forward()
        order = []
        stack.backward(after_gradients=order.append, defer_smallest=True)
        assert order == [1, 0, 2]          # the 1000- (40-) row gradient of the output layer goes last
    else:
        training_step(stack)
    wrapper.check_device_status()
    wmaxes = [float(np.abs(W).max()) for W in Ws]
    for i in range(3):
        e = orc.scaled_error(stack.y[i].ContentAsFloatArray(), a[i + 1], dims[i], 4.5, wmaxes[i])
        assert e <= TOL * (i + 1), (i, "y", e)       # layer i's input already carries i rounded products
    a_dev = _activations(stack)
    grads, gmax = _oracle_backward(a_dev, dy, Ws, oacts)
    _check_gradients(stack, grads, gmax, a_dev, batch)
    # one SGD step with momentum on the gradients just computed, on the device
    upd = SgdUpdate(stack, 0.05, batch, momentum=0.9)
    before = [t.ContentAsFloatArray().copy() for t in stack.W]
    dWs = [t.ContentAsFloatArray().copy() for t in stack.dW]
    for i in range(3):
        upd(wrapper.lib, wrapper.handle, stack, i)
    wrapper.check_device_status()
    for i in range(3):
        v = np.zeros_like(before[i])
        want = before[i].copy()
        orc.update_sgd_optimizer(want, 0.05 / batch, 0.9, False, dWs[i], v)
        np.testing.assert_allclose(stack.W[i].ContentAsFloatArray(), want, rtol=0, atol=1e-7)


def test_backward_as_two_calls_equals_one_call(wrapper):
    """dW / db first and dx in a second call (dW NULL) give the bits of the single call."""
    from sharpnet_b200 import ACT_RELU
    from sharpnet_b200.tensor import GPUTensor
    lib, h = wrapper.lib, wrapper.handle
    M, K, N = 512, 384, 256
    x, W, dy = orc.normal((M, K), 0, 1, 1), orc.glorot_uniform((N, K), 2), orc.normal((M, N), 0, 1, 3)
    y = np.maximum(orc.normal((M, N), 0, 1, 4), 0).astype(np.float32)
    X, Wt, DY, Y = (GPUTensor(v.shape, v, wrapper) for v in (x, W, dy, y))
    out = []
    for split in (False, True):
        DZ, DX, DW, DB = (GPUTensor(s, None, wrapper) for s in ((M, N), (M, K), (N, K), (N,)))
        if not split:
            st = lib.snb200_dense_bwd(h, 0, M, K, N, X.Pointer, Wt.Pointer, DY.Pointer, ACT_RELU, Y.Pointer, None, 1.0,
                                      DZ.Pointer, DX.Pointer, DW.Pointer, DB.Pointer)
            assert st == 0
        else:
            st = lib.snb200_dense_bwd(h, 0, M, K, N, X.Pointer, Wt.Pointer, DY.Pointer, ACT_RELU, Y.Pointer, None, 1.0,
                                      DZ.Pointer, None, DW.Pointer, DB.Pointer)
            assert st == 0
            st = lib.snb200_dense_bwd(h, 0, M, K, N, X.Pointer, Wt.Pointer, DZ.Pointer, 5, None, None, 1.0,
                                      None, DX.Pointer, None, None)
            assert st == 0
        wrapper.check_device_status()
        out.append([t.ContentAsFloatArray() for t in (DZ, DX, DW, DB)])
    for a, b in zip(*out):
        np.testing.assert_array_equal(a, b)
    # nothing to compute at all is an argument error
    assert lib.snb200_dense_bwd(h, 0, M, K, N, X.Pointer, Wt.Pointer, DY.Pointer, 5, None, None, 1.0, None, None, None,
                                None) == 7


def test_nccl_binding_with_one_rank(wrapper):
    """Both ways of building a communicator, with a single rank (the sum over one replica is the identity), so
    that the binding -- library load, id, init, all-reduce, grouped all-reduce, destroy -- runs on any machine."""
    import torch
    from sharpnet_b200.tensor import GPUWrapper
    lib = wrapper.lib
    w = GPUWrapper(0)                                   # a handle of its own: the communicator lives on it
    try:
        buf = torch.arange(100000, dtype=torch.float32, device=wrapper.device) * 0.25
        small = torch.full((37,), 3.0, dtype=torch.float32, device=wrapper.device)
        want = buf.clone()
        P = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
        assert lib.snb200_allreduce_sum(w.handle, P(buf), buf.numel()) == 1          # no communicator yet
        handles = (ctypes.c_void_p * 1)(w.handle)
        st = lib.snb200_comm_init_all(handles, 1)       # the thread-per-GPU form (Prod/Networks/Network.cs:71-83)
        if st == 15:
            pytest.skip("NCCL is not installed")
        assert st == 0
        assert lib.snb200_allreduce_sum(w.handle, P(buf), buf.numel()) == 0
        bufs = (ctypes.c_void_p * 2)(P(buf), P(small))
        counts = (ctypes.c_longlong * 2)(buf.numel(), small.numel())
        assert lib.snb200_allreduce_sum_group(w.handle, 2, bufs, counts) == 0
        w.check_device_status()
        assert torch.equal(buf, want) and float(small.min()) == 3.0 == float(small.max())
        assert lib.snb200_comm_init_all(handles, 1) == 7                              # already initialised
        assert lib.snb200_comm_destroy(w.handle) == 0
        ident = ctypes.create_string_buffer(128)        # the process-per-GPU form
        assert lib.snb200_comm_get_unique_id(ident) == 0
        assert lib.snb200_comm_init_rank(w.handle, 1, 0, ident) == 0
        assert lib.snb200_allreduce_sum(w.handle, P(buf), buf.numel()) == 0
        w.check_device_status()
        assert torch.equal(buf, want)
        assert lib.snb200_comm_init_rank(w.handle, 2, 5, ident) == 7                  # bad rank
        assert lib.snb200_allreduce_sum(w.handle, None, 5) == 7
        assert lib.snb200_comm_destroy(w.handle) == 0
    finally:
        lib.snb200_destroy(w.handle)
        w.handle = None


def test_wait_that_runs_out_is_reported_once(wrapper):
    """The failure path of the tensor-core kernels: a bounded wait gives up, the kernel returns normally, the host
    reads EXECUTION_FAILED once, and the handle keeps working."""
    from sharpnet_b200.tensor import GPUTensor
    lib, h = wrapper.lib, wrapper.handle
    wrapper.check_device_status()
    assert lib.snb200_selftest_wait_timeout(h, 0) == 7
    assert lib.snb200_selftest_wait_timeout(h, 1000) == 0        # one CTA waits 1 ms on a barrier nothing signals
    assert lib.snb200_check_device_status(h) == 13
    assert b"timed out" in lib.snb200_last_error_string(h)
    assert lib.snb200_check_device_status(h) == 0
    a, b = orc.uniform((256, 256), -1, 1, 5), orc.uniform((256, 256), -1, 1, 6)
    A, B, C = GPUTensor(a.shape, a, wrapper), GPUTensor(b.shape, b, wrapper), GPUTensor((256, 256), None, wrapper)
    C.Dot(A, False, B, True, 1.0, 0.0)
    wrapper.check_device_status()
    assert orc.scaled_error(C.ContentAsFloatArray(), a.astype(np.float64) @ b.astype(np.float64).T, 256, 1, 1) <= TOL


def test_stager_orders_copies_and_steps(wrapper):
    """Double-buffered mini-batch staging: step i reads the bytes of copy i although copy i+1 and i+2 are queued
    while it runs, and a slot is not overwritten before the step that reads it has finished (a long product is
    queued in front of every reader so that the readers run late)."""
    import torch
    from sharpnet_b200.tensor import GPUTensor
    lib, h = wrapper.lib, wrapper.handle
    rows, cols, steps, slots = 2048, 1024, 6, 2
    host = [torch.empty(rows, cols).pin_memory() for _ in range(steps)]
    for i, t in enumerate(host):
        t.copy_(torch.from_numpy(orc.uniform((rows, cols), -1, 1, 50 + i)))
    slot_buf = [GPUTensor((rows, cols), None, wrapper) for _ in range(slots)]
    sums = [GPUTensor((cols,), None, wrapper) for _ in range(steps)]
    big = GPUTensor((4096, 4096), orc.uniform((4096, 4096), -1, 1, 7), wrapper)
    big_out = GPUTensor((4096, 4096), None, wrapper)
    st = ctypes.c_void_p()
    assert lib.snb200_stager_create(h, slots, ctypes.byref(st)) == 0
    try:
        assert lib.snb200_stager_acquire(st, 0) == 7                     # nothing staged yet
        assert lib.snb200_stager_issue(st, 2, 0, None, None, None) == 7  # no such slot

        def issue(i):
            dst = (ctypes.c_void_p * 1)(slot_buf[i % slots].Pointer)
            src = (ctypes.c_void_p * 1)(host[i].data_ptr())
            n = (ctypes.c_longlong * 1)(rows * cols * 4)
            assert lib.snb200_stager_issue(st, i % slots, 1, dst, src, n) == 0
        issue(0)
        for i in range(steps):
            assert lib.snb200_stager_acquire(st, i % slots) == 0
            if i + 1 < steps:
                issue(i + 1)
            big_out.Dot(big, False, big, False, 1.0, 0.0)                 # ~0.5 ms in front of the reader
            slot_buf[i % slots].Compute_BiasGradient_from_dy(sums[i])
            assert lib.snb200_stager_release(st, i % slots) == 0
        wrapper.check_device_status()
        for i in range(steps):
            want = host[i].double().sum(0).numpy()
            assert np.abs(sums[i].ContentAsFloatArray() - want).max() <= 1e-5 * np.sqrt(rows) + 1e-6, i
    finally:
        assert lib.snb200_stager_destroy(st) == 0
    # page-locking caller memory
    arr = np.zeros(1 << 16, np.float32)
    assert lib.snb200_host_pin(ctypes.c_void_p(arr.ctypes.data), arr.nbytes) == 0
    assert lib.snb200_host_unpin(ctypes.c_void_p(arr.ctypes.data)) == 0
    assert lib.snb200_host_pin(None, 16) == 7


@pytest.mark.parametrize("batch,panels", [(256, 1), (1024, 4), (900, 3)])
def test_host_staging_class_feeds_the_stack(wrapper, batch, panels):
    # whole mini-batches, and x staged as row panels that the first layer consumes one by one (the ragged case:
    # 900 rows in panels of 384, 384 and 132)
    from sharpnet_b200 import ACT_IDENTITY, ACT_RELU
    from sharpnet_b200.data_parallel import DenseStack, HostStaging, training_step
    import torch
    dims = (128, 96, 32)
    x, dy, Ws, bs = _problem(batch, dims, 300)
    stack = DenseStack(wrapper, batch, dims, (ACT_RELU, ACT_IDENTITY), Ws)
    _load(stack, np.zeros_like(x), np.zeros_like(dy), bs)
    xh, dyh = torch.from_numpy(x).pin_memory(), torch.from_numpy(dy).pin_memory()
    staging = HostStaging(stack, xh, dyh, panels=panels)
    assert len(staging.panels) == panels and staging.panels[-1][1] == batch
    staging.issue(0)
    for i in range(3):
        staging.bind(i)
        if i + 1 < 3:
            staging.issue(i + 1)
        training_step(stack)
        staging.release(i)
    wrapper.check_device_status()
    staging.close()
    a_dev = _activations(stack)
    np.testing.assert_array_equal(a_dev[0], x)                   # the staged input is what the step read
    grads, gmax = _oracle_backward(a_dev, dy, Ws, (orc.ACT_RELU, orc.ACT_IDENTITY))
    _check_gradients(stack, grads, gmax, a_dev, batch)


# ------------------------------------------------------------------------------------------ two ranks
def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _two_gpus():
    import torch
    return torch.cuda.is_available() and torch.cuda.device_count() >= 2


_CHILD = r"""
import os, sys, json
import numpy as np
sys.path.insert(0, {root!r})
import torch
import torch.distributed as dist
from oracle import sharpnet_oracle as orc
from sharpnet_b200 import ACT_IDENTITY, ACT_RELU
from sharpnet_b200.data_parallel import DenseStack, GradientAllReduce, SgdUpdate, shard_rows, training_step
from sharpnet_b200.tensor import GPUWrapper
sys.path.insert(0, os.path.join({root!r}, "tests"))
from test_data_parallel_gpu import _problem, _load, _oracle_forward, _oracle_backward, _check_gradients, _activations
rank, world = int(sys.argv[1]), int(sys.argv[2])
os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = sys.argv[3]
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
torch.cuda.set_device(rank)
dist.init_process_group("gloo", rank=rank, world_size=world)
def bcast(b):
    obj = [b]; dist.broadcast_object_list(obj, src=0); return obj[0]
batch, dims = 768, (256, 192, 128, 40)
acts = (ACT_RELU, ACT_RELU, ACT_IDENTITY)
x, dy, Ws, bs = _problem(batch, dims, 500)
w = GPUWrapper.FromDeviceId(rank)
r0, r1 = shard_rows(batch, world, rank)
reducer = GradientAllReduce(rank, world, rank, bcast)
for with_update in (False, True):
    stack = DenseStack(w, r1 - r0, dims, acts, Ws)
    _load(stack, x[r0:r1], dy[r0:r1], bs)
    upd = SgdUpdate(stack, 0.05, batch, momentum=0.9) if with_update else None
    training_step(stack, reducer, torch.cuda.current_stream(), upd)
    torch.cuda.synchronize()
    w.check_device_status()
    # the activations of the whole batch, gathered from both replicas, then the oracle on the FULL batch
    mine = [torch.from_numpy(t) for t in _activations(stack)]
    full = []
    for t in mine:
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t)
        full.append(torch.cat(parts).numpy())
    oacts = (orc.ACT_RELU, orc.ACT_RELU, orc.ACT_IDENTITY)
    ref = _oracle_forward(x, Ws, bs, oacts)
    for i in range(1, 4):
        assert orc.scaled_error(full[i], ref[i], dims[i - 1], 4.5, 1.0) <= 1e-5 * i
    grads, gmax = _oracle_backward(full, dy, Ws, oacts)
    _check_gradients(stack, grads, gmax, full, batch)          # every replica holds the SUM over both shards
    if with_update:
        for i in range(3):
            want = Ws[i].copy(); v = np.zeros_like(want)
            orc.update_sgd_optimizer(want, 0.05 / batch, 0.9, False, stack.dW[i].ContentAsFloatArray(), v)
            np.testing.assert_allclose(stack.W[i].ContentAsFloatArray(), want, rtol=0, atol=1e-7)
# every replica holds the same bits
flat = torch.cat([t.storage[: t.Count] for t in stack.dW + stack.db]).cpu()
gathered = [torch.empty_like(flat) for _ in range(world)]
dist.all_gather(gathered, flat)
assert all(torch.equal(gathered[0], g) for g in gathered)
dist.barrier()
reducer.close()
dist.destroy_process_group()
print("rank", rank, "ok")
"""


@pytest.mark.skipif(not _two_gpus(), reason="needs two GPUs")
def test_two_rank_training_step_sums_gradients(tmp_path):
    """One process per GPU: each runs DenseStack on its row shard with GradientAllReduce (with and without the
    optimizer step on the side stream); dW, db and the updated W must equal the oracle's on the full batch."""
    script = tmp_path / "child.py"
    script.write_text(_CHILD.format(root=ROOT))
    port = str(_free_port())
    procs = [subprocess.Popen([sys.executable, str(script), str(r), "2", port], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {r} ok" in out, out[-3000:]


@pytest.mark.skipif(not _two_gpus(), reason="needs two GPUs")
def test_thread_per_gpu_communicator_sums():
    """snb200_comm_init_all: one process, one host thread per GPU -- SharpNet's own model
    (Prod/Networks/Network.cs:71-83)."""
    import torch
    from sharpnet_b200.tensor import GPUWrapper
    ws = [GPUWrapper(d) for d in range(2)]
    lib = ws[0].lib
    try:
        handles = (ctypes.c_void_p * 2)(ws[0].handle, ws[1].handle)
        st = lib.snb200_comm_init_all(handles, 2)
        if st == 15:
            pytest.skip("NCCL is not installed")
        assert st == 0
        bufs = [torch.full((1 << 20,), float(d + 1), dtype=torch.float32, device=f"cuda:{d}") for d in range(2)]
        status = [None, None]

        def run(d):
            status[d] = lib.snb200_allreduce_sum(ws[d].handle, ctypes.c_void_p(bufs[d].data_ptr()), bufs[d].numel())
            ws[d].check_device_status()
        threads = [threading.Thread(target=run, args=(d,)) for d in range(2)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(120)
        assert status == [0, 0]
        for b in bufs:
            assert float(b.min()) == 3.0 == float(b.max())
    finally:
        for w in ws:
            lib.snb200_comm_destroy(w.handle)
            lib.snb200_destroy(w.handle)
            w.handle = None
