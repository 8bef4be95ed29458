"""Host-side logic of the data-parallel Dense step, on CPU with two gloo ranks: row sharding as in
Prod/Networks/Network.cs:1229-1258 and gradient SUM across replicas as in
Prod/Networks/NetworkMultiGPUSupport.cs:161-173.  The per-replica arithmetic is the CPU oracle's
(this is a test); the reduction is a real torch.distributed all-reduce."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import sharpnet_oracle as orc
from sharpnet_b200.data_parallel import MLP_DIMS, mlp_step_flops, shard_rows

DIMS = (24, 16, 16, 5)
ACTS = (orc.ACT_RELU, orc.ACT_RELU, orc.ACT_IDENTITY)
BATCH = 12


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _grads(x, dy, Ws):
    a = [x]
    for i in range(3):
        a.append(orc.dense_forward(a[-1], Ws[i], np.zeros(DIMS[i + 1], np.float32), ACTS[i], orc.W_OUT_IN)[1])
    g, out = dy, []
    for i in (2, 1, 0):
        _, dW, db, g = orc.dense_backward(a[i], Ws[i], g, ACTS[i], a[i + 1], None, 1.0, orc.W_OUT_IN, need_dx=i > 0)
        out.append((dW, db))
    return out[::-1]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x = orc.normal((BATCH, DIMS[0]), 0, 1, 1)
    dy = orc.normal((BATCH, DIMS[-1]), 0, 1, 2)
    Ws = [orc.glorot_uniform((DIMS[i + 1], DIMS[i]), 3 + i) for i in range(3)]
    r0, r1 = shard_rows(BATCH, world, rank)
    local = _grads(x[r0:r1], dy[r0:r1], Ws)
    flat = torch.from_numpy(np.concatenate([np.concatenate([dW.ravel(), db.ravel()]) for dW, db in local]))
    dist.all_reduce(flat, op=dist.ReduceOp.SUM)          # what snb200_allreduce_sum does on the GPUs
    if rank == 0:
        full = _grads(x, dy, Ws)
        want = np.concatenate([np.concatenate([dW.ravel(), db.ravel()]) for dW, db in full])
        ret["err"] = float(np.max(np.abs(flat.numpy() - want)))
    dist.destroy_process_group()


def test_two_rank_gradient_sum_matches_full_batch():
    port = _free_port()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
        assert ret["err"] < 1e-5


def test_shard_rows_follows_the_reference_split():
    # master rows [0, b), worker i rows [(1+i) b, (2+i) b)
    assert [shard_rows(65536, 8, r) for r in range(8)] == [(r * 8192, (r + 1) * 8192) for r in range(8)]
    assert shard_rows(12, 1, 0) == (0, 12)
    with pytest.raises(ValueError):
        shard_rows(10, 4, 0)         # the batch must be a multiple of the number of workers
    with pytest.raises(ValueError):
        shard_rows(8, 2, 2)


def test_step_flops_match_the_stated_work():
    # 12.61 TFLOP per step for batch 65536, 4096 -> 4096 -> 4096 -> 1000
    assert abs(mlp_step_flops(65536, MLP_DIMS) / 1e12 - 12.61) < 0.01


class _FakeTensor:
    def __init__(self, count, name):
        self.Count, self.Pointer, self.Shape = count, name, [count]


class _FakeLib:
    """Records the C-ABI calls the host logic makes (no device needed): the order of the backward products, where
    the gradient hooks fire, and when SMs are kept free for the collective."""
    def __init__(self):
        self.calls = []

    def snb200_dense_fwd(self, h, layout, M, K, N, x, W, b, act, z, y):
        self.calls.append(("fwd", y))
        return 0

    def snb200_dense_bwd(self, h, layout, M, K, N, x, W, dy, act, y, z, mult, dz, dx, dW, db):
        self.calls.append(("bwd", dW, dx, db, act))
        return 0

    def snb200_dense_bwd_weight_rows(self, h, layout, M, K, N, x, dz, mult, row0, rows, dW):
        self.calls.append(("dw_rows", dW, None, None, (row0, rows)))
        return 0


class _FakeWrapper:
    def __init__(self):
        self.lib, self.handle, self.tuning = _FakeLib(), "h", []

    def set_tuning(self, key, value):
        self.tuning.append((len(self.lib.calls), key, value))


def _fake_stack(dims, acts):
    from sharpnet_b200.data_parallel import DenseStack
    s = DenseStack.__new__(DenseStack)
    s.w, s.batch, s.dims, s.acts, s.layout = _FakeWrapper(), 8, list(dims), list(acts), 0
    n = len(dims) - 1
    s.W = [_FakeTensor(dims[i] * dims[i + 1], f"W{i}") for i in range(n)]
    s.b = [_FakeTensor(dims[i + 1], f"b{i}") for i in range(n)]
    s.dW = [_FakeTensor(dims[i] * dims[i + 1], f"dW{i}") for i in range(n)]
    s.db = [_FakeTensor(dims[i + 1], f"db{i}") for i in range(n)]
    s.x = _FakeTensor(8 * dims[0], "x")
    s.y = [_FakeTensor(8 * dims[i + 1], f"y{i}") for i in range(n)]
    s.dz = [None if acts[i] == 5 else _FakeTensor(8 * dims[i + 1], f"dz{i}") for i in range(n)]
    s.dx = [None] + [_FakeTensor(8 * dims[i], f"dx{i}") for i in range(1, n)]
    s.dy = _FakeTensor(8 * dims[-1], "dy")
    s.reserve_pending = False
    s.input_panels = s.before_panel = s.before_backward = None
    s.dw_row_panels = 1
    for t, i in zip(s.W, range(n)):
        t.Shape = [dims[i + 1], dims[i]]
    return s


def test_backward_queues_gradients_before_dx_and_the_smallest_gradient_last():
    stack = _fake_stack((4096, 4096, 4096, 1000), (1, 1, 5))          # ReLU, ReLU, identity
    events = []
    stack.backward(after_gradients=lambda i: events.append(("grads", i, len(stack.w.lib.calls))),
                   after_layer=lambda i: events.append(("layer", i, len(stack.w.lib.calls))), defer_smallest=True)
    calls = stack.w.lib.calls
    # layer 2 (the smallest weights): db now, dx, dW at the very end; layers 1 and 0: dW + db, then dx
    assert [(c[1], c[2]) for c in calls] == [(None, None), (None, "dx2"), ("dW1", None), (None, "dx1"), ("dW0", None),
                                             ("dW2", None)]
    assert calls[0][3] == "db2" and calls[-1][3] is None            # the bias gradient is not recomputed
    assert calls[1][4] == 5 and calls[3][4] == 5                     # dx alone runs on the stored dz: no activation
    # the gradient hook fires right behind each dW product, before that layer's dx
    assert events == [("grads", 1, 3), ("layer", 1, 4), ("grads", 0, 5), ("layer", 0, 5), ("grads", 2, 6), ("layer", 2, 6)]
    # without deferral: layer order 2, 1, 0
    stack2 = _fake_stack((64, 32, 16), (1, 5))
    order = []
    stack2.backward(after_gradients=order.append)
    assert order == [1, 0]
    assert [(c[1], c[2]) for c in stack2.w.lib.calls] == [("dW1", None), (None, "dx1"), ("dW0", None)]


def test_last_large_weight_gradient_goes_out_in_row_panels():
    # layer 0's dW as two row panels, each followed by its reduction; the smallest layer's dW still comes last
    stack = _fake_stack((4096, 4096, 4096, 1000), (1, 1, 5))
    stack.dw_row_panels = 2
    events = []
    stack.backward(after_gradients=lambda i: events.append(("grads", i, len(stack.w.lib.calls))),
                   defer_smallest=True,
                   after_gradient_rows=lambda i, r0, n, last: events.append(("rows", i, r0, n, last, len(stack.w.lib.calls))))
    calls = stack.w.lib.calls
    assert [c[0] for c in calls] == ["bwd", "bwd", "bwd", "bwd", "bwd", "dw_rows", "dw_rows", "bwd"]
    assert calls[4][1] is None and calls[4][3] == "db0"              # dz and db of layer 0 without its dW
    assert [c[4] for c in calls[5:7]] == [(0, 2048), (2048, 2048)] and calls[7][1] == "dW2"
    assert events == [("grads", 1, 3), ("rows", 0, 0, 2048, False, 6), ("rows", 0, 2048, 2048, True, 7), ("grads", 2, 8)]
    # without a row hook the layer runs as one product
    stack = _fake_stack((64, 32, 16), (1, 5))
    stack.dw_row_panels = 2
    stack.backward(after_gradients=lambda i: None)
    assert [c[0] for c in stack.w.lib.calls] == ["bwd", "bwd", "bwd"]


def test_sm_reservation_covers_exactly_one_product_after_each_reduction():
    from sharpnet_b200 import _capi
    stack = _fake_stack((64, 32, 16), (1, 5))

    def fake_reduce(i):             # what GradientAllReduce.reduce_layer does on the compute handle
        stack.w.set_tuning(_capi.TUNE_SM_RESERVE, 16)
        stack.reserve_pending = True
    stack.backward(after_gradients=fake_reduce)
    # calls: dW1(+db1) | reduce -> reserve | dx1 -> release | dW0 | reduce -> reserve | end of the pass -> release
    assert stack.w.tuning == [(1, _capi.TUNE_SM_RESERVE, 16), (2, _capi.TUNE_SM_RESERVE, 0), (3, _capi.TUNE_SM_RESERVE, 16),
                              (3, _capi.TUNE_SM_RESERVE, 0)]


def test_reservation_is_made_only_where_the_collective_is_long_against_the_product():
    """At 8 GPUs the 67 MB reduction of a 4096 x 4096 layer takes about as long as a third of the product queued
    behind it, so that product leaves SMs free; at 2 GPUs the same product is four times longer and keeps them."""
    from sharpnet_b200.data_parallel import GradientAllReduce
    for world, rows, expected in ((8, 8192, True), (2, 32768, False)):
        stack = _fake_stack((4096, 4096, 4096, 1000), (1, 1, 5))
        stack.batch = rows
        r = object.__new__(GradientAllReduce)
        r.world, r.COLLECTIVE_CTAS = world, 16
        assert r._worth_reserving(stack, 1) is expected
        assert r._worth_reserving(stack, 2) is expected   # the 16 MB reduction of the output layer scales the same way


def test_host_binds_to_the_numa_node_of_its_gpu(tmp_path):
    # a fake sysfs: the GPU at 0000:1b:00.0 hangs off node 1 (CPUs 8-15,24-27); the process may use CPUs 0-11 and 24
    from sharpnet_b200.data_parallel import bind_host_to_device_node, _parse_cpulist
    dev = tmp_path / "bus" / "pci" / "devices" / "0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    node = tmp_path / "devices" / "system" / "node" / "node1"
    node.mkdir(parents=True)
    (node / "cpulist").write_text("8-15,24-27\n")
    assert _parse_cpulist("0-3,7,9-10") == {0, 1, 2, 3, 7, 9, 10}
    calls = []
    allowed = set(range(12)) | {24}
    got = bind_host_to_device_node("0000:1B:00.0", str(tmp_path), calls.append, lambda: allowed)
    assert got == {8, 9, 10, 11, 24} and calls == [got]
    # unknown node, missing device, or no CPU in common: nothing is changed
    (dev / "numa_node").write_text("-1\n")
    assert bind_host_to_device_node("0000:1b:00.0", str(tmp_path), calls.append, lambda: allowed) is None
    assert bind_host_to_device_node("0000:99:00.0", str(tmp_path), calls.append, lambda: allowed) is None
    (dev / "numa_node").write_text("1\n")
    assert bind_host_to_device_node("0000:1b:00.0", str(tmp_path), calls.append, lambda: {0, 1}) is None
    assert len(calls) == 1
