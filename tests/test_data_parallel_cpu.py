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
