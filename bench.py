#!/usr/bin/env python
"""Benchmark of the Tensor.Dot / Dense path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-shapes] [--no-cpu]
  (N > 1: launched by torch.distributed.run, one rank per GPU)

A step is one forward + backward pass of the 3-layer MLP of benchmark config 5
(batch 65536, 4096 -> 4096 -> 4096 -> 1000, ReLU, ReLU, identity; Glorot weights, zero biases,
x ~ N(0,1), upstream gradient ~ N(0,1)) through snb200_dense_fwd / snb200_dense_bwd, the batch rows
sharded over the N GPUs and the weight / bias gradients summed with one all-reduce per layer.
`value` is algorithmic TFLOP/s of the whole job (12.61 TFLOP per step), timed on the device with
inputs resident in HBM; `e2e` is the same step driven from pinned HOST buffers (x and the upstream
gradient copied in through double-buffered staging, the bias gradients copied out, every step).  `shapes` lists every Dot / batched /
Dense shape of benchmark configs 1-5 with its own TFLOP/s, roofline fraction and error vs fp64 (N = 1).

--impl reference times the reference's CPU path (MKL sgemm through the oracle) on a row sample of
the same step, with every host core.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

_emit = print
GLOBAL_BATCH = 65536
DIMS = (4096, 4096, 4096, 1000)
CPU_SAMPLE_ROWS = 4096
L2_BYTES = 126 * 1024 * 1024


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm": d["hbm_gbs"], "bf16_burst": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"],
                "src": "measured"}
    return {"hbm": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "src": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs (read-only)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.idx = device_index
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "100", "-i", str(self.idx)], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.p.terminate()
        self.p.wait()
        self.f.flush()
        rows = [r.strip().split(", ") for r in open(self.f.name) if r.strip()]
        os.unlink(self.f.name)
        sm, mx, pw, reasons = [], [], [], set()
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1])); mx.append(float(r[2])); pw.append(float(r[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.strip().lower() == "active":
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = sorted(s for s, p in zip(sm, pw) if p > 0.5 * max(pw)) or sorted(sm)
        return {"sm_mhz": busy[len(busy) // 2], "sm_max_mhz": max(mx), "power_w_max": max(pw), "samples": len(sm),
                "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------
# reference arm: the CPU path of SharpNet (MKL sgemm), through the oracle
# ------------------------------------------------------------------------------------------------
def cpu_step_sample(rows, seed=17):
    """One forward+backward of the MLP over `rows` batch rows with the CPU oracle; returns a closure."""
    import numpy as np
    import torch
    from oracle import sharpnet_oracle as orc
    torch.set_num_threads(os.cpu_count())
    x = orc.normal((rows, DIMS[0]), 0, 1, seed)
    dy = orc.normal((rows, DIMS[-1]), 0, 1, seed + 1)
    Ws = [orc.glorot_uniform((DIMS[i + 1], DIMS[i]), 14 + i) for i in range(3)]
    bs = [np.zeros(DIMS[i + 1], np.float32) for i in range(3)]
    acts = (orc.ACT_RELU, orc.ACT_RELU, orc.ACT_IDENTITY)

    def step(keep=None):
        a = [x]
        for i in range(3):
            _, y = orc.dense_forward(a[-1], Ws[i], bs[i], acts[i], orc.W_OUT_IN)
            a.append(y)
        g = dy
        for i in (2, 1, 0):
            _, dW, db, g = orc.dense_backward(a[i], Ws[i], g, acts[i], a[i + 1], None, 1.0, orc.W_OUT_IN,
                                              need_dx=(i > 0))
            if keep is not None:
                keep[i] = (dW, db)
        if keep is not None:
            keep["a"] = a
        return db
    step.inputs = (x, dy, Ws, bs, acts)
    return step


def time_cpu(rows, reps):
    """Times the oracle's step on `rows` rows; also returns the step's inputs and its results (MKL, fp32) so that
    the device's step on the same rows can be compared with them."""
    from sharpnet_b200.data_parallel import mlp_step_flops
    step = cpu_step_sample(rows)
    results = {}
    step(results)
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter()
        step()
        ts.append(time.perf_counter() - t0)
    t = sorted(ts)[len(ts) // 2]
    return mlp_step_flops(rows, DIMS) / t / 1e12, t, step.inputs, results


def step_parity(w, torch, inputs, cpu_results):
    """The device's training step on the rows the CPU baseline ran, compared with the oracle: the network output
    against the oracle's own forward pass (MKL, fp32), and every dW / db against the oracle's backward pass in
    float64 AND in MKL fp32, both evaluated on the device's activations (a pre-activation within rounding of zero
    may fall on either side of the ReLU on the two machines; the gradient mask must come from the same values)."""
    import numpy as np
    from oracle import sharpnet_oracle as orc
    from sharpnet_b200.data_parallel import MLP_ACTS, DenseStack, training_step
    x, dy, Ws, bs, acts = inputs
    rows = x.shape[0]
    stack = DenseStack(w, rows, DIMS, MLP_ACTS, Ws)
    stack.x.storage.copy_(torch.from_numpy(x).view(-1))
    stack.dy.storage.copy_(torch.from_numpy(dy).view(-1))
    training_step(stack)
    w.check_device_status()
    a_dev = [x] + [t.ContentAsFloatArray() for t in stack.y]
    out = {"rows": rows, "bound": 1e-5, "measure": "max|gpu - ref| / (sqrt(K) * a_max * b_max)"}
    worst = 0.0
    for i in range(3):
        e = orc.scaled_error(a_dev[i + 1], cpu_results["a"][i + 1], DIMS[i], float(np.abs(a_dev[i]).max()),
                             float(np.abs(Ws[i]).max()))
        out[f"y{i}_vs_mkl"] = float(f"{e:.3e}")
        worst = max(worst, e / (i + 1))          # layer i's input already carries i rounded products
    g64, g32 = dy, dy
    for i in (2, 1, 0):
        dz, dW64, db64, g64n = orc.dense_backward(a_dev[i], Ws[i], g64, acts[i], a_dev[i + 1], None, 1.0, orc.W_OUT_IN,
                                                  need_dx=i > 0, f64=True)
        _, dW32, db32, g32n = orc.dense_backward(a_dev[i], Ws[i], g32, acts[i], a_dev[i + 1], None, 1.0, orc.W_OUT_IN,
                                                 need_dx=i > 0)
        amax, gmax = float(np.abs(a_dev[i]).max()), float(np.abs(dz).max())
        got_dW, got_db = stack.dW[i].ContentAsFloatArray(), stack.db[i].ContentAsFloatArray()
        for name, got, r64, r32, am in (("dW", got_dW, dW64, dW32, amax), ("db", got_db, db64, db32, 1.0)):
            e64, e32 = orc.scaled_error(got, r64, rows, am, gmax), orc.scaled_error(got, r32, rows, am, gmax)
            out[f"{name}{i}_vs_f64"], out[f"{name}{i}_vs_mkl"] = float(f"{e64:.3e}"), float(f"{e32:.3e}")
            worst = max(worst, e64, e32)
        g64 = None if g64n is None else g64n.astype(np.float32)
        g32 = g32n
    out["worst"] = float(f"{worst:.3e}")
    out["ok"] = bool(worst <= 1e-5)
    del stack
    return out


def dp_check(w, torch, dist, world, rank, reducer, compute_stream):
    """One step of a small stack (batch 1024 per GPU, 512 -> 256 -> 64) through the same training_step and the
    same GradientAllReduce as the timed step; rank 0 compares the all-reduced dW / db it holds with the oracle on
    the FULL batch (float64, masks from the device's activations, gathered from every rank)."""
    import numpy as np
    from oracle import sharpnet_oracle as orc
    from sharpnet_b200 import ACT_IDENTITY, ACT_RELU
    from sharpnet_b200.data_parallel import DenseStack, shard_rows, training_step
    dims, batch = (512, 256, 64), 1024 * world
    acts = (ACT_RELU, ACT_IDENTITY)
    x, dy = orc.normal((batch, dims[0]), 0, 1, 31), orc.normal((batch, dims[-1]), 0, 1, 32)
    Ws = [orc.glorot_uniform((dims[i + 1], dims[i]), 33 + i) for i in range(2)]
    r0, r1 = shard_rows(batch, world, rank)
    stack = DenseStack(w, r1 - r0, dims, acts, Ws)
    stack.x.storage.copy_(torch.from_numpy(x[r0:r1]).reshape(-1))
    stack.dy.storage.copy_(torch.from_numpy(dy[r0:r1]).reshape(-1))
    training_step(stack, reducer, compute_stream)
    torch.cuda.synchronize()
    w.check_device_status()
    y0 = stack.y[0].storage[: stack.y[0].Count].view(r1 - r0, dims[1])
    if world > 1:
        parts = [torch.empty_like(y0) for _ in range(world)] if rank == 0 else None
        dist.gather(y0, parts, dst=0)
        y0_full = torch.cat(parts).cpu().numpy() if rank == 0 else None
    else:
        y0_full = y0.cpu().numpy()
    if rank != 0:
        return None
    a = [x, y0_full, None]
    worst, g = 0.0, dy
    for i in (1, 0):
        dz, dW, db, g = orc.dense_backward(a[i], Ws[i], g, (orc.ACT_RELU, orc.ACT_IDENTITY)[i], a[i + 1], None, 1.0,
                                           orc.W_OUT_IN, need_dx=i > 0, f64=True)
        amax, gmax = float(np.abs(a[i]).max()), float(np.abs(dz).max())
        worst = max(worst, orc.scaled_error(stack.dW[i].ContentAsFloatArray(), dW, batch, amax, gmax),
                    orc.scaled_error(stack.db[i].ContentAsFloatArray(), db, batch, 1.0, gmax))
        g = None if g is None else g.astype(np.float32)
    return {"scaled_err": float(f"{worst:.3e}"), "bound": 1e-5, "ok": bool(worst <= 1e-5), "ranks": world,
            "what": f"all-reduced dW/db of a {dims} stack, batch {batch} over {world} GPUs, vs the oracle on the full batch"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from sharpnet_b200.data_parallel import mlp_step_flops
    # every host thread this process may use: torchrun presets OMP_NUM_THREADS=1 for its children, which would time
    # MKL on one core (the other ranks have left, the cores are free)
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except (AttributeError, OSError):
        torch.set_num_threads(max(1, os.cpu_count() or 1))
    step = cpu_step_sample(CPU_SAMPLE_ROWS)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    v = mlp_step_flops(CPU_SAMPLE_ROWS, DIMS) / dt / 1e12
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": "dot_tflops", "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": dict(workload_config(args.gpus),
                       sample=f"1/{GLOBAL_BATCH // CPU_SAMPLE_ROWS} row sample: {CPU_SAMPLE_ROWS} of the {GLOBAL_BATCH} "
                              "batch rows per step (the rate, not the time, is what compares)"),
        "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": f"{CPU_SAMPLE_ROWS} of {GLOBAL_BATCH} batch rows per step, MKL sgemm via torch CPU "
                                   "(SharpNet's C# cannot be built here: no .NET)"},
        "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    _emit(json.dumps(line))


def workload_config(n):
    return {"workload": "benchmark config 5: 3-layer MLP training step (Dense fwd+bwd), batch 65536, "
                        "4096->4096->4096->1000, ReLU, fp32; rows sharded over the GPUs, dW/db all-reduced",
            "global_batch": GLOBAL_BATCH, "dims": list(DIMS), "parallelism": f"dp{n}",
            "math_mode": "3xTF32 (fp32-accurate)", "l2": "inputs (>1 GB per operand) exceed the 126 MB L2"}


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def time_gemm_shape(w, torch, peaks, name, M, N, K, tA, tB, beta, batch, lo, hi, mode, check_rows=64, min_calls=20,
                    cpu=True, compare=True, view_offset=0):
    """Times one Dot / BatchMatrixMultiplication shape.  The call cycles through enough distinct
    (A, B, C) sets that their total size exceeds twice the L2, so every call finds its operands in
    HBM; the whole loop is timed with one CUDA-event pair on the launching stream."""
    from sharpnet_b200 import MATH_3XTF32
    from sharpnet_b200.tensor import GPUTensor
    w.set_math_mode(mode)
    sa = (batch, K, M) if tA else (batch, M, K)
    sb = (batch, N, K) if tB else (batch, K, N)
    bytes_set = 4.0 * batch * (M * K + K * N + M * N)
    n_sets = int(min(64, max(1, math.ceil(2.0 * L2_BYTES / bytes_set))))
    sets = []
    for _ in range(n_sets):
        if view_offset:      # operands that start `view_offset` floats into their allocation: not 16-byte aligned
            na, nb = batch * sa[1] * sa[2], batch * sb[1] * sb[2]
            A = GPUTensor(sa, wrapper=w, storage=torch.empty(na + view_offset, device=w.device)[view_offset:])
            B = GPUTensor(sb, wrapper=w, storage=torch.empty(nb + view_offset, device=w.device)[view_offset:])
            C = GPUTensor((batch, M, N), None, w)
        else:
            A, B, C = GPUTensor(sa, None, w), GPUTensor(sb, None, w), GPUTensor((batch, M, N), None, w)
        A.storage.uniform_(lo, hi); B.storage.uniform_(lo, hi); C.storage.uniform_(lo, hi)
        sets.append((A, B, C))
    A, B, C = sets[0]
    rows = min(check_rows, M)
    # the rows of matrix 0 that get checked, copied out before the call overwrites C
    a0 = A.storage[: sa[1] * sa[2]].view(sa[1], sa[2])
    a_rows = (a0[:, :rows] if tA else a0[:rows]).contiguous().cpu().numpy()     # stored layout, `rows` rows of op(A)
    b0 = B.storage[: sb[1] * sb[2]].view(sb[1], sb[2]).cpu().numpy()
    c_rows = C.storage[: M * N].view(M, N)[:rows].cpu().numpy().copy()
    C.BatchMatrixMultiplication(A, tA, B, tB, 1.0, beta)
    got = C.storage[: M * N].view(M, N)[:rows].cpu().numpy()
    # error against the CPU oracle on those rows: MKL sgemm (what CpuTensor.Dot runs) and float64
    from oracle import sharpnet_oracle as orc
    errs = {}
    for key, f64 in (("mkl", False), ("f64", True)):
        ref = orc.batch_matrix_multiplication(a_rows[None], tA, b0[None], tB, c_rows[None].copy(), 1.0, beta, f64=f64)
        errs[key] = orc.scaled_error(got, ref[0], K, hi, hi)
    err = errs["f64"]
    del a0, b0, a_rows, c_rows, got
    calls = max(min_calls, n_sets) if bytes_set < 1e9 else 5
    # The timed loop calls the C ABI directly with arguments converted once, so that the host side of a
    # call is a few hundred nanoseconds, as it is for SharpNet's P/Invoke, and not Python bookkeeping.
    import ctypes
    lib, h = w.lib, w.handle
    fixed = (int(tA), int(tB), sa[1], sa[2], ctypes.c_longlong(sa[1] * sa[2]), sb[1], sb[2],
             ctypes.c_longlong(sb[1] * sb[2]), ctypes.c_longlong(M * N), batch, ctypes.c_float(1.0))
    argsets = [(h,) + fixed + (a.Pointer, b.Pointer, ctypes.c_float(beta), c.Pointer) for a, b, c in sets]
    gemm = lib.snb200_batched_gemm
    for i in range(min(3, calls)):
        if gemm(*argsets[i % n_sets]) != 0:
            raise RuntimeError(w.lib.snb200_last_error_string(h))
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(calls):
        gemm(*argsets[i % n_sets])
    e1.record()
    torch.cuda.synchronize()
    w.check_device_status()
    ms = e0.elapsed_time(e1) / calls
    flops = 2.0 * M * N * K * batch
    byts = bytes_set + (4.0 * batch * M * N if beta != 0 else 0.0)
    tpeak3 = peaks["bf16_burst"] / 2 / 3
    tens = tpeak3 * 3 if mode == 1 else tpeak3
    t_tensor, t_hbm = flops / (tens * 1e12), byts / (peaks["hbm"] * 1e9)
    return {"shape": name, "mode": {0: "3xTF32", 1: "TF32", 2: "FP32_SIMT", 3: "TF32+BF16x2"}[mode], "kernel": w.last_kernel(),
            "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 2), "gbs": round(byts / ms / 1e6, 1),
            "bound": "tensor" if t_tensor >= t_hbm else "hbm",
            "roofline_frac": round(max(t_tensor, t_hbm) / (ms * 1e-3), 3), "scaled_err_vs_f64": float(f"{err:.3e}"),
            "scaled_err_vs_mkl": float(f"{errs['mkl']:.3e}"), "checked_rows": rows,
            "operand_sets": n_sets, "calls": calls,
            **(library_comparators(torch, sets, sa, sb, M, N, K, tA, tB, beta, batch, mode, calls, ms, cpu)
               if compare else {})}


def _median(v):
    v = sorted(v)
    return v[len(v) // 2]


def library_comparators(torch, sets, sa, sb, M, N, K, tA, tB, beta, batch, mode, calls, our_ms, cpu):
    """What SharpNet runs today on the same operands, timed beside our kernel (bench-only: nothing in the library
    calls these).  cublas_sgemm_ms: torch on the device with TF32 off = cuBLAS sgemm default math, what
    GPUTensor.Dot / BatchMatrixMultiplication reach (Prod/GPU/GpuTensor.cs:1218,1192); in TF32 mode also cuBLAS with
    TF32 on.  mkl_ms: torch on the CPU (MKL sgemm, all host cores) = CpuTensor.Dot; a batch both as the reference's
    serial loop of Dot calls (Prod/CPU/CpuTensor.cs:3012-3024) and as one baddbmm."""
    out = {}
    views = []
    for A, B, C in sets:
        a = A.storage[: batch * sa[1] * sa[2]].view(batch, sa[1], sa[2])
        b = B.storage[: batch * sb[1] * sb[2]].view(batch, sb[1], sb[2])
        c = C.storage[: batch * M * N].view(batch, M, N)
        views.append((a.transpose(1, 2) if tA else a, b.transpose(1, 2) if tB else b, c))

    def dev_time(allow_tf32):
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = allow_tf32
        try:
            def call(i):
                a, b, c = views[i % len(views)]
                if beta != 0:
                    torch.baddbmm(c, a, b, beta=beta, alpha=1.0, out=c)
                else:
                    torch.bmm(a, b, out=c)
            for i in range(min(3, calls)):
                call(i)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(calls):
                call(i)
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / calls
        finally:
            torch.backends.cuda.matmul.allow_tf32 = prev
    sg = dev_time(False)
    out["cublas_sgemm_ms"] = round(sg, 4)
    out["x_vs_cublas_sgemm"] = round(sg / our_ms, 2)
    if mode == 1:
        tf = dev_time(True)
        out["cublas_tf32_ms"] = round(tf, 4)
        out["x_vs_cublas_tf32"] = round(tf / our_ms, 2)
    if cpu and mode == 0:        # once per shape, not per math mode
        a, b, c = (t.cpu() for t in views[0])
        big = 2.0 * M * N * K * batch > 2e12
        reps, warm = (1, 0) if big else (5, 3)

        def cpu_time(fn):
            for _ in range(warm):
                fn()
            ts = []
            for _ in range(reps):
                t0 = time.perf_counter()
                fn()
                ts.append(time.perf_counter() - t0)
            return _median(ts) * 1e3
        if batch == 1:
            fn = (lambda: torch.addmm(c[0], a[0], b[0], beta=beta, alpha=1.0, out=c[0])) if beta != 0 else \
                 (lambda: torch.mm(a[0], b[0], out=c[0]))
            out["mkl_ms"] = round(cpu_time(fn), 3)
        else:
            def loop():
                for i in range(batch):
                    torch.mm(a[i], b[i], out=c[i])
            out["mkl_serial_loop_ms"] = round(cpu_time(loop), 3)
            out["mkl_ms"] = round(cpu_time(lambda: torch.bmm(a, b, out=c)), 3)
        out["mkl_runs"] = "one run, no warm-up" if big else "median of 5 after 3 warm-ups"
        out["x_vs_mkl"] = round(out["mkl_ms"] / our_ms, 1)
    return out


def sharded_gemm(w, torch, world, rank, barrier, max_over_ranks, calls=5):
    """benchmark config 5a on N GPUs: C = A * B with 16384^3 operands, A and C sharded by rows of M over the ranks, B
    replicated; no collective on the data path.  Returns aggregate TFLOP/s = 2 * 16384^3 / (max over ranks of the
    device time per call)."""
    import ctypes
    from sharpnet_b200 import MATH_3XTF32
    n = 16384
    rows = n // world
    w.set_math_mode(MATH_3XTF32)
    g = torch.Generator(device="cuda").manual_seed(13 + rank)
    A = torch.empty(rows, n, device="cuda").uniform_(-1, 1, generator=g)
    B = torch.empty(n, n, device="cuda").uniform_(-1, 1, generator=torch.Generator(device="cuda").manual_seed(13))
    C = torch.empty(rows, n, device="cuda")
    P = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    call = lambda: w.lib.snb200_gemm(w.handle, 0, 0, rows, n, n, n, ctypes.c_float(1.0), P(A), P(B),  # noqa: E731
                                     ctypes.c_float(0.0), P(C))
    for _ in range(3):
        if call() != 0:
            raise RuntimeError(w.lib.snb200_last_error_string(w.handle))
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(calls):
        call()
    e1.record()
    barrier()
    w.check_device_status()
    ms = max_over_ranks(e0.elapsed_time(e1) / calls)
    return {"shape": f"cfg5a 16384^3 NN, rows of A and C sharded over {world} GPUs, B replicated, no collective",
            "mode": "3xTF32", "kernel": w.last_kernel(), "ms": round(ms, 4), "calls": calls,
            "tflops_aggregate": round(2.0 * n ** 3 / ms / 1e9, 2)}


def companion_table(w, torch, peaks):
    """Achieved HBM GB/s of the bandwidth-bound kernels of the path on config-sized tensors
    (16384 x 4096 fp32 = 256 MiB per tensor, so every call streams more than the L2 holds)."""
    import ctypes
    lib, h = w.lib, w.handle
    M, N = 16384, 4096          # 256 MiB per tensor: every call streams more than the L2 holds
    n = M * N
    t = [torch.empty(n, dtype=torch.float32, device=w.device).uniform_(0.1, 1.0) for _ in range(6)]
    db = torch.empty(N, dtype=torch.float32, device=w.device)
    P = lambda x: ctypes.c_void_p(x.data_ptr())  # noqa: E731
    f = ctypes.c_float
    cases = [
        ("bias_grad 16384x4096", 4 * n, lambda: lib.snb200_bias_grad(h, M, N, P(t[0]), P(db))),
        ("bias_add 16384x4096", 8 * n, lambda: lib.snb200_bias_add(h, M, N, P(db), P(t[1]))),
        ("activation_fwd swish", 8 * n, lambda: lib.snb200_activation_fwd(h, 6, n, P(t[0]), P(t[1]))),
        ("activation_bwd swish", 16 * n, lambda: lib.snb200_activation_bwd(h, 6, n, P(t[2]), P(t[0]), P(t[1]), P(t[3]))),
        ("axpy", 12 * n, lambda: lib.snb200_axpy(h, n, f(0.5), P(t[0]), P(t[4]))),
        ("sgd_update momentum", 20 * n, lambda: lib.snb200_sgd_update(h, n, f(1e-3), f(0.9), 0, P(t[0]), P(t[4]), P(t[5]))),
        ("adam_update", 28 * n, lambda: lib.snb200_adam_update(h, n, 1e-3, 0.9, 0.999, 1e-8, 0.0, 5, P(t[0]), P(t[4]), P(t[5]), P(t[3]))),
        # head split of 128 sequences x 512 steps x 16 heads x 64: [128, 512, 16, 64] -> [128, 16, 512, 64]
        ("transpose_second_third 128x512x16x64", 8 * n, lambda: lib.snb200_transpose_second_third(h, 128, 512, 16, 64, P(t[0]), P(t[1]))),
        ("softmax_fwd 524288x128", 8 * n, lambda: lib.snb200_softmax_fwd(h, n // 128, 128, P(t[0]), P(t[1]))),
    ]
    out = []
    for name, byts, call in cases:
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            call()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 20
        gbs = byts / ms / 1e6
        out.append({"kernel": name, "ms": round(ms, 4), "gbs": round(gbs, 1), "bound": "hbm",
                    "roofline_frac": round(gbs / peaks["hbm"], 3)})
    return out


def dense_and_attention_table(w, torch, peaks):
    """benchmark config 3 (Dense 4096 x 3072 -> 1024, bias, ReLU and Swish, forward and backward through the fused
    entry points) and an attention block of the reference's own timing sandbox
    (Tests/NonReg/ParallelRunWithTensorFlow.cs:415-490: 256 heads x [128 x 64]), timed like the Dot shapes."""
    import ctypes
    from sharpnet_b200 import ACT_RELU, ACT_SWISH, MATH_3XTF32
    lib, h = w.lib, w.handle
    w.set_math_mode(MATH_3XTF32)
    P = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    new = lambda *shape: torch.empty(*shape, dtype=torch.float32, device=w.device)  # noqa: E731
    tpeak3 = peaks["bf16_burst"] / 2 / 3
    out = []

    def timed(name, flops, byts, sets, call):
        for i in range(3):
            call(sets[i % len(sets)])
        torch.cuda.synchronize()
        n = max(10, len(sets))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            call(sets[i % len(sets)])
        e1.record()
        torch.cuda.synchronize()
        w.check_device_status()
        ms = e0.elapsed_time(e1) / n
        t_tensor, t_hbm = flops / (tpeak3 * 1e12), byts / (peaks["hbm"] * 1e9)
        out.append({"shape": name, "mode": "3xTF32", "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 2),
                    "gbs": round(byts / ms / 1e6, 1), "bound": "tensor" if t_tensor >= t_hbm else "hbm",
                    "roofline_frac": round(max(t_tensor, t_hbm) / (ms * 1e-3), 3), "operand_sets": len(sets)})

    M, K, N = 4096, 3072, 1024
    sets = []
    for _ in range(3):    # 3 x ~190 MB of operands: more than twice the L2
        d = {"x": new(M, K).normal_(), "W": new(K, N).uniform_(-0.038, 0.038), "b": new(N).zero_(), "dy": new(M, N).normal_(),
             "y": new(M, N), "z": new(M, N), "dz": new(M, N), "dx": new(M, K), "dW": new(K, N), "db": new(N)}
        sets.append(d)
    for act, an in ((ACT_RELU, "ReLU"), (ACT_SWISH, "Swish")):
        zarg = (lambda d: P(d["z"])) if act == ACT_SWISH else (lambda d: None)
        timed(f"cfg3 dense_fwd 4096x3072->1024 bias+{an} (W [in,out])", 2.0 * M * K * N,
              4.0 * (M * K + K * N + N + M * N * (2 if act == ACT_SWISH else 1)), sets,
              lambda d: lib.snb200_dense_fwd(h, 1, M, K, N, P(d["x"]), P(d["W"]), P(d["b"]), act, zarg(d), P(d["y"])))
        timed(f"cfg3 dense_bwd 4096x3072->1024 {an}: dz, db, dW, dx", 4.0 * M * K * N,
              4.0 * (2 * M * N + 2 * M * K + 2 * K * N + N), sets,
              lambda d: lib.snb200_dense_bwd(h, 1, M, K, N, P(d["x"]), P(d["W"]), P(d["dy"]), act, P(d["y"]), zarg(d),
                                             ctypes.c_float(1.0), P(d["dz"]), P(d["dx"]), P(d["dW"]), P(d["db"])))
    # what Linear + ActivationLayer do on the GPU today (Prod/Layers/Linear.cs:125-132, ActivationLayer.cs:32-38):
    # cuBLAS sgemm (default math), a bias pass and an activation pass -- library comparators, bench only
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        def unfused_fwd(d):
            torch.mm(d["x"], d["W"], out=d["y"])
            d["y"].add_(d["b"])
            torch.relu_(d["y"])
            return 0
        timed("cfg3 UNFUSED reference sequence fwd: cuBLAS sgemm + bias pass + ReLU pass (comparator)", 2.0 * M * K * N,
              4.0 * (M * K + K * N + N + M * N), sets, unfused_fwd)
        out[-1]["mode"] = "cuBLAS fp32"

        def unfused_bwd(d):
            torch.mul(d["dy"], (d["y"] > 0), out=d["dz"])           # activation backward pass
            torch.mm(d["x"].t(), d["dz"], out=d["dW"])              # dW
            torch.sum(d["dz"], 0, out=d["db"])                      # bias gradient pass
            torch.mm(d["dz"], d["W"].t(), out=d["dx"])              # dx
            return 0
        timed("cfg3 UNFUSED reference sequence bwd: ReLU' pass + 2 cuBLAS sgemm + column-sum pass (comparator)",
              4.0 * M * K * N, 4.0 * (2 * M * N + 2 * M * K + 2 * K * N + N), sets, unfused_bwd)
        out[-1]["mode"] = "cuBLAS fp32"
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    # the same sequence through this library's own separate entry points (Dot, bias add, activation)
    def own_unfused_fwd(d):
        st = lib.snb200_gemm(h, 0, 0, M, K, K, N, ctypes.c_float(1.0), P(d["x"]), P(d["W"]), ctypes.c_float(0.0), P(d["y"]))
        st = st or lib.snb200_bias_add(h, M, N, P(d["b"]), P(d["y"]))
        return st or lib.snb200_activation_fwd(h, ACT_RELU, M * N, P(d["y"]), P(d["y"]))
    timed("cfg3 unfused through this library: snb200_gemm + bias_add + activation_fwd (3 launches)", 2.0 * M * K * N,
          4.0 * (M * K + K * N + N + M * N), sets, own_unfused_fwd)
    B, T, E = 256, 128, 64
    asets = []
    for _ in range(8):    # 8 x 42 MB
        asets.append({k: new(B, T, E).uniform_(-1, 1) for k in ("Q", "K", "V", "dy", "y", "dQ", "dK", "dV")} |
                     {"w": new(B, T, T), "ds": new(B, T, T)})
    timed("attention fwd 256 x [128x64], scaled, causal", 4.0 * B * T * T * E, 4.0 * (4 * B * T * E + B * T * T), asets,
          lambda d: lib.snb200_sdpa_fwd(h, B, T, T, E, 1, 1, P(d["Q"]), P(d["K"]), P(d["V"]), P(d["w"]), P(d["y"])))
    timed("attention bwd 256 x [128x64]", 8.0 * B * T * T * E, 4.0 * (7 * B * T * E + B * T * T), asets,
          lambda d: lib.snb200_sdpa_bwd(h, B, T, T, E, 1, P(d["Q"]), P(d["K"]), P(d["V"]), P(d["dy"]), P(d["w"]),
                                        P(d["ds"]), P(d["dQ"]), P(d["dK"]), P(d["dV"])))
    # multi-head attention layer (Prod/Layers/MultiheadAttention.cs): 32 sequences x 128 steps, embed 512 = 8 heads x 64,
    # one snb200_mha_fwd / snb200_mha_bwd call each (4 Dense projections, head split / merge permutations, attention
    # core); every buffer allocated once, as the layer's memory pool does
    from sharpnet_b200 import _capi
    Bm, Tm, Em, Hm = 32, 128, 512, 8
    dm = Em // Hm
    desc = _capi.MhaDesc(0, Bm, Tm, Tm, Em, Hm, dm, dm, 1)
    wts = [new(Em, Em).uniform_(-0.05, 0.05) for _ in range(4)] + [new(Em).uniform_(-0.1, 0.1) for _ in range(4)]
    grads = [new(Em, Em) for _ in range(4)] + [new(Em) for _ in range(4)]
    xs = [new(Bm, Tm, Em).normal_() for _ in range(3)]
    dxs = [new(Bm, Tm, Em) for _ in range(3)]
    ym, dym = new(Bm, Tm, Em), new(Bm, Tm, Em).normal_()
    state = [new(Bm * Hm, Tm, dm), new(Bm * Hm, Tm, dm), new(Bm * Hm, Tm, dm), new(Bm, Tm, Em), new(Bm * Hm, Tm, Tm)]
    scr = new(lib.snb200_mha_scratch_floats(desc, 1))
    W_, S_, G_ = (_capi.MhaWeights(*[P(t) for t in wts]), _capi.MhaState(*[P(t) for t in state]),
                  _capi.MhaWeights(*[P(t) for t in grads]))
    proj = 2.0 * Bm * Tm * Em * Em * 4
    core = 4.0 * Bm * Hm * Tm * Tm * dm

    def mha_fwd(_):
        return lib.snb200_mha_fwd(h, desc, W_, P(xs[0]), P(xs[1]), P(xs[2]), S_, P(scr), P(ym))

    def mha_fwd_bwd(_):
        mha_fwd(_)
        return lib.snb200_mha_bwd(h, desc, W_, P(xs[0]), P(xs[1]), P(xs[2]), P(dym), S_, ctypes.c_float(1.0), P(scr), G_,
                                  P(dxs[0]), P(dxs[1]), P(dxs[2]))
    launches0 = w.launch_count()
    if mha_fwd_bwd(None) != 0:
        raise RuntimeError(lib.snb200_last_error_string(h))
    n_launch = w.launch_count() - launches0
    timed("multi-head attention fwd 32 x 128 x 512, 8 heads, causal (snb200_mha_fwd)", proj + core,
          4.0 * (4 * Bm * Tm * Em + 4 * Em * Em), [None], mha_fwd)
    timed(f"multi-head attention fwd + bwd 32 x 128 x 512, 8 heads, causal ({n_launch} kernels)", 3.0 * (proj + core),
          4.0 * (8 * Bm * Tm * Em + 8 * Em * Em), [None], mha_fwd_bwd)
    return out


def per_shape_table(w, torch, peaks, large, cpu=True):
    """TFLOP/s, roofline fraction and error vs fp64 of every Dot / batched shape in benchmark configs 1-4
    (`large` false) or of the 16384^3 product of config 5 (`large` true: 35 ms launches that drive the GPU into its
    power cap, so they run after the short kernels)."""
    from sharpnet_b200 import MATH_3XTF32, MATH_TF32
    out = []

    def one(name, M, N, K, tA, tB, beta, batch, lo, hi, mode, check_rows=64, view_offset=0):
        out.append(time_gemm_shape(w, torch, peaks, name, M, N, K, tA, tB, beta, batch, lo, hi, mode, check_rows, cpu=cpu,
                                   view_offset=view_offset))

    if large:
        # the opt-in TF32 + bf16 cross-term mode next to 3xTF32 on the layout it is implemented for
        from sharpnet_b200._capi import MATH_TF32_BF16X2
        for mode in (MATH_3XTF32, MATH_TF32_BF16X2):
            one("8192^3 NT", 8192, 8192, 8192, False, True, 0.0, 1, -1, 1, mode, check_rows=16)
        # SharpNet slices tensors at float granularity (Prod/GPU/GpuTensor.cs:1518-1521): operands TMA cannot load
        one("4096^3 NN, A and B views 4 bytes into their allocations", 4096, 4096, 4096, False, False, 0.0, 1, -1, 1,
            MATH_3XTF32, check_rows=16, view_offset=1)
        one("4096x4095x4097 NT (widths not multiples of 4 floats)", 4096, 4095, 4097, False, True, 0.0, 1, -1, 1,
            MATH_3XTF32, check_rows=16)
    for mode in (MATH_3XTF32, MATH_TF32):
        if large:
            one("cfg5a 16384^3 NN", 16384, 16384, 16384, False, False, 0.0, 1, -1, 1, mode, check_rows=8)
            continue
        one("cfg1 1024x1024x1024 NN", 1024, 1024, 1024, False, False, 0.0, 1, -1, 1, mode)
        for tA in (False, True):
            for tB in (False, True):
                tag = ("T" if tA else "N") + ("T" if tB else "N")
                one(f"cfg2 2048x1536x768 {tag} beta=1", 2048, 1536, 768, tA, tB, 1.0, 1, -1, 1, mode)
        for tA in (False, True):
            for tB in (False, True):
                tag = ("T" if tA else "N") + ("T" if tB else "N")
                one(f"cfg2 skinny 32x4096x4096 {tag} beta=1", 32, 4096, 4096, tA, tB, 1.0, 1, -1, 1, mode)
        one("cfg4a 64x[256x64]x[256x64]^T", 256, 256, 64, False, True, 0.0, 64, -0.1, 0.1, mode)
        one("cfg4b 256x4096x2048 NN (LSTM gates)", 256, 4096, 2048, False, False, 0.0, 1, -0.1, 0.1, mode)
    w.set_math_mode(MATH_3XTF32)
    return out


def cublas_tf32_rate(torch, seconds):
    """cuBLAS TF32 on 8192^3 through torch.matmul: best of 10 single calls (seconds = 0) or the average rate of
    back-to-back calls for `seconds` -- the two figures the pool's bf16 peak file is made of, for TF32."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        n = 8192
        a, b = torch.randn(n, n, device="cuda"), torch.randn(n, n, device="cuda")
        c = torch.empty(n, n, device="cuda")
        for _ in range(3):
            torch.mm(a, b, out=c)
        torch.cuda.synchronize()
        flops = 2.0 * n ** 3
        if seconds <= 0:
            best = 0.0
            for _ in range(10):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                torch.mm(a, b, out=c)
                e1.record()
                torch.cuda.synchronize()
                best = max(best, flops / e0.elapsed_time(e1) / 1e9)
            return best
        done, t_ms = 0, 0.0
        while t_ms < seconds * 1e3:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(100):
                torch.mm(a, b, out=c)
            e1.record()
            torch.cuda.synchronize()
            t_ms += e0.elapsed_time(e1)
            done += 100
        return done * flops / t_ms / 1e9
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def recorded_traffic(rows_per_gpu):
    """DRAM bytes per GEMM launch of the step, from the committed ncu capture of the step's eight GEMMs on a small
    case (profiles/mlp_step_gemm_dram_traffic.md: a few launches of one kernel, a few hundred MB on the device),
    scaled to this run's rows per GPU: every GEMM of the step has the batch rows as its M or its K, and the kernel
    walks both in blocks, so its traffic grows in proportion to them.  null when no capture is committed."""
    path = os.path.join(ROOT, "profiles", "mlp_step_gemm_dram_traffic.md")
    alg = None
    try:
        rec = None
        for ln in open(path):
            if ln.startswith("TRAFFIC_JSON "):
                rec = json.loads(ln[len("TRAFFIC_JSON "):])
        if rec is None:
            raise ValueError("no TRAFFIC_JSON line")
        scale = rows_per_gpu / rec["rows"]
        total = sum(g["read"] * scale + g["write"] * (scale if g["rows_are"] == "M" else 1.0) for g in rec["launches"])
        per_launch = total / len(rec["launches"])
        r = rows_per_gpu
        d = DIMS
        # algorithmic bytes of the 8 GEMMs: each operand touched once
        gemms = [(r, d[1], d[0]), (r, d[2], d[1]), (r, d[3], d[2]), (d[3], d[2], r), (r, d[2], d[3]), (d[2], d[1], r),
                 (r, d[1], d[2]), (d[1], d[0], r)]
        alg = sum(4.0 * (m * k + k * n + m * n) for m, n, k in gemms) / len(gemms)
        return {"traffic": per_launch, "algorithmic_bytes_per_launch": alg,
                "traffic_source": f"profiles/mlp_step_gemm_dram_traffic.md: ncu dram__bytes_read.sum + dram__bytes_write.sum "
                                  f"of the step's 8 GEMM launches captured at {rec['rows']} rows, scaled x {scale:g} to "
                                  f"{rows_per_gpu} rows (reads, and the writes of the products whose M is the rows, grow "
                                  "with the rows; the dW results do not), averaged per launch"}
    except (OSError, ValueError, KeyError) as e:
        return {"traffic": None, "algorithmic_bytes_per_launch": alg, "traffic_source": f"no committed capture ({e})"}


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from sharpnet_b200 import MATH_3XTF32
    from sharpnet_b200.data_parallel import (MLP_ACTS, DenseStack, GradientAllReduce, mlp_step_flops, shard_rows,
                                             training_step)
    from sharpnet_b200.tensor import GPUWrapper
    from oracle import sharpnet_oracle as orc

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    if world > 1:
        # the collective's CTA budget (see GradientAllReduce.COLLECTIVE_CTAS) must be in the environment before the
        # first NCCL communicator of the process reads it
        ctas = int(os.environ.get("SNB200_COLLECTIVE_CTAS", "0"))
        if ctas > 0:
            os.environ.setdefault("NCCL_MAX_CTAS", str(ctas))
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    if world > 1 and os.environ.get("SNB200_NO_NUMA_BIND", "0") != "1":
        # one process per GPU: keep each replica's staging buffers and host thread on its GPU's NUMA node (at N = 1
        # the process keeps every core: the CPU baseline legs use them)
        from sharpnet_b200.data_parallel import bind_host_to_device_node, device_pci_bus_id
        try:
            bound = bind_host_to_device_node(device_pci_bus_id(local))
        except Exception:          # a torch without the PCI fields: stay unbound
            bound = None
        print(f"rank {rank}: host bound to {len(bound) if bound else 0} CPUs of the GPU's NUMA node", file=sys.stderr)
    peaks = _peaks()
    w = GPUWrapper.FromDeviceId(local)
    w.set_math_mode(MATH_3XTF32)
    r0, r1 = shard_rows(GLOBAL_BATCH, world, rank)
    rows = r1 - r0
    weights = [orc.glorot_uniform((DIMS[i + 1], DIMS[i]), 14 + i) for i in range(3)]
    stack = DenseStack(w, rows, DIMS, MLP_ACTS, weights)
    # the first layer's weight gradient in row panels, each reduced while the next is computed (N > 1 only)
    stack.dw_row_panels = int(os.environ.get("SNB200_DW_PANELS", "1")) if world > 1 else 1
    # synthetic inputs of the named shape, generated on the host and pinned for the e2e leg
    g = torch.Generator().manual_seed(17 + rank)
    x_host = torch.randn(rows, DIMS[0], generator=g).pin_memory()
    dy_host = torch.randn(rows, DIMS[-1], generator=g).pin_memory()
    stack.x.storage.copy_(x_host.view(-1))
    stack.dy.storage.copy_(dy_host.view(-1))
    db_host = [torch.empty(DIMS[i + 1]).pin_memory() for i in range(3)]
    compute_stream = torch.cuda.default_stream()
    reducer = None
    if world > 1:
        def bcast(b):
            obj = [b]
            dist.broadcast_object_list(obj, src=0)
            return obj[0]
        reducer = GradientAllReduce(local, world, rank, bcast)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    # ---- is the data-parallel result right?  checked before anything is timed, at every N
    dp = dp_check(w, torch, dist, world, rank, reducer, compute_stream)
    if rank == 0:
        print(f"dp_check: {dp}", file=sys.stderr)

    # ---- the tensor roofline's denominator, measured the way the pool's bf16 peak was: cuBLAS TF32 8192^3, best of
    # 10 on the still cool GPU (burst); the 4-second back-to-back figure (sustained) is taken after the timed steps
    tf32_peak = None
    if rank == 0 and world == 1 and not args.no_shapes:
        tf32_peak = {"burst_tflops": cublas_tf32_rate(torch, seconds=0.0)}

    # ---- isolated kernels first (N = 1): every shape of configs 1-5, the Dense and attention entry points and the
    # bandwidth-bound companions, each timed alone before the long step heats the GPU into its power cap
    shapes = companions = None
    if world == 1 and not args.no_shapes:
        shapes = per_shape_table(w, torch, peaks, large=False, cpu=not args.no_cpu)
        shapes = shapes + dense_and_attention_table(w, torch, peaks)
        companions = companion_table(w, torch, peaks)
        shapes = shapes + per_shape_table(w, torch, peaks, large=True, cpu=not args.no_cpu)
        torch.cuda.synchronize()
        torch.cuda.empty_cache()

    sharded = None
    if world > 1 and not args.no_shapes:
        sharded = sharded_gemm(w, torch, world, rank, barrier, max_over_ranks)
        torch.cuda.empty_cache()

    step = lambda: training_step(stack, reducer, compute_stream)  # noqa: E731
    for _ in range(max(args.warmup, 3)):
        step()
    w.check_device_status()

    # ---- device-resident timing ------------------------------------------------------------
    sampler = ClockSampler(local)
    launches0 = w.launch_count()
    barrier()
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w.gemm_timing_begin()          # an event pair around every GEMM of the timed steps, on the launching stream
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    gemm_ms_total, gemm_calls = w.gemm_timing_end()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    launches = w.launch_count() - launches0
    w.check_device_status()
    flops = mlp_step_flops(GLOBAL_BATCH, DIMS)
    value = flops / ms / 1e9

    # ---- per-kernel timing of the GEMMs inside the step (events around every GEMM launch) ---
    gemm_ms = max_over_ranks(gemm_ms_total / args.steps)
    gemm_flops = mlp_step_flops(rows, DIMS)     # this rank's shard: all of the step's flops are in its GEMMs
    print(f"GEMMs in the timed steps: {gemm_calls} calls, {gemm_ms:.3f} ms per step", file=sys.stderr)

    # ---- end to end: host buffers in, bias gradients out, every step ----------------------
    # Every step's x and upstream gradient are copied from pinned host memory inside the timed region;
    # the copy of step i+1 runs on a copy stream while step i computes (double-buffered staging).
    from sharpnet_b200.data_parallel import HostStaging
    # x travels as four row panels: the first layer starts on a panel as soon as it has landed, which shortens the one
    # copy of the loop that nothing overlaps (the first) to a quarter
    # (panels of at least 16384 rows: below that the first layer's products get too small to run at full rate, measured
    # at 4 GPUs -- 4096-row panels cost 0.4 ms per step)
    panels = int(os.environ.get("SNB200_STAGE_PANELS", str(min(4, max(1, rows // 16384)))))
    staging = HostStaging(stack, x_host, dy_host, panels=panels)

    def e2e_loop(n):
        staging.issue(0)
        for i in range(n):
            staging.bind(i)
            if i + 1 < n:
                staging.issue(i + 1)
            step()
            staging.release(i)
            for j in range(3):
                db_host[j].copy_(stack.db[j].storage, non_blocking=True)
    e2e_loop(2)
    barrier()
    # how long one step's input copy takes on its own: the first step of the timed loop below has to wait for it
    # (nothing of the region runs before it), every later copy hides behind the step before
    c0 = torch.cuda.Event(enable_timing=True); c1 = torch.cuda.Event(enable_timing=True)
    c0.record()
    staging.issue(0)
    staging.bind(0)
    staging.wait()
    c1.record()
    staging.release(0)
    barrier()
    fill_ms = max_over_ranks(c0.elapsed_time(c1))
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    e2e_loop(args.steps)
    t1.record()
    barrier()
    e2e_ms = max_over_ranks(t0.elapsed_time(t1) / args.steps)
    h2d = (x_host.numel() + dy_host.numel()) * 4
    d2h = sum(t.numel() for t in db_host) * 4

    staging.close()
    # the sustained half of the TF32 peak: cuBLAS TF32 8192^3 back to back for 4 s, on the GPU the steps have heated
    if tf32_peak is not None:
        tf32_peak["sustained_tflops"] = cublas_tf32_rate(torch, seconds=4.0)
        tf32_peak["how"] = ("torch.matmul fp32 with TF32 allowed (cuBLAS), 8192^3, 2*N^3 flops: best of 10 single calls "
                            "before the tables (burst), back to back for 4 s after the timed steps (sustained)")
    cpu = parity = None
    if rank == 0 and world == 1 and not args.no_cpu:
        v, t, inputs, cpu_results = time_cpu(CPU_SAMPLE_ROWS, 3)
        cpu = {"value": v, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
               "sample": f"{CPU_SAMPLE_ROWS} of {GLOBAL_BATCH} batch rows of the same step, MKL sgemm via torch CPU, "
                         f"median of 3 ({t:.2f} s each)"}
        # the device's step on those same rows against what the CPU leg computed
        parity = step_parity(w, torch, inputs, cpu_results)
        print(f"parity: {parity}", file=sys.stderr)
    if rank == 0:
        peak3 = peaks["bf16_sustained"] / 2 / 3
        achieved = gemm_flops / gemm_ms / 1e9   # per-GPU rate of the GEMM kernel (this rank's shard)
        line = {
            "metric": "dot_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(world),
            "clocks": clocks,
            "e2e": {"value": flops / e2e_ms / 1e9, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d * world,
                    "d2h_bytes_per_step": d2h * world, "ms_per_step": e2e_ms,
                    "pipeline_fill_ms": fill_ms,
                    "note": "pipeline_fill_ms = one step's input copy on its own.  The timed loop starts with step 0's copy, "
                            f"which nothing of the region runs before; x travels as {panels} row panel(s) and the first layer "
                            "starts on each as it lands, so that fraction of it is exposed, once per run of `steps` steps; "
                            "every later copy runs behind the step before it"},
            "gpu_launches": launches * world,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak3, "unit": "TFLOP/s",
                         "frac": achieved / peak3,
                         **recorded_traffic(rows),
                         "kernel": "umma2_gemm_kernel (CTA-pair tcgen05 GEMM, 3xTF32), the 8 GEMM launches of the step",
                         "peak_source": f"{peaks['src']} bf16 sustained {peaks['bf16_sustained']} TFLOP/s / 2 (TF32) / 3 "
                                        "(three TF32 products per fp32 product); flops counted once (2*M*N*K)",
                         "gemm_ms_per_step": gemm_ms,
                         "gemm_timing": "CUDA-event pairs recorded by the library around every GEMM of the timed steps, "
                                        "on the launching stream",
                         "measured_tf32": tf32_peak,
                         "frac_vs_measured_tf32_sustained": (
                             None if not tf32_peak else achieved / (tf32_peak["sustained_tflops"] / 3.0)),
                         "frac_vs_measured_tf32_burst": (
                             None if not tf32_peak else achieved / (tf32_peak["burst_tflops"] / 3.0)),
                         # nominal dense TF32 rate (1100 TFLOP/s at 1965 MHz) scaled to the SM clock sampled during the
                         # timed steps, / 3: what the tensor cores can deliver to this arithmetic under the power cap
                         "nominal_tf32_at_sampled_clock_over_3": (
                             None if not clocks or not clocks.get("sm_mhz")
                             else 1100.0 * clocks["sm_mhz"] / 1965.0 / 3.0),
                         "note": "`peak` is the pool's measured cuBLAS bf16 rate / 2 / 3 (a proxy: the pool file holds no "
                                 "TF32 figure); measured_tf32 is cuBLAS TF32 on this GPU in this run, and the two "
                                 "frac_vs_measured_tf32_* use it / 3.  A fraction above 1 means this kernel keeps the tensor "
                                 "pipe busier than cuBLAS does; what remains is the SM clock under the 1000 W power cap"},
            "cpu_baseline": cpu,
            "dp_check": dp,
        }
        if parity is not None:
            line["parity"] = parity
        if shapes is not None:
            line["shapes"] = shapes
            line["companions"] = companions
        if sharded is not None:
            line["sharded_gemm"] = sharded
        _emit(json.dumps(line))
    if reducer is not None:
        reducer.close()
    if world > 1:
        dist.destroy_process_group()
    if rank == 0 and ((dp is not None and not dp["ok"]) or (parity is not None and not parity["ok"])):
        raise SystemExit("bench: a correctness check failed (dp_check / parity in the line above)")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-shapes", action="store_true", help="skip the per-shape table (N = 1 only)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--case", default=None, choices=["gemm", "sdpa", "step"],
                    help="time a single Dot shape, one attention core or the training step on --rows batch rows "
                         "instead of the full step (small cases for profiling)")
    ap.add_argument("--rows", type=int, default=8192, help="--case step: batch rows on the device")
    ap.add_argument("--mnk", type=int, nargs=3, default=[4096, 4096, 4096])
    ap.add_argument("--trans", default="NN", help="NN, NT, TN or TT")
    ap.add_argument("--beta", type=float, default=0.0)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--math", type=int, default=0, help="0 3xTF32, 1 TF32, 2 SIMT fp32, 3 TF32 + bf16 cross terms")
    ap.add_argument("--calls", type=int, default=20)
    args = ap.parse_args()
    # Libraries (NCCL's version banner, for one) write to file descriptor 1; the contract is ONE JSON line on
    # stdout, so everything but that line is sent to stderr.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    global _emit
    _emit = lambda text: os.write(real_stdout, (text + "\n").encode())  # noqa: E731
    if args.case == "gemm":
        import torch
        from sharpnet_b200.tensor import GPUWrapper
        M, N, K = args.mnk
        r = time_gemm_shape(GPUWrapper.FromDeviceId(0), torch, _peaks(), "case", M, N, K, args.trans[0] == "T",
                            args.trans[1] == "T", args.beta, args.batch, -1.0, 1.0, args.math, min_calls=args.calls,
                            cpu=False, compare=False)
        _emit(json.dumps(r))
    elif args.case == "step":
        # the training step of the benchmark on a fraction of its rows: 8 GEMM launches per step
        import torch
        from oracle import sharpnet_oracle as orc
        from sharpnet_b200.data_parallel import MLP_ACTS, DenseStack, mlp_step_flops, training_step
        from sharpnet_b200.tensor import GPUWrapper
        w = GPUWrapper.FromDeviceId(0)
        w.set_math_mode(args.math)
        stack = DenseStack(w, args.rows, DIMS, MLP_ACTS, [orc.glorot_uniform((DIMS[i + 1], DIMS[i]), 14 + i) for i in range(3)])
        stack.x.storage.normal_()
        stack.dy.storage.normal_()
        training_step(stack)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.calls):
            training_step(stack)
        e1.record()
        torch.cuda.synchronize()
        w.check_device_status()
        ms = e0.elapsed_time(e1) / args.calls
        _emit(json.dumps({"shape": f"MLP training step on {args.rows} rows", "calls": args.calls, "ms": round(ms, 4),
                          "tflops": round(mlp_step_flops(args.rows, DIMS) / ms / 1e9, 2)}))
    elif args.case == "sdpa":
        # one attention core, forward + backward: --batch heads, --mnk q_steps v_steps head_dim
        import ctypes
        import torch
        from sharpnet_b200.tensor import GPUWrapper
        w = GPUWrapper.FromDeviceId(0)
        w.set_math_mode(args.math)
        B, (Tq, Tk, E) = args.batch, args.mnk
        new = lambda *shape: torch.empty(*shape, dtype=torch.float32, device=w.device).uniform_(-1, 1)  # noqa: E731
        P = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
        Q, dy, y, dQ = (new(B, Tq, E) for _ in range(4))
        K, V, dK, dV = (new(B, Tk, E) for _ in range(4))
        wts, ds = new(B, Tq, Tk), new(B, Tq, Tk)

        def both():
            st = w.lib.snb200_sdpa_fwd(w.handle, B, Tq, Tk, E, 1, 1, P(Q), P(K), P(V), P(wts), P(y))
            return st or w.lib.snb200_sdpa_bwd(w.handle, B, Tq, Tk, E, 1, P(Q), P(K), P(V), P(dy), P(wts), P(ds), P(dQ),
                                               P(dK), P(dV))
        for _ in range(3):
            if both() != 0:
                raise RuntimeError(w.lib.snb200_last_error_string(w.handle))
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.calls):
            both()
        e1.record()
        torch.cuda.synchronize()
        w.check_device_status()
        _emit(json.dumps({"shape": f"sdpa fwd+bwd {B} x [{Tq} x {Tk} x {E}] causal", "calls": args.calls,
                          "ms": round(e0.elapsed_time(e1) / args.calls, 4)}))
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
