"""Data-parallel Dense training step: the host logic of SharpNet's multi-GPU support for the
Dense path, one process (or thread) per GPU.

SharpNet splits every mini-batch by rows among its workers -- worker 0 (the master) takes rows
[0, b), worker 1+i takes rows [(1+i)*b, (2+i)*b) (Prod/Networks/Network.cs:1121-1123,1229-1258) --
runs forward and backward on each replica, then SUMS the gradients of all replicas on the master
(Prod/Networks/NetworkMultiGPUSupport.cs:161-173) and divides by the global batch in the optimizer
(Prod/Optimizers/Optimizer.cs:26-29).  Here the sum is one all-reduce per layer over NVLink, issued
on a side stream as soon as that layer's dW is produced so that it overlaps the remaining backward
GEMMs; every replica ends the step with the same summed gradients.

Nothing in this file computes: the arithmetic is the C ABI's (GEMMs, fused Dense passes, NCCL).
"""
from . import _capi
from ._capi import ACT_IDENTITY, ACT_RELU, W_OUT_IN, check
from .tensor import GPUTensor, GPUWrapper


def shard_rows(global_batch, world_size, rank):
    """Row range [start, stop) of ``rank``: contiguous blocks in rank order, as the reference slices
    the mini-batch (Prod/Networks/Network.cs:1233,1243).  The batch must be a multiple of the
    number of workers (:1121-1122)."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} of {world_size}")
    if global_batch % world_size != 0:
        raise ValueError("the mini-batch size must be a multiple of the number of workers")
    b = global_batch // world_size
    return rank * b, (rank + 1) * b


def mlp_step_flops(global_batch, dims):
    """Algorithmic flops of one forward+backward step of a Dense stack ``dims[0] -> ... -> dims[-1]``
    over the whole batch: forward and dW for every layer, dx for every layer but the first
    (Prod/Layers/Linear.cs:184-187)."""
    pairs = list(zip(dims[:-1], dims[1:]))
    fwd = sum(2 * global_batch * i * o for i, o in pairs)
    dx = sum(2 * global_batch * i * o for i, o in pairs[1:])
    return fwd + fwd + dx


class DenseStack:
    """A stack of Dense layers with fused activations on one GPU: the buffers one replica needs for
    forward + backward, allocated once (the role of PropagationManager + TensorMemoryPool,
    Prod/Networks/PropagationManager.cs:46-145)."""

    def __init__(self, wrapper, local_batch, dims, activations, weights=None, w_layout=W_OUT_IN):
        assert len(activations) == len(dims) - 1
        self.w = wrapper
        self.batch = local_batch
        self.dims = list(dims)
        self.acts = list(activations)
        self.layout = w_layout
        n = len(dims) - 1
        shape = (lambda i: (dims[i + 1], dims[i])) if w_layout == W_OUT_IN else (lambda i: (dims[i], dims[i + 1]))
        self.W = [GPUTensor(shape(i), None if weights is None else weights[i], wrapper) for i in range(n)]
        self.b = [GPUTensor((dims[i + 1],), None, wrapper) for i in range(n)]
        self.dW = [GPUTensor(shape(i), None, wrapper) for i in range(n)]
        self.db = [GPUTensor((dims[i + 1],), None, wrapper) for i in range(n)]
        self.x = GPUTensor((local_batch, dims[0]), None, wrapper)
        self.y = [GPUTensor((local_batch, dims[i + 1]), None, wrapper) for i in range(n)]
        # dz scratch per activated layer, gradient w.r.t. each hidden activation
        self.dz = [None if activations[i] == ACT_IDENTITY else GPUTensor((local_batch, dims[i + 1]), None, wrapper)
                   for i in range(n)]
        self.dx = [None] + [GPUTensor((local_batch, dims[i]), None, wrapper) for i in range(1, n)]
        self.dy = GPUTensor((local_batch, dims[-1]), None, wrapper)
        self.reserve_pending = False
        # set by HostStaging when the input arrives as row panels: the first layer then runs panel by panel, each
        # product waiting only for its own rows, and the upstream gradient is waited for where the backward pass starts
        self.input_panels = None        # [(row0, row1), ...]
        # > 1: the weight-gradient product of the first layer -- the last large gradient of a backward pass -- is
        # cut into that many row panels, and `after_gradient_rows` (the reduction of one panel) runs behind each
        self.dw_row_panels = 1
        self.before_panel = None        # callable(k)
        self.before_backward = None     # callable()

    def forward(self):
        import ctypes
        lib, h = self.w.lib, self.w.handle
        src = self.x
        for i, W in enumerate(self.W):
            if i == 0 and self.input_panels:
                K, N = self.dims[0], self.dims[1]
                for k, (r0, r1) in enumerate(self.input_panels):
                    if self.before_panel is not None:
                        self.before_panel(k)
                    st = lib.snb200_dense_fwd(h, self.layout, r1 - r0, K, N,
                                              ctypes.c_void_p(src.Pointer.value + 4 * r0 * K), W.Pointer, self.b[0].Pointer,
                                              self.acts[0], None, ctypes.c_void_p(self.y[0].Pointer.value + 4 * r0 * N))
                    check(h, st)
            else:
                st = lib.snb200_dense_fwd(h, self.layout, self.batch, self.dims[i], self.dims[i + 1], src.Pointer,
                                          W.Pointer, self.b[i].Pointer, self.acts[i], None, self.y[i].Pointer)
                check(h, st)
            src = self.y[i]

    def _bwd(self, i, grad, act, dz, dx, dW, db):
        """One snb200_dense_bwd call on layer ``i``; every output is optional."""
        lib, h = self.w.lib, self.w.handle
        src = self.x if i == 0 else self.y[i - 1]
        p = lambda t: None if t is None else t.Pointer  # noqa: E731
        st = lib.snb200_dense_bwd(
            h, self.layout, self.batch, self.dims[i], self.dims[i + 1], src.Pointer, self.W[i].Pointer, grad.Pointer,
            act, None if act == ACT_IDENTITY else self.y[i].Pointer, None, 1.0, p(dz), p(dx), p(dW), p(db))
        check(h, st)
        if self.reserve_pending and (dx is not None or dW is not None):
            # one product has run beside the collective queued before it: back to every SM
            self.w.set_tuning(_capi.TUNE_SM_RESERVE, 0)
            self.reserve_pending = False

    def _bwd_weight_panels(self, dz, after_gradient_rows):
        """dW of layer 0 as ``dw_row_panels`` products over row panels of the result, each followed by its hook."""
        lib, h = self.w.lib, self.w.handle
        rows_total = self.W[0].Shape[0]
        per = -(-rows_total // self.dw_row_panels)
        per = -(-per // 256) * 256                      # whole tile rows of the CTA-pair kernel
        r0 = 0
        while r0 < rows_total:
            rows = min(per, rows_total - r0)
            check(h, lib.snb200_dense_bwd_weight_rows(h, self.layout, self.batch, self.dims[0], self.dims[1], self.x.Pointer,
                                                      dz.Pointer, 1.0, r0, rows, self.dW[0].Pointer))
            after_gradient_rows(0, r0, rows, r0 + rows >= rows_total)
            r0 += rows

    def backward(self, after_gradients=None, after_layer=None, defer_smallest=False, after_gradient_rows=None):
        """Backward through every layer, last to first.

        Per layer the two products are queued as two calls: first the activation gradient with the bias
        gradient and the weight gradient, then ``after_gradients(i)`` (the hook the gradient all-reduce hangs on:
        the reduction starts while the layer's dx product still runs), then dx alone, then ``after_layer(i)``
        (everything that reads W[i] is queued: the place for an optimizer step on another stream).

        ``defer_smallest``: the weight-gradient product of the layer with the fewest weights is queued last
        instead of in its turn (it depends only on that layer's dz and input, which stay in place), so that the
        reduction nothing is left to hide behind is the smallest one.  The arithmetic is the same in any order."""
        n = len(self.W)
        if self.before_backward is not None:
            self.before_backward()
        deferred = None
        if defer_smallest and n > 1:
            smallest = min(range(n), key=lambda i: self.W[i].Count)
            if smallest != 0:            # layer 0's dW is the last product anyway
                deferred = smallest
        grad = self.dy
        dz_of = {}
        for i in reversed(range(n)):
            act = self.acts[i]
            dz = grad if act == ACT_IDENTITY else self.dz[i]
            dz_of[i] = dz
            dx = None if i == 0 else self.dx[i]
            if i == deferred:
                self._bwd(i, grad, act, self.dz[i], None, None, self.db[i])     # dz and db now, dW at the end
            elif i == 0 and self.dw_row_panels > 1 and after_gradient_rows is not None:
                self._bwd(i, grad, act, self.dz[i], None, None, self.db[i])     # dz and db, then dW panel by panel
                self._bwd_weight_panels(dz, after_gradient_rows)
            else:
                self._bwd(i, grad, act, self.dz[i], None, self.dW[i], self.db[i])
                if after_gradients is not None:
                    after_gradients(i)
            if dx is not None:
                self._bwd(i, dz, ACT_IDENTITY, None, dx, None, None)
            if after_layer is not None and i != deferred:
                after_layer(i)
            grad = self.dx[i]
        if deferred is not None:
            self._bwd(deferred, dz_of[deferred], ACT_IDENTITY, None, None, self.dW[deferred], None)
            if after_gradients is not None:
                after_gradients(deferred)
            if after_layer is not None:
                after_layer(deferred)
        if self.reserve_pending:
            # nothing of this pass runs beside the last collective; what comes next gets every SM again
            self.w.set_tuning(_capi.TUNE_SM_RESERVE, 0)
            self.reserve_pending = False


class GradientAllReduce:
    """Sums dW and db of every layer over all replicas with NCCL, on a side stream.

    One process per GPU: rank 0 creates the NCCL id and ``broadcast_bytes`` (any callable that
    ships 128 bytes from rank 0 to everyone, e.g. built on torch.distributed) distributes it."""

    # Optional: CTAs the collective may use (NCCL_MAX_CTAS), and the SMs the product queued right behind a reduction
    # leaves free for it.  A persistent GEMM grid counts on every SM it was launched for, so a collective that has
    # to squeeze in displaces some of its CTAs for as long as it runs and the GEMM ends that much later.  Off by
    # default (0): measured at 2 and 4 GPUs, capping NCCL at 16 CTAs lengthened the exposed tail of the last
    # reduction by more than the reservation saved (13.82 against 13.67 ms per step at 4 GPUs).
    # SNB200_COLLECTIVE_CTAS=<n> turns it on.
    COLLECTIVE_CTAS = 0

    def __init__(self, device_id, world_size, rank, broadcast_bytes):
        import ctypes
        import os
        import torch
        self.torch = torch
        self.world = world_size
        # SNB200_COLLECTIVE_CTAS overrides the count; 0 leaves NCCL alone and reserves nothing (A/B measurements)
        self.COLLECTIVE_CTAS = int(os.environ.get("SNB200_COLLECTIVE_CTAS", self.COLLECTIVE_CTAS))
        if self.COLLECTIVE_CTAS > 0:
            os.environ.setdefault("NCCL_MAX_CTAS", str(self.COLLECTIVE_CTAS))
        self.comm_wrapper = GPUWrapper(device_id)          # a second handle: owns the communicator and its stream
        self.stream = torch.cuda.Stream(device=device_id)
        self.comm_wrapper.set_stream(self.stream)
        lib = _capi.load()
        ident = ctypes.create_string_buffer(128)
        if rank == 0:
            st = lib.snb200_comm_get_unique_id(ident)
            if st != 0:
                raise _capi.SharpNetB200Error(st, "NCCL could not be loaded")
        ident = ctypes.create_string_buffer(broadcast_bytes(bytes(ident.raw)), 128)
        check(self.comm_wrapper.handle,
              lib.snb200_comm_init_rank(self.comm_wrapper.handle, world_size, rank, ident))

    def reduce_layer(self, stack, i, compute_stream):
        """Queues the all-reduce of layer ``i``'s gradients (dW and db as one NCCL group, one launch) on the side
        stream, behind the work already on ``compute_stream``."""
        import ctypes
        ev = self.torch.cuda.Event()
        ev.record(compute_stream)
        self.stream.wait_event(ev)
        lib, h = self.comm_wrapper.lib, self.comm_wrapper.handle
        bufs = (ctypes.c_void_p * 2)(stack.dW[i].Pointer, stack.db[i].Pointer)
        counts = (ctypes.c_longlong * 2)(stack.dW[i].Count, stack.db[i].Count)
        check(h, lib.snb200_allreduce_sum_group(h, 2, bufs, counts))
        # the next product of the compute handle leaves room for the collective (see COLLECTIVE_CTAS) -- where that
        # pays: the product gives up COLLECTIVE_CTAS / 148 of its SMs for its whole duration, the collective needs
        # them for its own, so the reservation is made only when the collective is not short against the product
        if self.COLLECTIVE_CTAS > 0 and self._worth_reserving(stack, i):
            stack.w.set_tuning(_capi.TUNE_SM_RESERVE, self.COLLECTIVE_CTAS)
            stack.reserve_pending = True

    def reduce_rows(self, stack, i, row0, rows, last, compute_stream):
        """The same for rows [row0, row0 + rows) of layer ``i``'s weight gradient; the bias gradient travels with the
        last panel."""
        import ctypes
        ev = self.torch.cuda.Event()
        ev.record(compute_stream)
        self.stream.wait_event(ev)
        lib, h = self.comm_wrapper.lib, self.comm_wrapper.handle
        width = stack.dW[i].Count // stack.dW[i].Shape[0]
        bufs = (ctypes.c_void_p * 2)(stack.dW[i].Pointer.value + 4 * row0 * width, stack.db[i].Pointer)
        counts = (ctypes.c_longlong * 2)(rows * width, stack.db[i].Count)
        check(h, lib.snb200_allreduce_sum_group(h, 2 if last else 1, bufs, counts))

    def _worth_reserving(self, stack, i):
        """Rough durations: the all-reduce of layer ``i`` at ~350 GB/s of bus bandwidth against the product queued
        next (this layer's dx, or the next dW) at ~240 TFLOP/s.  Reserve when the collective takes at least as long
        as the slice of the product it would otherwise delay."""
        n = self.world
        t_collective = 2.0 * (n - 1) / n * 4.0 * (stack.dW[i].Count + stack.db[i].Count) / 350e9
        j = i if i > 0 else 0                                       # layer whose product follows
        t_product = 2.0 * stack.batch * stack.dims[j] * stack.dims[j + 1] / 240e12
        return t_collective >= t_product * self.COLLECTIVE_CTAS / 148.0 * 1.5

    def update_layer(self, stack, i, compute_stream, update):
        """Queues ``update(lib, handle, stack, i)`` -- the optimizer step of layer ``i`` -- on the side stream,
        behind that layer's reduction and behind everything on ``compute_stream`` that still reads W[i]."""
        ev = self.torch.cuda.Event()
        ev.record(compute_stream)
        self.stream.wait_event(ev)
        update(self.comm_wrapper.lib, self.comm_wrapper.handle, stack, i)

    def join(self, compute_stream):
        """Makes ``compute_stream`` wait for every queued all-reduce."""
        ev = self.torch.cuda.Event()
        ev.record(self.stream)
        compute_stream.wait_event(ev)

    def close(self):
        lib = self.comm_wrapper.lib
        lib.snb200_comm_destroy(self.comm_wrapper.handle)
        lib.snb200_destroy(self.comm_wrapper.handle)
        self.comm_wrapper.handle = None


def _parse_cpulist(text):
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def bind_host_to_device_node(pci_bus_id, sysfs_root="/sys", setaffinity=None, getaffinity=None):
    """Restricts the calling process to the CPUs of the NUMA node the GPU hangs off, so that pinned staging
    buffers allocated afterwards (first touched by this process) live in that node's memory and the copies of a
    replica do not cross the socket interconnect.  With one process per GPU, eight replicas otherwise stage through
    whatever node the scheduler put them on.  ``pci_bus_id`` is "domain:bus:device.function" as CUDA reports it.
    Returns the CPU set it bound to, or None when the node is unknown (no NUMA, no sysfs, an empty intersection
    with the CPUs the process may use): then nothing is changed."""
    import os
    setaffinity = setaffinity or (lambda cpus: os.sched_setaffinity(0, cpus))
    getaffinity = getaffinity or (lambda: os.sched_getaffinity(0))
    try:
        dev = os.path.join(sysfs_root, "bus", "pci", "devices", pci_bus_id.lower())
        with open(os.path.join(dev, "numa_node")) as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(os.path.join(sysfs_root, "devices", "system", "node", "node%d" % node, "cpulist")) as f:
            cpus = _parse_cpulist(f.read()) & set(getaffinity())
        if not cpus:
            return None
        setaffinity(cpus)
        return cpus
    except (OSError, ValueError):
        return None


def device_pci_bus_id(device_index):
    """"domain:bus:device.0" of a CUDA device, in the spelling of sysfs."""
    import torch
    p = torch.cuda.get_device_properties(device_index)
    return "%04x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)


class HostStaging:
    """Double-buffered host-to-device staging of a replica's mini-batch (x and the upstream gradient)
    through the library's stager (snb200_stager_*).

    SharpNet copies every mini-batch from pinned host memory to the device before it runs the
    step (Prod/Networks/Network.cs:1211-1258, Prod/GPU/GpuTensor.cs:68-80).  Here the copy of step
    i+1 runs on the stager's stream while step i computes; the compute stream only waits for the copy it
    is about to consume, and a buffer is not overwritten before the step that read it has finished."""

    def __init__(self, stack, x_host, dy_host, slots=2, panels=1):
        """``panels`` > 1 stages x as that many row panels (up to 15), each with an event of its own, and lets the
        stack's first layer start on a panel as soon as it has landed; the upstream gradient, copied last, is
        waited for where the backward pass starts.  Only the very first step of a loop gains (its copy has nothing
        to hide behind); every later copy overlaps the step before it either way."""
        import ctypes
        self.stack = stack
        self.x_host, self.dy_host = x_host, dy_host
        w = stack.w
        self.slots = slots
        self.buffers = [(stack.x, stack.dy)] + [(GPUTensor(stack.x.Shape, None, w), GPUTensor(stack.dy.Shape, None, w))
                                                for _ in range(slots - 1)]
        self.handle = ctypes.c_void_p()
        check(w.handle, w.lib.snb200_stager_create(w.handle, slots, ctypes.byref(self.handle)))
        rows, width = stack.batch, stack.dims[0]
        panels = max(1, min(int(panels), 15, rows // 256 if rows >= 256 else 1))
        per = -(-rows // panels)
        per = -(-per // 128) * 128 if panels > 1 else per          # whole tile rows per panel
        self.panels = [(r, min(rows, r + per)) for r in range(0, rows, per)]
        n = len(self.panels) + 1
        self._n = n
        self._src = (ctypes.c_void_p * n)(*[x_host.data_ptr() + 4 * r0 * width for r0, _ in self.panels], dy_host.data_ptr())
        self._bytes = (ctypes.c_longlong * n)(*[4 * (r1 - r0) * width for r0, r1 in self.panels], dy_host.numel() * 4)
        self._dst = [(ctypes.c_void_p * n)(*[bx.Pointer.value + 4 * r0 * width for r0, _ in self.panels], bdy.Pointer.value)
                     for bx, bdy in self.buffers]
        self._slot = 0

    def issue(self, i):
        """Queues the copy of step ``i``'s inputs into buffer ``i % slots``."""
        w = self.stack.w
        b = i % self.slots
        check(w.handle, w.lib.snb200_stager_issue(self.handle, b, self._n, self._dst[b], self._src, self._bytes))

    def _wait_panel(self, k):
        w = self.stack.w
        check(w.handle, w.lib.snb200_stager_acquire_part(self.handle, self._slot, k))

    def wait(self):
        """Makes the compute stream wait for everything staged into the bound buffer."""
        w = self.stack.w
        check(w.handle, w.lib.snb200_stager_acquire(self.handle, self._slot))

    def bind(self, i):
        """Points the stack at buffer ``i % slots`` and makes the compute stream wait for its copy: for all of it
        here, or (row panels) panel by panel inside the stack's first layer and before its backward pass."""
        w = self.stack.w
        b = i % self.slots
        self._slot = b
        self.stack.x, self.stack.dy = self.buffers[b]
        if len(self.panels) > 1:
            self.stack.input_panels = self.panels
            self.stack.before_panel = self._wait_panel
            self.stack.before_backward = self.wait
        else:
            check(w.handle, w.lib.snb200_stager_acquire(self.handle, b))

    def release(self, i):
        """Call after step ``i`` has been queued: marks when its buffer may be overwritten."""
        w = self.stack.w
        check(w.handle, w.lib.snb200_stager_release(self.handle, i % self.slots))

    def close(self):
        if self.handle is not None:
            self.stack.w.lib.snb200_stager_destroy(self.handle)
            self.handle = None
        self.stack.x, self.stack.dy = self.buffers[0]
        self.stack.input_panels = self.stack.before_panel = self.stack.before_backward = None


class SgdUpdate:
    """The optimizer step of every replica after the gradient sum: W -= lr / globalBatch * dW with optional
    (Nesterov) momentum -- SharpNet runs it on the master only and then re-broadcasts the parameters
    (Prod/Networks/Network.cs:1275-1290, NetworkMultiGPUSupport.cs:255); here every replica applies the
    identical update to identical sums, so no broadcast is needed."""

    def __init__(self, stack, learning_rate, global_batch, momentum=0.0, nesterov=False):
        self.lr = learning_rate / global_batch          # PonderedLearning, Prod/Optimizers/Optimizer.cs:26-29
        self.momentum, self.nesterov = momentum, nesterov
        self.vW = self.vb = None
        if momentum != 0.0:
            self.vW = [GPUTensor(t.Shape, None, stack.w) for t in stack.W]
            self.vb = [GPUTensor(t.Shape, None, stack.w) for t in stack.b]

    def __call__(self, lib, handle, stack, i):
        for W, g, v in ((stack.W[i], stack.dW[i], self.vW), (stack.b[i], stack.db[i], self.vb)):
            check(handle, lib.snb200_sgd_update(handle, W.Count, self.lr, self.momentum, int(self.nesterov), g.Pointer,
                                                W.Pointer, None if v is None else v[i].Pointer))


def training_step(stack, reducer=None, compute_stream=None, update=None, defer_smallest=True):
    """One forward + backward of ``stack`` on this replica's rows.  With a ``reducer`` the gradients of each layer
    are all-reduced on its side stream from the moment that layer's dW product is queued, overlapping the rest of
    the backward pass; ``update`` (the optimizer step of a layer) follows its reduction on the same stream once
    the products that read the layer's weights are queued."""
    stack.forward()
    if reducer is None:
        after = None if update is None else (lambda i: update(stack.w.lib, stack.w.handle, stack, i))
        stack.backward(after_layer=after)
        return
    stack.backward(after_gradients=lambda i: reducer.reduce_layer(stack, i, compute_stream),
                   after_layer=None if update is None else (lambda i: reducer.update_layer(stack, i, compute_stream, update)),
                   defer_smallest=defer_smallest,
                   after_gradient_rows=lambda i, r0, n, last: reducer.reduce_rows(stack, i, r0, n, last, compute_stream))
    reducer.join(compute_stream)


MLP_DIMS = (4096, 4096, 4096, 1000)
MLP_ACTS = (ACT_RELU, ACT_RELU, ACT_IDENTITY)
