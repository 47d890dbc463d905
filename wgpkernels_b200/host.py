"""The INT8 linear for activations that live in host memory: copy in, compute and copy out run as a pipeline over row chunks.

The reference has no counterpart (its callers hold the activations on the GPU).  A caller whose activations arrive from the host - an
offloading pipeline, a data loader, another process - pays two PCIe transfers per call; done one after the other around the linear they
cost several times the linear itself.  Here three streams work on different row chunks at the same time: chunk i + 1 is copied to the
device while chunk i is multiplied and chunk i - 1 travels back (PCIe is full duplex), with two device buffers on each side.
"""
import torch

from . import int8


class HostLinear:
    """y_host[rows] = linear(x_host[rows]) for pinned host tensors, pipelined over chunks of `chunk_rows` rows.  The device buffers and
    streams are kept between calls.  kwargs: those of `int8.linear` (mode, act, act_weight, eps, group, precise, residual_scale);
    a device `residual` (M, N) is read per chunk."""

    def __init__(self, weight, scale, bias=None, chunk_rows=4096, device=None):
        self.weight, self.scale, self.bias = weight, scale, bias
        self.chunk_rows = chunk_rows
        self.device = weight.device if device is None else device
        self.copy_in = torch.cuda.Stream(self.device)
        self.copy_out = torch.cuda.Stream(self.device)
        self._buffers = {}

    def _chunk_buffers(self, k, n, dtype):
        key = (k, n, dtype)
        if key not in self._buffers:
            self._buffers[key] = ([torch.empty((self.chunk_rows, k), dtype=dtype, device=self.device) for _ in range(2)],
                                  [torch.empty((self.chunk_rows, n), dtype=dtype, device=self.device) for _ in range(2)])
        return self._buffers[key]

    def __call__(self, x_host, out_host, residual=None, **kwargs):
        if not (x_host.is_pinned() and out_host.is_pinned()):
            raise ValueError("x_host and out_host must be pinned host tensors (asynchronous copies)")
        m, k = x_host.shape
        n = self.weight.shape[0]
        if tuple(out_host.shape) != (m, n) or out_host.dtype != x_host.dtype:
            raise ValueError("out_host must be (M, N) of x's dtype")
        xs, ys = self._chunk_buffers(k, n, x_host.dtype)
        compute = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(compute)
        self.copy_in.wait_event(start)   # the buffers may still be read by work queued before this call
        self.copy_out.wait_event(start)
        computed, stored = [None, None], [None, None]  # per buffer: the event after its last multiply / its last copy out
        for index, first in enumerate(range(0, m, self.chunk_rows)):
            rows = min(self.chunk_rows, m - first)
            slot = index % 2
            with torch.cuda.stream(self.copy_in):
                if computed[slot] is not None:
                    self.copy_in.wait_event(computed[slot])  # the multiply that read this input buffer two chunks ago
                xs[slot][:rows].copy_(x_host[first:first + rows], non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(self.copy_in)
            compute.wait_event(arrived)
            if stored[slot] is not None:
                compute.wait_event(stored[slot])  # the copy out that read this output buffer two chunks ago
            int8.linear(xs[slot][:rows], self.weight, self.scale, self.bias, out=ys[slot][:rows],
                        residual=None if residual is None else residual[first:first + rows], **kwargs)
            computed[slot] = torch.cuda.Event()
            computed[slot].record(compute)
            with torch.cuda.stream(self.copy_out):
                self.copy_out.wait_event(computed[slot])
                out_host[first:first + rows].copy_(ys[slot][:rows], non_blocking=True)
                stored[slot] = torch.cuda.Event()
                stored[slot].record(self.copy_out)
        for event in stored:
            if event is not None:
                compute.wait_event(event)  # the caller's stream sees the call as complete once every chunk is back on the host
        return out_host


def _shared_mapping(path, shape, dtype, create):
    """A host tensor backed by a file of shared memory that every process of the node maps (the same bytes in all processes: the
    ranks of a node fill and read one activation together).  create: make the file, sparse -- no page exists until somebody writes."""
    count = 1
    for extent in shape:
        count *= extent
    if create:
        with open(path, "wb") as handle:
            handle.truncate(count * torch.empty((), dtype=dtype).element_size())
    return torch.from_file(path, shared=True, size=count, dtype=dtype).view(shape)


def _register(tensor):
    """Pins the pages of a host tensor where they are and makes copies to and from it asynchronous."""
    code = torch.cuda.cudart().cudaHostRegister(tensor.data_ptr(), tensor.numel() * tensor.element_size(), 0)
    if int(code) != 0:
        raise RuntimeError(f"cudaHostRegister failed ({code})")


def _cpus_near(device):
    """The CPUs of the NUMA node a GPU hangs on (from sysfs), limited to those this process may run on; None when unknown."""
    import os
    try:
        props = torch.cuda.get_device_properties(device)
        address = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{address}/local_cpulist") as handle:
            text = handle.read().strip()
        cpus = set()
        for part in text.split(","):
            first, _, last = part.partition("-")
            cpus.update(range(int(first), int(last or first) + 1))
        cpus &= os.sched_getaffinity(0)
        return cpus or None
    except (OSError, ValueError, AttributeError, RuntimeError, AssertionError):
        return None


def _touch_near(device, tensors):
    """Writes zeros into host tensors that have no pages yet while the calling thread runs on the CPUs next to `device`: the kernel
    places a page on the NUMA node of the thread that first writes it, so the rows a GPU copies end up in the memory of its own socket
    and its PCIe traffic does not cross the link between the sockets.  The thread's CPU affinity is put back afterwards."""
    import os
    before = os.sched_getaffinity(0)
    near = _cpus_near(device)
    try:
        if near:
            os.sched_setaffinity(0, near)
        import ctypes
        for tensor in tensors:  # contiguous row bands; written by this very thread (a parallel fill would touch from other threads)
            ctypes.memset(tensor.data_ptr(), 0, tensor.numel() * tensor.element_size())
    finally:
        if near:
            os.sched_setaffinity(0, before)


class ShardedHostLinear:
    """The host-memory linear on all GPUs of a node: one process per GPU (torch.distributed initialised), the activation `x` (rows, K)
    and the output `y` (rows, N) live in host memory shared by the processes, and rank r moves and multiplies rows
    [r rows / g, (r + 1) rows / g) only, with the whole weight on every GPU (79 MB for the fused QKV projection: replicating it is
    cheap, moving activations between GPUs is not).  Every GPU has its own PCIe link, so the copies of the g bands run side by side:
    no bytes cross NVLink and no collective is involved.  Each band runs through HostLinear's three-stream pipeline.

    x and y are attributes: fill x (any rank; they are the same bytes), call the object on every rank, synchronize and barrier, read y."""

    def __init__(self, weight, scale, bias=None, rows=0, k=0, dtype=torch.bfloat16, chunk_rows=4096, group=None, tag="0"):
        import torch.distributed as dist
        self.group = group
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.rank, self.world = rank, world
        per_rank = -(-rows // world)
        self.start, self.stop = min(rank * per_rank, rows), min((rank + 1) * per_rank, rows)
        self._paths = [f"/dev/shm/wgpkernels_b200_{tag}_{name}" for name in ("x", "y")]
        shapes = ((rows, k), (rows, weight.shape[0]))
        # rank 0 makes the (sparse) files, every rank maps them, writes its own band first -- which places that band's pages in the host
        # memory next to its GPU -- and only then are the pages pinned, by every rank, where they lie
        if rank == 0:
            self.x, self.y = (_shared_mapping(path, shape, dtype, True) for path, shape in zip(self._paths, shapes))
        if world > 1:
            dist.barrier(group)
        if rank != 0:
            self.x, self.y = (_shared_mapping(path, shape, dtype, False) for path, shape in zip(self._paths, shapes))
        _touch_near(torch.cuda.current_device(), (self.x[self.start:self.stop], self.y[self.start:self.stop]))
        if world > 1:
            dist.barrier(group)
        _register(self.x)
        _register(self.y)
        self.inner = HostLinear(weight, scale, bias, chunk_rows=chunk_rows)
        self.h2d_bytes = self.x.numel() * self.x.element_size()
        self.d2h_bytes = self.y.numel() * self.y.element_size()

    def __call__(self, **kwargs):
        if self.stop > self.start:
            self.inner(self.x[self.start:self.stop], self.y[self.start:self.stop], **kwargs)
        return self.y

    def close(self):
        import os
        import torch.distributed as dist
        torch.cuda.synchronize()
        for tensor in (self.x, self.y):
            torch.cuda.cudart().cudaHostUnregister(tensor.data_ptr())
        if self.world > 1:
            dist.barrier(self.group)
        if self.rank == 0:
            for path in self._paths:
                try:
                    os.unlink(path)
                except OSError:
                    pass
