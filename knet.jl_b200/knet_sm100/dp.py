"""Host-side rules of the data-parallel training step (one process per GPU).
A `group` argument is either a torch.distributed process group or a `KnetComm` (the library's
own NCCL communicator behind the knet_dp_* C entry points).

Knet has no multi-GPU path; this is the batch-sharded step of the MLP benchmark: every rank
holds the same weights and optimizer state, takes a contiguous shard of the batch columns,
all-reduces (sum) each layer's gradient bucket as soon as it is final, and folds the 1/world
factor into the optimizer's read of the gradient.  The functions here are backend-agnostic
(NCCL on GPUs, gloo in the CPU tests).
"""
import os

import torch
import torch.distributed as dist


def init_from_env(backend):
    """Create the default process group from torchrun's environment; returns (rank, world)."""
    if "RANK" not in os.environ:
        return 0, 1
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if not dist.is_initialized():
        dist.init_process_group(backend=backend)
    return dist.get_rank(), dist.get_world_size()


def shard_range(n, rank, world):
    """Columns [lo, hi) of a batch of n that rank `rank` owns (contiguous, near-equal)."""
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def bucket_bounds(offsets):
    """[(start, stop)] per layer of a flat [W1,b1,W2,b2,...] buffer, in backward order."""
    return [(int(offsets[i]), int(offsets[i + 1])) for i in reversed(range(len(offsets) - 1))]


def allreduce_bucket(flat_g, bounds, group=None, async_op=True):
    """Sum one gradient bucket over the ranks in place; returns the work handle."""
    a, b = bounds
    if isinstance(group, KnetComm):
        return group.all_reduce(flat_g[a:b], async_op=async_op)
    return dist.all_reduce(flat_g[a:b], op=dist.ReduceOp.SUM, group=group, async_op=async_op)


# ---- sharded optimizer state: reduce-scatter -> update of the own shard -> all-gather ---------------
# Each layer bucket is padded to world * chunk elements (chunk a multiple of `align`, so that
# every shard starts on a 16-byte boundary); rank r owns [start + r*chunk, start + (r+1)*chunk).
# The optimizer then reads and writes 1/world of the weights, gradients and state per GPU.
def padded_offsets(counts, world, align=4):
    """Start of every bucket (and the total) when bucket i holds counts[i] elements padded up
    to a multiple of world * align."""
    out, o = [0], 0
    q = world * align
    for c in counts:
        o += (int(c) + q - 1) // q * q
        out.append(o)
    return out


def shard_bounds(bounds, rank, world):
    """The part of bucket [a, b) that `rank` owns; (b - a) must be a multiple of world."""
    a, b = bounds
    chunk, rem = divmod(b - a, world)
    if rem:
        raise ValueError(f"bucket of {b - a} elements does not split over {world} ranks")
    return a + rank * chunk, a + (rank + 1) * chunk


def reduce_scatter_bucket(flat_g, bounds, rank, world, group=None, async_op=True):
    """Sum bucket [a, b) over the ranks, leaving rank r's shard of the sum in place at its own
    position inside flat_g (the rest of the bucket is unspecified afterwards).  gloo has no
    reduce-scatter: there the whole bucket is all-reduced, which leaves the same shard."""
    a, b = bounds
    lo, hi = shard_bounds(bounds, rank, world)
    if isinstance(group, KnetComm):
        return group.reduce_scatter(flat_g[lo:hi], flat_g[a:b], async_op=async_op)
    if dist.get_backend(group) == "gloo":
        return dist.all_reduce(flat_g[a:b], op=dist.ReduceOp.SUM, group=group, async_op=async_op)
    return dist.reduce_scatter_tensor(flat_g[lo:hi], flat_g[a:b], op=dist.ReduceOp.SUM, group=group,
                                      async_op=async_op)


def allgather_bucket(flat_w, bounds, rank, world, group=None, async_op=True):
    """Every rank contributes its shard of bucket [a, b) of flat_w; afterwards the whole bucket
    is identical everywhere (in place: the shard already sits at its position)."""
    a, b = bounds
    lo, hi = shard_bounds(bounds, rank, world)
    if isinstance(group, KnetComm):
        return group.all_gather(flat_w[a:b], flat_w[lo:hi], async_op=async_op)
    if dist.get_backend(group) == "gloo":
        parts = [torch.empty(hi - lo, dtype=flat_w.dtype) for _ in range(world)]
        w = dist.all_gather(parts, flat_w[lo:hi].clone(), group=group)
        flat_w[a:b].copy_(torch.cat(parts))
        return w
    return dist.all_gather_into_tensor(flat_w[a:b], flat_w[lo:hi], group=group, async_op=async_op)


def gradient_scale(world):
    """Factor applied to the summed gradient: the mean over ranks of per-rank mean losses."""
    return 1.0 / world


def reduce_loss(total, count, group=None):
    """Global (sum, count) of the per-rank nll totals for reporting."""
    t = torch.stack([total.reshape(()).to(torch.float64), count.reshape(()).to(torch.float64)])
    if isinstance(group, KnetComm):
        group.all_reduce(t)
    else:
        dist.all_reduce(t, group=group)
    return float(t[0]), int(t[1])


# ---- the library's own communicator (knet_dp_* entry points) --------------------------------------
class _Done:
    """Handle of a collective launched on the communicator's side stream: wait() makes the
    caller's current stream wait for it (the host does not block)."""

    def __init__(self, event):
        self.event = event

    def wait(self):
        torch.cuda.current_stream().wait_event(self.event)


class KnetComm:
    """NCCL communicator created through libknet_sm100's knet_dp_* functions, usable wherever
    this module takes a `group`.  The 128-byte id travels from rank 0 to the others through
    an existing torch.distributed group (any backend; gloo is enough) or a caller-supplied
    `exchange(bytes_or_None) -> bytes` function, e.g. one backed by a file or a socket."""

    def __init__(self, rank, world, exchange=None, timeout_ms=60000, device=None):
        import ctypes as C
        from .lib import check, libknet
        self._C, self._lib, self._check = C, libknet, check
        self.rank, self.world = rank, world
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        ident = (C.c_ubyte * 128)()
        status = libknet.knet_dp_unique_id(ident) if rank == 0 else 0
        if exchange is None:
            # the id travels with rank 0's status, so that a failure there raises on every rank
            # instead of leaving the others waiting for the broadcast
            t = torch.tensor(list(bytes(ident)) + [1 if status else 0], dtype=torch.uint8)
            if dist.get_backend() == "nccl":
                t = t.to(self.device)
            dist.broadcast(t, 0)
            raw = bytes(t.cpu().tolist())
            if raw[128]:
                check(status if rank == 0 else -5, "knet_dp_unique_id (on rank 0)")
            raw = raw[:128]
        else:
            check(status, "knet_dp_unique_id")
            raw = exchange(bytes(ident) if rank == 0 else None)
        ident = (C.c_ubyte * 128).from_buffer_copy(raw)
        handle = C.c_void_p()
        with torch.cuda.device(self.device):
            check(libknet.knet_dp_init(ident, rank, world, int(timeout_ms), C.byref(handle)), "knet_dp_init")
            self.stream = torch.cuda.Stream()
        self.handle = handle

    def _launch(self, fn, name, async_op):
        """Run `fn(stream_pointer)` on the side stream after the work already queued on the
        caller's stream; returns a handle (async) or waits on the caller's stream."""
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream())
        self.stream.wait_event(ready)
        self._check(fn(self._C.c_void_p(self.stream.cuda_stream)), name)
        done = torch.cuda.Event()
        done.record(self.stream)
        h = _Done(done)
        if async_op:
            return h
        h.wait()
        return None

    def _sfx(self, t):
        return "32" if t.dtype == torch.float32 else "64"

    def all_reduce(self, t, async_op=False):
        f = getattr(self._lib, f"knet_dp_allreduce_sum_{self._sfx(t)}")
        p = self._C.c_void_p(t.data_ptr())
        t.record_stream(self.stream)
        return self._launch(lambda s: f(self.handle, p, t.numel(), s), "knet_dp_allreduce_sum", async_op)

    def reduce_scatter(self, out, inp, async_op=False):
        f = getattr(self._lib, f"knet_dp_reduce_scatter_sum_{self._sfx(inp)}")
        po, pi = self._C.c_void_p(out.data_ptr()), self._C.c_void_p(inp.data_ptr())
        inp.record_stream(self.stream)
        return self._launch(lambda s: f(self.handle, pi, po, out.numel(), s), "knet_dp_reduce_scatter_sum", async_op)

    def all_gather(self, out, inp, async_op=False):
        f = getattr(self._lib, f"knet_dp_allgather_{self._sfx(inp)}")
        po, pi = self._C.c_void_p(out.data_ptr()), self._C.c_void_p(inp.data_ptr())
        out.record_stream(self.stream)
        return self._launch(lambda s: f(self.handle, pi, po, inp.numel(), s), "knet_dp_allgather", async_op)

    def broadcast(self, t, root=0, async_op=False):
        f = getattr(self._lib, f"knet_dp_broadcast_{self._sfx(t)}")
        p = self._C.c_void_p(t.data_ptr())
        return self._launch(lambda s: f(self.handle, p, t.numel(), root, s), "knet_dp_broadcast", async_op)

    def destroy(self):
        if self.handle is not None:
            torch.cuda.synchronize(self.device)
            self._check(self._lib.knet_dp_destroy(self.handle), "knet_dp_destroy")
            self.handle = None
