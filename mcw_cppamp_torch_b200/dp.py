"""Mini-batch data parallelism: one process per GPU, full model replica per rank, the global batch
sharded by rows, gradients summed with an all-reduce, identical SGD update on every rank.

The reference has no multi-device code at all (its device functions are stubs,
gputorch/init.cpp:10-66); this follows the usual contract of Torch7 data-parallel training on top
of `Module:getParameters()` (mcw_nn/Module.lua:169-252): the flat gradient buffer is what crosses
the wire.  Collectives go through torch.distributed (NCCL over NVLink on GPUs, gloo on CPU for the
host-logic tests); the flat parameter / gradient buffers are torch tensors whose memory the
GPUTensor views borrow, so the collective and the CUDA kernels touch the same bytes."""
import torch
import torch.distributed as dist


def shard_rows(global_batch, rank, world):
    """Rows [lo, hi) of the global batch owned by `rank` (even shards required)."""
    if global_batch % world:
        raise ValueError("global batch %d does not divide over %d ranks" % (global_batch, world))
    per = global_batch // world
    return rank * per, (rank + 1) * per


class GradBuckets:
    """Contiguous slices of the flat gradient tensor, all-reduced (sum) independently so that a bucket
    whose gradients are complete can travel while the rest of backward still runs.  `bounds` are the
    element offsets where buckets start, in the order the buckets become ready."""

    def __init__(self, flat_grad, bounds):
        self.flat = flat_grad
        self.slices = []
        n = flat_grad.numel()
        for lo, hi in bounds:
            if not (0 <= lo < hi <= n):
                raise ValueError("bucket [%d, %d) outside the flat buffer of %d" % (lo, hi, n))
            self.slices.append(flat_grad[lo:hi])
        covered = sorted(bounds)
        pos = 0
        for lo, hi in covered:
            if lo != pos:
                raise ValueError("buckets must tile the flat buffer")
            pos = hi
        if pos != n:
            raise ValueError("buckets must tile the flat buffer")
        self.pending = []

    def launch(self, i):
        """Start the all-reduce of bucket i (asynchronous when a process group exists)."""
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            self.pending.append(dist.all_reduce(self.slices[i], op=dist.ReduceOp.SUM, async_op=True))

    def wait(self):
        for w in self.pending:
            w.wait()
        self.pending = []


def world():
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1
