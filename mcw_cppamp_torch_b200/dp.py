"""Mini-batch data parallelism: one process per GPU, full model replica per rank, the global batch sharded by
rows, the flat gradient buffer summed over the ranks bucket by bucket while backward still runs, each bucket's SGD
update right behind its all-reduce.

The reference has no multi-device code at all (its device functions are stubs, gputorch/init.cpp:10-66); this
follows the usual contract of Torch7 data-parallel training on top of `Module:getParameters()`
(mcw_nn/Module.lua:169-252): the flat gradient buffer is what crosses the wire.  The exchange itself lives in
libTHC.so (THGPUComm: NCCL communicator, own stream, event ordering, watchdog); this module is the thin host
wrapper.  The only thing a host must bring is a way to hand rank 0's 128-byte id to the other ranks."""
import ctypes as C

from ._lib import THGPUCommBackend, THCError, lib


def shard_rows(global_batch, rank, world):
    """Rows [lo, hi) of the global batch owned by `rank` (even shards required)."""
    if global_batch % world:
        raise ValueError("global batch %d does not divide over %d ranks" % (global_batch, world))
    per = global_batch // world
    return rank * per, (rank + 1) * per


def layer_buckets(net, min_elements=0):
    """Element ranges of the flat parameter / gradient buffer made by `net.getParameters()` in the order backward
    finishes them (last module first).  Returns (spans, owner): spans = [(begin, end)], owner = {index of the
    parametrised module, counted from the last one: (bucket, is_last_of_bucket)}.  With min_elements = 0 every
    parametrised module is a bucket of its own; otherwise consecutive modules are merged until a bucket holds at
    least min_elements (the remainder at the front of the net forms the last bucket): every collective is a point
    where the ranks wait for one another, so a few large buckets cost less than many small ones."""
    off, layers = 0, []
    for m in net.modules_list():
        p = m.parameters()
        if p:
            k = sum(t.nElement() for t in p[0])
            layers.append((off, off + k))
            off += k
    layers = layers[::-1]
    spans, owner = [], {}
    begin_idx = 0
    for i, (b, e) in enumerate(layers):
        lo = layers[i][0]                      # backward order walks the buffer downwards: the open bucket is [lo, hi)
        hi = layers[begin_idx][1]
        last = i == len(layers) - 1 or hi - lo >= max(min_elements, 1)
        owner[i] = (len(spans), last)
        if last:
            spans.append((lo, hi))
            begin_idx = i + 1
    return spans, owner


class Comm:
    """THGPUComm of this rank."""

    def __init__(self, handle, keep=None):
        self._h = handle
        self._keep = keep
        self.nbuckets = 0

    @classmethod
    def nccl(cls, world, rank, exchange, max_ctas=0):
        """`exchange(id_bytes_or_None) -> id_bytes`: called with the fresh id on rank 0 and with None elsewhere;
        returns rank 0's bytes on every rank (a broadcast over whatever the host has).  `max_ctas` > 0 caps the
        SMs a collective may occupy beside the backward pass (THGPUComm_newWithOptions)."""
        L = lib()
        buf = C.create_string_buffer(128)
        if rank == 0:
            L.THGPUComm_getUniqueId(buf)
        raw = exchange(buf.raw if rank == 0 else None)
        if len(raw) != 128:
            raise ValueError("the communicator id has 128 bytes")
        return cls(L.THGPUComm_newWithOptions(world, rank, C.create_string_buffer(raw, 128), int(max_ctas)))

    @classmethod
    def with_backend(cls, world, rank, **callbacks):
        """A communicator over caller-supplied transport callbacks (names as the fields of THGPUCommBackend)."""
        be = THGPUCommBackend()
        keep = []
        for name, ctype in (("all_reduce", be.ALL_REDUCE), ("set_update", be.SET_UPDATE), ("done", be.DONE),
                            ("join", be.JOIN), ("agree", be.AGREE), ("abort", be.ABORT), ("destroy", be.DESTROY)):
            if name in callbacks:
                fn = ctype(callbacks[name])
                keep.append(fn)
                setattr(be, name, fn)
        return cls(lib().THGPUComm_newWithBackend(world, rank, C.byref(be)), keep)

    def set_timeout(self, seconds):
        lib().THGPUComm_setTimeout(self._h, float(seconds))

    def set_buckets(self, flat_grad, bounds):
        arr = (C.c_long * (2 * len(bounds)))(*[v for lo_hi in bounds for v in lo_hi])
        lib().THGPUComm_setBuckets(self._h, flat_grad._p, arr, len(bounds))
        self.nbuckets = len(bounds)

    def set_update(self, flat_w, flat_v, lr, momentum):
        lib().THGPUComm_setUpdate(self._h, flat_w._p, flat_v._p if flat_v is not None else None, lr, momentum)

    def launch(self, bucket):
        lib().THGPUComm_allReduceAsync(self._h, bucket)

    def wait(self):
        lib().THGPUComm_wait(self._h)

    def error(self):
        e = lib().THGPUComm_error(self._h)
        return e.decode() if e else None

    def close(self):
        if self._h:
            lib().THGPUComm_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


__all__ = ["shard_rows", "layer_buckets", "Comm", "THCError"]
