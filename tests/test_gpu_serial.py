"""Serialisation of torch.GPUTensor / torch.GPUStorage: the byte layout of the records
(gputorch/torch/generic/Tensor.c:1150-1199, generic/Storage.c:180-200), round trips of views, large storages
that need several staging chunks, corrupt records, and `Module:clone()` / save / load of a network whose
parameters share one flat storage (mcw_nn/Module.lua:104-114, :169-252)."""
import io
import struct

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gt():
    import mcw_cppamp_torch_b200 as m
    m.lib().THGPUInit()
    return m


def test_record_layout_is_the_reference_s(gt):
    a = np.arange(24, dtype=np.float32).reshape(4, 6)
    view = gt.gpu(a).narrow(1, 2, 2).t()            # rows 1..2 of a, transposed: size (6, 2), stride (1, 6), offset 6
    buf = io.BytesIO()
    view.write(buf)
    raw = buf.getvalue()
    nd, = struct.unpack_from("i", raw, 0)
    size = struct.unpack_from("2l", raw, 4)
    stride = struct.unpack_from("2l", raw, 20)
    off1, has, ssize = struct.unpack_from("3l", raw, 36)
    assert (nd, size, stride, off1, has, ssize) == (2, (6, 2), (1, 6), 7, 1, 24)   # offset is written 1-based
    assert np.array_equal(np.frombuffer(raw, np.float32, 24, 60), a.ravel())       # the whole storage follows
    assert len(raw) == 60 + 96


def test_round_trip_of_views_empty_tensors_and_chunked_storages(gt):
    g = np.random.RandomState(0)
    a = g.standard_normal((5, 7, 3)).astype(np.float32)
    for make in (lambda x: x, lambda x: x.transpose(1, 3), lambda x: x.select(2, 4), lambda x: x.narrow(3, 2, 2)):
        t = make(gt.gpu(a))
        buf = io.BytesIO()
        t.write(buf)
        buf.seek(0)
        back = gt.GPUTensor().read(buf)
        assert back.size() == t.size() and back.stride() == t.stride() and back.storageOffset() == t.storageOffset()
        assert np.array_equal(back.float(), t.float())
    buf = io.BytesIO()
    gt.GPUTensor().write(buf)
    buf.seek(0)
    assert gt.GPUTensor(3).read(buf).dim() == 0
    big = g.standard_normal(5_000_003).astype(np.float32)       # more than one 16 MiB staging chunk
    buf = io.BytesIO()
    gt.gpu(big).write(buf)
    buf.seek(0)
    assert np.array_equal(gt.GPUTensor().read(buf).float(), big)


def test_corrupt_and_short_records_are_errors(gt):
    buf = io.BytesIO()
    gt.gpu(np.ones((3, 3), np.float32)).write(buf)
    raw = buf.getvalue()
    with pytest.raises(gt.THCError, match="read error"):
        gt.GPUTensor().read(io.BytesIO(raw[:-5]))
    with pytest.raises(gt.THCError, match="corrupt tensor record"):
        gt.GPUTensor().read(io.BytesIO(struct.pack("i", 99) + raw[4:]))
    bad = bytearray(raw)
    struct.pack_into("l", bad, 4, 1000)                         # a size that reaches beyond the storage
    with pytest.raises(gt.THCError, match="beyond its storage"):
        gt.GPUTensor().read(io.BytesIO(bytes(bad)))
    with pytest.raises(gt.THCError, match="not writable|write error"):
        gt.gpu(np.ones(4, np.float32)).write(_Closed())


class _Closed:
    def write(self, b):
        raise IOError("closed")

    def read(self, n):
        raise IOError("closed")


def _small_net(gt, g):
    net = gt.nn.Sequential()
    net.add(gt.nn.SpatialConvolutionMM(3, 8, 3, 3, 1, 1, 1, rng=g)).add(gt.nn.ReLU()).add(gt.nn.SpatialMaxPooling(2, 2))
    net.add(gt.nn.View(8 * 4 * 4)).add(gt.nn.Linear(8 * 4 * 4, 10, rng=g)).add(gt.nn.LogSoftMax())
    return net.gpu()


def test_module_clone_and_save_load_keep_shared_parameter_storage(gt, oracle_port, tmp_path):
    g = oracle_port.rng(12)
    net = _small_net(gt, g)
    fw, fg = net.getParameters()                               # all parameters become views of one storage
    x = gt.gpu(g.uniform((2, 3, 8, 8), -1, 1))
    want = net.forward(x).float()
    twin = net.clone()
    assert np.array_equal(twin.forward(x).float(), want)
    conv, lin = twin.modules[0], twin.modules[4]
    assert conv.weight.storage() is lin.weight.storage()        # still ONE flat storage after the round trip
    assert conv.weight.storage() is not net.modules[0].weight.storage()
    assert conv.weight.storage().size() == fw.nElement()
    conv.weight.fill(0)                                         # the clone is independent of the original
    assert np.array_equal(net.forward(x).float(), want)
    path = str(tmp_path / "net.t7")
    gt.save(net, path)
    again = gt.load(path)
    assert np.array_equal(again.forward(x).float(), want)
    assert again.modules[0].kW == 3 and again.modules[0].weight.storage() is again.modules[4].weight.storage()
