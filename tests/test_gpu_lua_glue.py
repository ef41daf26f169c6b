"""The Lua glue driven through the fake Lua stack on a GPU: every `gpunn_<Op>_<method>(lua_State*)` reads its
module table by field name, computes in place, returns the reference's result count, and raises library errors as
Lua errors; `luaopen_libgputorch` gives the device functions and the cross-type copy methods."""
import numpy as np
import pytest

from lua_glue import GPU, FakeLua
from util import close

pytestmark = pytest.mark.gpu
NN = "torch.GPUTensor.nn"


@pytest.fixture(scope="module")
def gt():
    import mcw_cppamp_torch_b200 as m
    m.lib().THGPUInit()
    return m


@pytest.fixture(scope="module")
def lua(gt):
    fl = FakeLua()
    assert fl.open("gpunn") == 1 and fl.open("gputorch") == 1
    return fl


def T(t):
    return (t._p, GPU)


def test_conv_relu_pool_block_through_the_lua_entry_points(gt, lua, oracle_port):
    g = oracle_port.rng(5)
    N, C, H, W, K, k, d, pad = 3, 3, 31, 31, 32, 5, 2, 2
    conv = gt.nn.SpatialConvolutionMM(C, K, k, k, d, d, pad, rng=g).gpu()
    relu, pool = gt.nn.ReLU(), gt.nn.SpatialMaxPooling(3, 3, 2, 2)
    x = g.uniform((N, C, H, W), -1, 1)
    w, b = conv.weight.float(), conv.bias.float()
    xg = gt.gpu(x)
    assert lua.call(NN, "SpatialConvolutionMM_updateOutput", [T(xg)], lua.module_fields(conv))[0] == 1
    assert lua.call(NN, "Threshold_updateOutput", [T(conv.output)], lua.module_fields(relu))[0] == 1
    assert lua.call(NN, "SpatialMaxPooling_updateOutput", [T(relu.output)], lua.module_fields(pool))[0] == 1
    c = oracle_port.conv_forward(x, w, b, k, k, d, d, pad)
    r = oracle_port.threshold_forward(c)
    p, ind = oracle_port.maxpool_forward(r, 3, 3, 2, 2)
    close(pool.output.float(), p)
    assert np.array_equal(pool.indices.float(), ind)
    go = g.normal(p.shape)
    gog = gt.gpu(go)
    assert lua.call(NN, "SpatialMaxPooling_updateGradInput", [T(relu.output), T(gog)], lua.module_fields(pool))[0] == 1
    assert lua.call(NN, "Threshold_updateGradInput", [T(conv.output), T(pool.gradInput)], lua.module_fields(relu))[0] == 1
    assert lua.call(NN, "SpatialConvolutionMM_updateGradInput", [T(xg), T(relu.gradInput)], lua.module_fields(conv))[0] == 1
    conv.zeroGradParameters()
    # the optional 4th argument is the scale; accGradParameters returns no Lua result
    assert lua.call(NN, "SpatialConvolutionMM_accGradParameters", [T(xg), T(relu.gradInput), 0.5], lua.module_fields(conv))[0] == 0
    g_r = oracle_port.maxpool_backward(go, ind, r.shape, 2, 2)
    g_c = oracle_port.threshold_backward(c, g_r)
    close(conv.gradInput.float(), oracle_port.conv_grad_input(g_c, w, x.shape, k, k, d, d, pad))
    gw, gb = np.zeros_like(w), np.zeros_like(b)
    oracle_port.conv_acc_grad(x, g_c, gw, gb, 0.5, k, k, d, d, pad)
    close(conv.gradWeight.float(), gw); close(conv.gradBias.float(), gb)
    conv.zeroGradParameters()
    lua.call(NN, "SpatialConvolutionMM_accGradParameters", [T(xg), T(relu.gradInput)], lua.module_fields(conv))   # scale defaults to 1
    close(conv.gradWeight.float(), 2 * gw, rtol=2e-4, atol=2e-5)


def test_classifier_tail_and_the_other_operators(gt, lua, oracle_port):
    g = oracle_port.rng(6)
    z = g.normal((6, 20), 0, 2)
    zg = gt.gpu(z)
    lsm, sm, crit = gt.nn.LogSoftMax(), gt.nn.SoftMax(), gt.nn.ClassNLLCriterion()
    assert lua.call(NN, "LogSoftMax_updateOutput", [T(zg)], lua.module_fields(lsm))[0] == 1
    want = oracle_port.logsoftmax_forward(z)
    close(lsm.output.float(), want)
    target = np.array([1, 20, 7, 7, 3, 12], np.float32)
    tg = gt.gpu(target)
    fields = lua.module_fields(crit)
    assert fields["sizeAverage"] is True
    assert lua.call(NN, "ClassNLLCriterion_updateOutput", [T(lsm.output), T(tg)], fields)[0] == 1
    assert abs(crit.outputTensor.float()[0] - oracle_port.classnll_forward(want, target)) < 1e-5
    assert lua.call(NN, "ClassNLLCriterion_updateGradInput", [T(lsm.output), T(tg)], fields)[0] == 1
    close(crit.gradInput.float(), oracle_port.classnll_backward(target, want.shape))
    assert lua.call(NN, "LogSoftMax_updateGradInput", [T(zg), T(crit.gradInput)], lua.module_fields(lsm))[0] == 1
    close(lsm.gradInput.float(), oracle_port.logsoftmax_backward(oracle_port.classnll_backward(target, want.shape), want))
    assert lua.call(NN, "SoftMax_updateOutput", [T(zg)], lua.module_fields(sm))[0] == 1
    close(sm.output.float(), oracle_port.softmax_forward(z), rtol=1e-6, atol=1e-7)
    ap = gt.nn.SpatialAveragePooling(2, 3, 2, 1)
    img = g.normal((2, 4, 9, 10))
    img_gpu = gt.gpu(img)                      # kept alive: T() only borrows the pointer
    assert lua.call(NN, "SpatialAveragePooling_updateOutput", [T(img_gpu)], lua.module_fields(ap))[0] == 1
    assert np.array_equal(ap.output.float(), oracle_port.sumpool_forward(img, 3, 2, 1, 2))


def test_library_errors_become_lua_errors_and_leave_nothing_pending(gt, lua):
    conv = gt.nn.SpatialConvolutionMM(4, 8, 3, 3).gpu()
    small = gt.GPUTensor(1, 4, 2, 2).fill(0)
    with pytest.raises(RuntimeError, match="smaller than kernel"):
        lua.call(NN, "SpatialConvolutionMM_updateOutput", [T(small)], lua.module_fields(conv))
    assert gt.lib().cdll.THGPUGetLastError() is None
    wrong = gt.GPUTensor(1, 3, 8, 8).fill(0)
    with pytest.raises(RuntimeError, match="input channels and nInputPlane dont match"):
        lua.call(NN, "SpatialConvolutionMM_updateOutput", [T(wrong)], lua.module_fields(conv))


def test_gputorch_table_and_copy_methods(gt, lua):
    assert ("<table>", "synchronize") in lua.registered() and ("torch.GPUTensor", "copy") in lua.registered()
    n, out = lua.call("<table>", "getDeviceCount")
    assert n == 1 and out[0] == gt.get_device_count() >= 1
    n, out = lua.call("<table>", "getDevice")
    assert n == 1 and out[0] == 1                                      # 1-based on the Lua side
    assert lua.call("<table>", "setDevice", [1])[0] == 0
    with pytest.raises(RuntimeError, match="device number out of range"):
        lua.call("<table>", "setDevice", [0])
    assert lua.call("<table>", "synchronize")[0] == 0
    # x:copy(y) with y a host DoubleTensor, then host IntTensor:copyGPU(x)
    from mcw_cppamp_torch_b200.tensor import _host_view
    a = np.arange(12, dtype=np.float64).reshape(3, 4) + 0.75
    name, h = _host_view(a)
    x = gt.GPUTensor(3, 4)
    import ctypes as C
    assert lua.call("torch.GPUTensor", "copy", [T(x), (C.pointer(h), b"torch.DoubleTensor")])[0] == 1
    assert np.array_equal(x.float(), a.astype(np.float32))
    back = np.zeros((3, 4), np.int32)
    name, hb = _host_view(back)
    assert lua.call("torch.IntTensor", "copyGPU", [(C.pointer(hb), b"torch.IntTensor"), T(x)])[0] == 1
    assert np.array_equal(back, np.trunc(a).astype(np.int32))
    with pytest.raises(RuntimeError, match=r"torch.\*Tensor expected"):
        lua.call("torch.GPUTensor", "copy", [T(x), (C.pointer(hb), b"torch.WeirdTensor")])
