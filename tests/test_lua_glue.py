"""The Lua glue (mcw_cppamp_torch_b200/lua) compiled against the fake Lua of tests/lua_shim: what it registers and
where, and the argument protocol, on machines without a GPU."""
import ctypes as C

import pytest

from lua_glue import GPU, FakeLua

NN_FUNCTIONS = {  # name -> number of Lua results (gputorch/lib/THC/gpunn-impl/*.cpp `return` of each function)
    "SpatialConvolutionMM_updateOutput": 1, "SpatialConvolutionMM_updateGradInput": 1,
    "SpatialConvolutionMM_accGradParameters": 0,
    "SpatialMaxPooling_updateOutput": 1, "SpatialMaxPooling_updateGradInput": 1,
    "Threshold_updateOutput": 1, "Threshold_updateGradInput": 1,
    "LogSoftMax_updateOutput": 1, "LogSoftMax_updateGradInput": 1,
    "SoftMax_updateOutput": 1, "SoftMax_updateGradInput": 1,
    "SpatialAveragePooling_updateOutput": 1, "SpatialAveragePooling_updateGradInput": 1,
    "ClassNLLCriterion_updateOutput": 1, "ClassNLLCriterion_updateGradInput": 1,
}


@pytest.fixture(scope="module")
def lua():
    fl = FakeLua()
    assert fl.open("gpunn") == 1
    return fl


def test_operators_are_registered_under_nn_of_the_gpu_tensor_metatable(lua):
    reg = lua.registered()
    assert sorted(n for o, n in reg if o == "torch.GPUTensor.nn") == sorted(NN_FUNCTIONS)
    assert all(o == "torch.GPUTensor.nn" for o, n in reg)


def test_argument_protocol_is_checked_before_any_compute(lua):
    from mcw_cppamp_torch_b200 import lib
    L = lib()
    st = L.THGPUStorage_newWithData(C.c_void_p(0x1000), 3 * 8 * 8)
    x = L.THGPUTensor_newWithStorage1d(st, 0, 3 * 8 * 8, 1)          # metadata only: no device is touched
    with pytest.raises(RuntimeError, match=r"#2 \(torch.GPUTensor expected\)"):
        lua.call("torch.GPUTensor.nn", "SpatialConvolutionMM_updateOutput", [None], {})
    with pytest.raises(RuntimeError, match=r"#2 \(torch.GPUTensor expected\)"):
        lua.call("torch.GPUTensor.nn", "Threshold_updateOutput", [(x, b"torch.FloatTensor")], {})
    with pytest.raises(RuntimeError, match="field dW does not exist"):
        lua.call("torch.GPUTensor.nn", "SpatialConvolutionMM_updateOutput", [(x, GPU)], {})
    fields = dict(dW=1, dH=1, kW=3, kH=3, nInputPlane=3, nOutputPlane=4, padding=0)
    with pytest.raises(RuntimeError, match="field weight does not exist"):
        lua.call("torch.GPUTensor.nn", "SpatialConvolutionMM_updateOutput", [(x, GPU)], fields)
    for k in ("weight", "bias", "finput", "fgradInput", "output"):
        fields[k] = (x, GPU)
    with pytest.raises(RuntimeError, match=r"#2 \(3D or 4D \(batch mode\) tensor is expected\)"):
        lua.call("torch.GPUTensor.nn", "SpatialConvolutionMM_updateOutput", [(x, GPU)], fields)
    with pytest.raises(RuntimeError, match="field sizeAverage is not a boolean"):
        lua.call("torch.GPUTensor.nn", "ClassNLLCriterion_updateOutput", [(x, GPU), (x, GPU)],
                 dict(outputTensor=(x, GPU), sizeAverage=1))
    with pytest.raises(KeyError):
        lua.call("torch.GPUTensor.nn", "SpatialConvolutionGPU_updateOutput", [], {})
    L.THGPUTensor_free(x)
    L.THGPUStorage_free(st)
