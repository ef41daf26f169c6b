"""B200-native gputorch/gpunn hot path: `torch.GPUTensor`, its math, and the nn modules on it.

    import mcw_cppamp_torch_b200 as gt
    x = gt.gpu(np_array)                 # host FloatTensor -> torch.GPUTensor
    net = gt.nn.Sequential(); net.add(gt.nn.SpatialConvolutionMM(3, 64, 11, 11, 4, 4, 2)) ...
    net.gpu(); y = net.forward(x)

Everything computes in libTHC.so (hand-written CUDA for sm_100a) through its C ABI."""
from .tensor import GPUTensor, GPUStorage, gpu, save, load, synchronize, set_device, get_device_count, set_math_mode  # noqa: F401
from ._lib import lib, THCError  # noqa: F401
from . import nn  # noqa: F401
