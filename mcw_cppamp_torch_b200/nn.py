"""The `nn` modules on the hot path, mirroring the reference's Lua classes over the C ABI.

Each class keeps the field names the reference's C operators read off the Lua module table
(`weight`, `bias`, `gradWeight`, `gradBias`, `finput`, `fgradInput`, `output`, `gradInput`,
`indices`, `kW`, `kH`, `dW`, `dH`, `padding`, `threshold`, `val`) and the `nn.Module` protocol of
mcw_nn/Module.lua:20-82 (forward / backward / updateOutput / updateGradInput / accGradParameters /
zeroGradParameters / updateParameters / parameters / getParameters).  Modules are built with host
(numpy) parameters, like the reference builds them with FloatTensors, and `:gpu()` moves them.
There is no CPU compute path: calling forward before `:gpu()` raises."""
import ctypes as C
import math

import numpy as np

from ._lib import lib
from .tensor import GPUTensor, gpu, _long_storage


class _NumpyRng:
    """Default host RNG for `reset()`; tests pass the TH-compatible generator instead."""

    def __init__(self, seed=0):
        self._g = np.random.default_rng(seed)

    def uniform(self, shape, a, b):
        return self._g.uniform(a, b, size=shape).astype(np.float32)


_default_rng = _NumpyRng()


def _need_gpu(t, what):
    if not isinstance(t, GPUTensor):
        raise TypeError("%s: torch.GPUTensor expected (this build has no CPU compute path; call :gpu())" % what)
    return t


class Module:
    """mcw_nn/Module.lua"""

    def __init__(self):
        self.output = GPUTensor()
        self.gradInput = GPUTensor()

    # -- protocol --
    def parameters(self):
        w, g = [], []
        if getattr(self, "weight", None) is not None:
            w += [self.weight]; g += [self.gradWeight]
        if getattr(self, "bias", None) is not None:
            w += [self.bias]; g += [self.gradBias]
        return (w, g) if w else None

    def updateOutput(self, input):
        return self.output

    def updateGradInput(self, input, gradOutput):
        return self.gradInput

    def accGradParameters(self, input, gradOutput, scale=1.0):
        pass

    def forward(self, input):
        return self.updateOutput(input)

    def backward(self, input, gradOutput, scale=1.0):
        self.updateGradInput(input, gradOutput)
        self.accGradParameters(input, gradOutput, scale)
        return self.gradInput

    def zeroGradParameters(self):
        p = self.parameters()
        if p:
            for g in p[1]:
                g.zero()

    def updateParameters(self, learningRate):
        p = self.parameters()
        if p:
            for w, g in zip(*p):
                w.add(-learningRate, g)

    def gpu(self):
        """Module:type('torch.GPUTensor'): converts every host tensor field (mcw_nn/Module.lua:116-148)."""
        for k, v in list(self.__dict__.items()):
            if isinstance(v, np.ndarray):
                setattr(self, k, gpu(v))
        return self

    def modules_list(self):
        return [self]

    def clone(self):
        """mcw_nn/Module.lua:104-114: the module written into a memory file and read back -- every GPU tensor
        goes through the library's storage / tensor records, tensors that share a storage still share one."""
        import io
        import pickle
        buf = io.BytesIO()
        pickle.dump(self, buf, protocol=4)
        buf.seek(0)
        return pickle.load(buf)

    def getParameters(self, flat=None):
        """Flattens all parameters (and gradients) into one storage each and re-points the modules'
        tensors at views of it (mcw_nn/Module.lua:169-252).  `flat` may carry two caller-owned
        device buffers `(w_ptr, g_ptr, n)` to flatten into (e.g. memory shared with a collective)."""
        L = lib()
        ws, gs = [], []
        for m in self.modules_list():
            p = m.parameters()
            if p:
                ws += p[0]; gs += p[1]
        n = sum(t.nElement() for t in ws)
        if flat is None:
            fw, fg = GPUTensor(n), GPUTensor(n)
        else:
            wptr, gptr, cap = flat
            assert cap >= n
            sw = L.THGPUStorage_newWithData(C.c_void_p(wptr), n)
            sg = L.THGPUStorage_newWithData(C.c_void_p(gptr), n)
            fw = GPUTensor(_ptr=L.THGPUTensor_newWithStorage1d(sw, 0, n, 1))
            fg = GPUTensor(_ptr=L.THGPUTensor_newWithStorage1d(sg, 0, n, 1))
            L.THGPUStorage_free(sw); L.THGPUStorage_free(sg)
        off = 0
        for t, g in zip(ws, gs):
            k = t.nElement()
            for flat_t, part in ((fw, t), (fg, g)):
                dst = flat_t.narrow(1, off + 1, k)
                dst.copy(part.contiguous().view(k))
                size = _long_storage(list(part.size()))
                L.THGPUTensor_setStorage(part._p, flat_t._p.contents.storage, off, C.byref(size), None)
            off += k
        return fw, fg


class Sequential(Module):
    """mcw_nn/Sequential.lua"""

    def __init__(self):
        super().__init__()
        self.modules = []

    def add(self, m):
        self.modules.append(m)
        return self

    def modules_list(self):
        out = []
        for m in self.modules:
            out += m.modules_list()
        return out

    def parameters(self):
        return None

    def gpu(self):
        for m in self.modules:
            m.gpu()
        return self

    def updateOutput(self, input):
        cur = input
        for m in self.modules:
            cur = m.updateOutput(cur)
        self.output = cur
        return cur

    def updateGradInput(self, input, gradOutput):
        cur = gradOutput
        for i in range(len(self.modules) - 1, 0, -1):
            cur = self.modules[i].updateGradInput(self.modules[i - 1].output, cur)
        cur = self.modules[0].updateGradInput(input, cur)
        self.gradInput = cur
        return cur

    def accGradParameters(self, input, gradOutput, scale=1.0):
        cur = gradOutput
        for i in range(len(self.modules) - 1, 0, -1):
            prev = self.modules[i - 1].output
            self.modules[i].accGradParameters(prev, cur, scale)
            cur = self.modules[i].gradInput
        self.modules[0].accGradParameters(input, cur, scale)

    def backward(self, input, gradOutput, scale=1.0):
        # mcw_nn/Sequential.lua backward: each module's backward in reverse order
        cur = gradOutput
        for i in range(len(self.modules) - 1, 0, -1):
            cur = self.modules[i].backward(self.modules[i - 1].output, cur, scale)
        cur = self.modules[0].backward(input, cur, scale)
        self.gradInput = cur
        return cur

    def zeroGradParameters(self):
        for m in self.modules:
            m.zeroGradParameters()

    def updateParameters(self, lr):
        for m in self.modules:
            m.updateParameters(lr)


class SpatialConvolutionMM(Module):
    """mcw_nn/SpatialConvolutionMM.lua over gpunn SpatialConvolutionMM_* (reference:
    gputorch/lib/THC/gpunn-impl/SpatialConvolutionMM.cpp:110-429)."""

    def __init__(self, nInputPlane, nOutputPlane, kW, kH, dW=1, dH=1, padding=0, rng=None):
        super().__init__()
        self.nInputPlane, self.nOutputPlane = nInputPlane, nOutputPlane
        self.kW, self.kH, self.dW, self.dH, self.padding = kW, kH, dW, dH, padding
        self.weight = np.empty((nOutputPlane, nInputPlane * kH * kW), np.float32)
        self.bias = np.empty((nOutputPlane,), np.float32)
        self.gradWeight = np.zeros_like(self.weight)
        self.gradBias = np.zeros_like(self.bias)
        self.finput = GPUTensor()
        self.fgradInput = GPUTensor()
        self.reset(rng=rng)

    def reset(self, stdv=None, rng=None):
        """uniform(-stdv, stdv), weight first then bias (mcw_nn/SpatialConvolutionMM.lua:29-46)."""
        rng = rng or _default_rng
        stdv = stdv * math.sqrt(3) if stdv else 1.0 / math.sqrt(self.kW * self.kH * self.nInputPlane)
        w = rng.uniform(tuple(self.weight.shape) if isinstance(self.weight, np.ndarray) else self.weight.size(), -stdv, stdv)
        b = rng.uniform((self.nOutputPlane,), -stdv, stdv)
        if isinstance(self.weight, np.ndarray):
            self.weight, self.bias = w, b
        else:
            self.weight.copy(w); self.bias.copy(b)

    def updateOutput(self, input):
        _need_gpu(input, "SpatialConvolutionMM"); _need_gpu(self.weight, "SpatialConvolutionMM.weight")
        lib().THGPUNN_SpatialConvolutionMM_updateOutput(input._p, self.output._p, self.weight._p, self.bias._p,
                                                        self.finput._p, self.fgradInput._p, self.kW, self.kH,
                                                        self.dW, self.dH, self.padding)
        return self.output

    def updateGradInput(self, input, gradOutput):
        if self.gradInput is None:
            return None
        lib().THGPUNN_SpatialConvolutionMM_updateGradInput(input._p, gradOutput._p, self.gradInput._p, self.weight._p,
                                                           self.finput._p, self.fgradInput._p, self.kW, self.kH,
                                                           self.dW, self.dH, self.padding)
        return self.gradInput

    def accGradParameters(self, input, gradOutput, scale=1.0):
        lib().THGPUNN_SpatialConvolutionMM_accGradParameters(input._p, gradOutput._p, self.gradWeight._p,
                                                             self.gradBias._p, self.finput._p, self.fgradInput._p,
                                                             self.kW, self.kH, self.dW, self.dH, self.padding, scale)


    def backward(self, input, gradOutput, scale=1.0):
        """updateGradInput + accGradParameters (mcw_nn/Module.lua backward) in one library call that
        transposes gradOutput once."""
        gi = self.gradInput._p if self.gradInput is not None else None
        lib().THGPUNN_SpatialConvolutionMM_backward(input._p, gradOutput._p, gi, self.weight._p, self.gradWeight._p,
                                                    self.gradBias._p, self.finput._p, self.fgradInput._p,
                                                    self.kW, self.kH, self.dW, self.dH, self.padding, scale)
        return self.gradInput


class SpatialMaxPooling(Module):
    """mcw_nn/SpatialMaxPooling.lua over gpunn SpatialMaxPooling_*."""

    def __init__(self, kW, kH, dW=None, dH=None):
        super().__init__()
        self.kW, self.kH = kW, kH
        self.dW, self.dH = dW or kW, dH or kH
        self.indices = GPUTensor()

    def updateOutput(self, input):
        _need_gpu(input, "SpatialMaxPooling")
        lib().THGPUNN_SpatialMaxPooling_updateOutput(input._p, self.output._p, self.indices._p, self.kW, self.kH,
                                                     self.dW, self.dH)
        return self.output

    def updateGradInput(self, input, gradOutput):
        lib().THGPUNN_SpatialMaxPooling_updateGradInput(input._p, gradOutput._p, self.gradInput._p, self.indices._p,
                                                        self.kW, self.kH, self.dW, self.dH)
        return self.gradInput


class Threshold(Module):
    """mcw_nn/Threshold.lua"""

    def __init__(self, th=1e-6, v=0.0):
        super().__init__()
        self.threshold, self.val = th, v

    def updateOutput(self, input):
        _need_gpu(input, "Threshold")
        lib().THGPUNN_Threshold_updateOutput(input._p, self.output._p, self.threshold, self.val)
        return self.output

    def updateGradInput(self, input, gradOutput):
        lib().THGPUNN_Threshold_updateGradInput(input._p, gradOutput._p, self.gradInput._p, self.threshold)
        return self.gradInput


class ReLU(Threshold):
    """mcw_nn/ReLU.lua:3-5: Threshold(0, 0)"""

    def __init__(self):
        super().__init__(0.0, 0.0)


class View(Module):
    """Reshape of a contiguous batch, e.g. [N,256,6,6] -> [N,9216] (mcw_nn/Reshape.lua / View)."""

    def __init__(self, *sizes):
        super().__init__()
        self.sizes = sizes

    def updateOutput(self, input):
        n = input.size(1)
        self.output = input.contiguous().view(n, *self.sizes)
        return self.output

    def updateGradInput(self, input, gradOutput):
        self.gradInput = gradOutput.contiguous().view(*input.size())
        return self.gradInput


class Linear(Module):
    """mcw_nn/Linear.lua:33-94, batch mode: addr for the bias broadcast, addmm for the products."""

    def __init__(self, inputSize, outputSize, rng=None):
        super().__init__()
        self.weight = np.empty((outputSize, inputSize), np.float32)
        self.bias = np.empty((outputSize,), np.float32)
        self.gradWeight = np.zeros_like(self.weight)
        self.gradBias = np.zeros_like(self.bias)
        self._ones = None
        self.reset(rng=rng)

    def reset(self, stdv=None, rng=None):
        rng = rng or _default_rng
        shape = tuple(self.weight.shape) if isinstance(self.weight, np.ndarray) else self.weight.size()
        stdv = stdv * math.sqrt(3) if stdv else 1.0 / math.sqrt(shape[1])
        w = rng.uniform(shape, -stdv, stdv)
        b = rng.uniform((shape[0],), -stdv, stdv)
        if isinstance(self.weight, np.ndarray):
            self.weight, self.bias = w, b
        else:
            self.weight.copy(w); self.bias.copy(b)

    def _ones_vec(self, n):
        if self._ones is None or self._ones.nElement() != n:
            self._ones = GPUTensor(n).fill(1)
        return self._ones

    def updateOutput(self, input):
        _need_gpu(input, "Linear"); _need_gpu(self.weight, "Linear.weight")
        assert input.dim() == 2, "batch (2-D) input expected"
        nframe, nunit = input.size(1), self.bias.size(1)
        self.output.resize(nframe, nunit)
        self.output.zero().addr(1, self._ones_vec(nframe), self.bias)
        self.output.addmm(1, input, self.weight.t())
        return self.output

    def updateGradInput(self, input, gradOutput):
        if self.gradInput is None:
            return None
        self.gradInput.resizeAs(input)
        self.gradInput.addmm(0, 1, gradOutput, self.weight)
        return self.gradInput

    def accGradParameters(self, input, gradOutput, scale=1.0):
        self.gradWeight.addmm(scale, gradOutput.t(), input)
        self.gradBias.addmv(scale, gradOutput.t(), self._ones_vec(input.size(1)))


class LogSoftMax(Module):
    """mcw_nn/LogSoftMax.lua"""

    def updateOutput(self, input):
        _need_gpu(input, "LogSoftMax")
        lib().THGPUNN_LogSoftMax_updateOutput(input._p, self.output._p)
        return self.output

    def updateGradInput(self, input, gradOutput):
        lib().THGPUNN_LogSoftMax_updateGradInput(input._p, gradOutput._p, self.gradInput._p, self.output._p)
        return self.gradInput


class SoftMax(Module):
    """mcw_nn/SoftMax.lua over gpunn SoftMax_* (gputorch/lib/THC/gpunn-impl/SoftMax.cpp)."""

    def updateOutput(self, input):
        _need_gpu(input, "SoftMax")
        lib().THGPUNN_SoftMax_updateOutput(input._p, self.output._p)
        return self.output

    def updateGradInput(self, input, gradOutput):
        lib().THGPUNN_SoftMax_updateGradInput(input._p, gradOutput._p, self.gradInput._p, self.output._p)
        return self.gradInput


class SpatialAveragePooling(Module):
    """mcw_nn/SpatialAveragePooling.lua:3-20 (dW, dH default to 1; the output is the window sum, as in the reference)."""

    def __init__(self, kW, kH, dW=1, dH=1):
        super().__init__()
        self.kW, self.kH, self.dW, self.dH = kW, kH, dW, dH

    def updateOutput(self, input):
        _need_gpu(input, "SpatialAveragePooling")
        lib().THGPUNN_SpatialAveragePooling_updateOutput(input._p, self.output._p, self.kW, self.kH, self.dW, self.dH)
        return self.output

    def updateGradInput(self, input, gradOutput):
        if self.gradInput is None:
            return None
        lib().THGPUNN_SpatialAveragePooling_updateGradInput(input._p, gradOutput._p, self.gradInput._p, self.kW, self.kH,
                                                            self.dW, self.dH)
        return self.gradInput


class ClassNLLCriterion:
    """mcw_nn/ClassNLLCriterion.lua GPU branch (:13-19, :42-50): targets are a GPU tensor of 1-based ids."""

    def __init__(self):
        self.sizeAverage = True
        self.outputTensor = GPUTensor(1)
        self.gradInput = GPUTensor()
        self.output = 0.0

    def updateOutput(self, input, target, read_back=True):
        lib().THGPUNN_ClassNLLCriterion_updateOutput(input._p, target._p, self.outputTensor._p, int(self.sizeAverage))
        if read_back:
            self.output = float(self.outputTensor.float()[0])
        return self.output

    forward = updateOutput

    def updateGradInput(self, input, target):
        lib().THGPUNN_ClassNLLCriterion_updateGradInput(input._p, target._p, self.gradInput._p, int(self.sizeAverage))
        return self.gradInput

    backward = updateGradInput
