"""The benchmark configurations as `nn` graphs: the AlexNet-style and VGG-A-style classifiers built
from SpatialConvolutionMM / ReLU / SpatialMaxPooling / Linear / LogSoftMax, and their algorithmic
FLOP counts (2*N*K*C*kH*kW*oH*oW per conv pass; padding, the 3xTF32 extra MMAs and index math never
count)."""
from . import nn

# (nIn, nOut, k, stride, pad, pool_after)
ALEXNET_CONVS = [(3, 64, 11, 4, 2, True), (64, 192, 5, 1, 2, True), (192, 384, 3, 1, 1, False),
                 (384, 256, 3, 1, 1, False), (256, 256, 3, 1, 1, True)]
ALEXNET_FC = [(9216, 4096), (4096, 4096), (4096, 1000)]
VGG_A_CONVS = [(3, 64, True), (64, 128, True), (128, 256, False), (256, 256, True), (256, 512, False),
               (512, 512, True), (512, 512, False), (512, 512, True)]
VGG_A_FC = [(25088, 4096), (4096, 4096), (4096, 1000)]


def alexnet(rng=None, first_layer_grad_input=False):
    """Conv 3->64 k11 s4 p2, 64->192 k5 p2, 192->384 k3 p1, 384->256 k3 p1, 256->256 k3 p1 (+ReLU each),
    max-pool 3/2 after conv1, conv2, conv5; Linear 9216->4096->4096->1000 with ReLU between; LogSoftMax.
    Parameters are drawn layer by layer in construction order (weight, then bias)."""
    net = nn.Sequential()
    for i, (ci, co, k, s, p, pool) in enumerate(ALEXNET_CONVS):
        conv = nn.SpatialConvolutionMM(ci, co, k, k, s, s, p, rng=rng)
        if i == 0 and not first_layer_grad_input:
            conv.gradInput = None   # the first layer's gradInput is not needed (Lua: self.gradInput = nil)
        net.add(conv).add(nn.ReLU())
        if pool:
            net.add(nn.SpatialMaxPooling(3, 3, 2, 2))
    net.add(nn.View(9216))
    for i, (fi, fo) in enumerate(ALEXNET_FC):
        net.add(nn.Linear(fi, fo, rng=rng))
        if i < 2:
            net.add(nn.ReLU())
    net.add(nn.LogSoftMax())
    return net


def vgg_a(rng=None):
    net = nn.Sequential()
    for i, (ci, co, pool) in enumerate(VGG_A_CONVS):
        conv = nn.SpatialConvolutionMM(ci, co, 3, 3, 1, 1, 1, rng=rng)
        if i == 0:
            conv.gradInput = None
        net.add(conv).add(nn.ReLU())
        if pool:
            net.add(nn.SpatialMaxPooling(2, 2, 2, 2))
    net.add(nn.View(25088))
    for i, (fi, fo) in enumerate(VGG_A_FC):
        net.add(nn.Linear(fi, fo, rng=rng))
        if i < 2:
            net.add(nn.ReLU())
    net.add(nn.LogSoftMax())
    return net


def _conv_out(h, k, s, p):
    return (h + 2 * p - k) // s + 1


def alexnet_flops_per_image():
    """(forward FLOPs, forward+backward FLOPs) per image; the first conv has no gradInput pass."""
    h = 224
    fwd = 0
    bwd = 0
    for i, (ci, co, k, s, p, pool) in enumerate(ALEXNET_CONVS):
        o = _conv_out(h, k, s, p)
        f = 2 * co * ci * k * k * o * o
        fwd += f
        bwd += f * (1 if i == 0 else 2)
        h = (o - 3) // 2 + 1 if pool else o
    for fi, fo in ALEXNET_FC:
        fwd += 2 * fi * fo
        bwd += 4 * fi * fo
    return fwd, fwd + bwd


def n_parameters(convs_fc):
    convs, fcs = convs_fc
    n = 0
    for c in convs:
        ci, co, k = c[0], c[1], (c[2] if len(c) > 3 else 3)
        n += co * ci * k * k + co
    for fi, fo in fcs:
        n += fi * fo + fo
    return n
