"""Host-side random numbers that follow Torch7's generator, so that "the same seeded inputs" means the same
numbers a Lua script draws with `torch.manualSeed(s); t:uniform(a, b)`.

TH's generator is MT19937 seeded by `init_genrand(seed)` (mcw_torch7_core/lib/TH/THRandom.c:96-118); a uniform
draw is one 32-bit output times 2^-32, scaled (`:170-199`); a normal draw is Box-Muller over two uniforms with the
second value of the pair cached, cosine branch first (`:201-220`); `THFloatTensor_uniform / normal` cast each double
draw to float in logical order (generic/THTensorRandom.c:38-46).  numpy's legacy `RandomState(seed)` is the same
MT19937 with the same seeding, and `RandomState.bytes` hands out its raw 32-bit outputs in order, which makes the
stream available at numpy speed."""
import numpy as np


class THGenerator:
    def __init__(self, seed):
        self.manualSeed(seed)

    def manualSeed(self, seed):
        self._rs = np.random.RandomState(int(seed) & 0xFFFFFFFF)
        self._cached = None          # (rho, x) of a normal pair whose sine branch is still to be handed out
        return self

    def _u01(self, n):
        raw = np.frombuffer(self._rs.bytes(4 * n), dtype="<u4")
        return raw.astype(np.float64) * (1.0 / 4294967296.0)

    def uniform(self, shape, a=0.0, b=1.0):
        n = int(np.prod(shape, dtype=np.int64))
        out = np.empty(n, np.float32)
        step = 1 << 24                                   # bounded temporaries for gigabyte-sized tensors
        for o in range(0, n, step):
            m = min(step, n - o)
            out[o:o + m] = self._u01(m) * (b - a) + a
        return out.reshape(shape)

    def normal(self, shape, mean=0.0, std=1.0):
        n = int(np.prod(shape, dtype=np.int64))
        out = np.empty(n, np.float32)
        o = 0
        if self._cached is not None and n > 0:
            rho, x = self._cached
            out[0] = rho * np.sin(2.0 * np.pi * x) * std + mean
            self._cached = None
            o = 1
        step = 1 << 22                                   # pairs per pass: bounded temporaries
        while o < n:
            pairs = min(step, (n - o + 1) // 2)
            u = self._u01(2 * pairs)
            x, y = u[0::2], u[1::2]
            rho = np.sqrt(-2.0 * np.log(1.0 - y))
            inter = np.empty(2 * pairs, np.float64)
            inter[0::2] = rho * np.cos(2.0 * np.pi * x) * std + mean
            inter[1::2] = rho * np.sin(2.0 * np.pi * x) * std + mean
            take = min(n - o, 2 * pairs)
            out[o:o + take] = inter[:take]
            if take < 2 * pairs:                          # the pair's second value stays cached
                self._cached = (rho[-1], x[-1])
            o += take
        return out.reshape(shape)

    def labels(self, n, classes):
        """n class ids in [1, classes] as floats (the form ClassNLLCriterion takes): floor(u * classes) + 1."""
        return (np.floor(self._u01(n) * classes) + 1.0).astype(np.float32)
