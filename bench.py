#!/usr/bin/env python
"""Benchmark of the gputorch/gpunn hot path on B200: one SGD step of the AlexNet-style classifier.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference            # the reference's CPU nn path on the host cores

Workload (all N): the data-parallel configuration -- global batch 1024 x 3 x 224 x 224 U[-1,1],
random-init AlexNet-style net, labels uniform in [1,1000], zeroGrad -> forward -> ClassNLL -> backward
-> gradient all-reduce (N > 1) -> SGD(lr 0.01, momentum 0.9); the batch is sharded by rows over the
ranks (strong scaling).  Prints ONE JSON line on rank 0."""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GLOBAL_BATCH = 1024
LR, MOMENTUM = 0.01, 0.9
SEED = 1234


def peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))), "measured"
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class NvmlClockSampler:
    """SM clock, power and throttle reasons of one GPU read through NVML from a thread of this process every
    100 ms.  Lighter than an `nvidia-smi -lms` child process, whose start-up and per-sample work was seen to
    stretch the timed region it ran beside."""

    def __init__(self, device):
        import threading
        import pynvml
        self.nv = pynvml
        pynvml.nvmlInit()
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        idx = device
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if device < len(ids) and ids[device].isdigit():
                idx = int(ids[device])
        self.h = pynvml.nvmlDeviceGetHandleByIndex(idx)
        self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        self.rows = []
        self.stop_flag = False
        self.sample()
        self.t = threading.Thread(target=self.loop, daemon=True)
        self.t.start()

    def sample(self, with_power=True):
        nv = self.nv
        try:
            reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
        except Exception:
            reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
        # the power reading goes through the GPU's management controller and can hold up the driver for
        # milliseconds: it is taken only by the calls made outside the sampling loop
        watts = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0 if with_power else 0.0
        self.rows.append((float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)), watts, int(reasons)))

    def loop(self):
        while not self.stop_flag:
            time.sleep(0.1)
            try:
                self.sample(with_power=False)
            except Exception:
                return

    def wait_first_row(self, timeout=5.0):
        pass

    def rows_so_far(self):
        return len(self.rows)

    def stop(self, first_row=0):
        self.stop_flag = True
        self.t.join(timeout=2)
        try:
            self.sample()
        except Exception:
            pass
        rows = self.rows[first_row:] if len(self.rows) > first_row else self.rows[-1:]
        nv = self.nv
        bits = {"hw_slowdown": nv.nvmlClocksThrottleReasonHwSlowdown,
                "hw_thermal_slowdown": nv.nvmlClocksThrottleReasonHwThermalSlowdown,
                "sw_thermal_slowdown": nv.nvmlClocksThrottleReasonSwThermalSlowdown,
                "sw_power_cap": nv.nvmlClocksThrottleReasonSwPowerCap}
        sm = sorted(r[0] for r in rows)
        out = {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": self.max_mhz,
               "reasons": [n for n, b in bits.items() if any(r[2] & b for r in rows)],
               "power_w_max": max(r[1] for r in rows), "samples": len(rows), "source": "nvml"}
        return out


def make_clock_sampler(device):
    try:
        return NvmlClockSampler(device)
    except Exception:
        return ClockSampler(device)


class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(device), "--query-gpu=" + self.Q,
                                       "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.f,
                                      stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def rows_so_far(self):
        try:
            return sum(1 for r in open(self.f.name) if r.count(",") >= 8)
        except Exception:
            return 0

    def wait_first_row(self, timeout=5.0):
        # nvidia-smi takes a while to start (NVML set-up); the timed region must not begin under it
        t0 = time.time()
        while self.p is not None and self.rows_so_far() == 0 and time.time() - t0 < timeout:
            time.sleep(0.05)

    def stop(self, first_row=0):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.p is None:
            return out
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:
            self.p.kill()
        self.f.flush()
        rows = [r.split(",") for r in open(self.f.name).read().strip().splitlines() if r.count(",") >= 8]
        os.unlink(self.f.name)
        rows = rows[first_row:] if len(rows) > first_row else rows[-1:]
        if not rows:
            return out
        sm = sorted(float(r[1]) for r in rows)
        out["sm_mhz"] = sm[len(sm) // 2]
        out["sm_max_mhz"] = float(rows[0][2])
        out["power_w_max"] = max(float(r[3]) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for i, n in enumerate(names):
            if any("Active" in r[5 + i] and "Not" not in r[5 + i] for r in rows):
                out["reasons"].append(n)
        out["samples"] = len(rows)
        return out


# ------------------------------------------------------------------ CPU legs (oracle / reference)
def cpu_alexnet_step(backend_name, n_images, seed=SEED, details=False):
    """One forward+backward+SGD step of the same net on the host cores over `n_images` images.
    backend 'reference': the reference's own TH/nn code (oracle/_ref); conv1 (stride 4) goes through its
    stride-capable nn.SpatialConvolution, the other convs through nn.SpatialConvolutionMM.
    backend 'port': the plain-C restatement (oracle/oracle.c).  Returns (seconds, loss); with details=True
    also the inputs, labels, initial parameters and their gradients (for the parity test of a whole step)."""
    import oracle
    from mcw_cppamp_torch_b200 import configs
    port, ref = oracle.port, oracle.ref
    use_ref = backend_name == "reference"
    from mcw_cppamp_torch_b200.random import THGenerator
    rs = THGenerator(seed)                       # TH's MT19937 stream, as a Lua script would draw the tensors
    x = rs.uniform((n_images, 3, 224, 224), -1, 1)
    labels = rs.labels(n_images, 1000)
    convs, fcs = [], []
    for ci, co, k, s, p, pool in configs.ALEXNET_CONVS:
        sd = 1.0 / np.sqrt(ci * k * k)
        convs.append((rs.uniform((co, ci * k * k), -sd, sd), rs.uniform((co,), -sd, sd)))
    for fi, fo in configs.ALEXNET_FC:
        sd = 1.0 / np.sqrt(fi)
        fcs.append((rs.uniform((fo, fi), -sd, sd), rs.uniform((fo,), -sd, sd)))
    init = [(w.copy(), b.copy()) for w, b in convs + fcs] if details else None
    be = ref if use_ref else port
    mods = []
    if use_ref:
        for (w, b), (ci, co, k, s, p, pool) in zip(convs, configs.ALEXNET_CONVS):
            mods.append(ref.ConvMM(ref, w, b, k, p) if s == 1 else None)
    t0 = time.perf_counter()
    acts = []
    cur = x
    for li, ((w, b), (ci, co, k, s, p, pool)) in enumerate(zip(convs, configs.ALEXNET_CONVS)):
        inp = cur
        if use_ref:
            c = mods[li].forward(inp) if s == 1 else ref.conv_strided(inp, w.reshape(co, ci, k, k), b, None, None, None, 1.0, s, s, p)[0]
        else:
            c = port.conv_forward(inp, w, b, k, k, s, s, p)
        r = be.threshold_forward(c)
        if pool:
            pl, ind = be.maxpool_forward(r, 3, 3, 2, 2)
            cur = pl
        else:
            ind, cur = None, r
        acts.append((inp, c, r, ind))
    flat = cur.reshape(n_images, -1)
    fc_acts = []
    h = flat
    for i, (w, b) in enumerate(fcs):
        z = be.addmm(1.0, np.tile(b, (n_images, 1)).astype(np.float32), 1.0, h, w.T)
        a = be.threshold_forward(z) if i < 2 else z
        fc_acts.append((h, z))
        h = a
    lsm = be.logsoftmax_forward(h)
    loss = port.classnll_forward(lsm, labels)
    g = port.classnll_backward(labels, lsm.shape)
    g = be.logsoftmax_backward(g, lsm)
    grads = []
    for i in range(2, -1, -1):
        hin, z = fc_acts[i]
        w, b = fcs[i]
        if i < 2:
            g = be.threshold_backward(z, g)
        gw = be.addmm(0.0, np.zeros_like(w), 1.0, np.ascontiguousarray(g.T), hin)
        gb = g.sum(0)
        g_in = be.addmm(0.0, np.zeros_like(hin), 1.0, g, w)
        grads.append((w, gw)); grads.append((b, gb))
        g = g_in
    g = g.reshape(cur.shape)
    for li in range(4, -1, -1):
        inp, c, r, ind = acts[li]
        w, b = convs[li]
        ci, co, k, s, p, pool = configs.ALEXNET_CONVS[li]
        if pool:
            g = ref.maxpool_backward(r, g, ind, 2, 2) if use_ref else port.maxpool_backward(g, ind, r.shape, 2, 2)
        g = be.threshold_backward(c, g)
        need_gi = li > 0
        if use_ref and s == 1:
            gi = mods[li].backward(inp, g, 1.0, need_gi)
            gw, gb = mods[li].grads()
        elif use_ref:
            _, gi, gw4, gb = ref.conv_strided(inp, w.reshape(co, ci, k, k), b, g, np.zeros((co, ci, k, k), np.float32),
                                              np.zeros(co, np.float32), 1.0, s, s, p)
            gw = gw4.reshape(co, -1)
        else:
            gi = port.conv_grad_input(g, w, inp.shape, k, k, s, s, p) if need_gi else None
            gw, gb = np.zeros_like(w), np.zeros_like(b)
            port.conv_acc_grad(inp, g, gw, gb, 1.0, k, k, s, s, p)
        grads.append((w, gw)); grads.append((b, gb))
        g = gi
    grad_copy = [gw.copy() for _, gw in grads] if details else None
    for w, gw in grads:
        w -= np.float32(LR) * gw.reshape(w.shape)
    dt = time.perf_counter() - t0
    for m in mods:
        if m is not None:
            m.close()
    if details:
        # grads were appended classifier first (fc8 w, b, fc7 ..., conv5 ..., conv1): return them layer by layer
        pairs = [(grad_copy[2 * i], grad_copy[2 * i + 1]) for i in range(len(grad_copy) // 2)][::-1]
        return dt, float(loss), {"x": x, "labels": labels, "params": init, "grads": pairs}
    return dt, float(loss)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    oracle.build()
    kind = "reference" if oracle.ref.available() else "port"
    cores = os.cpu_count()
    # torchrun exports OMP_NUM_THREADS=1 to its workers; this arm is the one rank that works and may use every core
    if os.environ.get("OMP_NUM_THREADS", "1") == "1":
        os.environ["OMP_NUM_THREADS"] = str(cores)
    sample = args.cpu_images
    for _ in range(args.warmup if args.warmup < 2 else 1):
        cpu_alexnet_step(kind, sample)
    times = []
    for _ in range(args.steps):
        dt, _ = cpu_alexnet_step(kind, sample)
        times.append(dt)
    total = sum(times)
    v = sample * args.steps / total
    line = {"impl": "reference", "metric": "alexnet_train_images_per_sec", "value": v, "unit": "images/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "alexnet-style SGD step, global batch %d (CPU leg: %d-image sample per step)" % (GLOBAL_BATCH, sample)},
            "cpu_baseline": {"value": v, "unit": "images/s", "cores": cores, "kind": kind,
                             "sample": "%d images per step, fwd+bwd+SGD, no BLAS (TH triple-loop SGEMM), OpenMP over images" % sample},
            "e2e": {"value": v, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


# ------------------------------------------------------------------ bandwidth-bound kernels (tensor-math configuration)
def tensor_math_report(gt, nn, torch, ts, hbm_gbs):
    """Achieved GB/s (algorithmic bytes / CUDA-event time) of the HBM-bound kernels on the tensor-math
    configuration's 8192 x 8192 N(0,1) operands (256 MiB each, larger than L2), the AlexNet-style pooling
    shapes at batch 1024 and the 61.1 M-parameter SGD update; addmm 4096^3 in TFLOP/s."""
    n = 8192
    from mcw_cppamp_torch_b200.random import THGenerator
    rs = THGenerator(7)
    X = gt.gpu(rs.normal((n, n)))
    Y = gt.gpu(rs.normal((n, n)))
    R = gt.GPUTensor(n, n)
    ne = n * n

    def time_op(fn, reps=5):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(ts)
        for _ in range(reps):
            fn()
        e1.record(ts)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e-3
    out = {}

    def bw(name, nbytes, fn):
        t = time_op(fn)
        out[name] = {"GB/s": nbytes / t / 1e9, "frac_of_measured_hbm": nbytes / t / 1e9 / hbm_gbs, "us": t * 1e6}
        if name in ("sumall", "maxall", "sumall_transposed", "normall_2"):
            # the kernel's own share: the scalar's round trip to the host taken off
            tk = max(t - out["scalar_readback"]["us"] * 1e-6, 1e-9)
            out[name]["frac_of_measured_hbm_without_readback"] = nbytes / tk / 1e9 / hbm_gbs
    relu = nn.ReLU()
    L = gt.lib()
    # what every scalar-returning call pays besides its kernel: one D2H copy of the scalar and a stream synchronisation
    t_rt = time_op(lambda: L.THGPUStorage_get(L.THGPUTensor_storage(X.cdata), 0))
    out["scalar_readback"] = {"us": t_rt * 1e6, "note": "host round trip contained in sumall / maxall / normall / dot"}
    bw("add_scalar", 8 * ne, lambda: R.add(X, 0.5))
    bw("cadd", 12 * ne, lambda: R.add(X, 0.5, Y))
    bw("cmul", 12 * ne, lambda: R.cmul(X, Y))
    bw("cadd_transposed_src", 12 * ne, lambda: R.add(X, 0.5, Y.t()))
    bw("cmul_transposed_dst", 12 * ne, lambda: R.t().cmul(X, Y))
    bw("copy_transposed", 8 * ne, lambda: R.copy(X.t()))
    bw("relu_fwd", 8 * ne, lambda: relu.updateOutput(X))
    bw("relu_bwd", 12 * ne, lambda: relu.updateGradInput(X, Y))
    bw("exp", 8 * ne, lambda: R.exp(X))                       # double-precision evaluation, rounded once
    bw("tanh", 8 * ne, lambda: R.tanh(X))
    bw("clamp", 8 * ne, lambda: R.clamp(X, -0.5, 0.5))
    bw("ltTensor", 12 * ne, lambda: R.lt(X, Y))
    bw("addcmul", 24 * ne, lambda: R.addcmul(X, 0.5, X, Y))    # product pass (12 B) + sum pass (12 B)
    bw("normall_2", 12 * ne, lambda: X.norm(2.0))             # squares pass (8 B) + sum (4 B)
    bw("sumall", 4 * ne, lambda: X.sum())
    bw("maxall", 4 * ne, lambda: X.max())
    bw("sumall_transposed", 4 * ne, lambda: X.t().sum())
    S = gt.GPUTensor()
    I = gt.GPUTensor()
    bw("sum_dim1", 4 * ne, lambda: L.THGPUTensor_sum(S.cdata, X.cdata, 0))
    bw("sum_dim2", 4 * ne, lambda: L.THGPUTensor_sum(S.cdata, X.cdata, 1))
    bw("max_dim1", 4 * ne, lambda: L.THGPUTensor_max(S.cdata, I.cdata, X.cdata, 0))
    bw("max_dim2", 4 * ne, lambda: L.THGPUTensor_max(S.cdata, I.cdata, X.cdata, 1))
    Xt = X.t()      # keep the view alive: .cdata is a raw pointer
    bw("sum_dim1_transposed", 4 * ne, lambda: L.THGPUTensor_sum(S.cdata, Xt.cdata, 0))
    # pooling at the AlexNet-style shapes, batch 1024
    for name, shape, k, d in (("pool3s2_64x55", (1024, 64, 55, 55), 3, 2), ("pool3s2_192x27", (1024, 192, 27, 27), 3, 2)):
        x = gt.GPUTensor(*shape).fill(0.5)
        pool = nn.SpatialMaxPooling(k, k, d, d)
        o = pool.updateOutput(x)
        nin, nout = x.nElement(), o.nElement()
        go = gt.GPUTensor(*o.size()).fill(1.0)
        bw(name + "_fwd", 4 * (nin + 3 * nout), lambda: pool.updateOutput(x))
        bw(name + "_bwd", 4 * (3 * nout + nin), lambda: pool.updateGradInput(x, go))
        del x, go, pool
    npar = 61100840
    w, g, v = gt.GPUTensor(npar).fill(0.1), gt.GPUTensor(npar).fill(0.01), gt.GPUTensor(npar).zero()
    bw("sgd_momentum", 20 * npar, lambda: L.THGPUNN_SGD_update(w.cdata, g.cdata, v.cdata, 0.01, 0.9))
    del w, g, v, R, Y
    m = 4096
    A = gt.gpu(rs.normal((m, m)))
    B = gt.gpu(rs.normal((m, m)))
    Cm = gt.GPUTensor(m, m).zero()
    t = time_op(lambda: Cm.addmm(0.0, 1.0, A, B))
    out["addmm_4096"] = {"TFLOP/s": 2.0 * m ** 3 / t / 1e12, "us": t * 1e6}
    t = time_op(lambda: Cm.addmm(0.0, 1.0, A.t(), B))
    out["addmm_4096_transposed_m1"] = {"TFLOP/s": 2.0 * m ** 3 / t / 1e12, "us": t * 1e6}
    return out


# ------------------------------------------------------------------ the CUDA arm
def tf32_yardstick(torch):
    """Dense TF32 rate of a LIBRARY GEMM in this very run (torch.matmul = cuBLAS with TF32 allowed, 8192^3, best of
    10): the denominator the 3xTF32 engine is measured against.  It is outside the product, which never calls it."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        n = 8192
        a = torch.randn(n, n, device="cuda")
        b = torch.randn(n, n, device="cuda")
        c = torch.empty(n, n, device="cuda")
        for _ in range(3):
            torch.matmul(a, b, out=c)
        torch.cuda.synchronize()
        best = None
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, b, out=c)
            e1.record()
            torch.cuda.synchronize()
            t = e0.elapsed_time(e1) * 1e-3
            best = t if best is None or t < best else best
        del a, b, c
        torch.cuda.empty_cache()
        return 2.0 * n ** 3 / best / 1e12
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def conv_block_report(gt, nn, torch, ts, rng):
    """The single-conv-block configuration: batch 16 x 3 x 224 x 224, conv 3->64 k11 s4 p2 -> ReLU -> max-pool 3/2,
    forward + backward with ALL THREE convolution passes (this configuration checks the first layer's gradInput).
    Reports algorithmic TFLOP/s of the three convolution launches and the time of the whole block."""
    N = 16
    conv = nn.SpatialConvolutionMM(3, 64, 11, 11, 4, 4, 2, rng=rng)
    net = nn.Sequential().add(conv).add(nn.ReLU()).add(nn.SpatialMaxPooling(3, 3, 2, 2))
    net.gpu()
    x = gt.gpu(rng.uniform((N, 3, 224, 224), -1, 1))
    out = net.forward(x)
    go = gt.gpu(rng.normal(out.size()))
    gconv = gt.GPUTensor(*conv.output.size()).fill(0.001)
    f = 2.0 * N * 64 * 3 * 11 * 11 * 55 * 55

    def timed(fn, reps=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(ts)
        for _ in range(reps):
            fn()
        e1.record(ts)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e-3

    def block():
        net.zeroGradParameters()
        net.forward(x)
        net.backward(x, go)
    t_f = timed(lambda: conv.updateOutput(x))
    t_d = timed(lambda: conv.updateGradInput(x, gconv))
    t_w = timed(lambda: conv.accGradParameters(x, gconv, 1.0))
    t_block = timed(block)
    return {"workload": "conv 3->64 k11 s4 p2 + ReLU + max-pool 3/2, batch 16, forward + backward (all three conv passes)",
            "conv_fwd_bwd_tflops": 3 * f / (t_f + t_d + t_w) / 1e12, "fwd_tflops": f / t_f / 1e12,
            "grad_input_tflops": f / t_d / 1e12, "grad_weight_tflops": f / t_w / 1e12,
            "block_ms": t_block * 1e3, "block_tflops": 3 * f / t_block / 1e12}


def vgg_report(gt, nn, torch, ts, rng, configs):
    """The VGG-A-style configuration: batch 64 x 3 x 224 x 224, forward + loss + whole backward pass."""
    N = 64
    net = configs.vgg_a(rng=rng)
    net.gpu()
    crit = nn.ClassNLLCriterion()
    x = gt.gpu(rng.uniform((N, 3, 224, 224), -1, 1))
    y = gt.gpu(rng.labels(N, 1000))
    layers = [m for m in net.modules if isinstance(m, (nn.SpatialConvolutionMM, nn.Linear))]

    def step():
        for m in layers:
            m.gradWeight.zero(); m.gradBias.zero()
        out = net.forward(x)
        crit.updateOutput(out, y, read_back=False)
        net.backward(x, crit.updateGradInput(out, y))
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    times = []
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(ts)
        step()
        e1.record(ts)
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    ms = times[len(times) // 2]
    # algorithmic FLOPs per image: convolutions 3x forward except the first layer (no gradInput), classifier 3x
    h, fwd, total = 224, 0.0, 0.0
    for i, (ci, co, pool) in enumerate(configs.VGG_A_CONVS):
        f = 2.0 * co * ci * 9 * h * h
        fwd += f
        total += f * (2 if i == 0 else 3)
        if pool:
            h //= 2
    for fi, fo in configs.VGG_A_FC:
        total += 6.0 * fi * fo
    loss = float(crit.outputTensor.float()[0])
    return {"workload": "VGG-A-style, batch 64, forward + ClassNLL + backward", "ms_per_step": ms, "ms_min": times[0],
            "images_per_sec": N / (ms * 1e-3), "tflops_algorithmic": N * total / (ms * 1e-3) / 1e12, "loss": loss}


class near_gpu:
    """Context manager: the calling thread runs on the CPUs NVML names as closest to CUDA device `index` (host
    memory allocated and first touched inside lands on that NUMA node), and gets its old affinity back on exit.
    Process CPU affinity only; no setting of the GPU is read-modified.  Does nothing when NVML cannot tell."""

    def __init__(self, index):
        self.index, self.old = index, None

    def __enter__(self):
        try:
            import pynvml
            import torch
            pr = torch.cuda.get_device_properties(self.index)
            bus = "%08x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
            words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
            cpus = {64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
            allowed = os.sched_getaffinity(0)
            if cpus & allowed:
                self.old = allowed
                os.sched_setaffinity(0, cpus & allowed)
        except Exception:
            self.old = None
        return self

    def __exit__(self, *exc):
        if self.old is not None:
            os.sched_setaffinity(0, self.old)
        return False


def run_ours(args):
    import ctypes as C
    import torch
    import torch.distributed as dist
    import mcw_cppamp_torch_b200 as gt
    from mcw_cppamp_torch_b200 import configs, dp, nn
    from mcw_cppamp_torch_b200.random import THGenerator
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU path)")
    torch.cuda.set_device(local)
    L = gt.lib()
    L.THGPUSetDevice(local)
    if world > 1:
        # torch.distributed is the rendezvous only (the communicator id, barriers, the MAX over ranks of the
        # timings); the gradient exchange itself is the library's THGPUComm
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ts = torch.cuda.Stream()
    L.THGPUSetStream(ts.cuda_stream)
    gt.set_math_mode(args.mode)

    lo, hi = dp.shard_rows(args.batch, rank, world)
    nloc = hi - lo
    # parameters and data come from Torch7's own generator (TH MT19937), as a Lua script would draw them
    net = configs.alexnet(rng=THGenerator(SEED))
    net.gpu()
    crit = nn.ClassNLLCriterion()
    nparam = sum(t.nElement() for m in net.modules_list() if m.parameters() for t in m.parameters()[0])
    with torch.cuda.stream(ts):
        flat_w = torch.empty(nparam, device="cuda", dtype=torch.float32)
        flat_g = torch.zeros(nparam, device="cuda", dtype=torch.float32)
        vel = torch.zeros(nparam, device="cuda", dtype=torch.float32)
        fw, fg = net.getParameters(flat=(flat_w.data_ptr(), flat_g.data_ptr(), nparam))
        sv = L.THGPUStorage_newWithData(C.c_void_p(vel.data_ptr()), nparam)
        fv = gt.GPUTensor(_ptr=L.THGPUTensor_newWithStorage1d(sv, 0, nparam, 1))
    torch.cuda.synchronize()

    # gradient buckets: one per parametrised layer, in the order backward finishes them
    spans, owner = dp.layer_buckets(net, min_elements=int(args.bucket_mb * 2 ** 20 / 4))
    bucket_of = {}      # module -> bucket to launch once its backward is queued (the last module of each bucket)
    param_mods = [m for m in net.modules_list() if m.parameters()]
    for i, m in enumerate(param_mods[::-1]):
        b, last = owner[i]
        if last:
            bucket_of[id(m)] = b
    comm = None
    if world > 1 or args.comm_alone:
        def exchange(raw):
            if world == 1:
                return raw
            box = [raw]
            dist.broadcast_object_list(box, src=0)
            return box[0]
        comm = dp.Comm.nccl(world, rank, exchange, max_ctas=args.comm_ctas)
        comm.set_buckets(fg, spans)
        # gradients are sums over ranks of per-rank batch means: lr / world gives the global mean
        comm.set_update(fw, fv, LR / world, MOMENTUM)
        if world > 1:
            with torch.cuda.stream(ts):
                dist.broadcast(flat_w, 0)
        torch.cuda.synchronize()

    # synthetic shard in pinned host memory (the e2e leg copies it every step) and resident in HBM: every rank
    # draws the whole global batch from one stream and keeps its rows
    gen = THGenerator(SEED + 1)
    with near_gpu(local):   # pages of the staging buffers on the NUMA node the GPU hangs off
        x_pin = torch.empty((nloc, 3, 224, 224), dtype=torch.float32).pin_memory()
        y_pin = torch.empty((nloc,), dtype=torch.float32).pin_memory()
        x_pin.zero_()
    xa, ya = x_pin.numpy(), y_pin.numpy()
    for r0 in range(0, args.batch, 64):
        blk = gen.uniform((min(64, args.batch - r0), 3, 224, 224), -1, 1)
        a, b = max(r0, lo), min(r0 + 64, hi)
        if a < b:
            xa[a - lo:b - lo] = blk[a - r0:b - r0]
    labels = gen.labels(args.batch, 1000)
    ya[:] = labels[lo:hi]
    x_dev, y_dev = gt.GPUTensor(nloc, 3, 224, 224), gt.GPUTensor(nloc)
    x_dev.copy(xa); y_dev.copy(ya)

    # End-to-end leg: every step's inputs travel from pinned host memory inside the timed region.  Two device
    # buffers and a copy stream let the copy of step i+1 run under the kernels of step i.
    copy_stream = torch.cuda.Stream()
    xbuf = [torch.empty((nloc, 3, 224, 224), device="cuda"), torch.empty((nloc, 3, 224, 224), device="cuda")]
    ybuf = [torch.empty((nloc,), device="cuda"), torch.empty((nloc,), device="cuda")]

    def wrap(t, *shape):
        st = L.THGPUStorage_newWithData(C.c_void_p(t.data_ptr()), t.numel())
        return gt.GPUTensor(_ptr=L.THGPUTensor_newWithStorage1d(st, 0, t.numel(), 1)).view(*shape)
    xg = [wrap(xbuf[0], nloc, 3, 224, 224), wrap(xbuf[1], nloc, 3, 224, 224)]
    yg = [wrap(ybuf[0], nloc), wrap(ybuf[1], nloc)]
    ready = [torch.cuda.Event(), torch.cuda.Event()]
    freed = [torch.cuda.Event(), torch.cuda.Event()]
    e2e_state = {"next_copy": 0, "next_step": 0}
    # the loss of every step lands in a pinned slot through an event-ordered copy; the host reads a slot only
    # when it waits for that step anyway, so the read-back never drains the queue by itself
    loss_pin = torch.zeros(4, dtype=torch.float32).pin_memory()
    loss_dev = torch.zeros(1, device="cuda")
    loss_view = wrap(loss_dev, 1)

    def prefetch():
        i = e2e_state["next_copy"] % 2
        e2e_state["next_copy"] += 1
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(freed[i])               # the step that last read this buffer has finished with it
            xbuf[i].copy_(x_pin, non_blocking=True)
            ybuf[i].copy_(y_pin, non_blocking=True)
            ready[i].record(copy_stream)

    def compute(x_in, y_in):
        fg.zero()
        out = net.forward(x_in)
        crit.updateOutput(out, y_in, read_back=False)
        g = crit.updateGradInput(out, y_in)
        mods = net.modules
        for i in range(len(mods) - 1, -1, -1):
            inp = mods[i - 1].output if i > 0 else x_in
            g = mods[i].backward(inp, g, 1.0)
            if comm is not None and id(mods[i]) in bucket_of:
                comm.launch(bucket_of[id(mods[i])])        # this layer's gradients travel while backward goes on
        if comm is not None:
            comm.wait()                                     # all-reduce + SGD of every bucket, ordered on the stream
        else:
            L.THGPUNN_SGD_update(fw.cdata, fg.cdata, fv.cdata, LR, MOMENTUM)

    step_no = {"n": 0}
    step_done = [torch.cuda.Event(), torch.cuda.Event(), torch.cuda.Event()]

    def step(e2e):
        """Queues one step.  At most two steps are in flight: before step i is queued the host waits for step i - 2
        (what a training loop that logs its loss does); in the end-to-end leg that wait is also where the loss
        of step i - 2 is read from its pinned slot."""
        n = step_no["n"]
        step_no["n"] += 1
        loss = None
        if n >= 2:
            step_done[(n - 2) % 3].synchronize()
            if e2e:
                loss = float(loss_pin[(n - 2) % 4])
        with torch.cuda.stream(ts):
            if not e2e:
                compute(x_dev, y_dev)
            else:
                while e2e_state["next_copy"] < e2e_state["next_step"] + 2:
                    prefetch()                              # this step's inputs and the next one's
                i = e2e_state["next_step"] % 2
                e2e_state["next_step"] += 1
                ts.wait_event(ready[i])
                compute(xg[i], yg[i])
                freed[i].record(ts)
                loss_view.copy(crit.outputTensor)
                loss_pin[n % 4:n % 4 + 1].copy_(loss_dev, non_blocking=True)   # D2H of the loss, asynchronous
            step_done[n % 3].record(ts)
        return loss

    def drain():
        torch.cuda.synchronize()
        step_no["n"] = 0

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(n, e2e):
        """EXACTLY n steps between two barriers; device time between the events around them, MAX over ranks."""
        drain()
        barrier()
        if e2e:
            e2e_state["next_copy"] = e2e_state["next_step"]   # nothing prefetched: step 1's copy is inside the region too
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(ts)
        for _ in range(n):
            step(e2e)
        e1.record(ts)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def median(v):
        v = sorted(v)
        return v[len(v) // 2]

    # the clock sampler starts before the warm-up steps: its start-up would otherwise fall into the timed region
    sampler = make_clock_sampler(local) if rank == 0 else None
    if sampler:
        sampler.wait_first_row()
    warm = max(args.warmup, 3)
    for _ in range(warm):
        step(False)
    drain()
    row0 = sampler.rows_so_far() if sampler else 0
    l0, a0 = L.THGPUKernelLaunchCount(), L.THGPUDeviceAllocCount()
    NREG = args.regions
    regions = [timed(args.steps, False) for _ in range(NREG)]
    launches = (L.THGPUKernelLaunchCount() - l0) // NREG
    allocs = (L.THGPUDeviceAllocCount() - a0) / float(NREG * args.steps)
    ms = median(regions)
    for _ in range(2):
        step(True)
    e2e_regions = [timed(args.steps, True) for _ in range(3)]
    ms_e2e = median(e2e_regions)
    loss = float(loss_pin[(args.steps - 1) % 4])
    clocks = sampler.stop(row0) if sampler else None
    if clocks is not None:
        clocks["regions_ms_per_step"] = [r / args.steps for r in regions]
        clocks["e2e_regions_ms_per_step"] = [r / args.steps for r in e2e_regions]
        clocks["note"] = ("%d device-timed and 3 end-to-end regions of %d steps each were sampled; value / e2e are the "
                          "median regions" % (NREG, args.steps))
    L.THGPUSynchronize()

    value = args.batch * args.steps / (ms * 1e-3)
    e2e_value = args.batch * args.steps / (ms_e2e * 1e-3)
    fwd_flops, step_flops = configs.alexnet_flops_per_image()

    # ---- roofline of the dominant kernel (the tcgen05 implicit-GEMM / GEMM engine): every GEMM-shaped
    # op of one step timed on its own with CUDA events, algorithmic FLOPs / summed duration
    roof = None
    layers = []
    if rank == 0:
        def time_op(fn, reps=3):
            fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(ts)
            for _ in range(reps):
                fn()
            e1.record(ts)
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / reps * 1e-3
        mods = net.modules
        tot_f, tot_t, conv_f, conv_t = 0.0, 0.0, 0.0, 0.0
        with torch.cuda.stream(ts):
            for i, m in enumerate(mods):
                inp = mods[i - 1].output if i > 0 else x_dev
                if isinstance(m, nn.SpatialConvolutionMM):
                    o = m.output.size()
                    f = 2.0 * nloc * m.nOutputPlane * m.nInputPlane * m.kH * m.kW * o[2] * o[3]
                    go = gt.GPUTensor(*o).fill(0.001)
                    t_f = time_op(lambda: m.updateOutput(inp))
                    t_w = time_op(lambda: m.accGradParameters(inp, go, 1.0))
                    t_d = time_op(lambda: m.updateGradInput(inp, go)) if m.gradInput is not None else 0.0
                    nf = 3 if m.gradInput is not None else 2
                    layers.append({"layer": "conv%dx%d %d->%d" % (m.kH, m.kW, m.nInputPlane, m.nOutputPlane),
                                   "fwd_tflops": f / t_f / 1e12, "wgrad_tflops": f / t_w / 1e12,
                                   "dgrad_tflops": (f / t_d / 1e12) if t_d else None})
                    tot_f += nf * f; tot_t += t_f + t_w + t_d
                    conv_f += nf * f; conv_t += t_f + t_w + t_d
                elif isinstance(m, nn.Linear):
                    fo, fi = m.weight.size()
                    f = 2.0 * nloc * fo * fi
                    go = gt.GPUTensor(nloc, fo).fill(0.001)
                    t_f = time_op(lambda: m.updateOutput(inp))
                    t_b = time_op(lambda: m.backward(inp, go, 1.0))
                    layers.append({"layer": "linear %d->%d" % (fi, fo), "fwd_tflops": f / t_f / 1e12, "bwd_tflops": 2 * f / t_b / 1e12})
                    tot_f += 3 * f; tot_t += t_f + t_b
        pk, src = peaks()
        tf32_run = tf32_yardstick(torch)
        ach = tot_f / tot_t / 1e12
        roof = {"bound": "tensor", "achieved": ach, "peak": tf32_run, "unit": "TFLOP/s", "frac": ach / tf32_run,
                # DRAM bytes of the GEMM-shaped launches of one step (ncu dram__bytes_read.sum + dram__bytes_write.sum
                # over the 23 tc2r_kernel launches of a step captured at batch 128): 831 MB in the three classifier
                # layers, whose traffic is their weights and does not grow with the batch, and 7.09 MB per image
                # in the convolution layers, scaled to this rank's batch
                "traffic": 0.831e9 + 7.09e6 * nloc,
                "kernel": "thc::mm::tc2r_kernel (persistent two-SM tcgen05 3xTF32 GEMM / implicit GEMM over raw FP32 operands)",
                "peak_source": "dense TF32 rate of a library GEMM measured in this run (torch.matmul / cuBLAS, TF32 allowed, "
                               "8192^3, best of 10; outside the product); %s bf16_tflops (burst) / 2 would be %.1f" % (
                                   src, pk["bf16_tflops"] / 2.0),
                "peak_bf16_half": pk["bf16_tflops"] / 2.0, "frac_of_bf16_half": ach / (pk["bf16_tflops"] / 2.0),
                "executed_mma_frac": 3 * ach / tf32_run,
                "conv_fwd_bwd_tflops": conv_f / conv_t / 1e12, "gemm_time_share_of_step": tot_t / (ms * 1e-3 / args.steps)}

    # the opt-in BF16 math mode, reported separately: the same step with every GEMM-shaped op on BF16 tensor
    # cores (one plane, no split); everything else (pooling, ReLU, loss, SGD) is unchanged FP32
    bf16 = None
    if rank == 0 and world == 1 and not args.no_extras and args.mode == "fp32x3":
        gt.set_math_mode("bf16")
        for _ in range(3):
            step(False)
        ms_b = median([timed(args.steps, False) for _ in range(3)])
        conv_f = conv_t = 0.0
        with torch.cuda.stream(ts):
            for i, m in enumerate(net.modules):
                if isinstance(m, nn.SpatialConvolutionMM) and m.gradInput is not None:
                    inp = net.modules[i - 1].output
                    o = m.output.size()
                    f = 2.0 * nloc * m.nOutputPlane * m.nInputPlane * m.kH * m.kW * o[2] * o[3]
                    go = gt.GPUTensor(*o).fill(0.001)
                    for fn in (lambda: m.updateOutput(inp), lambda: m.accGradParameters(inp, go, 1.0), lambda: m.updateGradInput(inp, go)):
                        fn(); torch.cuda.synchronize()
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record(ts)
                        for _ in range(3):
                            fn()
                        e1.record(ts); torch.cuda.synchronize()
                        conv_f += f; conv_t += e0.elapsed_time(e1) / 3 * 1e-3
        for _ in range(3):
            step(True)
        drain()
        loss_b = float(loss_pin[2])
        gt.set_math_mode(args.mode)
        pk = peaks()[0]
        bf16 = {"images_per_sec": args.batch * args.steps / (ms_b * 1e-3), "ms_per_step": ms_b / args.steps, "loss": loss_b,
                "conv_fwd_bwd_tflops": conv_f / conv_t / 1e12, "frac_of_measured_bf16_peak": conv_f / conv_t / 1e12 / pk["bf16_tflops"],
                "note": "layers 2-5 (fwd + gradInput + gradWeight), algorithmic FLOPs / CUDA-event time incl. the BF16 plane transforms"}

    tmath = None
    other = None
    if rank == 0 and world == 1 and not args.no_extras:
        with torch.cuda.stream(ts):
            tmath = tensor_math_report(gt, nn, torch, ts, peaks()[0]["hbm_gbs"])
            # the other configurations the metric is quoted on: single conv block (batch 16) and VGG-A-style (batch 64)
            other = {"conv_block_b16": conv_block_report(gt, nn, torch, ts, THGenerator(SEED + 2)),
                     "vgg_a_b64": vgg_report(gt, nn, torch, ts, THGenerator(SEED + 3), configs)}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        import oracle
        oracle.build()
        kind = "reference" if oracle.ref.available() else "port"
        dt, _ = cpu_alexnet_step(kind, args.cpu_images)
        cpu = {"value": args.cpu_images / dt, "unit": "images/s", "cores": os.cpu_count(), "kind": kind,
               "sample": "%d images, one fwd+bwd+SGD step (%.1f s), no BLAS, OpenMP" % (args.cpu_images, dt)}

    if rank == 0:
        line = {"metric": "alexnet_train_images_per_sec", "value": value, "unit": "images/s", "n_gpus": world,
                "steps": args.steps, "warmup": warm, "ms_per_step": ms / args.steps,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic",
                "config": {"workload": "alexnet-style SGD step (5 conv + 3 fc, LogSoftMax + ClassNLL, SGD momentum 0.9), "
                                       "global batch %d sharded by rows" % args.batch,
                           "global_batch": args.batch, "per_gpu_batch": nloc, "math_mode": args.mode,
                           "parallelism": "dp%d" % world,
                           "inputs": "TH MT19937 stream (seed %d parameters, %d data), U[-1,1] images, labels in [1,1000]" % (SEED, SEED + 1),
                           "in_flight": "at most two steps queued ahead of the device",
                           "l2": "per-step inputs + activations (%.0f MB input shard) exceed the 126 MB L2" % (nloc * 150528 * 4 / 1e6)},
                "tflops_algorithmic": value * step_flops / 1e12,
                "regions": {"ms_per_step": [r / args.steps for r in regions], "median": ms / args.steps,
                            "min": min(regions) / args.steps, "max": max(regions) / args.steps},
                "e2e": {"value": e2e_value, "unit": "images/s", "h2d_bytes_per_step": int(nloc * (150528 + 1) * 4),
                        "d2h_bytes_per_step": 4, "ms_per_step": ms_e2e / args.steps,
                        "regions_ms_per_step": [r / args.steps for r in e2e_regions]},
                "gpu_launches": int(launches), "device_allocs_per_step": allocs, "clocks": clocks, "roofline": roof,
                "cpu_baseline": cpu, "layers": layers, "configs": other, "bf16_mode": bf16, "tensor_math": tmath, "loss": loss}
        print(json.dumps(line))
    if comm is not None:
        comm.close()
    if world > 1:
        dist.destroy_process_group()

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=GLOBAL_BATCH, help="global batch (rows are sharded over ranks)")
    ap.add_argument("--mode", default="fp32x3", choices=["fp32x3", "simt", "bf16"])
    ap.add_argument("--cpu-images", type=int, default=8, help="images in the bounded CPU sample")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extras", action="store_true", help="skip the tensor-math / pooling bandwidth report")
    ap.add_argument("--bucket-mb", type=float, default=25.0,
                    help="gradient buckets of at least this many MiB (consecutive layers merged; measured at 8 GPUs: 4.76 ms "
                         "per step with 25, 4.79 with 200, 4.91 with one bucket per layer); 0: one bucket per layer")
    ap.add_argument("--comm-alone", action="store_true",
                    help="one GPU: run the bucketed exchange (a one-rank communicator, per-bucket update on its stream) to measure what it costs without peers")
    ap.add_argument("--comm-ctas", type=int, default=0, help="cap on the SMs a gradient all-reduce may occupy (0: NCCL's default)")
    ap.add_argument("--regions", type=int, default=5, help="device-timed regions of --steps steps each (the median is reported)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
