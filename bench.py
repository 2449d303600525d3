#!/usr/bin/env python
"""Benchmark of the B200 mshadow evaluation engine.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload reductions|all] [--no-table]

Prints ONE JSON line.  Headline workload (N GPUs, weak scaling): the reductions config,
one step = `sumall_except_dim<1>` over a (256,512,28,28) fp32 tensor plus `sum_rows` over a
65536x4096 fp32 matrix per GPU, followed (N > 1) by one NCCL all-reduce of the 512 + 4096 result
floats (double-buffered, so that it overlaps the next step's kernels).  Inputs are seeded synthetic data generated once on the host and
copied to the device, so that the CPU reference sees the same bits.

value        Gelem/s over all GPUs, inputs resident in HBM, timed with CUDA events
e2e          the same metric through the C ABI with inputs in page-locked HOST memory:
             every step copies its inputs host->device and its results device->host
roofline     live CUDA-event time of the dominant kernel (the 65536x4096 column sum)
cpu_baseline the reference's CPU evaluator on the host cores, same data (N = 1 only)
kernels      per-kernel table for every config of the path (N = 1 only, outside the timed
             region): algorithmic GB/s and fraction of the measured HBM copy bandwidth

--impl reference times the reference CPU implementation alone (see cpu_reference_arm).
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import numpy as np  # noqa: E402

C2A_SHAPE = (256, 512, 28, 28)
C2B_SHAPE = (65536, 4096)
ELEMS_PER_STEP = int(np.prod(C2A_SHAPE)) + int(np.prod(C2B_SHAPE))
METRIC = "reduction throughput: sumall_except_dim<1> (256,512,28,28) + sum_rows 65536x4096, fp32"
UNIT = "Gelem/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0

# DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum) from
# the ncu capture summarised in profiles/reduce_keep_lowest_sum_rows.md: 268.45 MB read + 4.2 MB
# written on a 16384x4096 case; reads grow with the rows, the partial-row writes do not, so a
# 65536x4096 launch moves 4 * 268.45 MB + 4.2 MB.
NCU_TRAFFIC_KEEP_LOWEST = 4 * 268.45e6 + 4.2e6


# where the JSON line goes; main() re-points it at the real stdout after moving fd 1 to stderr (see claim_stdout)
OUT = sys.stdout


def claim_stdout():
    """Keeps stdout for the one JSON line: returns a file on the original fd 1 and points fd 1 at
    stderr, so that banners which libraries write to stdout (NCCL prints its version there) do
    not end up next to the result."""
    sys.stdout.flush()
    real = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    return real


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# --------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------
class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while work runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap", 0x80: "hw_power_brake"}

    def __init__(self, index, period=0.01):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.stop_flag, self.window = [], False, [None, None]
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.max_mhz = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) \
                    if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") \
                    else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((time.perf_counter(), mhz, reasons))
            except Exception:
                pass
            time.sleep(self.period)

    def summary(self):
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        t0, t1 = self.window
        inside = [s for s in self.samples if t0 is not None and t0 <= s[0] <= t1]
        use = inside if len(inside) >= 3 else self.samples
        mask = 0
        for s in use:
            mask |= s[2]
        reasons = [name for bit, name in self.REASONS.items() if mask & bit]
        return {"sm_mhz": float(np.median([s[1] for s in use])), "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(use), "in_timed_region": len(inside)}


# --------------------------------------------------------------------------------------
# host data
# --------------------------------------------------------------------------------------
def make_host_inputs(lib, rank):
    """Seeded N(0,1) inputs in page-locked host memory, as numpy views."""
    import ctypes as C
    out = []
    for ordinal, shape in enumerate((C2A_SHAPE, C2B_SHAPE)):
        n = int(np.prod(shape))
        ptr = lib.alloc_host(n * 4)
        arr = np.ctypeslib.as_array((C.c_float * n).from_address(ptr)).reshape(shape)
        rng = np.random.default_rng(2000 + 10 * rank + ordinal)
        step = 1 << 24
        flat = arr.reshape(-1)
        for lo in range(0, n, step):
            hi = min(n, lo + step)
            flat[lo:hi] = rng.standard_normal(hi - lo, dtype=np.float32)
        out.append((ptr, arr))
    return out


# --------------------------------------------------------------------------------------
# reference arm: the reference's own CPU evaluator
# --------------------------------------------------------------------------------------
def load_cpu_checker():
    import cpu_checkers as cc
    ref = cc.load("ref")
    if ref is not None:
        return ref, "reference"
    return cc.load("orc"), "port"


def cpu_step(chk, t4, m, out512, out4096):
    chk.reduce_keep_highdim(out512, t4)
    chk.reduce_keep_lowest(out4096, m)


def reference_gpu_table(peak):
    """The reference's OWN CUDA kernels (oracle/_ref/libmshadow_ref_gpu.so: the unmodified
    mshadow headers recompiled for sm_100a) timed on this GPU at the BASELINE configs, with the
    same algorithmic byte counts as the `kernels` table of the other arm.  Returns None where
    there is no GPU or the library was not built.  None of this repository's kernels run here:
    inputs come from torch, the sorted index list from torch.sort."""
    import ctypes as C
    path = os.path.join(ROOT, "oracle", "_ref", "libmshadow_ref_gpu.so")
    try:
        import torch
    except Exception:
        return None
    if not os.path.exists(path) or not torch.cuda.is_available():
        return None
    dll = C.CDLL(path)
    dll.refgpu_last_error.restype = C.c_char_p
    vp, i64 = C.c_void_p, C.c_int64

    def call(name, *args):
        conv = [vp(a.data_ptr()) if hasattr(a, "data_ptr") else a for a in args]
        if getattr(dll, name)(*conv, None) != 0:
            raise RuntimeError(dll.refgpu_last_error().decode("utf-8", "replace"))

    for name, types in {
        "refgpu_expr_case0": [vp] * 5 + [i64] * 2, "refgpu_sum_rows": [vp] * 2 + [i64] * 2,
        "refgpu_sumall_except_dim1": [vp] * 2 + [i64] * 4, "refgpu_softmax": [vp] * 2 + [i64] * 2,
        "refgpu_softmax_grad": [vp] * 3 + [i64] * 2, "refgpu_pool_max": [vp] * 2 + [i64] * 3 + [C.c_int] * 4,
        "refgpu_unpool_max": [vp] * 4 + [i64] * 3 + [C.c_int] * 4, "refgpu_chpool_sum": [vp] * 2 + [i64] * 4 + [C.c_int],
        "refgpu_addtakegrad_largebatch": [vp] * 4 + [i64] * 3,
    }.items():
        getattr(dll, name).argtypes = types + [vp]
        getattr(dll, name).restype = C.c_int
    dev = torch.device("cuda")
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    rows = []

    def run(key, label, nbytes, fn, iters):
        try:
            seconds = time_kernel(torch, fn, iters=iters, warm=2)
            gbs = nbytes / seconds / 1e9
            rows.append({"key": key, "kernel": label, "ms": seconds * 1e3, "GBps": round(gbs, 1),
                         "frac_of_measured_peak": round(gbs / peak, 3)})
        except Exception as e:  # the reference refused the shape (its CHECKs throw)
            rows.append({"key": key, "kernel": label, "error": str(e)[:200]})

    n = 8192
    A, B, Cm = (torch.rand(n, n, device=dev, generator=g) * 2 - 1 for _ in range(3))
    bias, D = torch.randn(n, device=dev, generator=g), torch.empty(n, n, device=dev)
    run("map", "C1 map", 16 * n * n + 4 * n, lambda: call("refgpu_expr_case0", D, A, B, Cm, bias, n, n), 10)
    del A, B, Cm, D
    T = torch.randn(C2A_SHAPE, device=dev, generator=g)
    o = torch.zeros(C2A_SHAPE[1], device=dev)
    run("keep_highdim", "C2a sumall_except_dim<1>", 4 * T.numel(),
        lambda: call("refgpu_sumall_except_dim1", o, T, *C2A_SHAPE), 10)
    del T
    M = torch.randn(C2B_SHAPE, device=dev, generator=g)
    o2 = torch.zeros(C2B_SHAPE[1], device=dev)
    run("keep_lowest", "C2b sum_rows", 4 * M.numel(), lambda: call("refgpu_sum_rows", o2, M, *C2B_SHAPE), 10)
    del M
    r, c = 32768, 32000
    L = torch.randn(r, c, device=dev, generator=g) * 2
    P = torch.empty(r, c, device=dev)
    run("softmax", "C3 Softmax", 8 * r * c, lambda: call("refgpu_softmax", P, L, r, c), 5)
    lab = torch.randint(0, c, (r,), device=dev, generator=g).float()
    run("softmax_grad", "C3 SoftmaxGrad", 8 * r * c, lambda: call("refgpu_softmax_grad", L, P, lab, r, c), 5)
    del L, P
    planes = 256 * 256
    X = torch.rand(planes, 56, 56, device=dev, generator=g)
    Pm = torch.empty(planes, 27, 27, device=dev)
    run("pool", "C4 pool<max> 3x3/2", 4 * X.numel() + 4 * Pm.numel(),
        lambda: call("refgpu_pool_max", Pm, X, planes, 56, 56, 3, 3, 2, 2), 5)
    gP = torch.rand(planes, 27, 27, device=dev, generator=g)
    G = torch.empty_like(X)
    run("unpool", "C4 unpool<max> 3x3/2", 8 * X.numel() + 8 * Pm.numel(),
        lambda: call("refgpu_unpool_max", G, X, Pm, gP, planes, 56, 56, 3, 3, 2, 2), 5)
    run("chpool", "C4 chpool<sum> 5", 8 * X.numel(), lambda: call("refgpu_chpool_sum", G, X, 256, 256, 56, 56, 5), 5)
    del X, Pm, gP, G
    k, d, nidx = 262144, 1024, 1 << 20
    p = (np.arange(k) + 1.0) ** -1.1
    idx = np.random.default_rng(5).choice(k, size=nidx, p=p / p.sum()).astype(np.int32)
    uniq = int(np.unique(idx).size)
    keys, order = torch.sort(torch.from_numpy(idx).to(dev), stable=True)
    keys, order = keys.contiguous(), order.to(torch.int32).contiguous()
    src = torch.randn(nidx, d, device=dev, generator=g)
    table = torch.zeros(k, d, device=dev)
    run("addtakegrad", "C5 AddTakeGradLargeBatch", 4 * nidx * d + 8 * nidx + 8 * uniq * d,
        lambda: call("refgpu_addtakegrad_largebatch", table, keys, order, src, k, d, nidx), 3)
    return rows


def cpu_reference_arm(args):
    """Times sumall_except_dim<1> + sum_rows of the reference CPU path on the host cores.

    Each step processes a bounded sample of the workload (the leading images / rows), sized
    from one probe step so that the whole run stays within a couple of minutes.
    """
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    chk, kind = load_cpu_checker()
    rng = np.random.default_rng(2000)
    t4 = rng.standard_normal(C2A_SHAPE, dtype=np.float32)
    rng = np.random.default_rng(2001)
    m = rng.standard_normal(C2B_SHAPE, dtype=np.float32)
    o1, o2 = np.zeros(C2A_SHAPE[1], np.float32), np.zeros(C2B_SHAPE[1], np.float32)
    t = time.perf_counter()
    cpu_step(chk, t4, m, o1, o2)
    probe = time.perf_counter() - t
    budget = 100.0
    frac = min(1.0, budget / max(1e-9, probe * (args.steps + args.warmup)))
    n_img = max(1, int(C2A_SHAPE[0] * frac))
    n_row = max(32, int(C2B_SHAPE[0] * frac))
    t4s, ms = t4[:n_img], m[:n_row]
    elems = t4s.size + ms.size
    for _ in range(args.warmup):
        cpu_step(chk, t4s, ms, o1, o2)
    t = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(chk, t4s, ms, o1, o2)
    dt = time.perf_counter() - t
    value = elems * args.steps / dt / 1e9
    sample = "first %d of %d images and first %d of %d rows per step" % (n_img, C2A_SHAPE[0], n_row, C2B_SHAPE[0])
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "reductions: sumall_except_dim<1> (256,512,28,28) + sum_rows 65536x4096",
                   "device": "host CPU"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": chk.num_threads(), "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if not args.no_table:
        # second baseline: the reference's own CUDA kernels recompiled for this GPU (not part of `value`)
        peak, _ = measured_peak()
        table = reference_gpu_table(peak)
        if table is not None:
            line["reference_gpu_kernels"] = table
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# per-kernel table (N = 1)
# --------------------------------------------------------------------------------------
def time_kernel(torch, fn, iters=20, warm=5):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(iters + 1)]
    evs[0].record()
    for i in range(iters):
        fn()
        evs[i + 1].record()
    torch.cuda.synchronize()
    times = [evs[i].elapsed_time(evs[i + 1]) for i in range(iters)]
    return float(np.median(times)) * 1e-3


def kernel_cases(lib, torch, small=False):
    """Yields (key, label, algorithmic bytes, elements, callable, iterations) for every kernel
    of the path, at its BASELINE config or, with small=True, at a reduced size that still
    exceeds the L2 cache (for profiler captures).  Tensors of a case die when the next starts."""
    dev = torch.device("cuda")
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    # C1: fused element-wise, 16 B/elem
    rows, n = (2048, 8192) if small else (8192, 8192)
    A, B, Cm = (torch.rand(rows, n, device=dev, generator=g) * 2 - 1 for _ in range(3))
    bias = torch.randn(n, device=dev, generator=g)
    D = torch.empty(rows, n, device=dev)
    yield ("map", "C1 map: sigmoid(A*B+0.5*C)+repmat(bias) %dx%d" % (rows, n), 16 * rows * n + 4 * n, rows * n,
           lambda: lib.expr_case(0, D, A, B, Cm, bias), 20)
    del A, B, Cm, D
    # C2: reductions, 4 B/elem
    shape = (64,) + C2A_SHAPE[1:] if small else C2A_SHAPE
    T = torch.randn(shape, device=dev, generator=g)
    o = torch.zeros(shape[1], device=dev)
    yield ("keep_highdim", "C2a sumall_except_dim<1> %s" % (shape,), 4 * T.numel() + 4 * o.numel(), T.numel(),
           lambda: lib.reduce_keep_highdim(o, T), 20)
    del T
    shape = (16384, 4096) if small else C2B_SHAPE
    M = torch.randn(shape, device=dev, generator=g)
    o2 = torch.zeros(shape[1], device=dev)
    yield ("keep_lowest", "C2b sum_rows %dx%d" % shape, 4 * M.numel() + 4 * o2.numel(), M.numel(),
           lambda: lib.reduce_keep_lowest(o2, M), 20)
    del M
    # C3: softmax + grad, 8 B/elem each
    r, c = (2048, 32000) if small else (32768, 32000)
    L = torch.randn(r, c, device=dev, generator=g) * 2
    P = torch.empty(r, c, device=dev)
    yield ("softmax", "C3 Softmax %dx%d" % (r, c), 8 * r * c, r * c, lambda: lib.softmax(P, L), 10)
    lab = torch.randint(0, c, (r,), device=dev, generator=g).float()
    yield ("softmax_grad", "C3 SoftmaxGrad %dx%d" % (r, c), 8 * r * c + 4 * r, r * c,
           lambda: lib.softmax_grad(L, P, lab), 10)
    # beyond the reference API: both in one pass (reads the logits, writes the gradient)
    Gd = P
    yield ("softmax_grad_fused", "Softmax+SoftmaxGrad fused %dx%d" % (r, c), 8 * r * c + 4 * r, r * c,
           lambda: lib.softmax_grad_fused(Gd, L, lab), 10)
    del L, P, Gd
    # C4: pooling
    imgs = 32 if small else 256
    X = torch.rand(imgs * 256, 56, 56, device=dev, generator=g)
    Pm = torch.empty(imgs * 256, 27, 27, device=dev)
    yield ("pool", "C4 pool<max> 3x3/2 (%d,256,56,56)" % imgs, 4 * X.numel() + 4 * Pm.numel(), X.numel(),
           lambda: lib.pool(Pm, X, 3, 3, 2, 2), 20)
    gP = torch.rand(imgs * 256, 27, 27, device=dev, generator=g)
    G = torch.empty_like(X)
    yield ("unpool", "C4 unpool<max> 3x3/2 (%d,256,56,56)" % imgs, 8 * X.numel() + 8 * Pm.numel(), X.numel(),
           lambda: lib.unpool(G, X, Pm, gP, 3, 3, 2, 2), 20)
    X4, G4 = X.view(imgs, 256, 56, 56), G.view(imgs, 256, 56, 56)
    yield ("chpool", "C4 chpool<sum> nsize 5 (%d,256,56,56)" % imgs, 8 * X.numel(), X.numel(),
           lambda: lib.chpool(G4, X4, 5), 20)
    del X, Pm, gP, G, X4, G4
    # C5: embedding backward
    k, d, nidx = (262144, 1024, 1 << 17) if small else (262144, 1024, 1 << 20)
    p = (np.arange(k) + 1.0) ** -1.1
    idx = np.random.default_rng(5).choice(k, size=nidx, p=p / p.sum()).astype(np.int32)
    uniq = int(np.unique(idx).size)
    keys = torch.from_numpy(idx).to(dev)
    vals = torch.arange(nidx, dtype=torch.int32, device=dev)
    lib.sort_by_key(keys, vals, True)
    src = torch.randn(nidx, d, device=dev, generator=g)
    table = torch.zeros(k, d, device=dev)
    yield ("addtakegrad", "C5 AddTakeGradLargeBatch 262144x1024, %d Zipf(1.1) indices" % nidx,
           4 * nidx * d + 8 * nidx + 8 * uniq * d, nidx * d,
           lambda: lib.addtakegrad_largebatch(table, keys, vals, src), 10)
    # the step before it: unsorted indices in, clip + stable radix sort + segmented sum in one call
    raw = torch.from_numpy(idx).to(dev)
    yield ("addtakegrad_unsorted", "C5 AddTakeGrad (unsorted, clipped) 262144x1024, %d Zipf(1.1) indices" % nidx,
           4 * nidx * d + 12 * nidx + 8 * uniq * d, nidx * d,
           lambda: lib.addtakegrad(table, raw, src), 10)
    k2, v2 = raw.clone(), vals.clone()
    yield ("sort_by_key", "SortByKey %d int32 pairs" % nidx, 16 * nidx, nidx,
           lambda: lib.sort_by_key(k2, v2, True), 10)
    del src, table
    # gradient of the channel pooling.  For red::sum the mask PartialGrad is the constant 1, so only
    # the pooled gradient is read (8 B/elem); for red::maximum src and pooled are compared as well.
    imgs = 32 if small else 256
    X4 = torch.rand(imgs, 256, 56, 56, device=dev, generator=g)
    P4 = torch.empty_like(X4)
    lib.chpool(P4, X4, 5)
    gP4 = torch.rand(imgs, 256, 56, 56, device=dev, generator=g)
    G4 = torch.empty_like(X4)
    yield ("ch_unpool", "ch_unpool<sum> nsize 5 (%d,256,56,56)" % imgs, 8 * X4.numel(), X4.numel(),
           lambda: lib.ch_unpool(G4, X4, P4, gP4, 5), 10)
    lib.chpool(P4, X4, 5, reducer=1)
    yield ("ch_unpool_max", "ch_unpool<max> nsize 5 (%d,256,56,56)" % imgs, 16 * X4.numel(), X4.numel(),
           lambda: lib.ch_unpool(G4, X4, P4, gP4, 5, reducer=1), 10)
    del X4, P4, gP4, G4
    # softmax over the middle axis (per-pixel classification shape: 21 classes, 256x256 positions)
    b3, c3, n3 = (32 if small else 64), 21, 256 * 256
    L3 = torch.randn(b3, c3, n3, device=dev, generator=g) * 2
    P3 = torch.empty_like(L3)
    yield ("softmax3d", "Softmax 3-D (%d,%d,%d)" % (b3, c3, n3), 8 * L3.numel(), L3.numel(),
           lambda: lib.softmax3d(P3, L3), 10)
    lab3 = torch.randint(0, c3, (b3, n3), device=dev, generator=g).float()
    yield ("softmax_grad3d", "SoftmaxGrad 3-D (%d,%d,%d)" % (b3, c3, n3), 8 * L3.numel() + 4 * lab3.numel(),
           L3.numel(), lambda: lib.softmax_grad3d(L3, P3, lab3), 10)
    del L3, P3, lab3
    # IndexFill: 2^18 distinct rows of 1024 floats written into a 262144-row table
    kf, df, nf = 262144, 1024, (1 << 16 if small else 1 << 18)
    fidx = torch.randperm(kf, device=dev, generator=g)[:nf].to(torch.int32)
    fsrc = torch.randn(nf, df, device=dev, generator=g)
    ftab = torch.zeros(kf, df, device=dev)
    yield ("index_fill", "IndexFill %d rows of %d into %dx%d" % (nf, df, kf, df), 8 * nf * df + 8 * nf + 4 * kf,
           nf * df, lambda: lib.index_fill(ftab, fidx, fsrc), 10)
    del fidx, fsrc, ftab
    # index-remapping expressions: a permutation that keeps the last axis (128-bit path), one that
    # moves it (element path), and a mirrored copy
    rs = (32, 256, 56, 56) if small else (256, 256, 56, 56)
    RA = torch.rand(rs, device=dev, generator=g)
    RB = torch.empty_like(RA)
    RD = torch.empty_like(RA)
    for cid, name in ((7, "transpose(A,(0,2,1,3))"), (6, "swapaxis<3,1>(A)"), (12, "mirror(A)")):
        yield ("remap_%d" % cid, "%s %s" % (name, rs), 8 * RA.numel(), RA.numel(),
               lambda cid=cid: lib.remap_case(cid, RD, RA, RB), 10)
    # a plan without 16-byte evaluation (zero padding): groups assembled from element evaluations
    RP = torch.empty(lib.remap_shape(9, rs, 2, 4), device=dev)
    yield ("remap_9", "pad(A, 2, 4) %s" % (rs,), 4 * RA.numel() + 4 * RP.numel(), RP.numel(),
           lambda: lib.remap_case(9, RP, RA, RB, 2, 4), 10)
    del RP
    # folding and repeating an axis: sum over the channels, and a new axis of extent 2 behind the first
    RS = torch.empty(lib.axis_shape(4, rs, 1, 0), device=dev)
    yield ("axis_4", "reduce_with_axis<sum>(A, 1) %s" % (rs,), 4 * RA.numel() + 4 * RS.numel(), RA.numel(),
           lambda: lib.axis_case(4, RS, RA, 1, 0), 10)
    del RS, RD
    RW = torch.empty(lib.axis_shape(7, rs, 1, 2), device=dev)
    yield ("axis_7", "broadcast_with_axis(A3, 0, 2) %s" % (rs,), 4 * RA.numel() + 4 * RW.numel(), RW.numel(),
           lambda: lib.axis_case(7, RW, RA, 1, 2), 10)
    del RW
    RD = None
    del RA, RB, RD
    # complex product of two interleaved (re, im) matrices
    cr, ccn = (4096, 8192) if small else (8192, 8192)
    CA = torch.rand(cr, ccn, device=dev, generator=g)
    CB = torch.rand(cr, ccn, device=dev, generator=g)
    CD = torch.empty_like(CA)
    yield ("complex_0", "complex_mul_cc %dx%d floats" % (cr, ccn), 12 * CA.numel(), CA.numel(),
           lambda: lib.complex_case(0, CD, CA, CB), 10)
    del CA, CB, CD
    # embedding look-up (the forward of AddTakeGrad): rows of a table gathered by an index vector
    tr, tc = (65536, 1024) if small else (262144, 1024)
    TA = torch.randn(tr, tc, device=dev, generator=g)
    TD = torch.empty_like(TA)
    tidx = torch.randint(0, tr, (tr,), device=dev, generator=g).float()
    tic = torch.zeros(tr, device=dev)
    yield ("take", "take(index, table) %d rows of %d from a %dx%d table" % (tr, tc, tr, tc), 8 * tr * tc + 4 * tr,
           tr * tc, lambda: lib.select_case(0, TD, TA, TA, tidx, tic), 10)
    del TA, TD, tidx, tic
    # patch -> column (im2col) of a (64, 64, 56, 56) batch with 3 x 3 patches, stride 1: the matrix is nine
    # times the image (minus the border), so the write dominates
    pn = 8 if small else 64
    PI = torch.rand(pn, 64, 56, 56, device=dev, generator=g)
    PM = torch.empty(9 * 64, 54 * 54 * pn, device=dev)
    yield ("unpack_patch2col", "unpack_patch2col 3x3/1 (%d,64,56,56)" % pn, 4 * PI.numel() + 4 * PM.numel(), PM.numel(),
           lambda: lib.unpack_patch2col(PM, PI, 3, 3, 1, 1), 10)
    PG = torch.empty_like(PI)
    yield ("pack_col2patch", "pack_col2patch 3x3/1 (%d,64,56,56)" % pn, 4 * PI.numel() + 4 * PM.numel(), PM.numel(),
           lambda: lib.pack_col2patch(PG, PM, 3, 3, 1, 1), 10)
    del PI, PM, PG
    torch.cuda.empty_cache()


def kernel_table(lib, torch, peak, only=None, small=False, iters=None, warm=None):
    """Algorithmic GB/s of every kernel of the path (one GPU)."""
    rows = []
    for key, label, nbytes, elems, fn, n_it in kernel_cases(lib, torch, small):
        if only is not None and key != only:
            continue
        seconds = time_kernel(torch, fn, iters=iters or n_it, warm=warm if warm is not None else 3)
        gbs = nbytes / seconds / 1e9
        rows.append({"kernel": label, "key": key, "ms": seconds * 1e3, "GBps": round(gbs, 1),
                     "frac_of_measured_peak": round(gbs / peak, 3), "frac_of_8TBps": round(gbs / NOMINAL_HBM_GBS, 3),
                     "Gelem_per_s": round(elems / seconds / 1e9, 2)})
    return rows


# --------------------------------------------------------------------------------------
# embedding backward with the table sharded by rows (strong scaling; --workload embed_sharded)
# --------------------------------------------------------------------------------------
def embed_sharded_arm(args, torch, lib, dist, rank, world, dev):
    """AddTakeGradLargeBatch on a 262144 x 1024 table whose rows are spread over the ranks, for the
    same 2^20 Zipf(1.1) indices at every N (total work fixed).  The source rows are replicated on
    every rank, the sorted index list is routed on the host before the timed region (its time is
    reported separately).  Two ownership schemes are timed:
      contiguous   rank r owns a contiguous range of rows; every row keeps its accumulation order
      cyclic_hot   row i is owned by rank i % N and the 64 most frequent rows are handled by all
                   ranks: each sums the hot entries of its slice of the batch into a 64 x 1024
                   table, one NCCL all-reduce combines them, owners add their rows
    Time per step = max over ranks (CUDA events); rank 0 prints one JSON line."""
    from mshadow_b200 import sharding
    k, d, nidx, hot_count = 262144, 1024, 1 << 20, 64
    p = (np.arange(k) + 1.0) ** -1.1
    idx = np.random.default_rng(5).choice(k, size=nidx, p=p / p.sum()).astype(np.int32)
    order = np.argsort(idx, kind="stable").astype(np.int32)
    keys = idx[order]
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    src = torch.randn(nidx, d, device=dev, generator=g)
    steps, warm = max(3, min(args.steps, 30)), max(3, min(args.warmup, 5))

    def timed(fn):
        for _ in range(warm):
            fn()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def spread(count):
        c = torch.tensor([float(count)], device=dev, dtype=torch.float64)
        hi = c.clone()
        if dist is not None:
            dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        return int(hi.item())

    def checksum(table):
        s = table.double().sum().reshape(1)
        if dist is not None:
            dist.all_reduce(s)
        return float(s.item())

    out = {}
    # contiguous ranges
    t0 = time.perf_counter()
    lk, lo, rb, re = sharding.route_sorted_indices(keys, order, k, rank, world)
    route_ms = (time.perf_counter() - t0) * 1e3
    shard = torch.zeros(re - rb, d, device=dev)
    dk, do = torch.from_numpy(lk).to(dev), torch.from_numpy(lo).to(dev)
    if lk.size:
        lib.addtakegrad_largebatch(shard, dk, do, src)
    ref_sum = checksum(shard)
    ms = timed(lambda: lib.addtakegrad_largebatch(shard, dk, do, src) if lk.size else None)
    out["contiguous"] = {"ms_per_step": ms, "max_entries_on_a_rank": spread(lk.size), "host_routing_ms": route_ms}
    del shard, dk, do
    # cyclic ownership, hot rows replicated
    t0 = time.perf_counter()
    hot = sharding.hot_rows(keys, hot_count)
    tk, to, hk, ho = sharding.route_cyclic_with_hot_rows(keys, order, nidx, rank, world, hot)
    route_ms = (time.perf_counter() - t0) * 1e3
    rows_mine = (k - rank + world - 1) // world
    shard = torch.zeros(rows_mine, d, device=dev)
    dtk, dto = torch.from_numpy(tk).to(dev), torch.from_numpy(to).to(dev)
    dhk, dho = torch.from_numpy(hk).to(dev), torch.from_numpy(ho).to(dev)
    partial = torch.zeros(max(1, hot.size), d, device=dev)
    mine = np.nonzero(hot % world == rank)[0]
    # my hot rows as a (sorted local row, position in `partial`) list: one more sorted scatter-add
    mine_pos = torch.from_numpy(mine.astype(np.int32)).to(dev)
    mine_rows = torch.from_numpy((hot[mine] // world).astype(np.int32)).to(dev)

    def hot_step(stream=None):
        if tk.size:
            lib.addtakegrad_largebatch(shard, dtk, dto, src, stream=stream)
        partial.zero_()
        if hk.size:
            lib.addtakegrad_largebatch(partial, dhk, dho, src, stream=stream)
        if dist is not None:
            dist.all_reduce(partial)
        if mine.size:
            lib.addtakegrad_largebatch(shard, mine_rows, mine_pos, partial, stream=stream)

    hot_step()
    hot_sum = checksum(shard)
    ms = timed(hot_step)
    out["cyclic_hot"] = {"ms_per_step": ms, "hot_rows": int(hot.size), "max_entries_on_a_rank": spread(tk.size + hk.size),
                         "host_routing_ms": route_ms, "allreduce_bytes": int(hot.size) * d * 4}
    # the same step captured once into a CUDA graph: its dozen dependent launches (two multi-level
    # segmented sums, the clear, the all-reduce, the scatter-add) are then issued by one graph launch
    # instead of one host call each.  The library's scratch buffers are per stream, so the warm-up
    # runs on the capture stream before the capture starts (nothing may allocate inside it).
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            hot_step(side.cuda_stream)
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        hot_step(side.cuda_stream)
    torch.cuda.current_stream().wait_stream(side)
    ms = timed(graph.replay)
    out["cyclic_hot_graph"] = {"ms_per_step": ms, "hot_rows": int(hot.size)}
    if rank == 0:
        best = min(v["ms_per_step"] for v in out.values())
        line = {"metric": "AddTakeGradLargeBatch 262144x1024 table sharded by rows, 2^20 Zipf(1.1) indices, fp32",
                "value": nidx * d / (best * 1e-3) / 1e9, "unit": "Gelem/s", "n_gpus": world, "steps": steps,
                "warmup": warm, "ms_per_step": best, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic", "config": {"workload": "embed_sharded", "source_rows": "replicated",
                                                               "index_routing": "host, outside the timed region"},
                "schemes": out,
                "checksum_rel_diff_between_schemes": abs(hot_sum - ref_sum) / max(1e-30, abs(ref_sum))}
        print(json.dumps(line), file=OUT, flush=True)


# --------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-table", action="store_true", help="skip the per-kernel table")
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--cpu-reps", type=int, default=5)
    ap.add_argument("--only", default=None,
                    help="run one kernel of the table alone (map, keep_highdim, keep_lowest, softmax, softmax_grad, "
                         "pool, unpool, chpool, addtakegrad) for --steps launches after --warmup; for profiling")
    ap.add_argument("--small", action="store_true", help="with --only: reduced size that still exceeds L2")
    ap.add_argument("--workload", default="reductions", choices=["reductions", "embed_sharded"],
                    help="reductions: the headline workload; embed_sharded: AddTakeGradLargeBatch with the table "
                         "sharded by rows over the ranks (strong scaling, see embed_sharded_arm)")
    args = ap.parse_args()
    if args.only is not None:
        import torch
        import mshadow_b200
        lib = mshadow_b200.load()
        lib.init(0)
        peak, _ = measured_peak()
        print(json.dumps({"only": args.only, "small": args.small,
                          "kernels": kernel_table(lib, torch, peak, only=args.only, small=args.small,
                                                  iters=args.steps, warm=args.warmup)}), flush=True)
        return
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        cpu_reference_arm(args)
        return

    import torch
    import mshadow_b200

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the engine has no CPU path")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        global OUT
        OUT = claim_stdout()
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    lib = mshadow_b200.load()
    lib.init(local_rank)
    dev = torch.device("cuda", local_rank)
    peak, peak_kind = measured_peak()
    if args.workload == "embed_sharded":
        embed_sharded_arm(args, torch, lib, dist, rank, world, dev)
        if dist is not None:
            dist.destroy_process_group()
        return

    (p4, h4), (pm, hm) = make_host_inputs(lib, rank)
    T = torch.empty(C2A_SHAPE, device=dev)
    M = torch.empty(C2B_SHAPE, device=dev)
    # both results of a step live in one buffer so that one all-reduce combines them; two
    # buffers alternate so that the all-reduce of step i overlaps the kernels of step i+1
    nres = C2A_SHAPE[1] + C2B_SHAPE[1]
    outs = [torch.zeros(nres, device=dev) for _ in range(2)]
    o512s = [o[:C2A_SHAPE[1]] for o in outs]
    o4096s = [o[C2A_SHAPE[1]:] for o in outs]
    pending = [None, None]
    n4, nm = int(np.prod(C2A_SHAPE)), int(np.prod(C2B_SHAPE))
    lib.copy_2d(T, n4, p4, n4, 1, n4, mshadow_b200.capi.H2D)
    lib.copy_2d(M, nm, pm, nm, 1, nm, mshadow_b200.capi.H2D)
    torch.cuda.synchronize()

    def combine(j):
        if dist is not None:
            pending[j] = dist.all_reduce(outs[j], async_op=True)

    def reuse(j):
        # the buffer's previous all-reduce must be done before kernels overwrite it
        if pending[j] is not None:
            pending[j].wait()
            pending[j] = None

    def step(i=0):
        j = i & 1
        reuse(j)
        lib.reduce_keep_highdim(o512s[j], T)
        lib.reduce_keep_lowest(o4096s[j], M)
        combine(j)

    def barrier():
        reuse(0)
        reuse(1)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()
    for i in range(args.warmup):
        step(i)
    barrier()

    # timed region: events around the whole run and around each kernel of each step
    k = args.steps
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(k)]
    launches0 = lib.launch_count()
    sampler.window[0] = time.perf_counter()
    e_start.record()
    for i in range(k):
        j = i & 1
        reuse(j)
        ev[i][0].record()
        lib.reduce_keep_highdim(o512s[j], T)
        ev[i][1].record()
        lib.reduce_keep_lowest(o4096s[j], M)
        ev[i][2].record()
        combine(j)
    reuse(0)
    reuse(1)
    e_end.record()
    barrier()
    sampler.window[1] = time.perf_counter()
    launches = lib.launch_count() - launches0
    seconds = e_start.elapsed_time(e_end) * 1e-3
    t_high = float(np.mean([ev[i][0].elapsed_time(ev[i][1]) for i in range(k)])) * 1e-3
    t_low = float(np.mean([ev[i][1].elapsed_time(ev[i][2]) for i in range(k)])) * 1e-3
    if dist is not None:
        t = torch.tensor([seconds], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        seconds = float(t.item())
    value = ELEMS_PER_STEP * world * k / seconds / 1e9

    # end to end: host buffers in, host results out, through the C ABI
    res_ptr = lib.alloc_host((C2A_SHAPE[1] + C2B_SHAPE[1]) * 4)
    ke = max(1, min(args.e2e_steps, k))

    def e2e_step():
        lib.copy_2d(T, n4, p4, n4, 1, n4, mshadow_b200.capi.H2D)
        lib.copy_2d(M, nm, pm, nm, 1, nm, mshadow_b200.capi.H2D)
        lib.reduce_keep_highdim(o512s[0], T)
        lib.reduce_keep_lowest(o4096s[0], M)
        if dist is not None:
            dist.all_reduce(outs[0])
        lib.copy_2d(res_ptr, nres, outs[0], nres, 1, nres, mshadow_b200.capi.D2H)
        lib.stream_wait(None)

    e2e_step()
    barrier()
    t0 = time.perf_counter()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for _ in range(ke):
        e2e_step()
    s1.record()
    barrier()
    e2e_seconds = max(s0.elapsed_time(s1) * 1e-3, 0.0)
    wall = time.perf_counter() - t0
    if dist is not None:
        t = torch.tensor([e2e_seconds], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_seconds = float(t.item())
    e2e_value = ELEMS_PER_STEP * world * ke / e2e_seconds / 1e9
    sampler.stop_flag = True
    sampler.join(timeout=1.0)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    bytes_low = 4 * nm + 4 * C2B_SHAPE[1]
    achieved = bytes_low / t_low / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": k, "warmup": args.warmup,
        "ms_per_step": seconds / k * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "reductions: sumall_except_dim<1> (256,512,28,28) + sum_rows 65536x4096 per GPU"
                               + ("; one NCCL all-reduce of the 4608 result floats per step, overlapped with the next step"
                                  if world > 1 else ""),
                   "l2": "inputs (411 MB and 1074 MB) exceed the 126 MB L2; no flush needed",
                   "inputs": "N(0,1), seeded, generated on the host, resident in HBM before timing"},
        "clocks": sampler.summary(),
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 4 * (n4 + nm),
                "d2h_bytes_per_step": 4 * (C2A_SHAPE[1] + C2B_SHAPE[1]), "steps": ke,
                "ms_per_step": e2e_seconds / ke * 1e3, "wall_ms_per_step": wall / ke * 1e3},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "kernel": "ReduceKeepLowestKernel (sum_rows 65536x4096)",
                     "achieved": achieved, "peak": peak, "peak_kind": "of " + peak_kind, "unit": "GB/s",
                     "frac": achieved / peak, "frac_of_8TBps": achieved / NOMINAL_HBM_GBS,
                     "traffic": NCU_TRAFFIC_KEEP_LOWEST, "algorithmic_bytes": bytes_low,
                     "launch_ms": t_low * 1e3,
                     "other": {"kernel": "ReduceKeepHighDimKernel (256,512,28,28)", "launch_ms": t_high * 1e3,
                               "achieved": (4 * n4 + 2048) / t_high / 1e9,
                               "frac": (4 * n4 + 2048) / t_high / 1e9 / peak}},
    }
    if world == 1:
        chk, kind = load_cpu_checker()
        c1, c2 = np.zeros(C2A_SHAPE[1], np.float32), np.zeros(C2B_SHAPE[1], np.float32)
        cpu_step(chk, h4, hm, c1, c2)
        t = time.perf_counter()
        for _ in range(args.cpu_reps):
            cpu_step(chk, h4, hm, c1, c2)
        cpu_s = (time.perf_counter() - t) / args.cpu_reps
        line["cpu_baseline"] = {"value": ELEMS_PER_STEP / cpu_s / 1e9, "unit": UNIT, "cores": chk.num_threads(),
                                "kind": kind, "sample": "%d repetitions of the full step on the same inputs"
                                                        % args.cpu_reps,
                                "ms_per_step": cpu_s * 1e3}
        # parity of this very run: GPU results against the CPU evaluation of the same inputs
        g1, g2 = o512s[0].cpu().numpy(), o4096s[0].cpu().numpy()
        def scaled(a, b):
            s = np.maximum(np.abs(b), np.sqrt(np.mean(b.astype(np.float64) ** 2)))
            return float(np.max(np.abs(a.astype(np.float64) - b) / s))
        line["parity"] = {"sumall_except_dim_max_scaled_err": scaled(g1, c1), "sum_rows_max_scaled_err": scaled(g2, c2)}
        if not args.no_table:
            lib.free_host(p4)
            lib.free_host(pm)
            del T, M
            torch.cuda.empty_cache()
            line["kernels"] = kernel_table(lib, torch, peak)
    print(json.dumps(line), file=OUT, flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
