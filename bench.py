#!/usr/bin/env python
"""Benchmark of the B200 mshadow evaluation engine.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--no-table] [--no-parity] [--no-sharded]

Prints ONE JSON line.  Headline workload (N GPUs, weak scaling): the reductions config, one step =
`sumall_except_dim<1>` over a (256,512,28,28) fp32 tensor plus `sum_rows` over a 65536x4096 fp32
matrix per GPU, followed (N > 1) by the exchange of the 512 + 4096 result floats: every rank
stores them into every other GPU's window over NVLink (mshadow::ps::PeerModel) and adds the N
contributions in rank order; the pull of step i is enqueued behind the kernels of step i + 1.
Inputs are seeded synthetic data generated once on the host and copied to the device, so that the
CPU reference sees the same bits.

value        Gelem/s over all GPUs, inputs resident in HBM, timed with CUDA events
e2e          the same metric through the C ABI with inputs in page-locked HOST memory: every step
             copies its inputs host->device and its results device->host
roofline     live CUDA-event time of the dominant kernel (the 65536x4096 column sum), per rank
cpu_baseline the reference's CPU evaluator on the host cores, same data (N = 1 only)
kernels      per-kernel table for every config of the path and the operators next to it (N = 1,
             outside the timed region)
configs      the nine kernels of the five BASELINE configs: ms, fractions of the measured and the
             nominal HBM bandwidth, the reference CPU evaluator's time at the same full size
sharded      strong scaling: every BASELINE tensor split on its leading dimension over the N ranks
             (embedding table: by rows), time of the slowest rank
parity       GPU results against the reference CPU evaluator at the full BASELINE sizes, with the
             stated tolerances and a pass flag each (N = 1 only; last key of the line)

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
NRES = C2A_SHAPE[1] + C2B_SHAPE[1]
METRIC = "reduction throughput: sumall_except_dim<1> (256,512,28,28) + sum_rows 65536x4096, fp32"
UNIT = "Gelem/s"
WORKLOAD = "reductions: sumall_except_dim<1> (256,512,28,28) + sum_rows 65536x4096 per GPU"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
L2_BYTES = 126e6

# DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum of one
# ncu capture): 268.45 MB read + 4.2 MB written on a 16384x4096 case; reads grow with the rows, the
# partial-row writes do not, so a 65536x4096 launch moves 4 * 268.45 MB + 4.2 MB.
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


def host_cores():
    """Cores this process may run on (a launcher's OMP_NUM_THREADS does not change that)."""
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def cpu_model():
    try:
        for ln in open("/proc/cpuinfo"):
            if ln.startswith("model name"):
                return ln.split(":", 1)[1].strip()
    except Exception:
        pass
    return "unknown"


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
        self.samples, self.stop_flag, self.window, self.tail_window = [], False, [None, None], [None, None]
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
        t2, t3 = self.tail_window
        tail = [s for s in self.samples if t2 is not None and t2 <= s[0] <= t3]
        use = inside if len(inside) >= 3 else (inside + tail if len(inside + tail) >= 3 else self.samples)
        mask = 0
        for s in use:
            mask |= s[2]
        reasons = [name for bit, name in self.REASONS.items() if mask & bit]
        return {"sm_mhz": float(np.median([s[1] for s in use])), "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(use), "in_timed_region": len(inside),
                "in_the_same_steps_continued_untimed": len(tail)}


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
    """The reference CPU build if present, else the C port; with one OpenMP thread per core this
    process may use, whatever OMP_NUM_THREADS a launcher exported (torchrun sets it to 1)."""
    import cpu_checkers as cc
    ref = cc.load("ref")
    chk, kind = (ref, "reference") if ref is not None else (cc.load("orc"), "port")
    chk.set_num_threads(host_cores())
    return chk, kind


def cpu_step(chk, t4, m, out512, out4096):
    chk.reduce_keep_highdim(out512, t4)
    chk.reduce_keep_lowest(out4096, m)


def best_of(fn, reps=3):
    """Smallest wall time of `reps` calls, in seconds."""
    best = float("inf")
    for _ in range(reps):
        t = time.perf_counter()
        fn()
        best = min(best, time.perf_counter() - t)
    return best


def reference_gpu_table(peak, fastmath=False):
    """The reference's OWN CUDA kernels (oracle/_ref/libmshadow_ref_gpu.so: the unmodified
    mshadow headers recompiled for sm_100a) timed on this GPU at the BASELINE configs, with the
    same algorithmic byte counts as the `kernels` table of the other arm.  fastmath=True uses the
    build with --use_fast_math, as the reference's examples ship (guide/neuralnet/Makefile:9): a
    speed row only, its arithmetic is not the one parity is judged on.  Returns None where
    there is no GPU or the library was not built.  None of this repository's kernels run here:
    inputs come from torch, the sorted index list from torch.sort."""
    import ctypes as C
    path = os.path.join(ROOT, "oracle", "_ref",
                        "libmshadow_ref_gpu_fastmath.so" if fastmath else "libmshadow_ref_gpu.so")
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

    Rank 0 alone works (the other ranks of a multi-process launch return at once), with one OpenMP
    thread per core of the box.  Each step processes the full workload unless one probe step shows
    that the run would take longer than 100 seconds; then every step processes the leading images / rows
    only, and `sample` says how many.
    """
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    chk, kind = load_cpu_checker()
    cores = chk.num_threads()
    rng = np.random.default_rng(2000)
    t4 = rng.standard_normal(C2A_SHAPE, dtype=np.float32)
    rng = np.random.default_rng(2001)
    m = rng.standard_normal(C2B_SHAPE, dtype=np.float32)
    o1, o2 = np.zeros(C2A_SHAPE[1], np.float32), np.zeros(C2B_SHAPE[1], np.float32)
    cpu_step(chk, t4, m, o1, o2)  # first touch of the pages and of the thread pool
    t = time.perf_counter()
    cpu_step(chk, t4, m, o1, o2)
    probe = time.perf_counter() - t
    limit_s = 100.0
    frac = min(1.0, limit_s / max(1e-9, probe * (args.steps + args.warmup)))
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
        "config": {"workload": WORKLOAD, "device": "host CPU: %d threads on %s" % (cores, cpu_model())},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample,
                         "cpu_model": cpu_model()},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if not args.no_table:
        # second baseline: the reference's own CUDA kernels recompiled for this GPU (not part of `value`),
        # as parity is judged (IEEE division and expf) and as the reference's examples ship them
        peak, _ = measured_peak()
        table = reference_gpu_table(peak)
        if table is not None:
            line["reference_gpu_kernels"] = table
        fast = reference_gpu_table(peak, fastmath=True)
        if fast is not None:
            line["reference_gpu_kernels_use_fast_math"] = [
                {"key": r["key"], "ms": round(r["ms"], 4), "frac_of_measured_peak": r["frac_of_measured_peak"]}
                if "ms" in r else {"key": r["key"], "error": r["error"][:80]} for r in fast]
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
    time_kernel.spread = (float(np.min(times)), float(np.max(times)))   # ms, of the launches just timed
    # the same launches with nothing between them: an event record between two kernels keeps the second
    # from being placed on the SMs while the first drains (gpu_rt::LaunchAfterDrain), so the per-launch
    # times above carry a launch gap that a stream of kernels does not
    evs[0].record()
    for i in range(iters):
        fn()
    evs[1].record()
    torch.cuda.synchronize()
    time_kernel.back_to_back = evs[0].elapsed_time(evs[1]) / iters
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
    # rows beyond one CTA's registers: held by a cluster of four CTAs (131072 columns), and rows beyond that
    # (2^20 columns: one pass with a running max and sum, second read from the L2)
    for key, (rl, cl) in (("softmax_long", (512, 1 << 17) if small else (2048, 1 << 17)),
                          ("softmax_very_long", (16, 1 << 20) if small else (64, 1 << 20))):
        LL = torch.randn(rl, cl, device=dev, generator=g) * 2
        PLr = torch.empty(rl, cl, device=dev)
        yield (key, "Softmax %dx%d" % (rl, cl), 8 * rl * cl, rl * cl, lambda: lib.softmax(PLr, LL), 10)
        del LL, PLr
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
    # pooling of planes that do not fit shared memory (224 x 224): bands of rows instead of whole planes
    pl = (8 if small else 64) * 64
    XL = torch.rand(pl, 224, 224, device=dev, generator=g)
    PL = torch.empty(pl, 111, 111, device=dev)
    yield ("pool_large", "pool<max> 3x3/2 (%d,224,224) planes" % pl, 4 * XL.numel() + 4 * PL.numel(), XL.numel(),
           lambda: lib.pool(PL, XL, 3, 3, 2, 2), 10)
    gPL = torch.rand(pl, 111, 111, device=dev, generator=g)
    GL = torch.empty_like(XL)
    yield ("unpool_large", "unpool<max> 3x3/2 (%d,224,224) planes" % pl, 8 * XL.numel() + 8 * PL.numel(), XL.numel(),
           lambda: lib.unpool(GL, XL, PL, gPL, 3, 3, 2, 2), 10)
    del XL, PL, gPL, GL
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
    # local response normalisation in one pass each way (beta 0.75 by roots: the bit-exact power functor)
    XN = torch.rand(imgs, 256, 56, 56, device=dev, generator=g)
    ON, NN = torch.empty_like(XN), torch.empty_like(XN)
    yield ("lrn_forward", "LRN forward nsize 5 (%d,256,56,56), norm not kept" % imgs, 8 * XN.numel(), XN.numel(),
           lambda: lib.lrn_forward(ON, None, XN, 5, 0.0001, 0.75, 1.0, 1), 10)
    yield ("lrn_forward_norm", "LRN forward nsize 5 (%d,256,56,56), norm kept" % imgs, 12 * XN.numel(), XN.numel(),
           lambda: lib.lrn_forward(ON, NN, XN, 5, 0.0001, 0.75, 1.0, 1), 10)
    yield ("lrn_forward_fast", "LRN forward nsize 5 (%d,256,56,56), fast power functor" % imgs, 8 * XN.numel(),
           XN.numel(), lambda: lib.lrn_forward(ON, None, XN, 5, 0.0001, 0.75, 1.0, 2), 10)
    GN = torch.rand(imgs, 256, 56, 56, device=dev, generator=g)
    yield ("lrn_backward", "LRN backward nsize 5 (%d,256,56,56)" % imgs, 16 * XN.numel(), XN.numel(),
           lambda: lib.lrn_backward(ON, GN, XN, NN, 5, 0.0001, 0.75, 1), 10)
    yield ("lrn_backward_fast", "LRN backward nsize 5 (%d,256,56,56), fast power functor" % imgs, 16 * XN.numel(),
           XN.numel(), lambda: lib.lrn_backward(ON, GN, XN, NN, 5, 0.0001, 0.75, 2), 10)
    del XN, ON, NN, GN
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


def launch_trace(lib, torch, key, small, launches, per_bin=20):
    """One kernel launched `launches` times back to back, timed launch by launch, with the SM clock and
    the throttle reasons sampled every 0.5 ms: per bin of `per_bin` launches the median time, the median
    clock and the reasons seen.  Shows how a kernel's time moves with the clock over a long burst."""
    sampler = ClockSampler(torch.cuda.current_device(), period=0.0005)
    sampler.start()
    bins = []
    for k, label, nbytes, elems, fn, n_it in kernel_cases(lib, torch, small):
        if k != key:
            continue
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        for b in range(max(1, launches // per_bin)):
            evs = [torch.cuda.Event(enable_timing=True) for _ in range(per_bin + 1)]
            t0 = time.perf_counter()
            evs[0].record()
            for i in range(per_bin):
                fn()
                evs[i + 1].record()
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            ms = [evs[i].elapsed_time(evs[i + 1]) for i in range(per_bin)]
            inside = [x for x in sampler.samples if t0 <= x[0] <= t1]
            mask = 0
            for x in inside:
                mask |= x[2]
            mhz = float(np.median([x[1] for x in inside])) if inside else None
            bins.append({"launches": [b * per_bin, (b + 1) * per_bin - 1], "ms_median": round(float(np.median(ms)), 4),
                         "ms_min": round(float(np.min(ms)), 4), "ms_max": round(float(np.max(ms)), 4), "sm_mhz": mhz,
                         "ms_x_ghz": round(float(np.median(ms)) * mhz / 1e3, 4) if mhz else None,
                         "reasons": [name for bit, name in ClockSampler.REASONS.items() if mask & bit]})
        break
    sampler.stop_flag = True
    sampler.join(timeout=1.0)
    return bins


def kernel_table(lib, torch, peak, only=None, small=False, iters=None, warm=None):
    """Algorithmic GB/s of every kernel of the path (one GPU)."""
    rows = []
    for key, label, nbytes, elems, fn, n_it in kernel_cases(lib, torch, small):
        if only is not None and key != only:
            continue
        seconds = time_kernel(torch, fn, iters=iters or n_it, warm=warm if warm is not None else 3)
        gbs = nbytes / seconds / 1e9
        rows.append({"kernel": label, "key": key, "ms": seconds * 1e3, "ms_min": round(time_kernel.spread[0], 5),
                     "ms_max": round(time_kernel.spread[1], 5), "ms_back_to_back": round(time_kernel.back_to_back, 5),
                     "frac_back_to_back": round(nbytes / (time_kernel.back_to_back * 1e-3) / 1e9 / peak, 3),
                     "GBps": round(gbs, 1),
                     "frac_of_measured_peak": round(gbs / peak, 3), "frac_of_8TBps": round(gbs / NOMINAL_HBM_GBS, 3),
                     "Gelem_per_s": round(elems / seconds / 1e9, 2)})
    return rows




# --------------------------------------------------------------------------------------
# exchange of per-rank results (N > 1)
# --------------------------------------------------------------------------------------
def make_peer_model(dist, rank, world, local_rank, own_stream=False):
    """mshadow::ps::PeerModel of this rank, connected to the others: key 0 carries the headline's
    4608 result floats, key 1 the 512 channel sums of the strong-scaling case, key 2 the partial
    sums of the embedding table's hot rows.  The window handles travel through torch.distributed.
    own_stream: the model's kernels run on a stream of its own, beside the caller's."""
    from mshadow_b200 import ps
    m = ps.PeerModel(rank=rank, world=world, device=local_rank, depth=4, wait_limit_ms=20000, own_stream=own_stream)
    if world > 1:
        handles = [None] * world
        dist.all_gather_object(handles, m.export_handle())
        m.connect(handles)
    m.init_key(0, (NRES,))
    m.init_key(1, (C2A_SHAPE[1],))
    m.init_key(2, (HOT_ROWS, EMBED_D))
    return m


def gather_floats(torch, dist, dev, values):
    """values (list of floats) of every rank -> list of lists, on every rank."""
    t = torch.tensor(values, device=dev, dtype=torch.float64)
    if dist is None:
        return [t.tolist()]
    out = [torch.zeros_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t)
    return [o.tolist() for o in out]


class Lagged:
    """Delivery of step i, then pull of step i - 1: the wait for the peers hides behind a step's
    kernels.  The delivery is either a push kernel (step) or done by the reduction kernels
    themselves through sinks (sinks, then delivered)."""

    def __init__(self, peer, key):
        self.peer, self.key, self.outstanding = peer, key, 0

    def step(self, src, dst):
        self.peer.push(src, self.key)
        self.delivered(dst)

    def sinks(self, *segments):
        """One sink per (offset, count) segment of the step that the first segment opens."""
        return [self.peer.next_sink(self.key, off, cnt) for off, cnt in segments]

    def delivered(self, dst):
        self.outstanding += 1
        if self.outstanding > 1:
            self.peer.pull_req(dst, self.key)
            self.outstanding -= 1

    def drain(self, dst):
        while self.outstanding > 0:
            self.peer.pull_req(dst, self.key)
            self.outstanding -= 1
        self.peer.pull_wait(self.key)


def exchange_variants(torch, lib, dist, peer, peer_side, dev, T, M, outs, sums, steps):
    """The headline step with five ways of combining the ranks' 4608 results, `steps` steps each,
    CUDA events around every kernel: which exchange costs what, and what it does to the column sum
    that runs beside it.  Times are the maximum over the ranks."""
    o512s = [o[:C2A_SHAPE[1]] for o in outs]
    o4096s = [o[C2A_SHAPE[1]:] for o in outs]
    pending = [None, None]
    lag = Lagged(peer, 0)

    def peer_lagged(j):
        lag.step(outs[j], sums[j ^ 1])

    lag_side = Lagged(peer_side, 0)

    def peer_side_stream(j):
        # the fence names the pull issued one step ago (step i - 2): behind it the buffers of step
        # i + 1 are free, and nothing this step's push or pull does can hold up the main stream
        peer_side.pull_fence(0)
        lag_side.step(outs[j], sums[j ^ 1])

    def nccl_blocking(j):
        dist.all_reduce(outs[j])

    def nccl_overlapped(j):
        pending[j] = dist.all_reduce(outs[j], async_op=True)

    def before(j):
        if pending[j] is not None:
            pending[j].wait()
            pending[j] = None

    def finish():
        before(0)
        before(1)
        lag.drain(sums[0])
        lag_side.drain(sums[0])

    def fused_lagged(j):
        lag.delivered(sums[j ^ 1])

    result = {}
    for name, combine in (("push_and_pull_kernels_on_the_models_own_stream", peer_side_stream),
                          ("sinks_in_the_reductions_pull_lagging_one_step", fused_lagged),
                          ("push_kernel_pull_lagging_one_step", peer_lagged),
                          ("nccl_allreduce_blocking", nccl_blocking), ("nccl_allreduce_overlapped", nccl_overlapped)):
        fused = combine is fused_lagged

        def one(i, ev=None):
            j = i & 1
            before(j)
            s_hi, s_lo = lag.sinks((0, C2A_SHAPE[1]), (C2A_SHAPE[1], C2B_SHAPE[1])) if fused else (None, None)
            if ev is not None:
                ev[0].record()
            lib.reduce_keep_highdim(o512s[j], T, sink=s_hi)
            if ev is not None:
                ev[1].record()
            lib.reduce_keep_lowest(o4096s[j], M, sink=s_lo)
            if ev is not None:
                ev[2].record()
            combine(j)
        for i in range(6):
            one(i)
        finish()
        dist.barrier()
        torch.cuda.synchronize()
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            one(i, ev[i])
        finish()
        e1.record()
        torch.cuda.synchronize()
        mine = [e0.elapsed_time(e1) / steps,
                float(np.mean([ev[i][0].elapsed_time(ev[i][1]) for i in range(steps)])),
                float(np.mean([ev[i][1].elapsed_time(ev[i][2]) for i in range(steps)]))]
        allr = np.array(gather_floats(torch, dist, dev, mine))
        result[name] = {"ms_per_step": round(float(allr[:, 0].max()), 5),
                        "sumall_ms_max": round(float(allr[:, 1].max()), 5),
                        "sum_rows_ms_max": round(float(allr[:, 2].max()), 5),
                        "sum_rows_ms_min": round(float(allr[:, 2].min()), 5)}
    result["steps"] = steps
    return result


# --------------------------------------------------------------------------------------
# strong scaling: the BASELINE tensors split over the ranks
# --------------------------------------------------------------------------------------
HOT_ROWS = 64
EMBED_K, EMBED_D, EMBED_N = 262144, 1024, 1 << 20


def zipf_batch():
    """The config-5 index batch: 2^20 draws from Zipf(1.1) over 262144 rows, seeded; with its stable sort."""
    p = (np.arange(EMBED_K) + 1.0) ** -1.1
    idx = np.random.default_rng(5).choice(EMBED_K, size=EMBED_N, p=p / p.sum()).astype(np.int32)
    order = np.argsort(idx, kind="stable").astype(np.int32)
    return idx, idx[order], order


def make_cyclic_hot_step(torch, lib, dist, peer, keys, order, src, rank, world, dev):
    """Embedding backward with table row r owned by rank r % world and the HOT_ROWS most frequent
    rows summed by all ranks (see mshadow_b200/sharding.py).  Returns (step, shard, info).
    The hot rows' partial sums are combined through the peer-store exchange when `peer` is given,
    else by one NCCL all-reduce.  The rank's part of the sorted list is selected on the device
    (msb_frequent_rows_i32, msb_route_cyclic_hot_i32) and checked against the host routing."""
    from mshadow_b200 import sharding
    rows_mine = (EMBED_K - rank + world - 1) // world
    n = int(keys.size)
    dk_all, do_all = torch.from_numpy(keys).to(dev), torch.from_numpy(order).to(dev)
    hot_rows_dev = torch.zeros(HOT_ROWS, dtype=torch.int32, device=dev)
    hot_counts_dev = torch.zeros(HOT_ROWS, dtype=torch.int32, device=dev)
    out_keys = torch.empty(n, dtype=torch.int32, device=dev)
    out_rows = torch.empty(n, dtype=torch.int32, device=dev)
    totals = torch.zeros(2, dtype=torch.int32, device=dev)
    b, e = sharding.shard_range(EMBED_N, rank, world)

    def route_on_device():
        lib.frequent_rows(hot_rows_dev, hot_counts_dev, dk_all)
        found = hot_rows_dev.cpu().numpy()[hot_counts_dev.cpu().numpy() > 0]
        hot_dev = torch.from_numpy(np.sort(found)).to(dev)
        lib.route_cyclic_hot(out_keys, out_rows, totals, dk_all, do_all, hot_dev if found.size else None, world, rank,
                             b, e, rows_mine)
        nt, nh = (int(v) for v in totals.cpu().numpy())
        return np.sort(found), nt, nh

    route_on_device()                      # first call: scratch allocation, kernel loading
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    hot, nt, nh = route_on_device()
    device_route_ms = (time.perf_counter() - t0) * 1e3
    t0 = time.perf_counter()
    hot_host = sharding.hot_rows(keys, HOT_ROWS)
    tk, to, hk, ho = sharding.route_cyclic_with_hot_rows(keys, order, EMBED_N, rank, world, hot_host)
    route_ms = (time.perf_counter() - t0) * 1e3
    # One destination for both parts: the rank's table rows followed by the partial rows of the hot
    # rows.  The tail list (local rows, ascending) followed by the hot list (positions offset by
    # rows_mine) is again sorted, so ONE segmented sum serves both, with half the launches.
    dkeys, dorder = out_keys[:nt + nh], out_rows[:nt + nh]
    same = bool(np.array_equal(hot, hot_host) and nt == tk.size and nh == hk.size and
                np.array_equal(dkeys.cpu().numpy(), np.concatenate([tk, hk + np.int32(rows_mine)])) and
                np.array_equal(dorder.cpu().numpy(), np.concatenate([to, ho])))
    ext = torch.zeros(rows_mine + HOT_ROWS, EMBED_D, device=dev)
    shard, partial = ext[:rows_mine], ext[rows_mine:]
    mine = np.nonzero(hot % world == rank)[0]
    # my hot rows as a (sorted local row, position in `partial`) list: one more sorted scatter-add
    mine_pos = torch.from_numpy(mine.astype(np.int32)).to(dev)
    mine_rows = torch.from_numpy((hot[mine] // world).astype(np.int32)).to(dev)

    def step(stream=None):
        partial.zero_()
        if dkeys.numel():
            lib.addtakegrad_largebatch(ext, dkeys, dorder, src, stream=stream)
        if world > 1:
            if peer is not None:
                peer.push(partial, 2, stream=stream)
                peer.pull_req(partial, 2, stream=stream)
            elif dist is not None:
                dist.all_reduce(partial)
        if mine.size:
            lib.addtakegrad_largebatch(shard, mine_rows, mine_pos, partial, stream=stream)

    info = {"hot_rows": int(hot.size), "entries_on_this_rank": int(nt + nh), "host_routing_ms": route_ms,
            "device_routing_ms": device_route_ms, "device_routing_equals_host_routing": same}
    return step, shard, info


def make_batch_sharded_step(torch, lib, dist, idx_all, src, rank, world, dev):
    """Embedding backward when the SOURCE rows are spread over the ranks by batch position (rank r
    holds rows [b, e) of the batch and their indices) and table row t lives on rank t % world.
    Nothing is prepared outside the step: every call
      1. builds a composite key (owner, local row) per local entry and sorts the entries by it
         (this engine's radix sort), numbers the runs of equal keys (msb_run_index_i32),
      2. sums the local source rows into a compact matrix with one partial row per distinct table
         row (AddTakeGradLargeBatch with the run numbers as keys); the matrix is ordered by owner,
      3. hands every owner its partial rows and their local row numbers (two NCCL all-to-alls with
         uneven splits, after an all-to-all of the counts),
      4. sorts what it received by row (stable: contributions to a row stay in rank order) and adds
         it to its shard of the table (AddTakeGradLargeBatch again).
    Returns (step, shard, info); info["phases"] holds the last call's split into routing (1 and the
    count exchange), local sum (2), exchange (3) and owner's sum (4), from CUDA events."""
    from mshadow_b200 import sharding
    b, e = sharding.shard_range(EMBED_N, rank, world)
    n_loc = e - b
    kp = (EMBED_K + world - 1) // world
    rows_mine = (EMBED_K - rank + world - 1) // world
    idx = torch.from_numpy(np.ascontiguousarray(idx_all[b:e])).to(dev)
    src_loc = src[b:e]
    shard = torch.zeros(rows_mine, EMBED_D, device=dev)
    iota = torch.arange(n_loc, dtype=torch.int32, device=dev)
    pos = torch.empty_like(iota)
    run_of, run_keys = torch.empty_like(iota), torch.empty_like(iota)
    total = torch.zeros(1, dtype=torch.int32, device=dev)
    partial = torch.empty(min(n_loc, EMBED_K), EMBED_D, device=dev)
    edges = torch.arange(world + 1, dtype=torch.int32, device=dev) * kp
    info = {"entries_on_this_rank": n_loc, "phases": {}}
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)]

    def step():
        ev[0].record()
        ck = ((idx % world) * kp + idx // world).to(torch.int32)
        pos.copy_(iota)
        lib.sort_by_key(ck, pos)
        lib.run_index(run_of, run_keys, total, ck)
        u = int(total.item())
        keys_u = run_keys[:u]
        bounds = torch.searchsorted(keys_u, edges, right=False)
        send = (bounds[1:] - bounds[:-1]).to(torch.int64)
        recv = torch.empty_like(send)
        if world > 1:
            dist.all_to_all_single(recv, send)
        else:
            recv.copy_(send)
        send_l, recv_l = send.tolist(), recv.tolist()
        ev[1].record()
        part = partial[:u]
        part.zero_()
        if u:
            lib.addtakegrad_largebatch(part, run_of, pos, src_loc)
        ev[2].record()
        got = int(sum(recv_l))
        local_rows = keys_u % kp                     # the owner's numbering of its rows
        if world > 1:
            rows_in = torch.empty(got, EMBED_D, device=dev)
            keys_in = torch.empty(got, dtype=torch.int32, device=dev)
            dist.all_to_all_single(rows_in, part, recv_l, send_l)
            dist.all_to_all_single(keys_in, local_rows.contiguous(), recv_l, send_l)
        else:
            rows_in, keys_in = part, local_rows.clone()
        ev[3].record()
        if got:
            order_in = torch.arange(got, dtype=torch.int32, device=dev)
            lib.sort_by_key(keys_in, order_in)
            lib.addtakegrad_largebatch(shard, keys_in, order_in, rows_in)
        ev[4].record()
        info["distinct_rows_in_the_local_batch"] = u
        info["partial_rows_received"] = got
        info["bytes_sent_to_other_ranks"] = int((u - send_l[rank]) * (EMBED_D * 4 + 4))

    def phases():
        torch.cuda.synchronize()
        names = ("routing_sort_runs_counts", "local_sum", "exchange_of_partial_rows", "owner_sort_and_sum")
        return {n: round(ev[i].elapsed_time(ev[i + 1]), 4) for i, n in enumerate(names)}

    info["phases_fn"] = phases
    return step, shard, info


def make_batch_sharded_peer_step(torch, lib, dist, idx_all, src, rank, world, local_rank, dev):
    """The placement of make_batch_sharded_step with the exchange done by the segmented-sum kernel
    itself: the sum of every run is stored straight into its row of a receive block in the OWNER's
    memory (16-byte stores over NVLink into a window mapped with CUDA IPC), the owner's row numbers
    beside it, and the counts travel as a small key of the peer-store exchange pushed behind those
    kernels -- whoever has pulled that key finds the rows in place.  No library collective, no
    send-side host synchronisation; the owner reads its counts back once per step to size its sum.
    Receive blocks are double-buffered: a rank starts writing step i + 1 only after it has pulled
    step i's counts, which every owner pushed after it had finished reading step i - 1.
    Returns (step, shard, info, model)."""
    from mshadow_b200 import ps, sharding
    b, e = sharding.shard_range(EMBED_N, rank, world)
    n_loc = e - b
    kp = (EMBED_K + world - 1) // world
    rows_mine = (EMBED_K - rank + world - 1) // world
    key_bits, row_bits = max(1, int(world * kp - 1).bit_length()), max(1, int(kp - 1).bit_length())
    slots = world * kp                                  # rows a rank can receive per step: kp from every sender
    row_bytes, key_bytes = 2 * slots * EMBED_D * 4, 2 * slots * 4
    m = ps.PeerModel(rank=rank, world=world, device=local_rank, depth=4, wait_limit_ms=20000,
                     window_bytes=row_bytes + key_bytes + (1 << 20))
    if world > 1:
        handles = [None] * world
        dist.all_gather_object(handles, m.export_handle())
        m.connect(handles)
    m.init_key(0, (world * world,))
    off_rows, off_keys = m.reserve(row_bytes), m.reserve(key_bytes)
    my_rows, my_keys = m.window(rank, off_rows), m.window(rank, off_keys)

    def blocks(parity):
        """Where this rank writes in every owner's window: sender `rank`'s kp rows of the given parity."""
        at = (parity * world + rank) * kp
        return ([m.window(q, off_rows) + at * EMBED_D * 4 for q in range(world)],
                [m.window(q, off_keys) + at * 4 for q in range(world)])

    targets = [blocks(0), blocks(1)]
    idx = torch.from_numpy(np.ascontiguousarray(idx_all[b:e])).to(dev)
    src_loc = src[b:e]
    shard = torch.zeros(rows_mine, EMBED_D, device=dev)
    iota = torch.arange(n_loc, dtype=torch.int32, device=dev)
    pos, run_of, run_keys = torch.empty_like(iota), torch.empty_like(iota), torch.empty_like(iota)
    total = torch.zeros(1, dtype=torch.int32, device=dev)
    first = torch.zeros(world + 1, dtype=torch.int32, device=dev)
    mine = torch.zeros(world * world, device=dev)
    counts = torch.zeros(world * world, device=dev)
    keys_all = torch.empty(slots, dtype=torch.int32, device=dev)
    lane = torch.arange(kp, dtype=torch.int32, device=dev)
    info = {"entries_on_this_rank": n_loc, "window_bytes": row_bytes + key_bytes + (1 << 20)}
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    state = {"step": 0}
    from mshadow_b200 import capi as _capi

    def step():
        parity = state["step"] & 1
        state["step"] += 1
        row_blocks, key_blocks = targets[parity]
        ev[0].record()
        ck = ((idx % world) * kp + idx // world).to(torch.int32)
        pos.copy_(iota)
        lib.sort_by_key(ck, pos, bits=key_bits)
        lib.run_index(run_of, run_keys, total, ck)
        lib.run_bounds(first, run_keys, total, world, kp)
        ev[1].record()
        # sums of this rank's source rows, stored into the owners' memory; then the owners' row numbers
        lib.take_sum_to_owners(row_blocks, first, run_of, pos, src_loc, world)
        lib.run_keys_to_owners(key_blocks, first, run_keys, world, kp)
        mine.zero_()
        mine[rank * world:(rank + 1) * world] = (first[1:] - first[:-1]).float()
        m.push(mine, 0)                      # behind the storing kernels on this stream: the completion signal
        m.pull_req(counts, 0)
        ev[2].record()
        m.pull_wait(0)
        got = counts.view(world, world)[:, rank].to(torch.int64).tolist()      # rows from every sender
        lib.copy_2d(keys_all, slots, my_keys + parity * slots * 4, slots, 1, slots, _capi.D2D)
        parts_k, parts_o = [], []
        for r, c in enumerate(got):
            if c:
                parts_k.append(keys_all[r * kp:r * kp + c])
                parts_o.append(lane[:c] + (parity * slots + r * kp))
        if parts_k:
            keys_in, order_in = torch.cat(parts_k), torch.cat(parts_o)
            lib.sort_by_key(keys_in, order_in, bits=row_bits)
            lib.call("msb_addtakegrad_largebatch_f32_i32", shard.data_ptr(), keys_in.data_ptr(), order_in.data_ptr(),
                     my_rows, rows_mine, EMBED_D, keys_in.shape[0], None)
        ev[3].record()
        info["partial_rows_received"] = int(sum(got))

    def phases():
        torch.cuda.synchronize()
        names = ("routing_sort_runs_bounds", "local_sum_stored_into_the_owners_and_signal", "owner_wait_sort_and_sum")
        return {n: round(ev[i].elapsed_time(ev[i + 1]), 4) for i, n in enumerate(names)}

    info["phases_fn"] = phases
    info["first"] = first
    return step, shard, info, m


def sharded_block(args, torch, lib, dist, peer, peer_side, rank, world, dev, peak):
    """Every BASELINE tensor split on its leading dimension over the ranks (strong scaling: the total
    work is that of one GPU's config), inputs resident per rank before timing, launches back to
    back, time = the slowest rank.  A shard that would fit the 126 MB L2 is rotated through several
    copies of its inputs, so that every launch reads from HBM like the unsharded case does."""
    from mshadow_b200 import sharding
    g = torch.Generator(device=dev)
    g.manual_seed(100 + rank)
    out = {}

    def timed(fn, iters):
        for i in range(3):
            fn(i)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(iters):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def copies(nbytes):
        return 1 if nbytes >= 4 * L2_BYTES else int(min(8, -(-4 * L2_BYTES // nbytes)))

    def entry(key, ms, total_elems, rank_bytes, ncopies, extra=None):
        e = {"ms": round(ms, 5), "Gelem_per_s": round(total_elems / ms / 1e6, 1),
             "frac_of_measured_peak_per_rank": round(rank_bytes / (ms * 1e-3) / 1e9 / peak, 3),
             "input_copies_rotated": ncopies, "shard_fits_l2": bool(rank_bytes < L2_BYTES)}
        if extra:
            e.update(extra)
        out[key] = e

    iters = 50
    # C1: rows of the 8192 x 8192 matrices
    b, e_ = sharding.shard_range(8192, rank, world)
    r, n = e_ - b, 8192
    nb = 16 * r * n
    R = copies(nb)
    sets = [tuple(torch.rand(r, n, device=dev, generator=g) * 2 - 1 for _ in range(3)) + (torch.empty(r, n, device=dev),)
            for _ in range(R)]
    bias = torch.randn(n, device=dev, generator=g)
    entry("C1_map", timed(lambda i: lib.expr_case(0, sets[i % R][3], sets[i % R][0], sets[i % R][1], sets[i % R][2], bias),
                          iters), 8192 * n, nb, R)
    del sets
    # C3: rows of the 32768 x 32000 logits
    b, e_ = sharding.shard_range(32768, rank, world)
    r, c = e_ - b, 32000
    L = torch.randn(r, c, device=dev, generator=g) * 2
    P = torch.empty(r, c, device=dev)
    lab = torch.randint(0, c, (r,), device=dev, generator=g).float()
    entry("C3_softmax", timed(lambda i: lib.softmax(P, L), 20), 32768 * c, 8 * r * c, 1)
    entry("C3_softmax_grad", timed(lambda i: lib.softmax_grad(L, P, lab), 20), 32768 * c, 8 * r * c, 1)
    del L, P
    # C4: images of the (256,256,56,56) batch
    b, e_ = sharding.shard_range(256, rank, world)
    imgs = e_ - b
    nin, nout = imgs * 256 * 56 * 56, imgs * 256 * 27 * 27
    R = copies(4 * nin)
    Xs = [torch.rand(imgs * 256, 56, 56, device=dev, generator=g) for _ in range(R)]
    Pm = torch.empty(imgs * 256, 27, 27, device=dev)
    gP = torch.rand(imgs * 256, 27, 27, device=dev, generator=g)
    G = torch.empty(imgs * 256, 56, 56, device=dev)
    total_in = 256 * 256 * 56 * 56
    entry("C4_pool", timed(lambda i: lib.pool(Pm, Xs[i % R], 3, 3, 2, 2), iters), total_in, 4 * nin + 4 * nout, R)
    lib.pool(Pm, Xs[0], 3, 3, 2, 2)
    entry("C4_unpool", timed(lambda i: lib.unpool(G, Xs[0], Pm, gP, 3, 3, 2, 2), iters), total_in, 8 * nin + 8 * nout, 1)
    G4 = G.view(imgs, 256, 56, 56)
    entry("C4_chpool", timed(lambda i: lib.chpool(G4, Xs[i % R].view(imgs, 256, 56, 56), 5), iters), total_in, 8 * nin, R)
    del Xs, Pm, gP, G, G4
    # C2a: the (256,512,28,28) tensor itself split on dim 0, the 512 partial sums exchanged every step
    b, e_ = sharding.shard_range(256, rank, world)
    imgs = e_ - b
    nb = 4 * imgs * 512 * 28 * 28
    R = copies(nb)
    Ts = [torch.randn(imgs, 512, 28, 28, device=dev, generator=g) for _ in range(R)]
    part = [torch.zeros(512, device=dev) for _ in range(2)]
    total = [torch.zeros(512, device=dev) for _ in range(2)]
    lag = Lagged(peer_side, 1) if world > 1 else None

    def c2a(i):
        # the reduction on the main stream; push of its 512 results and pull of the previous step's
        # sum on the exchange model's own stream (the fence before them names the pull of step i - 2)
        j = i & 1
        lib.reduce_keep_highdim(part[j], Ts[i % R])
        if lag is not None:
            peer_side.pull_fence(1)
            lag.step(part[j], total[j ^ 1])

    ms = timed(c2a, 200)
    if lag is not None:
        lag.drain(total[0])
    entry("C2a_sumall_except_dim", ms, 256 * 512 * 28 * 28, nb, R,
          {"exchange": "512 floats per step: push and pull kernels on the exchange model's own stream, pull lagging "
                       "one step" if world > 1 else "none"})
    if world > 1:
        # the same with the reduction kernel delivering its results itself (sink) and the pull in-stream
        lag2 = Lagged(peer, 1)

        def c2a_sink(i):
            j = i & 1
            lib.reduce_keep_highdim(part[j], Ts[i % R], sink=lag2.sinks((0, 512))[0])
            lag2.delivered(total[j ^ 1])

        ms2 = timed(c2a_sink, 200)
        lag2.drain(total[0])
        out["C2a_sumall_except_dim"]["ms_with_sink_in_the_kernel_and_pull_in_stream"] = round(ms2, 5)
    if world > 1:
        # correctness of the exchange: the pulled sum equals the rank-order sum of the ranks' partials
        lib.reduce_keep_highdim(part[0], Ts[0])
        peer.push(part[0], 1)
        peer.pull_req(total[0], 1)
        peer.pull_wait(1)
        parts = [torch.zeros(512, device=dev) for _ in range(world)]
        dist.all_gather(parts, part[0])
        want = sharding.rank_order_sum([p.cpu().numpy() for p in parts])
        out["C2a_sumall_except_dim"]["exchange_bit_exact_vs_rank_order_sum"] = bool(
            np.array_equal(want.view(np.uint32), total[0].cpu().numpy().view(np.uint32)))
    del Ts
    # C5: table rows owned cyclically, hot rows by everyone
    idx, keys, order = zipf_batch()
    uniq = int(np.unique(idx).size)
    src = torch.randn(EMBED_N, EMBED_D, device=dev, generator=torch.Generator(device=dev).manual_seed(1))
    step, shard, info = make_cyclic_hot_step(torch, lib, dist, peer if world > 1 else None, keys, order, src, rank,
                                             world, dev)
    ms = timed(lambda i: step(), 20)
    if world > 1:
        peer.pull_wait(2)
    most = torch.tensor([float(info["entries_on_this_rank"])], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(most, op=dist.ReduceOp.MAX)
    total_bytes = 4 * EMBED_N * EMBED_D + 8 * EMBED_N + 8 * uniq * EMBED_D
    # correctness: one step from a zero table against the unsharded call on this rank's own GPU
    # (rows r, r + N, ...); the two differ only in the order the hot rows' entries are added
    shard.zero_()
    step()
    if world > 1:
        peer.pull_wait(2)
    whole = torch.zeros(EMBED_K, EMBED_D, device=dev)
    lib.addtakegrad_largebatch(whole, torch.from_numpy(keys).to(dev), torch.from_numpy(order).to(dev), src)
    want = whole[rank::world]
    scale = torch.maximum(want.abs(), want.pow(2).mean(dim=1, keepdim=True).sqrt()).clamp_min(1e-30)
    worst = torch.tensor([float(((shard - want).abs() / scale).max().item())], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    del whole, want, scale
    entry("C5_addtakegrad_cyclic_hot", ms, EMBED_N * EMBED_D, total_bytes / world, 1,
          {"hot_rows": info["hot_rows"], "max_entries_on_a_rank": int(most.item()),
           "max_rel_diff_vs_unsharded_call": float(worst.item()), "within_1e-5": bool(worst.item() <= 1e-5),
           "routing_ms_outside_timing": {"on_the_device_with_its_two_readbacks": round(info["device_routing_ms"], 3),
                                         "numpy_on_the_host": round(info["host_routing_ms"], 2),
                                         "same_lists": info["device_routing_equals_host_routing"]},
           "source_rows": "replicated"})
    del shard
    # C5 with contiguous row ranges per rank (the plain scheme: rank 0 owns the head of the Zipf distribution)
    lk, lo, rb, re_ = sharding.route_sorted_indices(keys, order, EMBED_K, rank, world)
    shard_c = torch.zeros(re_ - rb, EMBED_D, device=dev)
    dk, do = torch.from_numpy(lk).to(dev), torch.from_numpy(lo).to(dev)
    ms_c = timed(lambda i: lib.addtakegrad_largebatch(shard_c, dk, do, src) if lk.size else None, 20)
    most_c = torch.tensor([float(lk.size)], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(most_c, op=dist.ReduceOp.MAX)
    entry("C5_addtakegrad_contiguous_rows", ms_c, EMBED_N * EMBED_D, total_bytes / world, 1,
          {"max_entries_on_a_rank": int(most_c.item()), "source_rows": "replicated",
           "routing": "numpy on the host, outside the timed region"})
    del shard_c, dk, do
    # C5 again with the placement a data-parallel job has: source rows and indices sharded by batch position
    step_b, shard_b, info_b = make_batch_sharded_step(torch, lib, dist, idx, src, rank, world, dev)
    ms_b = timed(lambda i: step_b(), 10)
    shard_b.zero_()
    step_b()
    ph = info_b["phases_fn"]()
    whole = torch.zeros(EMBED_K, EMBED_D, device=dev)
    lib.addtakegrad_largebatch(whole, torch.from_numpy(keys).to(dev), torch.from_numpy(order).to(dev), src)
    want = whole[rank::world]
    scale = torch.maximum(want.abs(), want.pow(2).mean(dim=1, keepdim=True).sqrt()).clamp_min(1e-30)
    worst = torch.tensor([float(((shard_b - want).abs() / scale).max().item())], device=dev, dtype=torch.float64)
    sent = torch.tensor([float(info_b["bytes_sent_to_other_ranks"])], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        dist.all_reduce(sent, op=dist.ReduceOp.MAX)
    del whole, want, scale
    entry("C5_addtakegrad_source_sharded_by_batch", ms_b, EMBED_N * EMBED_D, total_bytes / world, 1,
          {"placement": "source rows and indices sharded by batch position, table rows cyclic; sort, routing and "
                        "exchange inside the timed step",
           "exchange": "NCCL all-to-all of partial rows (uneven splits)" if world > 1 else "none",
           "phases_ms_on_rank_0": ph, "distinct_rows_in_rank_0s_batch": info_b["distinct_rows_in_the_local_batch"],
           "max_bytes_sent_by_a_rank": int(sent.item()),
           "max_rel_diff_vs_unsharded_call": float(worst.item()), "within_1e-5": bool(worst.item() <= 1e-5)})
    del shard_b
    # the same placement with the segmented-sum kernel storing its sums straight into the owners' memory
    local_rank = dev.index if dev.index is not None else 0
    step_p, shard_p, info_p, model_p = make_batch_sharded_peer_step(torch, lib, dist, idx, src, rank, world, local_rank, dev)
    ms_p = timed(lambda i: step_p(), 10)
    shard_p.zero_()
    step_p()
    ph = info_p["phases_fn"]()
    f = info_p["first"].cpu().numpy()
    stored = torch.tensor([float((f[world] - (f[rank + 1] - f[rank])) * (EMBED_D * 4 + 4))], device=dev, dtype=torch.float64)
    whole = torch.zeros(EMBED_K, EMBED_D, device=dev)
    lib.addtakegrad_largebatch(whole, torch.from_numpy(keys).to(dev), torch.from_numpy(order).to(dev), src)
    want = whole[rank::world]
    scale = torch.maximum(want.abs(), want.pow(2).mean(dim=1, keepdim=True).sqrt()).clamp_min(1e-30)
    worst = torch.tensor([float(((shard_p - want).abs() / scale).max().item())], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        dist.all_reduce(stored, op=dist.ReduceOp.MAX)
        dist.barrier()
    model_p.close()
    del whole, want, scale
    entry("C5_addtakegrad_source_sharded_by_batch_peer_stores", ms_p, EMBED_N * EMBED_D, total_bytes / world, 1,
          {"placement": "as C5_addtakegrad_source_sharded_by_batch",
           "exchange": "the segmented-sum kernel stores every run's sum into its owner's window over NVLink; counts "
                       "through the peer-store exchange; no library collective" if world > 1 else "none (own window)",
           "phases_ms_on_rank_0": ph, "max_bytes_stored_into_other_ranks": int(stored.item()),
           "window_bytes_per_rank": info_p["window_bytes"],
           "max_rel_diff_vs_unsharded_call": float(worst.item()), "within_1e-5": bool(worst.item() <= 1e-5)})
    del src, shard_p
    torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------------------
# parity at the full BASELINE sizes (N = 1), and the reference CPU evaluator's time per config
# --------------------------------------------------------------------------------------
def full_size_parity(torch, lib, chk, dev, h4, hm, T, M, g1, g2):
    """Runs each BASELINE config at its stated size on the GPU (through the C ABI) and on the CPU
    checker, on the same seeded inputs, and compares under the stated tolerance: bit-exact for
    pooling and all index work and for SoftmaxGrad, <= 1 ulp for the element-wise expression,
    relative 1e-5 for sums, softmax and the embedding backward.  Comparisons run on the GPU (the
    CPU result is uploaded).  Returns (parity, cpu_ms): cpu_ms holds the best of three wall times
    of the CPU evaluator per kernel."""
    g = torch.Generator(device=dev)
    g.manual_seed(7)
    parity, cpu_ms = {}, {}

    def host(t):
        return t.cpu().numpy()

    def up(a):
        return torch.from_numpy(a).to(dev)

    def ordered(t):  # float bits as integers that sort like the floats
        i = t.view(torch.int32).to(torch.int64)
        return torch.where(i >= 0, i, -(i & 0x7fffffff))

    def bit_mismatches(a, b):
        return int((a.view(torch.int32) != b.view(torch.int32)).sum().item())

    def scaled(a, b):  # max |a - b| / max(|b|, rms(b)), in binary64
        a, b = a.double(), b.double()
        s = torch.maximum(b.abs(), b.pow(2).mean().sqrt())
        return float(((a - b).abs() / s).max().item())

    # ---- C1: <= 1 ulp on all 8192^2 results -------------------------------------------------
    n = 8192
    A, B, Cm = (torch.rand(n, n, device=dev, generator=g) * 2 - 1 for _ in range(3))
    bias = torch.randn(n, device=dev, generator=g)
    D = lib.expr_case(0, torch.empty(n, n, device=dev), A, B, Cm, bias)
    hA, hB, hC, hb = host(A), host(B), host(Cm), host(bias)
    want = np.empty((n, n), np.float32)
    cpu_ms["map"] = best_of(lambda: chk.expr_case(0, want, hA, hB, hC, hb)) * 1e3
    W = up(want)
    ulp = (ordered(D) - ordered(W)).abs()
    # cancellation: the bias removed at least three leading bits of the sigmoid
    cancel = W.abs() * 8 < bias.abs()[None, :]
    mx = int(ulp.max().item())
    parity["C1_map"] = {"tolerance": "<= 1 ulp", "elements": n * n, "max_ulp": mx,
                        "ulp_histogram": {"0": int((ulp == 0).sum().item()), "1": int((ulp == 1).sum().item()),
                                          ">1": int((ulp > 1).sum().item())},
                        "cancellation_cases": int(cancel.sum().item()),
                        "max_ulp_in_cancellation_cases": int(ulp[cancel].max().item()) if bool(cancel.any()) else 0,
                        "pass": mx <= 1}
    del A, B, Cm, D, W, ulp, cancel, hA, hB, hC, want

    # ---- C2: sums against the CPU and both against binary64 ---------------------------------
    c1, c2 = np.zeros(C2A_SHAPE[1], np.float32), np.zeros(C2B_SHAPE[1], np.float32)
    cpu_ms["keep_highdim"] = best_of(lambda: chk.reduce_keep_highdim(c1, h4)) * 1e3
    cpu_ms["keep_lowest"] = best_of(lambda: chk.reduce_keep_lowest(c2, hm)) * 1e3
    for name, gpu_res, cpu_res, truth in (("C2a_sumall_except_dim", g1, c1, T.double().sum(dim=(0, 2, 3))),
                                          ("C2b_sum_rows", g2, c2, M.double().sum(dim=0))):
        gr, cr = up(gpu_res), up(cpu_res)
        gc, gt, ct = scaled(gr, cr), scaled(gr, truth), scaled(cr, truth)
        parity[name] = {"tolerance": "1e-5 of max(|ref|, rms); the CPU's own distance from a binary64 sum is allowed for",
                        "gpu_vs_cpu": gc, "gpu_vs_f64": gt, "cpu_vs_f64": ct,
                        "pass": bool(gt <= max(ct, 1e-5) and gc <= 1e-5 + ct)}

    # ---- C3: softmax relative 1e-5, SoftmaxGrad bit-exact -----------------------------------
    r, c = 32768, 32000
    L = torch.randn(r, c, device=dev, generator=g) * 2
    lab = torch.randint(0, c, (r,), device=dev, generator=g).float()
    P = lib.softmax(torch.empty(r, c, device=dev), L)
    hL, hlab = host(L), host(lab)
    cP = np.empty((r, c), np.float32)
    cpu_ms["softmax"] = best_of(lambda: chk.softmax(cP, hL)) * 1e3
    dP = up(cP)
    rel, rel64_gpu, rel64_cpu = 0.0, 0.0, 0.0
    for lo in range(0, r, 2048):
        a, b = P[lo:lo + 2048], dP[lo:lo + 2048]
        rel = max(rel, float(((a - b).abs() / b.clamp_min(1.2e-38)).max().item()))
        # the CPU adds a row's 32000 exponentials one after the other in binary32; how far that
        # (and the GPU's pairwise sum) is from a binary64 evaluation says whose rounding a difference is
        truth = torch.softmax(L[lo:lo + 2048].double(), dim=1)
        rel64_gpu = max(rel64_gpu, float(((a.double() - truth).abs() / truth).max().item()))
        rel64_cpu = max(rel64_cpu, float(((b.double() - truth).abs() / truth).max().item()))
        del truth
    parity["C3_softmax"] = {"tolerance": "relative 1e-5 per element; the CPU's own distance from a binary64 "
                                         "evaluation is allowed for",
                            "elements": r * c, "gpu_vs_cpu": rel, "gpu_vs_f64": rel64_gpu, "cpu_vs_f64": rel64_cpu,
                            "pass": bool(rel64_gpu <= max(rel64_cpu, 1e-5) and rel <= 1e-5 + rel64_cpu)}
    del P
    # the gradient of the same probabilities on both sides: prob - onehot(label), exact
    Gd = lib.softmax_grad(L, dP, lab)  # L is no longer needed: it receives the gradient
    cG = hL
    cpu_ms["softmax_grad"] = best_of(lambda: chk.softmax_grad(cG, cP, hlab)) * 1e3
    dG = up(cG)
    bad = 0
    for lo in range(0, r, 4096):
        bad += bit_mismatches(Gd[lo:lo + 4096], dG[lo:lo + 4096])
    parity["C3_softmax_grad"] = {"tolerance": "bit-exact", "elements": r * c, "mismatches": bad, "pass": bad == 0}
    del L, Gd, dG, dP, cP, cG, hL

    # ---- C4: pooling family, bit-exact -------------------------------------------------------
    planes = 256 * 256
    X = torch.rand(planes, 56, 56, device=dev, generator=g)
    gP = torch.rand(planes, 27, 27, device=dev, generator=g)
    Pm = lib.pool(torch.empty(planes, 27, 27, device=dev), X, 3, 3, 2, 2)
    hX, hgP = host(X), host(gP)
    cPm = np.empty((planes, 27, 27), np.float32)
    cpu_ms["pool"] = best_of(lambda: chk.pool(cPm, hX, 3, 3, 2, 2)) * 1e3
    bad_pool = bit_mismatches(Pm, up(cPm))
    win = X.unfold(1, 3, 2).unfold(2, 3, 2)  # (planes, 27, 27, 3, 3) view
    tied = 0
    for lo in range(0, planes, 8192):
        hits = (win[lo:lo + 8192] == Pm[lo:lo + 8192, :, :, None, None]).sum(dim=(3, 4))
        tied += int((hits > 1).sum().item())
    G = lib.unpool(torch.empty(planes, 56, 56, device=dev), X, Pm, gP, 3, 3, 2, 2)
    cG = np.empty((planes, 56, 56), np.float32)
    cpu_ms["unpool"] = best_of(lambda: chk.unpool(cG, hX, cPm, hgP, 3, 3, 2, 2)) * 1e3
    bad_unpool = bit_mismatches(G, up(cG))
    X4 = X.view(256, 256, 56, 56)
    Lr = lib.chpool(G.view(256, 256, 56, 56), X4, 5)
    hX4 = hX.reshape(256, 256, 56, 56)
    cL = cG.reshape(256, 256, 56, 56)
    cpu_ms["chpool"] = best_of(lambda: chk.chpool(cL, hX4, 5)) * 1e3
    bad_chpool = bit_mismatches(Lr, up(cL))
    parity["C4_pooling"] = {"tolerance": "bit-exact", "shape": [256, 256, 56, 56],
                            "pool_mismatches": bad_pool, "unpool_mismatches": bad_unpool,
                            "chpool_mismatches": bad_chpool, "windows_with_a_tied_maximum": tied,
                            "pass": bad_pool == 0 and bad_unpool == 0 and bad_chpool == 0}
    del X, gP, Pm, G, X4, Lr, win, hX, hgP, cPm, cG, cL, hX4

    # ---- C5: embedding backward, relative 1e-5 per table row, index work exact ---------------
    idx = zipf_batch()[0]
    ck, cv = idx.copy(), np.arange(EMBED_N, dtype=np.int32)
    keys = torch.from_numpy(idx.copy()).to(dev)
    vals = torch.arange(EMBED_N, dtype=torch.int32, device=dev)
    lib.sort_by_key(keys, vals, True)
    cpu_ms["sort_by_key"] = best_of(lambda: chk.sort_by_key(ck, cv, True), 1) * 1e3  # in place: one run
    bad_sort = int((keys.cpu().numpy() != ck).sum() + (vals.cpu().numpy() != cv).sum())
    src = torch.randn(EMBED_N, EMBED_D, device=dev, generator=g)
    table = lib.addtakegrad_largebatch(torch.zeros(EMBED_K, EMBED_D, device=dev), keys, vals, src)
    hsrc = host(src)
    ctab = np.zeros((EMBED_K, EMBED_D), np.float32)

    def cpu_embed(reps):  # the table is cleared outside the timed call
        best = float("inf")
        for _ in range(reps):
            ctab[...] = 0
            best = min(best, best_of(lambda: chk.addtakegrad_largebatch(ctab, ck, cv, hsrc), 1))
        return best * 1e3

    cpu_ms["addtakegrad"] = cpu_embed(2)
    threads = chk.num_threads()
    chk.set_num_threads(1)
    cpu_ms["addtakegrad_one_thread"] = cpu_embed(1)
    chk.set_num_threads(threads)
    dC = up(ctab)
    # binary64 accumulation of the same rows: the CPU adds the 135 619 entries of the hottest row one
    # after the other in binary32, so its own rounding exceeds 1e-5 there
    truth = torch.zeros(EMBED_K, EMBED_D, device=dev, dtype=torch.float64)
    for lo in range(0, EMBED_N, 1 << 18):
        truth.index_add_(0, keys[lo:lo + (1 << 18)].long(), src[vals[lo:lo + (1 << 18)].long()].double())

    def row_scaled(a, b):  # per table row: max |a - b| / max(|b|, rms of the row of b)
        a, b = a.double(), b.double()
        rms = b.pow(2).mean(dim=1, keepdim=True).sqrt()
        return float(((a - b).abs() / torch.maximum(b.abs(), rms).clamp_min(1e-30)).max().item())

    gc, gt, ct = row_scaled(table, dC), row_scaled(table, truth), row_scaled(dC, truth)
    touched = torch.zeros(EMBED_K, dtype=torch.bool, device=dev)
    touched[keys.long()] = True
    untouched_bad = bit_mismatches(table[~touched], dC[~touched])
    seg = np.bincount(ck, minlength=EMBED_K)
    parity["C5_addtakegrad_largebatch"] = {
        "tolerance": "1e-5 of max(|ref|, rms of the table row), the CPU's own distance from a binary64 sum allowed "
                     "for; untouched rows and the sort bit-exact",
        "indices": EMBED_N, "distinct_rows": int(touched.sum().item()), "longest_segment": int(seg.max()),
        "gpu_vs_cpu": gc, "gpu_vs_f64": gt, "cpu_vs_f64": ct,
        "untouched_row_mismatches": untouched_bad, "sort_by_key_mismatches": bad_sort,
        "pass": bool(gt <= max(ct, 1e-5) and gc <= 1e-5 + ct and untouched_bad == 0 and bad_sort == 0)}
    del src, table, dC, truth, hsrc, ctab
    torch.cuda.empty_cache()
    parity["pass"] = all(v["pass"] for v in parity.values() if isinstance(v, dict))
    return parity, {k: round(v, 2) for k, v in cpu_ms.items()}


BASELINE_KERNELS = ("map", "keep_highdim", "keep_lowest", "softmax", "softmax_grad", "pool", "unpool", "chpool",
                    "addtakegrad")


def configs_block(kernels, cpu_ms):
    """The nine kernels of the five BASELINE configs in compact form."""
    rows = {r["key"]: r for r in kernels}
    out = []
    for key in BASELINE_KERNELS:
        if key not in rows:
            continue
        r = rows[key]
        e = {"key": key, "ms": round(r["ms"], 4), "frac_of_measured_peak": r["frac_of_measured_peak"],
             "frac_of_8TBps": r["frac_of_8TBps"], "ms_back_to_back": round(r["ms_back_to_back"], 4),
             "frac_back_to_back": r["frac_back_to_back"]}
        if cpu_ms and key in cpu_ms:
            e["cpu_ms"] = cpu_ms[key]
        out.append(e)
    return out


# --------------------------------------------------------------------------------------
# embedding backward with the table sharded by rows (strong scaling; --workload embed_sharded)
# --------------------------------------------------------------------------------------
def embed_sharded_arm(args, torch, lib, dist, peer, rank, world, dev):
    """AddTakeGradLargeBatch on a 262144 x 1024 table whose rows are spread over the ranks, for the
    same 2^20 Zipf(1.1) indices at every N (total work fixed).  The source rows are replicated on
    every rank, the sorted index list is routed on the host before the timed region (its time is
    reported separately).  Ownership schemes:
      contiguous        rank r owns a contiguous range of rows; every row keeps its accumulation order
      cyclic_hot        row i is owned by rank i % N and the 64 most frequent rows are handled by all
                        ranks: each sums the hot entries of its slice of the batch into a 64 x 1024
                        table, the ranks' tables are combined by peer stores, owners add their rows
      cyclic_hot_nccl   the same with one NCCL all-reduce as the combine
    Time per step = max over ranks (CUDA events); rank 0 prints one JSON line."""
    from mshadow_b200 import sharding
    idx, keys, order = zipf_batch()
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    src = torch.randn(EMBED_N, EMBED_D, device=dev, generator=g)
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
        if dist is not None:
            dist.all_reduce(c, op=dist.ReduceOp.MAX)
        return int(c.item())

    def checksum(table):
        s = table.double().sum().reshape(1)
        if dist is not None:
            dist.all_reduce(s)
        return float(s.item())

    if args.emulate_rank_of > 1 and world == 1:
        # rank 0's step of a group of `emulate_rank_of` ranks, alone on this GPU and without the exchange:
        # what the kernels of one shard cost (for launch lists; a single-rank command can be profiled)
        w = args.emulate_rank_of
        step, shard, info = make_cyclic_hot_step(torch, lib, None, None, keys, order, src, 0, w, dev)
        ms = timed(step)
        print(json.dumps({"workload": "embed_sharded", "emulated": "rank 0 of %d, no exchange" % w, "ms_per_step": ms,
                          "entries_on_this_rank": info["entries_on_this_rank"], "steps": steps, "warmup": warm}),
              file=OUT, flush=True)
        return
    out = {}
    t0 = time.perf_counter()
    lk, lo, rb, re = sharding.route_sorted_indices(keys, order, EMBED_K, rank, world)
    route_ms = (time.perf_counter() - t0) * 1e3
    shard = torch.zeros(re - rb, EMBED_D, device=dev)
    dk, do = torch.from_numpy(lk).to(dev), torch.from_numpy(lo).to(dev)
    if lk.size:
        lib.addtakegrad_largebatch(shard, dk, do, src)
    ref_sum = checksum(shard)
    ms = timed(lambda: lib.addtakegrad_largebatch(shard, dk, do, src) if lk.size else None)
    out["contiguous"] = {"ms_per_step": ms, "max_entries_on_a_rank": spread(lk.size), "host_routing_ms": route_ms}
    del shard, dk, do
    hot_sum = None
    for name, use_peer in (("cyclic_hot", True), ("cyclic_hot_nccl", False)):
        if world == 1 and not use_peer:
            continue
        step, shard, info = make_cyclic_hot_step(torch, lib, dist, peer if (use_peer and world > 1) else None, keys,
                                                 order, src, rank, world, dev)
        step()
        if hot_sum is None:
            hot_sum = checksum(shard)
        ms = timed(step)
        if use_peer and world > 1:
            peer.pull_wait(2)
        out[name] = {"ms_per_step": ms, "hot_rows": info["hot_rows"],
                     "max_entries_on_a_rank": spread(info["entries_on_this_rank"]),
                     "host_routing_ms": info["host_routing_ms"], "device_routing_ms": info["device_routing_ms"],
                     "device_routing_equals_host_routing": info["device_routing_equals_host_routing"],
                     "exchange_bytes": HOT_ROWS * EMBED_D * 4}
        del shard
    if rank == 0:
        best = min(v["ms_per_step"] for v in out.values())
        line = {"metric": "AddTakeGradLargeBatch 262144x1024 table sharded by rows, 2^20 Zipf(1.1) indices, fp32",
                "value": EMBED_N * EMBED_D / (best * 1e-3) / 1e9, "unit": "Gelem/s", "n_gpus": world, "steps": steps,
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
    ap.add_argument("--no-parity", action="store_true", help="skip the full-size parity leg (N = 1)")
    ap.add_argument("--no-sharded", action="store_true", help="skip the strong-scaling block")
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--variant-steps", type=int, default=200,
                    help="steps per exchange variant in the N > 1 diagnostic block (0 = skip)")
    ap.add_argument("--only", default=None,
                    help="run one kernel of the table alone (map, keep_highdim, keep_lowest, softmax, softmax_grad, "
                         "pool, unpool, chpool, addtakegrad, ...) for --steps launches after --warmup; for profiling")
    ap.add_argument("--small", action="store_true", help="with --only: reduced size that still exceeds L2")
    ap.add_argument("--trace-launches", action="store_true",
                    help="with --only: time --steps launches one by one and report them in bins of 20 beside the "
                         "sampled SM clock and throttle reasons")
    ap.add_argument("--emulate-rank-of", type=int, default=0,
                    help="with --workload embed_sharded on one GPU: run rank 0's step of a group of this many ranks, "
                         "without the exchange")
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
        if args.trace_launches:
            print(json.dumps({"only": args.only, "small": args.small,
                              "launch_trace": launch_trace(lib, torch, args.only, args.small, args.steps)}), flush=True)
            return
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
    # the ranks' results are combined by peer stores; NCCL (through torch.distributed) carries the
    # barriers, the max-over-ranks of the timings and the window handles
    peer = make_peer_model(dist, rank, world, local_rank) if world > 1 else None
    peer_side = make_peer_model(dist, rank, world, local_rank, own_stream=True) if world > 1 else None
    if args.workload == "embed_sharded":
        embed_sharded_arm(args, torch, lib, dist, peer, rank, world, dev)
        if dist is not None:
            dist.barrier()
            peer.close()
            peer_side.close()
            dist.destroy_process_group()
        return

    # The strong-scaling block and (N > 1) the comparison of exchange schemes run first: they are
    # part of the job anyway, and the headline's short timed region then starts on a GPU that has
    # been busy for a while instead of one that idled through the host-side set-up.
    (p4, h4), (pm, hm) = make_host_inputs(lib, rank)
    sharded = None
    if not args.no_sharded:
        sharded = sharded_block(args, torch, lib, dist, peer, peer_side, rank, world, dev, peak)
    T = torch.empty(C2A_SHAPE, device=dev)
    M = torch.empty(C2B_SHAPE, device=dev)
    # both results of a step live in one buffer so that one exchange combines them; two buffers
    # alternate, and the sum over the ranks of step i arrives in sums[i & 1]
    outs = [torch.zeros(NRES, device=dev) for _ in range(2)]
    sums = [torch.zeros(NRES, device=dev) for _ in range(2)]
    o512s = [o[:C2A_SHAPE[1]] for o in outs]
    o4096s = [o[C2A_SHAPE[1]:] for o in outs]
    n4, nm = int(np.prod(C2A_SHAPE)), int(np.prod(C2B_SHAPE))
    lib.copy_2d(T, n4, p4, n4, 1, n4, mshadow_b200.capi.H2D)
    lib.copy_2d(M, nm, pm, nm, 1, nm, mshadow_b200.capi.H2D)
    torch.cuda.synchronize()
    variants = None
    if world > 1 and args.variant_steps > 0:
        variants = exchange_variants(torch, lib, dist, peer, peer_side, dev, T, M, outs, sums, args.variant_steps)
    lag = Lagged(peer_side, 0) if peer_side is not None else None

    def reductions(i, ev=None):
        """Step i: both reductions into outs[i & 1]; then, on the exchange model's own stream and
        beside the next step's reductions, the push of the 4608 results into every GPU's window and
        the pull of step i - 1 (the sum over the ranks) into sums[(i - 1) & 1]."""
        j = i & 1
        if ev is not None:
            ev[0].record()
        lib.reduce_keep_highdim(o512s[j], T)
        if ev is not None:
            ev[1].record()
        lib.reduce_keep_lowest(o4096s[j], M)
        if ev is not None:
            ev[2].record()
        if lag is not None:
            # The fence names the most recent pull, that of step i - 2: once it is done, so is the
            # push that read outs[(i + 1) & 1], which the next step overwrites.  Placed here, before
            # this step's push and pull are issued, it cannot make the main stream wait for them.
            peer_side.pull_fence(0)
            lag.step(outs[j], sums[j ^ 1])
        if ev is not None:
            ev[3].record()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()
    sampler.period = 0.002            # the timed region may last only milliseconds
    for i in range(args.warmup):
        reductions(i)
    barrier()

    # timed region: events around the whole run and around each kernel of each step; the end event
    # follows the last step's pull, so K steps carry K complete exchanges
    k = args.steps
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(k)]
    launches0 = lib.launch_count()
    sampler.window[0] = time.perf_counter()
    e_start.record()
    for s in range(k):
        reductions(args.warmup + s, ev[s])
    if lag is not None:
        peer_side.pull_fence(0)
    e_end.record()
    barrier()
    sampler.window[1] = time.perf_counter()
    launches = lib.launch_count() - launches0 + (2 * k if lag is not None else 0)  # + push and pull kernels
    seconds = e_start.elapsed_time(e_end) * 1e-3
    t_high = float(np.mean([ev[s][0].elapsed_time(ev[s][1]) for s in range(k)])) * 1e-3
    t_low = float(np.mean([ev[s][1].elapsed_time(ev[s][2]) for s in range(k)])) * 1e-3
    t_xchg = float(np.mean([ev[s][2].elapsed_time(ev[s][3]) for s in range(k)])) * 1e-3
    per_rank = np.array(gather_floats(torch, dist, dev, [seconds, t_high, t_low, t_xchg]))
    seconds = float(per_rank[:, 0].max())
    # One NVML query takes milliseconds, so a short timed region may hold no clock sample at all:
    # the same steps carry on, untimed, for a twentieth of a second (the same number on every rank),
    # and the clock record says which samples fall where.
    extra = int(min(5000, max(0, 0.05 / max(1e-6, seconds / k) - k)))
    sampler.tail_window[0] = time.perf_counter()
    for s in range(extra):
        reductions(args.warmup + k + s)
    if lag is not None:
        peer_side.pull_fence(0)
    barrier()
    sampler.tail_window[1] = time.perf_counter()
    k_done = k + extra
    sampler.period = 0.01
    if lag is not None:
        lag.drain(sums[(args.warmup + k_done - 1) & 1])
    value = ELEMS_PER_STEP * world * k / seconds / 1e9
    exchange_ok = None
    if peer is not None:
        # the last step's sum over the ranks against the rank-order sum of the gathered results
        from mshadow_b200 import sharding
        last = (args.warmup + k_done - 1) & 1
        parts = [torch.zeros(NRES, device=dev) for _ in range(world)]
        dist.all_gather(parts, outs[last])
        want = sharding.rank_order_sum([p.cpu().numpy() for p in parts])
        exchange_ok = bool(np.array_equal(want.view(np.uint32), sums[last].cpu().numpy().view(np.uint32)))

    # end to end: host buffers in, host results out, through the C ABI
    res_ptr = lib.alloc_host(NRES * 4)
    ke = max(1, min(args.e2e_steps, k))

    def e2e_step():
        lib.copy_2d(T, n4, p4, n4, 1, n4, mshadow_b200.capi.H2D)
        lib.copy_2d(M, nm, pm, nm, 1, nm, mshadow_b200.capi.H2D)
        lib.reduce_keep_highdim(o512s[0], T)
        lib.reduce_keep_lowest(o4096s[0], M)
        res = outs[0]
        if peer_side is not None:
            peer_side.push(outs[0], 0)
            peer_side.pull_req(sums[0], 0)
            peer_side.pull_fence(0)
            res = sums[0]
        lib.copy_2d(res_ptr, NRES, res, NRES, 1, NRES, mshadow_b200.capi.D2H)
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
    e2e_seconds = float(np.array(gather_floats(torch, dist, dev, [e2e_seconds]))[:, 0].max())
    e2e_value = ELEMS_PER_STEP * world * ke / e2e_seconds / 1e9
    sampler.stop_flag = True
    sampler.join(timeout=1.0)
    if peer_side is not None:
        peer_side.pull_wait(0)

    g1, g2 = o512s[0].cpu().numpy().copy(), o4096s[0].cpu().numpy().copy()

    if rank != 0:
        if dist is not None:
            dist.barrier()
            peer.close()
            peer_side.close()
            dist.destroy_process_group()
        return

    bytes_low = 4 * nm + 4 * C2B_SHAPE[1]
    bytes_high = 4 * n4 + 4 * C2A_SHAPE[1]
    achieved = bytes_low / t_low / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": k, "warmup": args.warmup,
        "ms_per_step": seconds / k * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD
                               + ("; the 4608 result floats of every step are stored into every GPU's window over NVLink "
                                  "and added in rank order by two small kernels on the exchange model's own stream "
                                  "(mshadow::ps::PeerModel), beside the next step's reductions"
                                  if world > 1 else ""),
                   "l2": "inputs (411 MB and 1074 MB) exceed the 126 MB L2; no flush needed",
                   "inputs": "N(0,1), seeded, generated on the host, resident in HBM before timing"},
        "clocks": sampler.summary(),
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 4 * (n4 + nm),
                "d2h_bytes_per_step": 4 * NRES, "steps": ke,
                "ms_per_step": e2e_seconds / ke * 1e3, "wall_ms_per_step": wall / ke * 1e3},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "kernel": "ReduceKeepLowestKernel (sum_rows 65536x4096)",
                     "achieved": achieved, "peak": peak, "peak_kind": "of " + peak_kind, "unit": "GB/s",
                     "frac": achieved / peak, "frac_of_8TBps": achieved / NOMINAL_HBM_GBS,
                     "traffic": NCU_TRAFFIC_KEEP_LOWEST, "algorithmic_bytes": bytes_low,
                     "launch_ms": t_low * 1e3,
                     "other": {"kernel": "ReduceKeepHighDimKernel (256,512,28,28)", "launch_ms": t_high * 1e3,
                               "achieved": bytes_high / t_high / 1e9, "frac": bytes_high / t_high / 1e9 / peak},
                     "per_rank": {"sum_rows_ms": {"max": round(float(per_rank[:, 2].max()) * 1e3, 5),
                                                  "min": round(float(per_rank[:, 2].min()) * 1e3, 5)},
                                  "sumall_ms": {"max": round(float(per_rank[:, 1].max()) * 1e3, 5),
                                                "min": round(float(per_rank[:, 1].min()) * 1e3, 5)},
                                  "exchange_ms": {"max": round(float(per_rank[:, 3].max()) * 1e3, 5),
                                                  "min": round(float(per_rank[:, 3].min()) * 1e3, 5)},
                                  "step_ms": {"max": round(float(per_rank[:, 0].max()) / k * 1e3, 5),
                                              "min": round(float(per_rank[:, 0].min()) / k * 1e3, 5)}}},
    }
    if exchange_ok is not None:
        line["exchange_bit_exact_vs_rank_order_sum"] = exchange_ok
    if variants is not None:
        line["exchange_variants"] = variants
    parity = None
    if world == 1:
        chk, kind = load_cpu_checker()
        c1, c2 = np.zeros(C2A_SHAPE[1], np.float32), np.zeros(C2B_SHAPE[1], np.float32)
        cpu_step(chk, h4, hm, c1, c2)
        cpu_s = best_of(lambda: cpu_step(chk, h4, hm, c1, c2), 3)
        line["cpu_baseline"] = {"value": ELEMS_PER_STEP / cpu_s / 1e9, "unit": UNIT, "cores": chk.num_threads(),
                                "kind": kind, "sample": "best of 3 repetitions of the full step on the same inputs",
                                "ms_per_step": cpu_s * 1e3, "cpu_model": cpu_model()}
        cpu_ms = None
        if not args.no_parity:
            parity, cpu_ms = full_size_parity(torch, lib, chk, dev, h4, hm, T, M, g1, g2)
        lib.free_host(p4)
        lib.free_host(pm)
        del T, M
        torch.cuda.empty_cache()
        if not args.no_table:
            kernels = kernel_table(lib, torch, peak)
            line["kernels"] = kernels
            line["configs"] = configs_block(kernels, cpu_ms)
            # the driver's record keeps the known keys whole: a compact copy rides inside `roofline`
            # per kernel: [ms alone, fraction of the measured peak, ms back to back, fraction back to back]
            line["roofline"]["configs"] = {c["key"]: [c["ms"], c["frac_of_measured_peak"], c["ms_back_to_back"],
                                                      c["frac_back_to_back"]] for c in line["configs"]}
    if sharded is not None:
        line["sharded"] = sharded
        line["roofline"]["sharded_Gelem_per_s"] = {key: v["Gelem_per_s"] for key, v in sharded.items()}
    if parity is not None:
        line["roofline"]["parity_pass"] = {key: v["pass"] for key, v in parity.items() if isinstance(v, dict)}
        line["parity"] = parity
    print(json.dumps(line), file=OUT, flush=True)
    if dist is not None:
        dist.barrier()
        peer.close()
        peer_side.close()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
