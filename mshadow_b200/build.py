"""Builds libmshadow_b200.so (and the conformance test library) in-tree with nvcc for sm_100a."""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    # a*b+c in user functors must round twice, as on the host, for bit-identical results
    "-fmad=false",
    "-Xcompiler", "-fPIC", "-shared",
    # failed CHECKs become exceptions that the C layer turns into status codes
    "-DDMLC_LOG_FATAL_THROW=1",
    "-I" + os.path.join(ROOT, "include"),
    "-I" + os.path.join(HERE, "include"),
]

TARGETS = [
    (os.path.join(HERE, "libmshadow_b200.so"),
     [os.path.join(HERE, "csrc", "capi.cu"), os.path.join(HERE, "csrc", "noalloc.cu")], []),
    (os.path.join(ROOT, "tests", "cxx", "libmsb_api_suite.so"),
     [os.path.join(ROOT, "tests", "cxx", "api_suite.cu")], []),
    # the checked build of the engine (tensor leaves refuse and record accesses outside their storage)
    (os.path.join(ROOT, "tests", "cxx", "libmsb_bounds_suite.so"),
     [os.path.join(ROOT, "tests", "cxx", "bounds_suite.cu")], ["-DMSHADOW_B200_CHECK_BOUNDS=1"]),
    # the multi-GPU synchronisation model; the only part that needs NCCL
    (os.path.join(HERE, "libmshadow_b200_ps.so"), [os.path.join(HERE, "csrc", "ps_capi.cu")], ["-lnccl"]),
]


# the headers evaluated on Tensor<cpu> by the host compiler alone (tests of the plans' index arithmetic)
HOST_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-shared", "-ffp-contract=off", "-DMSHADOW_USE_CUDA=0",
              "-DDMLC_LOG_FATAL_THROW=1", "-I" + os.path.join(HERE, "include")]
HOST_TARGETS = [
    (os.path.join(ROOT, "tests", "cxx", "libmsb_host_suite.so"), [os.path.join(ROOT, "tests", "cxx", "host_suite.cc")]),
]


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return exe


def _stale(out, deps):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    for d in deps:
        for base, _, files in os.walk(d) if os.path.isdir(d) else [(os.path.dirname(d), [], [os.path.basename(d)])]:
            for f in files:
                if os.path.getmtime(os.path.join(base, f)) > t:
                    return True
    return False


def build_all(force=False, verbose=True, only=None):
    """Builds every stale target; independent targets compile side by side.  `only` restricts the
    build to targets whose output file name contains that text."""
    from concurrent.futures import ThreadPoolExecutor
    deps_common = [os.path.join(HERE, "include"), os.path.join(ROOT, "include"), os.path.join(HERE, "csrc")]
    cmds = []
    for out, srcs, extra in TARGETS:
        if not all(os.path.exists(s) for s in srcs) or (only and only not in os.path.basename(out)):
            continue
        if not force and not _stale(out, srcs + deps_common):
            continue
        cmds.append([_nvcc()] + NVCC_FLAGS + ["-o", out] + srcs + extra)
    for out, srcs in HOST_TARGETS:
        if not all(os.path.exists(s) for s in srcs) or (only and only not in os.path.basename(out)):
            continue
        if not force and not _stale(out, srcs + deps_common):
            continue
        cmds.append([shutil.which("g++") or "g++"] + HOST_FLAGS + ["-o", out] + srcs)

    def run(cmd):
        if verbose:
            print("[build]", " ".join(cmd), flush=True)
        subprocess.check_call(cmd)

    if cmds:
        with ThreadPoolExecutor(max_workers=min(len(cmds), os.cpu_count() or 1)) as pool:
            list(pool.map(run, cmds))


if __name__ == "__main__":
    build_all(force="--force" in sys.argv,
              only=next((a.split("=", 1)[1] for a in sys.argv if a.startswith("--only=")), None))
