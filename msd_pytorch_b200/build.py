"""Builds libmsd_b200.so (hand-written sm_100a CUDA + the C ABI) in-tree with nvcc.

The shared object lands in ``msd_pytorch_b200/lib/`` next to the sources, so a copy
of the source tree carries the binary with it.  No torch headers are involved: the
library is plain CUDA C++ behind ``include/msd_b200.h``.
"""
import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
OBJDIR = os.path.join(PKG, "build")
LIB = os.path.join(LIBDIR, "libmsd_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-DMSD_B200_BUILD",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-O3",
    "--expt-relaxed-constexpr",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; the msd_b200 library cannot be built")


def _sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _deps_mtime():
    files = glob.glob(os.path.join(CSRC, "*")) + [os.path.join(PKG, "..", "include", "msd_b200.h"), __file__]
    return max(os.path.getmtime(f) for f in files)


def is_current():
    return os.path.exists(LIB) and os.path.getmtime(LIB) >= _deps_mtime()


def build_library(force=False, verbose=False, ptxas_info=False):
    """Compile every ``csrc/*.cu`` for sm_100a and link ``lib/libmsd_b200.so``."""
    if not force and is_current():
        return LIB
    nvcc = _nvcc()
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    hdr_mtime = max(os.path.getmtime(f) for f in glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh"))
                    + [os.path.join(PKG, "..", "include", "msd_b200.h"), __file__])

    def compile_one(src):
        obj = os.path.join(OBJDIR, os.path.basename(src)[:-3] + ".o")
        if not force and os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src), hdr_mtime):
            return obj, ""
        extra = os.environ.get("MSD_EXTRA_NVCC_FLAGS", "").split()
        cmd = [nvcc] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if ptxas_info else []) + ["-c", src, "-o", obj]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, p.stdout, p.stderr))
        return obj, p.stderr

    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        results = list(ex.map(compile_one, _sources()))
    objs = [o for o, _ in results]
    log = "".join(l for _, l in results)
    cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", "-lcuda"]
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise RuntimeError("link failed:\n%s\n%s" % (p.stdout, p.stderr))
    if verbose or ptxas_info:
        sys.stderr.write(log)
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv))
