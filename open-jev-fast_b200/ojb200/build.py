"""In-tree build of libojb200.so (CUDA kernels + C ABI) with nvcc for sm_100a.

    python -m ojb200.build            # rebuild what is out of date
    python -m ojb200.build --force
    python -m ojb200.build --force --probes      # with the GEMM measurement knobs (-DOJB_GEMM_PROBES); never shipped

The library lands next to this file so that it travels with the source tree; nothing is installed anywhere else.
"""
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.normpath(os.path.join(HERE, "..", "csrc"))
INCLUDE = os.path.normpath(os.path.join(HERE, "..", "..", "include"))
OBJ_DIR = os.path.join(CSRC, "build")
LIB_PATH = os.path.join(HERE, "libojb200.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v", "-I", INCLUDE]
EXTRA_FLAGS = []


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libojb200.so cannot be built")
    return exe


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))


def _deps():
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hdrs += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    return hdrs


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(src, force, log):
    obj = os.path.join(OBJ_DIR, os.path.basename(src) + ".o")
    if not force and not _stale(obj, [src] + _deps()):
        return obj
    cmd = [_nvcc()] + NVCC_FLAGS + EXTRA_FLAGS + ["-x", "cu", "-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    with open(os.path.join(OBJ_DIR, os.path.basename(src) + ".log"), "w") as f:
        f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stderr[-4000:]}")
    if log:
        print(f"[ojb200.build] compiled {os.path.basename(src)}", flush=True)
    return obj


def build(force=False, log=True):
    """Compile every source under csrc/ and link libojb200.so. Returns the library path."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, force, log), srcs))
    if force or _stale(LIB_PATH, objs):
        cmd = [_nvcc(), "-shared", "-o", LIB_PATH] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stderr[-4000:])
        if log:
            print(f"[ojb200.build] linked {LIB_PATH}", flush=True)
    return LIB_PATH


if __name__ == "__main__":
    if "--probes" in sys.argv:
        EXTRA_FLAGS.append("-DOJB_GEMM_PROBES")
    build(force="--force" in sys.argv)
