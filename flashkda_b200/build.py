"""Build libfkda.so (the C-ABI library with the sm_100a kernels) in-tree with nvcc.

    python -m flashkda_b200.build [--force] [--verbose]

nvcc cross-compiles for sm_100a without a GPU.  The library lands next to this file so that it
travels with the source tree; it is never installed into site-packages.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libfkda.so")
SOURCES = ["fkda_api.cu", "fkda_prepare.cu", "fkda_prepare_tc.cu", "fkda_scan.cu", "fkda_scan2.cu", "fkda_scan_short.cu", "fkda_segscan.cu", "fkda_short16.cu", "fkda_refmode.cu", "fkda_aux.cu", "fkda_static_ws.cu"]
HEADERS = [os.path.join(CSRC, "fkda_common.cuh"), os.path.join(os.path.dirname(HERE), "include", "fkda.h"),
           os.path.join(os.path.dirname(HERE), "include", "fkda_testing.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]
# extra compiler flags, e.g. FKDA_NVCC_EXTRA="-DFKDA_TUNING" for a build with the phase-skip timing aid of the prepare kernel
NVCC_FLAGS += os.environ.get("FKDA_NVCC_EXTRA", "").split()


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    sources = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    logs = {}

    def compile_one(src):
        path = os.path.join(CSRC, src)
        obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        if force or _stale(obj, [path] + HEADERS):
            r = subprocess.run([nvcc] + NVCC_FLAGS + ["-c", path, "-o", obj], capture_output=True, text=True)
            logs[src] = r.stderr
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=len(sources)) as ex:
        objs = list(ex.map(compile_one, sources))
    if force or _stale(LIB, objs):
        r = subprocess.run([nvcc, "-shared", "-o", LIB] + objs + ["-lcudart"], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    if verbose:
        for src, log in logs.items():
            print(f"==== {src}\n{log}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
