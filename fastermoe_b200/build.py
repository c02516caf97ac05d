"""Builds libfmoe_b200.so (sm_100a) from csrc/ with nvcc.

Run as ``python -m fastermoe_b200.build`` or call :func:`build`.  Objects are
compiled in parallel and only when their sources changed; the shared library
is written next to this file so that it is loaded from the source tree.
"""
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "build")
LIB_PATH = os.path.join(HERE, "libfmoe_b200.so")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nccl_include():
    try:
        import nvidia.nccl  # type: ignore

        for base in nvidia.nccl.__path__:
            inc = os.path.join(base, "include")
            if os.path.exists(os.path.join(inc, "nccl.h")):
                return inc
    except Exception:
        pass
    if os.path.exists("/usr/include/nccl.h"):
        return "/usr/include"
    raise RuntimeError("nccl.h not found (looked in the nvidia.nccl wheel and /usr/include)")


def _nvcc():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found")
    return nvcc


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose=False, force=False, ptxas_info=False):
    """Compile every .cu under csrc/ for sm_100a and link libfmoe_b200.so."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(HERE, "..", "include", "fmoe_b200.h"))
    sources = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    common = [nvcc, *ARCH_FLAGS, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "-I", _nccl_include()]
    if ptxas_info:
        common += ["-Xptxas", "-v"]
    jobs = []
    for src in sources:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ_DIR, src[:-3] + ".o")
        if force or _newer(o, [s, *headers]):
            jobs.append((common + ["-c", s, "-o", o], src))

    def run(job):
        cmd, name = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        return name, r

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for name, r in ex.map(run, jobs):
            if verbose or r.returncode != 0 or ptxas_info:
                sys.stderr.write(f"[nvcc {name}]\n{r.stdout}{r.stderr}\n")
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {name}")
    objs = [os.path.join(OBJ_DIR, s[:-3] + ".o") for s in sources]
    if force or jobs or _newer(LIB_PATH, objs):
        cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", LIB_PATH, *objs, "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link of libfmoe_b200.so failed")
    return LIB_PATH


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="-f" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)
