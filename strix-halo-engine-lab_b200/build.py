"""Builds libb200moe.so (the CUDA kernels + the C ABI) for sm_100a, in-tree, with nvcc.

nvcc cross-compiles without a GPU. Flags: the exact-arithmetic set the reference uses for its bit-exact kernels
(--fmad=false -prec-div=true -prec-sqrt=true -ftz=false, cmake/QwenCuda.cmake:49) plus -lineinfo for profilers.
"""
import concurrent.futures as cf
import glob
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libb200moe.so")
OBJ = os.path.join(HERE, "build")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--fmad=false", "-prec-div=true",
              "-prec-sqrt=true", "-ftz=false", "-Xcompiler", "-fPIC"]


def nvcc():
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found")
    return path


def stale(sources):
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = sources + glob.glob(os.path.join(CSRC, "*.cuh")) + [os.path.join(HERE, "..", "include", "b200moe.h"), __file__]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    if not force and not stale(sources):
        return OUT
    os.makedirs(OBJ, exist_ok=True)
    cc = nvcc()

    def compile_one(src):
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        cmd = [cc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr)
        return obj

    with cf.ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, sources))
    libs = []
    if any("nccl" in open(s).read() for s in sources):
        libs = ["-lnccl"]
    r = subprocess.run([cc, "-shared", "-o", OUT] + objs + libs, capture_output=True, text=True)
    if r.returncode:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return OUT


if __name__ == "__main__":
    import sys
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
