"""Builds libdyb200.so (all CUDA kernels + the C ABI) in-tree with nvcc for sm_100a.

Usage: python -m dynet_b200.build [--force] [--verbose]
"""
import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libdyb200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "--use_fast_math=false", "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function", "-Xptxas", "-v"]
FLAGS = [f for f in FLAGS if f != "--use_fast_math=false"]


def _deps_mtime():
    hdrs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    return max(os.path.getmtime(h) for h in hdrs)


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    hdr_t = _deps_mtime()
    objs, jobs = [], []
    for s in srcs:
        o = os.path.join(OBJ, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_t):
            jobs.append((s, o))

    def compile_one(job):
        s, o = job
        p = subprocess.run([NVCC] + FLAGS + ["-c", s, "-o", o], capture_output=True, text=True)
        if verbose or p.returncode != 0:
            sys.stderr.write(p.stdout + p.stderr)
        if p.returncode != 0:
            raise RuntimeError("nvcc failed on " + s)
        with open(o + ".ptxas.txt", "w") as f:  # registers / spills / shared memory per kernel
            f.write(p.stderr)

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(compile_one, jobs))
    if jobs or not os.path.exists(LIB):
        subprocess.check_call([NVCC, "-shared", "-o", LIB] + objs + ["-lcudart"])
    build_host(force or bool(jobs))
    return LIB


HOST = os.path.join(HERE, "host")
HOST_LIB = os.path.join(HERE, "libdyb200_host.so")


def build_host(force=False):
    """C++ host layer above the C ABI: the node classes mirroring the reference interface and
    the LSTM language-model step driver (g++, links libdyb200.so and cudart)."""
    srcs = sorted(glob.glob(os.path.join(HOST, "*.cc")))
    deps = srcs + glob.glob(os.path.join(HOST, "*.h")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    if not force and os.path.exists(HOST_LIB) and os.path.getmtime(HOST_LIB) >= max(os.path.getmtime(d) for d in deps):
        return HOST_LIB
    cuda_home = os.path.dirname(os.path.dirname(NVCC))
    subprocess.check_call(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-o", HOST_LIB] + srcs +
                          ["-I" + os.path.join(cuda_home, "include"), "-L" + HERE, "-ldyb200",
                           "-L" + os.path.join(cuda_home, "lib64"), "-lcudart", "-Wl,-rpath,$ORIGIN"])
    return HOST_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
