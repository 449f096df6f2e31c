"""Build recipe for the in-tree native libraries (no network, no JIT cache):

  rusttensor_b200/librt_b200.so       the C-ABI CUDA library (include/rt_b200.h), sm_100a only
  rusttensor_b200/librt_b200_host.so  the C++ host engine over that ABI (rth_* functions)

nvcc cross-compiles without a GPU, so this runs on a CPU-only machine as well.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "librt_b200.so")
HOST_LIB = os.path.join(HERE, "librt_b200_host.so")

CU_SOURCES = ["rt_context.cu", "k_elementwise.cu", "k_reduce.cu", "k_pool.cu", "k_optim.cu", "k_gemm.cu", "k_gemm_tc.cu", "k_conv_tc.cu", "k_conv_thin.cu", "k_lstm.cu", "k_tc_probe.cu", "k_conv_dw_tc.cu", "k_random.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function"]


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def _headers():
    out = [os.path.join(HERE, "..", "include", "rt_b200.h")]
    for root, _, files in os.walk(CSRC):
        out += [os.path.join(root, f) for f in files if f.endswith((".cuh", ".hpp", ".h"))]
    return out


def build(verbose=False, force=False):
    os.makedirs(BUILD, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    cxx = os.environ.get("CXX", "g++")
    hdrs = _headers()
    objs = []
    procs = []
    for src in CU_SOURCES:
        path = os.path.join(CSRC, src)
        obj = os.path.join(BUILD, src.replace(".cu", ".o"))
        objs.append(obj)
        if force or _newer(obj, [path] + hdrs):
            cmd = [nvcc] + NVCC_FLAGS + ["-c", path, "-o", obj]
            if verbose:
                print(" ".join(cmd), file=sys.stderr)
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out.decode()}")
    if force or _newer(LIB, objs):
        cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-ldl"]
        subprocess.run(cmd, check=True)
    host_src = os.path.join(CSRC, "host", "harness.cpp")
    if force or _newer(HOST_LIB, [host_src, LIB] + hdrs):
        cmd = [cxx] + HOST_FLAGS + ["-shared", "-o", HOST_LIB, host_src, "-L" + HERE, "-lrt_b200", "-Wl,-rpath,$ORIGIN"]
        if verbose:
            print(" ".join(cmd), file=sys.stderr)
        subprocess.run(cmd, check=True)
    return LIB, HOST_LIB


if __name__ == "__main__":
    print(build(verbose=True, force="--force" in sys.argv))
