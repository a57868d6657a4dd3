"""Build recipe for the native parts of the package (in-tree, sm_100a only).

    python -m tbb_test_b200.build            # libb200mlp.so + host library/driver
    python -m tbb_test_b200.build --force

Outputs (git-ignored, next to their sources):
    tbb_test_b200/csrc/libb200mlp.so    CUDA kernels + C ABI (include/b200mlp.h)
    tbb_test_b200/host/libb2host.so     C++ host mirror of the reference's
                                        Partition / TwistedHyperCube / driver code
    tbb_test_b200/host/mlp_cuda         driver binary (counterpart of mlp_omp)
"""
import glob
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
HOST = os.path.join(PKG, "host")
LIB = os.path.join(CSRC, "libb200mlp.so")
HOST_LIB = os.path.join(HOST, "libb2host.so")
DRIVER = os.path.join(HOST, "mlp_cuda")

NVCC = os.environ.get("B2_NVCC", "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("B2_CXX", "/usr/bin/g++")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-ccbin", CXX]


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed:\n" + " ".join(cmd) + "\n" + r.stdout)
    if verbose and r.stdout.strip():
        print(r.stdout)


def build_cuda(force=False, verbose=False, ptxas_info=False):
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    deps = srcs + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + \
        glob.glob(os.path.join(ROOT, "include", "*.h"))
    if not force and not _stale(LIB, deps):
        return LIB
    objs = []
    for s in srcs:
        o = s[:-3] + ".o"
        if force or _stale(o, deps):
            cmd = [NVCC] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + ["-c", s, "-o", o]
            _run(cmd, verbose or ptxas_info)
        objs.append(o)
    _run([NVCC, "-shared", "-o", LIB] + objs + ["-ldl", "-ccbin", CXX], verbose)
    return LIB


def build_host(force=False, verbose=False):
    srcs = sorted(glob.glob(os.path.join(HOST, "*.cc")))
    if not srcs:
        return None
    deps = srcs + glob.glob(os.path.join(HOST, "*.h")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    lib_srcs = [s for s in srcs if os.path.basename(s) != "mlp_cuda.cc"]
    flags = ["-std=c++17", "-O2", "-fPIC", "-Wall", "-I", os.path.join(ROOT, "include"), "-I", HOST]
    if force or _stale(HOST_LIB, deps):
        _run([CXX] + flags + ["-shared", "-o", HOST_LIB] + lib_srcs + ["-lpthread"], verbose)
    main = os.path.join(HOST, "mlp_cuda.cc")
    if os.path.exists(main) and (force or _stale(DRIVER, deps + [LIB])):
        _run([CXX] + flags + ["-o", DRIVER, main, "-L", HOST, "-lb2host", "-L", CSRC, "-lb200mlp",
                              "-Wl,-rpath,$ORIGIN", "-Wl,-rpath,$ORIGIN/../csrc", "-lpthread", "-ldl"], verbose)
    return HOST_LIB


def build_all(force=False, verbose=False):
    build_cuda(force, verbose)
    build_host(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
    print("built", LIB)
