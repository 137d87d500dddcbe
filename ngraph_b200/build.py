"""Builds the in-tree native libraries with nvcc / g++ (no JIT cache: the .so files sit next to
the sources so they travel with the repository snapshot to the GPU machine).

    python -m ngraph_b200.build            # kernels (+ the nGraph plugin when libngraph is present)
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
KERNEL_LIB = os.path.join(HERE, "libb200_kernels.so")
KERNEL_SOURCES = ["abi.cu", "quantize.cu", "qcontract.cu", "layout.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler",
              "-fPIC,-fvisibility=hidden", "-I" + os.path.join(ROOT, "include")]


def _newer(target, deps):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _deps():
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    files.append(os.path.join(ROOT, "include", "b200_kernels.h"))
    return files


def build_kernels(force=False, verbose=False):
    """Compile every CUDA translation unit for sm_100a and link libb200_kernels.so."""
    if not force and _newer(KERNEL_LIB, _deps()):
        return KERNEL_LIB
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    objs, procs = [], []
    for src in KERNEL_SOURCES:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        objs.append(obj)
        cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    for cmd, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out.decode())
        if p.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    subprocess.check_call(["nvcc", "-shared", "-o", KERNEL_LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"])
    return KERNEL_LIB


if __name__ == "__main__":
    print(build_kernels(force="--force" in sys.argv, verbose="-v" in sys.argv))
