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
KERNEL_SOURCES = ["abi.cu", "quantize.cu", "qcontract.cu", "layout.cu", "glue_f32.cu", "zero_points.cu"]
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


PLUGIN_LIB = os.path.join(HERE, "libb200_backend.so")
NGRAPH_LIB_DIR = os.path.join(ROOT, "oracle", "_ref", "lib")


def ngraph_checkout():
    """Root of the nGraph source tree, or None: $NGRAPH_REF, else the default the reference build recipe names
    (`REF ?= ...` in oracle/Makefile.ngraph, the one place that default is written down)."""
    cands = [os.environ.get("NGRAPH_REF", "")]
    try:
        for line in open(os.path.join(ROOT, "oracle", "Makefile.ngraph")):
            if line.startswith("REF ?="):
                cands.append(line.split("=", 1)[1].strip())
    except OSError:
        pass
    for d in cands:
        if d and os.path.isdir(os.path.join(d, "src", "ngraph")):
            return d
    return None


def ngraph_include_dir():
    """nGraph's public headers (the plugin compiles against them, like every nGraph backend): $NGRAPH_SRC, else the src
    directory of the checkout."""
    d = os.environ.get("NGRAPH_SRC", "")
    if d and os.path.exists(os.path.join(d, "ngraph", "runtime", "backend.hpp")):
        return d
    root = ngraph_checkout()
    return os.path.join(root, "src") if root else None


def host_cxx_flags(inc):
    return ["-std=c++14", "-O2", "-fPIC", "-w", "-include", "cstdint", "-include", "limits", "-DNGRAPH_JSON_DISABLE",
            "-I" + inc, "-I" + os.path.join(ROOT, "include"), "-I/usr/local/cuda/include"]


def build_plugin(force=False):
    """g++ the nGraph backend plugin against nGraph's headers and libngraph.so.  Skipped (returns None)
    where nGraph's headers or library are not available: the prebuilt .so is used there."""
    inc = ngraph_include_dir()
    cpp = ("b200_backend.cpp", "quant_fusion.cpp", "graph_passes.cpp", "function_io.cpp", "batch_split.cpp", "multi_device.cpp")
    src = [os.path.join(HERE, "backend", f) for f in cpp + ("b200_backend.hpp", "quant_fusion.hpp", "graph_passes.hpp", "function_io.hpp",
                                                            "batch_split.hpp", "multi_device.hpp")]
    if inc is None or not os.path.exists(os.path.join(NGRAPH_LIB_DIR, "libngraph.so")):
        return PLUGIN_LIB if os.path.exists(PLUGIN_LIB) else None
    build_kernels()
    if not force and _newer(PLUGIN_LIB, src + [KERNEL_LIB]):
        return PLUGIN_LIB
    cmd = ["/usr/bin/g++"] + host_cxx_flags(inc) + ["-shared", "-fvisibility=hidden"] + src[:len(cpp)] + ["-o", PLUGIN_LIB,
           "-L" + HERE, "-lb200_kernels", "-L" + NGRAPH_LIB_DIR, "-lngraph", "-L/usr/local/cuda/lib64", "-lcudart_static",
           "-ldl", "-lrt", "-lpthread", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath,$ORIGIN/../oracle/_ref/lib"]
    subprocess.check_call(cmd)
    return PLUGIN_LIB


CAPI_LIB = os.path.join(HERE, "libng_capi.so")


def build_capi(force=False):
    """The C facade over nGraph's C++ API that the Python tests and the benchmark drive (ctypes)."""
    inc = ngraph_include_dir()
    # the plugin's device-free graph passes are compiled in as well (tests look at the graph compile() would lower)
    srcs = [os.path.join(HERE, "harness", "ng_capi.cpp"), os.path.join(HERE, "harness", "bert_int8.cpp"),
            os.path.join(HERE, "backend", "graph_passes.cpp"), os.path.join(HERE, "backend", "quant_fusion.cpp"),
            os.path.join(HERE, "backend", "function_io.cpp"), os.path.join(HERE, "backend", "batch_split.cpp")]
    if inc is None or not os.path.exists(os.path.join(NGRAPH_LIB_DIR, "libngraph.so")):
        return CAPI_LIB if os.path.exists(CAPI_LIB) else None
    if not force and _newer(CAPI_LIB, srcs + [os.path.join(HERE, "backend", "graph_passes.hpp"), os.path.join(HERE, "backend", "quant_fusion.hpp"),
                                           os.path.join(HERE, "backend", "batch_split.hpp")]):
        return CAPI_LIB
    flags = [f for f in host_cxx_flags(inc) if f != "-std=c++14"] + ["-std=c++11"]
    cmd = ["/usr/bin/g++"] + flags + ["-shared"] + srcs + ["-o", CAPI_LIB, "-L" + NGRAPH_LIB_DIR, "-lngraph", "-ldl",
                             "-Wl,-rpath,$ORIGIN/../oracle/_ref/lib"]
    subprocess.check_call(cmd)
    return CAPI_LIB


if __name__ == "__main__":
    print(build_kernels(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_plugin(force="--force" in sys.argv))
    print(build_capi(force="--force" in sys.argv))
