"""Builds libpink_b200.so (the CUDA kernels and their C ABI) for sm_100a, in-tree.

Usage: python -m pink_b200.build [--force]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libpink_b200.so")
SOURCES = ["capi.cu", "operands.cu", "distance_tc.cu", "distance_f32.cu", "filter_f32.cu", "update.cu", "train_steps.cu", "rotshare.cu", "group.cu", "mma_peak.cu", "host_tables.cpp"]
HEADERS = ["kernels.cuh", "ptx.cuh", "record.cuh", "quant.cuh", "tensormap.cuh", os.path.join("..", "..", "include", "pink_b200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compile every .cu to an object and link the shared library; returns its path."""
    nvcc = os.environ.get("NVCC", "nvcc")
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    headers = [os.path.join(CSRC, h) for h in HEADERS]
    objs, procs = [], []
    for src in SOURCES:
        path = os.path.join(CSRC, src)
        obj = os.path.join(objdir, os.path.splitext(src)[0] + ".o")
        objs.append(obj)
        if force or _stale(obj, [path] + headers):
            cmd = [nvcc] + NVCC_FLAGS + ["-Xcompiler", "-ffp-contract=off"] \
                + (["-Xptxas", "-v"] if verbose else []) + ["-c", path, "-o", obj]
            procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(out)
        if p.returncode:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    if force or procs or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-ldl"]
        subprocess.check_call(cmd)
    build_cli(force)
    build_module(force)
    return LIB


CLI = os.path.join(HERE, "Pink")


def build_cli(force=False):
    """The command line program (host C++ only) next to the library it drives."""
    host = os.path.join(HERE, "host")
    srcs = [os.path.join(host, "pink_cli.cpp"), os.path.join(host, "pink_files.hpp"),
            os.path.join(HERE, "..", "include", "pink_b200.h")]
    if force or _stale(CLI, srcs + [LIB]):
        cxx = os.environ.get("CXX", "g++")
        subprocess.check_call([cxx, "-O2", "-std=c++17", "-pthread", srcs[0], "-o", CLI, "-L" + HERE, "-lpink_b200",
                               "-Wl,-rpath,$ORIGIN"])
    return CLI


def module_path():
    import sysconfig
    return os.path.join(HERE, "_pink" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_module(force=False):
    """The compiled Python module `_pink` (pybind11) next to the library it binds."""
    import sysconfig
    import pybind11
    src = os.path.join(HERE, "host", "pink_module.cpp")
    out = module_path()
    if force or _stale(out, [src, os.path.join(HERE, "..", "include", "pink_b200.h"), LIB]):
        cxx = os.environ.get("CXX", "g++")
        subprocess.check_call([cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
                               "-I" + sysconfig.get_paths()["include"], "-I" + pybind11.get_include(), src, "-o", out,
                               "-L" + HERE, "-lpink_b200", "-Wl,-rpath,$ORIGIN"])
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
