"""Builds the native parts of megcc_b200 in-tree with nvcc for sm_100a.

    python -m megcc_b200.build            # libmegcc_b200.so (+ compile-side library)

The shared objects land next to this file so that they travel with the source tree.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libmegcc_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-Wno-deprecated-gpu-targets", "-O3", "-std=c++17",
    "-fmad=false", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-Xcompiler", "-Wall", "-Xptxas", "-v",
]


COMPILER_DIR = os.path.join(HERE, "compiler")
COMPILER_LIB = os.path.join(HERE, "libmegcc_b200_compiler.so")


def _sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC)
                  if f.endswith((".cu", ".cpp")))


def build_compiler(verbose=False, force=False):
    """The compile-side library (KernelGen CUDA pack, planner, tinynn writer): host C++ only."""
    srcs = sorted(os.path.join(COMPILER_DIR, f) for f in os.listdir(COMPILER_DIR)
                  if f.endswith(".cpp"))
    deps = srcs + [os.path.join(COMPILER_DIR, f) for f in os.listdir(COMPILER_DIR)
                   if f.endswith(".h")]
    deps += [os.path.join(CSRC, "tinynn_format.h"),
             os.path.join(os.path.dirname(HERE), "include", "megcc_b200_compiler.h")]
    if not force and not _stale(COMPILER_LIB, deps):
        return COMPILER_LIB
    # the distribution compiler: a g++ that links libstdc++ statically into a shared object
    # yields a library that crashes when loaded next to another C++ runtime
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else os.environ.get("CXX", "g++")
    cmd = [cxx, "-std=c++17", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall",
           "-o", COMPILER_LIB] + srcs
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or r.returncode:
        sys.stderr.write(r.stdout)
    if r.returncode:
        raise RuntimeError("building the compiler library failed")
    return COMPILER_LIB


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose=False, force=False):
    build_compiler(verbose, force)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    srcs = _sources()
    deps = srcs + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    deps += [os.path.join(os.path.dirname(HERE), "include", f)
             for f in os.listdir(os.path.join(os.path.dirname(HERE), "include"))]
    if not force and not _stale(LIB, deps):
        return LIB
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    procs = []
    objs = []
    for s in srcs:
        o = os.path.join(objdir, os.path.basename(s) + ".o")
        objs.append(o)
        if force or _stale(o, deps):
            cmd = [nvcc] + NVCC_FLAGS + ["-x", "cu", "-c", s, "-o", o]
            procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE,
                                              stderr=subprocess.STDOUT, text=True)))
    for s, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(out)
        if p.returncode:
            raise RuntimeError(f"nvcc failed on {s}")
    cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs + [
        "-lcudart", "-ldl"]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
