"""In-tree build of the CUDA library for sm_100a (nvcc cross-compiles without a GPU).

The shared object lands beside the sources (hipster_b200/libhipster_b200.so); it has a plain C ABI
(include/hipster_b200.h) and links the CUDA runtime statically, so it carries no torch dependency.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libhipster_b200.so")
OBJ = os.path.join(HERE, "csrc", "_obj")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--fmad=false", "-Xcompiler", "-fPIC,-ffp-contract=off,-fno-fast-math",
    "-Xptxas", "-v", "-I", os.path.join(HERE, "..", "include"),
]


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose=False, force=False):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libhipster_b200.so")
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(HERE, "..", "include", "hipster_b200.h"))
    objs = []
    env = dict(os.environ)
    env.pop("CXX", None); env.pop("CC", None)
    for src in sources():
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src[:-3] + ".o")
        objs.append(o)
        if force or _stale(o, [s] + headers):
            cmd = [nvcc] + NVCC_FLAGS + ["-c", s, "-o", o]
            r = subprocess.run(cmd, capture_output=True, text=True, env=env)
            if verbose or r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError("nvcc failed on " + src)
            with open(o + ".ptxas.txt", "w") as f:
                f.write(r.stderr)
    if force or _stale(LIB, objs):
        # NCCL is loaded with dlopen at run time (expert parallelism only): nothing but libdl is linked for it
        cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-cudart", "static", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True, env=env)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    build_driver(force)
    return LIB


DRIVER_SRC = os.path.join(HERE, "driver", "spec_driver.cpp")
DRIVER = os.path.join(HERE, "driver", "spec_driver")


def build_driver(force=False):
    """The C++ MTP driver: compiled against include/hipster_b200.h and linked with libhipster_b200.so only."""
    if not (force or _stale(DRIVER, [DRIVER_SRC, LIB, os.path.join(HERE, "..", "include", "hipster_b200.h")])):
        return DRIVER
    cxx = shutil.which("g++") or "g++"
    cmd = [cxx, "-O2", "-std=c++17", "-I", os.path.join(HERE, "..", "include"), DRIVER_SRC, "-o", DRIVER,
           "-L", HERE, "-lhipster_b200", "-Wl,-rpath,$ORIGIN/.."]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("building the C++ driver failed")
    return DRIVER


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
