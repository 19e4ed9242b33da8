"""Builds tscale2_b200/libts2b200.so from csrc/*.cu with nvcc for sm_100a (in-tree,
so that the library travels with the source tree)."""
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libts2b200.so")
OBJ = os.path.join(HERE, "build")


def _nccl_paths():
    import importlib.util
    spec = importlib.util.find_spec("nvidia.nccl")
    if spec and spec.submodule_search_locations:
        base = list(spec.submodule_search_locations)[0]
        inc, lib = os.path.join(base, "include"), os.path.join(base, "lib")
        if os.path.exists(os.path.join(inc, "nccl.h")):
            return inc, lib
    return "/usr/include", "/usr/lib/x86_64-linux-gnu"


def build(verbose=False, force=False):
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    hdrs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    newest = max(os.path.getmtime(f) for f in srcs + hdrs)
    os.makedirs(OBJ, exist_ok=True)
    nccl_inc, nccl_lib = _nccl_paths()
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
             "-I" + nccl_inc, "--expt-relaxed-constexpr"]
    if verbose:
        flags += ["-Xptxas", "-v"]
    objs, procs = [], []
    for s in srcs:
        o = os.path.join(OBJ, os.path.basename(s) + ".o")
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < newest:
            procs.append((s, subprocess.Popen([nvcc, *flags, "-c", s, "-o", o], stdout=subprocess.PIPE,
                                              stderr=subprocess.STDOUT, text=True)))
    failed = False
    for s, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            print(out)
        if p.returncode:
            print(f"nvcc failed on {s}", file=sys.stderr)
            failed = True
    if failed:
        raise RuntimeError("build failed")
    if procs or not os.path.exists(OUT):
        # libnccl.so.2 is resolved at run time from the python environment (torch loads it first) or the system
        cmd = [nvcc, "-shared", "-o", OUT, *objs, "-lcudart", "-L" + nccl_lib, "-l:libnccl.so.2",
               "-Xlinker", "-rpath," + nccl_lib, "-Xlinker", "-rpath,/usr/lib/x86_64-linux-gnu"]
        subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
