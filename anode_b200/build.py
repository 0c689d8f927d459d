"""Builds libanode_routines_gpu.so in-tree with plain nvcc (sm_100a only).

The flags follow the reference's own recipe where they matter for numerics
(build.rs:47-48: -prec-div=true -prec-sqrt=true); the architecture list is replaced by the
single sm_100a target.  Usage: `python -m anode_b200.build [--force]`.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libanode_routines_gpu.so")
SOURCES = ["bn_fused.cu", "bn_legacy.cu", "bn_sync.cu", "bn_static.cu", "bn_hoststep.cu", "bn_segres.cu", "bn_infer.cu", "bn_resident.cu", "bn_resident_diag.cpp"]
HEADERS = ["bn_plan.h", "bn_device.cuh", "bn_fused.cuh", "bn_ring.cuh", "bn_resident_plan.h", "bn_host.h", "bn_sync.h",
           os.path.join("..", "..", "include", "anode_routines_gpu.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-prec-div=true", "-prec-sqrt=true",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fno-strict-aliasing",
]


def _sources():
    return [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _nccl_include():
    """nccl.h is only needed for types; the library itself is resolved at run time."""
    try:
        import nvidia.nccl as n
        inc = os.path.join(list(n.__path__)[0], "include")
        if os.path.exists(os.path.join(inc, "nccl.h")):
            return inc
    except Exception:
        pass
    return "/usr/include"


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in _sources()] + [os.path.join(CSRC, h) for h in HEADERS]
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def build_library(force=False, verbose=False):
    if not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    objs = []
    procs = []
    for s in _sources():
        obj = os.path.join(CSRC, os.path.splitext(s)[0] + ".o")
        cmd = [nvcc] + NVCC_FLAGS + ["-I", _nccl_include(), "-c", os.path.join(CSRC, s), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for s, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(out)
        if p.returncode:
            raise RuntimeError("nvcc failed on %s" % s)
    # the CUDA runtime is linked statically (nvcc's default); NCCL is looked up with dlopen
    # link to a temporary name and rename: a reader (or a copy of the tree) never sees a half-written library
    tmp = LIB + ".tmp%d" % os.getpid()
    link = [nvcc, "-shared", "-o", tmp] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-Xlinker", "-Bsymbolic", "-ldl"]
    subprocess.check_call(link)
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
