"""Builds libqtip_b200.so (the C-ABI library) in-tree with nvcc for sm_100a."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = ["tables.cu", "viterbi.cu", "ldlq.cu", "hadamard.cu", "epilogue_residual.cu", "epilogue_gateup.cu", "elementwise.cu", "decode.cu", "fp8.cu", "gemm_tc.cu",
           "trellis_tc.cu", "block_ldl.cu", "group.cu", "checkpoint.cpp"]
LIB = os.path.join(HERE, "libqtip_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
EXTRA = os.environ.get("QTIP_NVCC_FLAGS", "").split()
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "--expt-relaxed-constexpr", "-ccbin", "/usr/bin/g++"]


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(HERE, "csrc", f) for f in os.listdir(os.path.join(HERE, "csrc"))]
    deps.append(os.path.join(HERE, "..", "include", "qtip_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compile every CUDA source to one shared library. Objects go to build/ (git-ignored)."""
    if not force and not _stale():
        return LIB
    obj_dir = os.path.join(HERE, "..", "build", "obj")
    os.makedirs(obj_dir, exist_ok=True)
    procs = []
    for src in SOURCES:
        obj = os.path.join(obj_dir, os.path.splitext(src)[0] + ".o")
        cmd = [NVCC, *FLAGS, *EXTRA, "-c", os.path.join(HERE, "csrc", src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objs = []
    for src, obj, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(out)
        if p.returncode:
            raise RuntimeError("nvcc failed on %s" % src)
        objs.append(obj)
    subprocess.check_call([NVCC, "-shared", "-Wno-deprecated-gpu-targets", "-o", LIB, *objs, "-ccbin", "/usr/bin/g++"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
