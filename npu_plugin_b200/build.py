"""Builds npu_plugin_b200/csrc/libb200const.so with nvcc for sm_100a (cross-compiles without a GPU)."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
SOURCES = ["api.cu", "plan.cu", "fold_kernels.cu", "rowquant_kernels.cu", "tile_kernels.cu", "dequant_kernels.cu", "sparsity_kernels.cu", "codec_kernels.cu", "synth_kernels.cu",
           "infer.cpp"]
HEADERS = ["ctype.h", "view.h", "runtime.h", "plan.h", "codec.h", os.path.join("..", "..", "include", "b200const.h")]
LIB = os.path.join(CSRC, "libb200const.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


def stale(lib=LIB):
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    return any(os.path.getmtime(os.path.join(CSRC, f)) > t for f in SOURCES + HEADERS)


def build(force=False, verbose=False, extra=(), out=LIB):
    """nvcc -gencode arch=compute_100a,code=sm_100a ... -shared -> libb200const.so"""
    if not force and not stale(out):
        return out
    cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
           "-ccbin", "/usr/bin/g++", "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall", "-Xcompiler", "-ffp-contract=off",
           "--fmad=false", "-cudart", "shared", "-o", out]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += list(extra)
    cmd += [os.path.join(CSRC, f) for f in SOURCES]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("nvcc failed")
    if verbose:
        sys.stderr.write(r.stderr)
    return out


if __name__ == "__main__":
    build(force=True, verbose="-v" in sys.argv)
    print(LIB)
