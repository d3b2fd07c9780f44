"""Builds npu_plugin_b200/csrc/libb200const.so with nvcc for sm_100a (cross-compiles without a GPU).

Every source is compiled to its own object file (in parallel, only when it or a header changed) and the
objects are linked into the shared library."""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_obj")
SOURCES = ["api.cu", "plan.cu", "fold_kernels.cu", "rowquant_kernels.cu", "tile_kernels.cu", "dequant_kernels.cu",
           "sparsity_kernels.cu", "codec_kernels.cu", "synth_kernels.cu", "probe_kernels.cu", "exchange_kernels.cu",
           "infer.cpp"]
HEADERS = ["ctype.h", "view.h", "runtime.h", "plan.h", "codec.h", os.path.join("..", "..", "include", "b200const.h")]
LIB = os.path.join(CSRC, "libb200const.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-ccbin", "/usr/bin/g++",
         "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall", "-Xcompiler", "-ffp-contract=off", "--fmad=false"]


def _sources():
    return [f for f in SOURCES if os.path.exists(os.path.join(CSRC, f))]


def _headers_mtime():
    return max(os.path.getmtime(os.path.join(CSRC, h)) for h in HEADERS if os.path.exists(os.path.join(CSRC, h)))


def _obj(src):
    return os.path.join(OBJ, os.path.splitext(src)[0] + ".o")


def _stale_objects():
    ht = _headers_mtime()
    out = []
    for s in _sources():
        o = _obj(s)
        if not os.path.exists(o) or os.path.getmtime(o) < max(ht, os.path.getmtime(os.path.join(CSRC, s))):
            out.append(s)
    return out


def stale(lib=LIB):
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    return _headers_mtime() > t or any(os.path.getmtime(os.path.join(CSRC, f)) > t for f in _sources())


def _compile(src, verbose):
    cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", os.path.join(CSRC, src), "-o", _obj(src)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    return src, r


def build(force=False, verbose=False, out=LIB):
    """nvcc -gencode arch=compute_100a,code=sm_100a ... -> one object per source -> libb200const.so"""
    if not force and not stale(out):
        return out
    os.makedirs(OBJ, exist_ok=True)
    todo = _sources() if force else _stale_objects()
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(todo)))) as pool:
        results = list(pool.map(lambda s: _compile(s, verbose), todo))
    failed = False
    for src, r in results:
        if r.returncode != 0:
            sys.stderr.write(f"---- {src}\n{r.stdout}{r.stderr}")
            failed = True
        elif verbose:
            sys.stderr.write(f"---- {src}\n{r.stderr}")
    if failed:
        raise RuntimeError("nvcc failed")
    cmd = [NVCC, "-shared", "-cudart", "shared", "-ccbin", "/usr/bin/g++", "-o", out] + [_obj(s) for s in _sources()] + ["-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed")
    return out


if __name__ == "__main__":
    only = [a for a in sys.argv[1:] if not a.startswith("-")]
    if only:  # python -m npu_plugin_b200.build codec_kernels.cu -v : recompile the named sources, then link
        os.makedirs(OBJ, exist_ok=True)
        for s in only:
            _, r = _compile(s, "-v" in sys.argv)
            sys.stderr.write(r.stdout + r.stderr)
            if r.returncode != 0:
                sys.exit(1)
        build(force=False)
    else:
        build(force="-f" in sys.argv or "-v" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
