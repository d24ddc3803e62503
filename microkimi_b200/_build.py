"""Builds libmk_b200.so in-tree with nvcc for sm_100a (no other target).

    python -m microkimi_b200._build [--force] [--verbose]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libmk_b200.so")
SOURCES = ["mk_api.cu", "qgemv.cu", "weights.cu", "moe.cu", "mla.cu", "spine.cu", "gather.cu", "vq.cu", "kda.cu", "binfile.cu", "model.cu"]
HEADERS = [os.path.join(CSRC, "mk_common.cuh"), os.path.join(HERE, "..", "include", "mk_cuda.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    # IEEE arithmetic everywhere: no fast-math, denormals kept, exact divide/sqrt
    "-ftz=false", "-prec-div=true", "-prec-sqrt=true", "-fmad=true",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build_variant(out, defines):
    """Side build with extra -D flags (kernel studies); objects go next to `out`."""
    nvcc = _nvcc()
    srcs = [os.path.join(CSRC, s) for s in SOURCES]
    subprocess.check_call([nvcc] + NVCC_FLAGS + ["-D" + d for d in defines] + ["-shared", "-o", out] + srcs)
    return out


def build(force=False, verbose=False):
    nvcc = _nvcc()
    objs = []
    hdrs = HEADERS + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")]
    for s in SOURCES:
        src = os.path.join(CSRC, s)
        obj = os.path.join(CSRC, s.replace(".cu", ".o"))
        objs.append(obj)
        if force or _stale(obj, [src] + hdrs):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            if verbose:
                print(" ".join(cmd))
            subprocess.check_call(cmd)
    if force or _stale(OUT, objs):
        cmd = [nvcc, "-shared", "-o", OUT] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
