"""Builds libgpt2_linear.so (the C-ABI library) for sm_100a with nvcc, in-tree.

    python gpt2.cu_b200/build.py [--force] [--verbose]

The library is written next to this file (gpt2.cu_b200/lib/libgpt2_linear.so). nvcc
cross-compiles, so this works on a machine without a GPU.
"""
import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIBDIR, "libgpt2_linear.so")
SOURCES = ["linear_tcgen05.cu", "linear_tcgen05_pair.cu", "linear_simt.cu", "api.cu", "megakernel.cu", "step_schedule.cu", "noalloc.cu", "layers.cu", "attention_gemm.cu", "attention_flash.cu", "attention_api.cu", "model.cu"]
HEADERS = ["linear_internal.h", "ptx_sm100.cuh", "kernel_common.cuh", "epilogue.cuh", "attention_flash.cuh", "layers.h", "step_rowops.cuh", "schedule_internal.h", "model_internal.h",
           os.path.join(ROOT, "include", "gpt2_model.h"), os.path.join(ROOT, "include", "gpt2_linear.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
    "-I", os.path.join(ROOT, "include"), "-I", CSRC,
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _fingerprint():
    h = hashlib.sha256()
    for name in SOURCES + HEADERS:
        path = name if os.path.isabs(name) else os.path.join(CSRC, name)
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force=False, verbose=False):
    """Compiles the library if the sources changed since the last build. Returns its path."""
    os.makedirs(LIBDIR, exist_ok=True)
    stamp = os.path.join(LIBDIR, "build.stamp")
    fp = _fingerprint()
    if not force and os.path.exists(LIB) and os.path.exists(stamp):
        with open(stamp) as f:
            if f.read().strip() == fp:
                return LIB
    cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else [])
    cmd += [os.path.join(CSRC, s) for s in SOURCES] + ["-o", LIB]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libgpt2_linear.so")
    with open(stamp, "w") as f:
        f.write(fp)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
