"""The mlp.h compatibility header: a program written against the reference's linear-layer names
compiles against it and links with the library (CPU check), and produces correct results (GPU check)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "compat_mlp_check.cu")
LIBDIR = os.path.join(ROOT, "gpt2.cu_b200", "lib")


def build(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    exe = str(tmp_path / "compat_mlp_check")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O1",
           "-I", os.path.join(ROOT, "include", "compat"), "-I", os.path.join(ROOT, "include"),
           SRC, "-o", exe, "-L", LIBDIR, "-lgpt2_linear", f"-Xlinker=-rpath={LIBDIR}", "-lcuda"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    return exe


def test_reference_style_call_sites_compile_and_link(built, tmp_path):
    assert os.path.exists(build(tmp_path))


@pytest.mark.gpu
def test_reference_style_call_sites_give_correct_results(gpu, tmp_path):
    exe = build(tmp_path)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "compat ok" in r.stdout, r.stdout + r.stderr
