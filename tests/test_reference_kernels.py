"""GPU tests against the reference's OWN kernels (include/gpt2/layers/mlp.h compiled unmodified
into oracle/_ref/libref_mlp.so): they pin the CPU oracle's fp32 flavour, and they are the
parity target the specification names for the new kernels."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = {0: 1e-2, 1: 2e-3}


@pytest.fixture(scope="module")
def ref(orc):
    L = orc.ref_lib()
    assert L is not None, "oracle/_ref/libref_mlp.so missing: run `make -C oracle ref` where the reference tree is"
    return L


def seeded(M, K, N, seed):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn((M, K), device="cuda", generator=gen)
    w = torch.randn((K, N), device="cuda", generator=gen) * 0.02
    b = torch.randn((N,), device="cuda", generator=gen) * 0.02
    dy = torch.randn((M, N), device="cuda", generator=gen) * 0.01
    return x, w, b, dy


def ref_run(ref, x, w, b, dy):
    M, K = x.shape
    N = w.shape[1]
    y = torch.empty((M, N), device="cuda")
    dx = torch.empty((M, K), device="cuda")
    dw = torch.empty((K, N), device="cuda")
    db = torch.empty((N,), device="cuda")
    assert ref.ref_mlp_forward(y.data_ptr(), x.data_ptr(), w.data_ptr(), b.data_ptr() if b is not None else None,
                               1, M, K, N, None) == 0
    assert ref.ref_mlp_backward_input(dx.data_ptr(), dy.data_ptr(), w.data_ptr(), 1, M, K, N, None) == 0
    assert ref.ref_mlp_backward_weight(dw.data_ptr(), db.data_ptr(), dy.data_ptr(), x.data_ptr(), 1, M, K, N,
                                       None) == 0
    torch.cuda.synchronize()
    return y, dx, dw, db


@pytest.mark.parametrize("M,K,N", [(64, 48, 80), (100, 70, 33), (256, 768, 768)])
def test_oracle_f32_matches_reference_kernels(gpu, orc, ref, M, K, N):
    """Same order of operations (ascending k, FMA): the CPU restatement reproduces the
    reference's CUDA kernels to the last bits."""
    x, w, b, dy = seeded(M, K, N, seed=M)
    y, dx, dw, db = (t.cpu().numpy() for t in ref_run(ref, x, w, b, dy))
    xn, wn, bn, dyn = (t.cpu().numpy() for t in (x, w, b, dy))
    assert orc.max_rel_err(orc.forward(xn, wn, bn), y) <= 1e-6
    assert orc.max_rel_err(orc.backward_input(dyn, wn), dx) <= 1e-6
    gw, gb = orc.backward_weight(dyn, xn)
    assert orc.max_rel_err(gw, dw) <= 1e-6
    assert orc.max_rel_err(gb, db) <= 1e-6


def rel(a, b):
    return ((a - b).abs().max() / b.abs().max()).item()


# GPT-2 small layer shapes at M = B*T = 8*1024 (lm_head with the padded vocabulary)
FULL = [("qkv", 768, 2304), ("attn_proj", 768, 768), ("fc", 768, 3072), ("fc_proj", 3072, 768),
        ("lm_head", 768, 50304)]


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("name,K,N", FULL)
def test_new_kernels_match_reference_kernels_at_full_size(gpu, ref, name, K, N, mode):
    M = 8192
    x, w, b, dy = seeded(M, K, N, seed=K + N)
    if name == "lm_head":
        b = None
        w[:, 50257:] = 0  # padded vocabulary columns
    ry, rdx, rdw, rdb = ref_run(ref, x, w, b, dy)
    y = torch.empty_like(ry)
    dx = torch.empty_like(rdx)
    dw = torch.empty_like(rdw)
    db = torch.empty_like(rdb) if b is not None else None
    o = gpu.make_opts(mode=mode)
    gpu.check("forward", gpu.forward(y, x, w, b, 8, 1024, K, N, o))
    gpu.check("backward_input", gpu.backward_input(dx, dy, w, 8, 1024, K, N, o))
    gpu.check("backward_weight", gpu.backward_weight(dw, db, dy, x, 8, 1024, K, N, o))
    torch.cuda.synchronize()
    st, rec = gpu.last_status()
    assert st == 0, rec
    assert rel(y, ry) <= TOL[mode]
    assert rel(dx, rdx) <= TOL[mode]
    assert rel(dw, rdw) <= TOL[mode]
    if db is not None:
        assert rel(db, rdb) <= TOL[mode]
