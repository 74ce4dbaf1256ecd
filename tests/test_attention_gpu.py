"""GPU tests of the attention layer (include/gpt2_attention.h): the three implementations against a
float64 causal attention written out in torch on the CPU, forward and backward, on seeded inputs.

Tolerances (max |err| / max |truth| per tensor): TF32 implementations 2e-3 (3e-3 on the gradients, which
chain two TF32 contractions), 3xTF32 and fp32 implementations 2e-5."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def truth(qkv, dout, B, T, NH, C):
    """float64 reference: softmax(q k^T / 8, causal) v per head, and its gradient w.r.t. qkv"""
    x = torch.tensor(qkv, dtype=torch.float64, requires_grad=True)
    q, k, v = x.view(B, T, 3, NH, 64).permute(2, 0, 3, 1, 4)  # each [B, NH, T, 64]
    s = q @ k.transpose(-1, -2) / 8.0
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    s = s.masked_fill(~mask, float("-inf"))
    o = (torch.softmax(s, -1) @ v).permute(0, 2, 1, 3).reshape(B * T, C)
    o.backward(torch.tensor(dout, dtype=torch.float64))
    return o.detach().numpy(), x.grad.numpy()


def rel(a, b):
    return float(np.abs(a - b).max() / np.abs(b).max())


CASES = [
    # impl, mode, T, forward tol, backward tol
    ("flash", 0, 128, 2e-3, 3e-3), ("flash", 0, 256, 2e-3, 3e-3), ("flash", 0, 640, 2e-3, 3e-3), ("flash", 0, 1024, 2e-3, 3e-3),
    ("gemm", 0, 256, 2e-3, 3e-3), ("gemm", 1, 160, 2e-5, 2e-5), ("gemm", 1, 256, 2e-5, 2e-5),
    ("simt", 0, 200, 2e-5, 2e-5),
]


@pytest.mark.parametrize("impl,mode,T,tol_f,tol_b", CASES)
def test_attention_against_float64(gpu, impl, mode, T, tol_f, tol_b):
    B, NH = 2, 3
    C = NH * 64
    rng = np.random.default_rng(T)
    qkv = rng.standard_normal((B * T, 3 * C)).astype(np.float32)
    qkv[:, :C] *= 2.0  # sharper softmax: rows with a dominant key as well as flat ones
    dout = (rng.standard_normal((B * T, C)) * 0.1).astype(np.float32)
    want_o, want_g = truth(qkv, dout, B, T, NH, C)
    code = {"flash": gpu.ATT_FLASH, "gemm": gpu.ATT_GEMM, "simt": gpu.ATT_SIMT}[impl]
    assert gpu.lib.gpt2_attention_supported(code, T, C, NH) == 1
    d_qkv, d_dout = torch.from_numpy(qkv).cuda(), torch.from_numpy(dout).cuda()
    out = torch.full((B * T, C), float("nan"), device="cuda")
    lse = torch.zeros((B, NH, T), device="cuda")
    probs = torch.zeros((B, NH, T, T), device="cuda") if impl == "gemm" else None
    tt = torch.zeros((B, NH, T, T), device="cuda") if impl == "gemm" else None
    row = torch.zeros((B, NH, T), device="cuda")
    g = torch.full((B * T, 3 * C), float("nan"), device="cuda")
    assert gpu.attention_forward(out, lse, probs, d_qkv, B, T, NH, C, code, mode) == 0
    assert gpu.attention_backward(g, d_dout, d_qkv, out, lse, probs, row, tt, B, T, C, NH, code, mode) == 0
    torch.cuda.synchronize()
    assert gpu.lib.gpt2_attention_status() == 0
    got_o, got_g = out.cpu().numpy(), g.cpu().numpy()
    assert np.isfinite(got_o).all() and np.isfinite(got_g).all()
    assert rel(got_o, want_o) <= tol_f, rel(got_o, want_o)
    for name, sl in (("dq", slice(0, C)), ("dk", slice(C, 2 * C)), ("dv", slice(2 * C, 3 * C))):
        e = rel(got_g[:, sl], want_g[:, sl])
        assert e <= tol_b, (name, e)


def test_attention_shape_checks(gpu):
    assert gpu.lib.gpt2_attention_supported(gpu.ATT_FLASH, 192, 128, 2) == 0   # T % 128
    assert gpu.lib.gpt2_attention_supported(gpu.ATT_GEMM, 100, 128, 2) == 0    # T % 32
    assert gpu.lib.gpt2_attention_supported(gpu.ATT_SIMT, 100, 128, 2) == 1
    assert gpu.lib.gpt2_attention_supported(gpu.ATT_FLASH, 128, 100, 2) == 0   # head size 64 only
    x = torch.zeros((192, 384), device="cuda")
    o = torch.zeros((192, 128), device="cuda")
    l = torch.zeros((2, 192), device="cuda")
    assert gpu.attention_forward(o, l, None, x, 1, 192, 2, 128, gpu.ATT_FLASH) == gpu.ERR_BAD_ARG
    assert gpu.attention_forward(o, None, None, x, 1, 192, 2, 128, gpu.ATT_SIMT) == gpu.ERR_BAD_ARG


def test_flash_attention_properties_at_full_sequence_length(gpu):
    """Size-independent properties at T = 1024, 12 heads (the benchmark's sequence length): with V = 1 every
    output is 1 (the probabilities of a row sum to one); the output at position t depends on positions
    <= t only (bitwise, after perturbing everything from t = 512 on); and the gradient with respect to a
    position vanishes when only earlier positions receive a gradient."""
    B, NH, T = 2, 12, 1024
    C = NH * 64
    gen = torch.Generator(device="cuda").manual_seed(3)
    qkv = torch.randn(B * T, 3 * C, device="cuda", generator=gen)
    out = torch.empty(B * T, C, device="cuda")
    lse = torch.empty(B, NH, T, device="cuda")

    ones = qkv.clone()
    ones[:, 2 * C:] = 1.0
    assert gpu.attention_forward(out, lse, None, ones, B, T, NH, C, gpu.ATT_FLASH, 0) == 0
    torch.cuda.synchronize()
    assert float((out - 1.0).abs().max()) <= 1e-5

    assert gpu.attention_forward(out, lse, None, qkv, B, T, NH, C, gpu.ATT_FLASH, 0) == 0
    ref = out.clone()
    lse_ref = lse.clone()
    pert = qkv.clone().view(B, T, 3 * C)
    pert[:, 512:, :] = torch.randn(B, T - 512, 3 * C, device="cuda", generator=gen)
    out2 = torch.empty_like(out)
    lse2 = torch.empty_like(lse)
    assert gpu.attention_forward(out2, lse2, None, pert.view(B * T, 3 * C), B, T, NH, C, gpu.ATT_FLASH, 0) == 0
    torch.cuda.synchronize()
    assert torch.equal(out2.view(B, T, C)[:, :512], ref.view(B, T, C)[:, :512])
    assert not torch.equal(out2.view(B, T, C)[:, 512:], ref.view(B, T, C)[:, 512:])

    # a gradient that arrives only at positions < 512 leaves q, k, v of positions >= 512 without gradient
    dout = torch.zeros(B, T, C, device="cuda")
    dout[:, :512] = torch.randn(B, 512, C, device="cuda", generator=gen) * 0.1
    g = torch.full((B * T, 3 * C), float("nan"), device="cuda")
    row = torch.empty(B, NH, T, device="cuda")
    assert gpu.attention_backward(g, dout.view(B * T, C), qkv, ref, lse_ref, None, row, None, B, T, C, NH,
                                  gpu.ATT_FLASH, 0) == 0
    torch.cuda.synchronize()
    assert gpu.lib.gpt2_attention_status() == 0
    g3 = g.view(B, T, 3 * C)
    assert torch.isfinite(g3).all()
    assert float(g3[:, 512:].abs().max()) == 0.0
    assert float(g3[:, :512].abs().max()) > 0.0


def test_flash_attention_against_the_reference_kernels(gpu, orc):
    """The fused tensor-core attention against the reference's own attention_forward / attention_backward
    (src/layers/attention.cu:213-218, 366-371, compiled unmodified into oracle/_ref/libref_train.so) at the
    benchmarked sequence length: T = 1024, B = 1, 12 heads, seeded inputs. Same tolerances as against the
    float64 restatement (the reference computes in fp32 with --use_fast_math)."""
    L = orc.ref_train_lib()
    if L is None:
        pytest.skip("oracle/_ref/libref_train.so was not built (no reference tree at build time)")
    B, T, NH = 1, 1024, 12
    C = NH * 64
    gen = torch.Generator(device="cuda").manual_seed(21)
    qkv = torch.randn((B * T, 3 * C), device="cuda", generator=gen)
    qkv[:, :C] *= 2.0
    dout = torch.randn((B * T, C), device="cuda", generator=gen) * 0.1
    ref_out = torch.zeros((B * T, C), device="cuda")
    preatt = torch.zeros((B, NH, T, T), device="cuda")
    att = torch.zeros((B, NH, T, T), device="cuda")
    g_ref = torch.zeros((B * T, 3 * C), device="cuda")
    g_preatt, g_att = torch.zeros_like(preatt), torch.zeros_like(att)
    torch.cuda.synchronize()
    assert L.ref_attention_forward(ref_out.data_ptr(), preatt.data_ptr(), att.data_ptr(), qkv.data_ptr(), B, T, NH, C) == 0
    assert L.ref_attention_backward(g_ref.data_ptr(), g_preatt.data_ptr(), g_att.data_ptr(), dout.data_ptr(),
                                    qkv.data_ptr(), att.data_ptr(), B, T, C, NH) == 0
    out = torch.full((B * T, C), float("nan"), device="cuda")
    lse = torch.zeros((B, NH, T), device="cuda")
    row = torch.zeros((B, NH, T), device="cuda")
    g = torch.full((B * T, 3 * C), float("nan"), device="cuda")
    assert gpu.attention_forward(out, lse, None, qkv, B, T, NH, C, gpu.ATT_FLASH, 0) == 0
    assert gpu.attention_backward(g, dout, qkv, out, lse, None, row, None, B, T, C, NH, gpu.ATT_FLASH, 0) == 0
    torch.cuda.synchronize()
    assert gpu.lib.gpt2_attention_status() == 0
    assert torch.isfinite(out).all() and torch.isfinite(g).all()
    assert rel(out.cpu().numpy(), ref_out.cpu().numpy()) <= 2e-3
    for name, sl in (("dq", slice(0, C)), ("dk", slice(C, 2 * C)), ("dv", slice(2 * C, 3 * C))):
        assert rel(g[:, sl].cpu().numpy(), g_ref[:, sl].cpu().numpy()) <= 3e-3, name
