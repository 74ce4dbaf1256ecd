"""GPU tests of the lm_head with softmax and cross-entropy folded in (gpt2_linear_forward_xent and the
xent_* fields of gpt2_linear_opts): the loss and the two gradients against float64 torch on the same seeded
inputs, and against the unfused calls (gpt2_linear_forward, an explicit dlogits tensor, then
gpt2_linear_backward_input / _backward_weight).

Tolerances are the parity thresholds of the GEMMs themselves (max |err| / max |truth|: 1e-2 in TF32 mode,
2e-3 in 3xTF32 mode); the per-row losses and log-sum-exps are fp32 reductions of the GEMM's output and are held
to 2e-3 / 2e-5 absolute."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = {0: 1e-2, 1: 2e-3}
TOL_LOSS = {0: 2e-3, 1: 2e-5}


def rel(a, b):
    return ((a.double() - b.double()).abs().max() / b.double().abs().max()).item()


# (M, K, N padded, V true): two tile rows and ragged rows; vocabulary padding; a wide weight gradient
# (N >= 8192 and N >= 8 K: computed from a transposed activation copy)
SHAPES = [(512, 256, 1024, 1000), (300, 192, 640, 611), (256, 128, 8192, 8100)]


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("shape", SHAPES)
def test_fused_cross_entropy_against_float64(gpu, mode, shape):
    M, K, N, V = shape
    gen = torch.Generator(device="cuda").manual_seed(7 + M)
    x = torch.randn((M, K), device="cuda", generator=gen)
    w = torch.randn((K, N), device="cuda", generator=gen) * 0.1
    w[:, V:] = 0  # pad columns of the embedding matrix are kept at zero
    tgt = torch.randint(0, V, (M,), dtype=torch.int32, device="cuda", generator=gen)
    o = gpu.make_opts(mode=mode)
    logits = torch.full((M, N), float("nan"), device="cuda")
    losses = torch.full((M,), float("nan"), device="cuda")
    lse = torch.full((M,), float("nan"), device="cuda")
    gpu.check("forward_xent", gpu.forward_xent(logits, losses, lse, x, w, tgt, 1, M, K, N, V, o))
    torch.cuda.synchronize()
    st, rec = gpu.last_status()
    assert st == 0, rec
    # ---- truth in float64
    xd = x.double().requires_grad_(True)
    wd = w.double().requires_grad_(True)
    z = xd @ wd
    loss64 = torch.nn.functional.cross_entropy(z[:, :V], tgt.long(), reduction="none")
    loss64.mean().backward()
    assert rel(logits, z.detach()) <= TOL[mode]
    assert (losses.double() - loss64.detach()).abs().max().item() <= TOL_LOSS[mode] * max(1.0, loss64.max().item())
    lse64 = torch.logsumexp(z.detach()[:, :V], dim=1) / np.log(2.0)
    assert (lse.double() - lse64).abs().max().item() <= TOL_LOSS[mode] * 10
    # ---- unfused: the same GEMM without the statistics gives the same logits bit for bit (unsplit, as the call with
    # statistics always is: left to itself the plain call may split a short reduction, which rounds differently)
    plain = torch.empty((M, N), device="cuda")
    gpu.check("forward", gpu.forward(plain, x, w, None, 1, M, K, N, gpu.make_opts(mode=mode, split_k=1)))
    torch.cuda.synchronize()
    assert torch.equal(plain, logits)
    # ---- gradients from the stored logits
    ox = gpu.make_opts(mode=mode, xent_lse=lse, xent_targets=tgt, xent_vocab=V, xent_scale=1.0 / M)
    dx = torch.full((M, K), float("nan"), device="cuda")
    dw = torch.full((K, N), float("nan"), device="cuda")
    gpu.check("backward_input", gpu.backward_input(dx, logits, w, 1, M, K, N, ox))
    gpu.check("backward_weight", gpu.backward_weight(dw, None, logits, x, 1, M, K, N, ox))
    torch.cuda.synchronize()
    st, rec = gpu.last_status()
    assert st == 0, rec
    assert torch.equal(plain, logits)  # the logits tensor itself is left alone
    assert rel(dx, xd.grad) <= TOL[mode], rel(dx, xd.grad)
    assert rel(dw, wd.grad) <= TOL[mode], rel(dw, wd.grad)
    assert torch.all(dw[:, V:] == 0)  # no gradient reaches the pad columns
    # ---- and against the unfused backward calls on an explicit dlogits tensor
    p = torch.softmax(logits[:, :V].double(), dim=1)
    dl = torch.zeros((M, N), dtype=torch.float64, device="cuda")
    dl[:, :V] = p
    dl[torch.arange(M), tgt.long()] -= 1.0
    dl = (dl / M).float()
    dx2 = torch.empty((M, K), device="cuda")
    dw2 = torch.empty((K, N), device="cuda")
    gpu.check("backward_input", gpu.backward_input(dx2, dl, w, 1, M, K, N, o))
    gpu.check("backward_weight", gpu.backward_weight(dw2, None, dl, x, 1, M, K, N, o))
    torch.cuda.synchronize()
    assert rel(dx, dx2) <= (1e-4 if mode == 1 else TOL[mode])
    assert rel(dw, dw2) <= (1e-4 if mode == 1 else TOL[mode])


def test_fused_cross_entropy_argument_checks(gpu):
    M, K, N, V = 128, 64, 256, 250
    x = torch.zeros((M, K), device="cuda")
    w = torch.zeros((K, N), device="cuda")
    t = torch.zeros((M,), dtype=torch.int32, device="cuda")
    lg = torch.zeros((M, N), device="cuda")
    ls = torch.zeros((M,), device="cuda")
    assert gpu.forward_xent(lg, ls, ls, x, w, t, 1, M, K, N, N + 1) == gpu.ERR_BAD_ARG     # V > N
    assert gpu.forward_xent(lg, None, ls, x, w, t, 1, M, K, N, V) == gpu.ERR_BAD_ARG
    assert gpu.forward_xent(lg, ls, ls, x, w, t, 1, M, K, N, V, gpu.make_opts(force_simt=1)) == gpu.ERR_BAD_ARG
    ox = gpu.make_opts(xent_lse=ls, xent_targets=None, xent_vocab=V, xent_scale=1.0)
    assert gpu.backward_input(x, lg, w, 1, M, K, N, ox) == gpu.ERR_BAD_ARG                # no targets
    ox = gpu.make_opts(xent_lse=ls, xent_targets=t, xent_vocab=V, xent_scale=1.0)
    assert gpu.forward(lg, x, w, None, 1, M, K, N, ox) == gpu.ERR_BAD_ARG                 # forward has its own entry


def test_model_with_fused_cross_entropy_equals_the_separate_kernel(gpu, monkeypatch):
    """One forward + backward of a two-layer model at GPT-2 small's width (3xTF32): the three ways the loss
    can run (GPT2_XENT = fused | stats | separate: gradient inside the backward GEMMs; statistics in the lm_head
    epilogue + one elementwise pass; the stand-alone softmax / cross-entropy kernel) give the same loss (1e-6)
    and the same gradients (1e-5 of each tensor's largest entry)."""
    import os, sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import gpt2_ref
    n_layer, n_head, n_embd, vocab, padded, block, B, T = 2, 12, 768, 1000, 1024, 128, 2, 128
    params = gpt2_ref.to_flat(gpt2_ref.init_params(vocab, block, n_layer, n_head, n_embd), n_layer, padded)
    rng = np.random.default_rng(9)
    tok = torch.from_numpy(rng.integers(0, vocab, B * T).astype(np.int32)).cuda()
    tgt = torch.from_numpy(rng.integers(0, vocab, B * T).astype(np.int32)).cuda()
    res = {}
    for kind in ("fused", "stats", "separate"):
        monkeypatch.setenv("GPT2_XENT", kind)
        m = gpu.Model(vocab, padded, n_layer, n_head, n_embd, block, B, T, mode=1)
        m.set_params(params)
        assert m.forward(tok, tgt) == 0
        loss = m.mean_loss()
        assert m.backward() == 0
        torch.cuda.synchronize()
        st, rec = gpu.last_status()
        assert st == 0, rec
        g = np.empty_like(params)
        m.get_grads(g)
        bounds = m.offsets() + [m.num_params]
        res[kind] = (loss, g)
        m.close()
    monkeypatch.delenv("GPT2_XENT")
    for kind in ("fused", "stats"):
        assert abs(res[kind][0] - res["separate"][0]) <= 1e-6
        a, b = res[kind][1], res["separate"][1]
        assert np.isfinite(a).all()
        for i in range(len(bounds) - 1):
            x, y = a[bounds[i]:bounds[i + 1]], b[bounds[i]:bounds[i + 1]]
            assert np.abs(x - y).max() <= 1e-5 * max(np.abs(y).max(), 1e-12), (kind, i, np.abs(x - y).max(), np.abs(y).max())
