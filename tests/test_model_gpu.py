"""GPU tests of the training step built around the GEMM path (include/gpt2_model.h): losses and
gradients against what the reference's PyTorch model (scripts/llm.py) produced for the same seeded
parameters and tokens — the fixtures written by tests/golden/make_golden_train.py."""
import numpy as np
import pytest
import torch

import os, sys
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import gpt2_ref  # noqa: E402
from conftest import golden

pytestmark = pytest.mark.gpu


def build(gpu, z, mode):
    n_layer, n_head, n_embd, vocab, padded, block, B, T, steps = (int(v) for v in z["meta"])
    params = gpt2_ref.to_flat(gpt2_ref.init_params(vocab, block, n_layer, n_head, n_embd), n_layer, padded)
    cs = z["init_checksum"]
    assert abs(float(np.sum(params.astype(np.float64))) - cs[0]) <= 1e-6 * max(1.0, abs(cs[0]))
    assert abs(float(np.sum(np.abs(params).astype(np.float64))) - cs[1]) <= 1e-9 * cs[1]
    m = gpu.Model(vocab, padded, n_layer, n_head, n_embd, block, B, T, mode=mode)
    assert m.num_params == params.size
    m.set_params(params)
    tok = torch.from_numpy(z["tokens"].reshape(-1)).cuda()
    tgt = torch.from_numpy(z["targets"].reshape(-1)).cuda()
    return m, params, tok, tgt, steps


def train(m, tok, tgt, steps, hyper):
    lr, b1, b2, eps, wd = (float(v) for v in hyper)
    losses = []
    for t in range(1, steps + 1):
        assert m.forward(tok, tgt) == 0
        losses.append(m.mean_loss())
        assert m.backward() == 0
        assert m.update(lr, b1, b2, eps, wd, t) == 0
    torch.cuda.synchronize()
    return np.array(losses, np.float64)


@pytest.mark.parametrize("mode", [1, 0])
def test_tiny_model_losses_and_first_gradient(gpu, mode):
    z = golden("llm_train_tiny.npz")
    m, params, tok, tgt, steps = build(gpu, z, mode)
    assert m.forward(tok, tgt) == 0
    loss0 = m.mean_loss()
    assert m.backward() == 0
    torch.cuda.synchronize()
    st, rec = gpu.last_status()
    assert st == 0, rec
    grads = np.empty_like(params)
    m.get_grads(grads)
    want = z["grad1"]
    tol_l, tol_g = {1: (1e-5, 2e-4), 0: (2e-3, 2e-2)}[mode]
    assert abs(loss0 - z["losses"][0]) <= tol_l
    # per tensor: max error relative to the tensor's largest gradient
    offs = m.offsets() + [m.num_params]
    for i in range(len(offs) - 1):
        a, b = grads[offs[i]:offs[i + 1]], want[offs[i]:offs[i + 1]]
        denom = np.abs(b).max()
        if denom == 0:
            assert np.abs(a).max() == 0, i
        else:
            assert np.abs(a - b).max() / denom <= tol_g, (i, np.abs(a - b).max() / denom)
    # the whole curve
    m.set_params(params)
    m2, _, _, _, _ = build(gpu, z, mode)
    losses = train(m2, tok, tgt, steps, z["hyper"])
    assert np.abs(losses - z["losses"]).max() <= {1: 1e-3, 0: 1e-2}[mode], losses - z["losses"]
    m.close()
    m2.close()


def test_gpt2_small_20_steps_loss_curve(gpu):
    """GPT-2 small (124M), B=4, T=64, AdamW lr 1e-4: the per-step loss must agree with the reference's
    PyTorch model within 1e-3 over 20 steps (3xTF32 GEMMs)."""
    z = golden("llm_train_124M.npz")
    m, params, tok, tgt, steps = build(gpu, z, 1)
    losses = train(m, tok, tgt, steps, z["hyper"])
    st, rec = gpu.last_status()
    assert st == 0, rec
    diff = np.abs(losses - z["losses"])
    assert diff.max() <= 1e-3, (losses, z["losses"])
    # pad columns of wte stay exactly zero through AdamW
    after = np.empty_like(params)
    m.get_params(after)
    C, Vp, V = 768, 50304, 50257
    assert np.all(after[: C * Vp].reshape(C, Vp)[:, V:] == 0)
    m.close()


def test_gpt2_small_tf32_mode_tracks_the_curve(gpu):
    z = golden("llm_train_124M.npz")
    m, params, tok, tgt, steps = build(gpu, z, 0)
    losses = train(m, tok, tgt, steps, z["hyper"])
    assert np.abs(losses - z["losses"]).max() <= 2e-2, losses - z["losses"]
    m.close()


def test_tensor_core_attention_matches_cuda_core_attention(gpu, monkeypatch):
    """T = 256 (two 128-row blocks per head: skipped tiles, clipped reductions) and T = 160 (ragged
    blocks): the batched-GEMM attention and the flash-style CUDA-core attention give the same loss
    and the same gradients."""
    for T in (256, 160):
        n_layer, n_head, n_embd, vocab, block, B = 2, 2, 128, 96, 256, 2
        params = gpt2_ref.to_flat(gpt2_ref.init_params(vocab, block, n_layer, n_head, n_embd), n_layer, vocab)
        rng = np.random.default_rng(T)
        tok = torch.from_numpy(rng.integers(0, vocab, B * T).astype(np.int32)).cuda()
        tgt = torch.from_numpy(rng.integers(0, vocab, B * T).astype(np.int32)).cuda()
        res = {}
        for kind in ("gemm", "simt"):
            monkeypatch.setenv("GPT2_ATTENTION", kind)
            m = gpu.Model(vocab, vocab, n_layer, n_head, n_embd, block, B, T, mode=1)
            m.set_params(params)
            assert m.forward(tok, tgt) == 0
            loss = m.mean_loss()
            assert m.backward() == 0
            torch.cuda.synchronize()
            st, rec = gpu.last_status()
            assert st == 0, rec
            g = np.empty_like(params)
            m.get_grads(g)
            res[kind] = (loss, g)
            m.close()
        monkeypatch.delenv("GPT2_ATTENTION")
        assert abs(res["gemm"][0] - res["simt"][0]) <= 1e-5, T
        a, b = res["gemm"][1], res["simt"][1]
        assert np.isfinite(a).all()
        assert np.abs(a - b).max() / np.abs(b).max() <= 1e-4, (T, np.abs(a - b).max() / np.abs(b).max())
