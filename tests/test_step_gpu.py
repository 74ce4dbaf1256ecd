"""GPU tests of the training step as a schedule of the persistent kernel (gpt2_schedule_instructions /
gpt2_megakernel_step, include/gpt2_model.h): the same losses, gradients and parameters as the step made of
separate launches, the loss curves of the reference's PyTorch model (fixtures of
tests/golden/make_golden_train.py), and a clean end when a dependency can never be satisfied."""
import os
import sys
import time

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import gpt2_ref  # noqa: E402
from conftest import golden
from test_model_gpu import build, _sampled_gradient_errors

pytestmark = pytest.mark.gpu

IN_KERNEL = [False, True]


def run_steps(gpu, m, tok, tgt, steps, hyper, in_kernel):
    lr, b1, b2, eps, wd = (float(v) for v in hyper)
    st = gpu.Step(m, tok, tgt, with_update=True, attention_in_kernel=in_kernel)
    losses = []
    for t in range(1, steps + 1):
        assert st.run(lr, b1, b2, eps, wd, t) == 0
        losses.append(m.mean_loss())
    torch.cuda.synchronize()
    assert st.status() == 0
    info = st.info()
    st.close()
    return np.array(losses, np.float64), info


@pytest.mark.parametrize("in_kernel", IN_KERNEL)
def test_step_gradients_equal_the_separate_launches(gpu, in_kernel):
    """Two layers at GPT-2 small's width, T = 256 (two 128-row blocks per sequence), 3xTF32: one step without
    the update leaves the same loss and the same gradients as gpt2_model_forward + gpt2_model_backward, up
    to the order of the floating-point sums (split reductions and column sums are combined in a different
    order: measured 1.4e-4 of a tensor's largest gradient after two blocks; bound 5e-4, loss 5e-6)."""
    os.environ["GPT2_ATTENTION"] = "flash"
    try:
        n_layer, n_head, n_embd, vocab, block, B, T = 2, 12, 768, 1024, 256, 2, 256
        params = gpt2_ref.to_flat(gpt2_ref.init_params(vocab, block, n_layer, n_head, n_embd), n_layer, vocab)
        rng = np.random.default_rng(3)
        tok = torch.from_numpy(rng.integers(0, vocab, B * T).astype(np.int32)).cuda()
        tgt = torch.from_numpy(rng.integers(0, vocab, B * T).astype(np.int32)).cuda()
        res = []
        for which in ("separate", "step"):
            m = gpu.Model(vocab, vocab, n_layer, n_head, n_embd, block, B, T, mode=1)
            m.set_params(params)
            if which == "separate":
                assert m.forward(tok, tgt) == 0 and m.backward() == 0
            else:
                st = gpu.Step(m, tok, tgt, with_update=False, attention_in_kernel=in_kernel)
                assert st.run() == 0
                torch.cuda.synchronize()
                assert st.status() == 0
                info = st.info()
                assert info["launches"] == (1 if in_kernel else 1 + 2 * n_layer + 3 * n_layer)
                st.close()
            loss = m.mean_loss()
            g = np.empty_like(params)
            m.get_grads(g)
            res.append((loss, g))
            m.close()
        assert gpu.lib.gpt2_attention_status() == 0
        assert abs(res[0][0] - res[1][0]) <= 5e-6, (res[0][0], res[1][0])
        a, b = res[1][1], res[0][1]
        assert np.isfinite(a).all()
        offs = gpu.Model(vocab, vocab, n_layer, n_head, n_embd, block, B, T, mode=1)
        bounds = offs.offsets() + [offs.num_params]
        offs.close()
        for i in range(len(bounds) - 1):
            x, y = a[bounds[i]:bounds[i + 1]], b[bounds[i]:bounds[i + 1]]
            assert np.abs(x - y).max() <= 5e-4 * max(np.abs(y).max(), 1e-12), (i, np.abs(x - y).max(), np.abs(y).max())
    finally:
        os.environ.pop("GPT2_ATTENTION", None)


def test_tiny_model_curve_through_the_step(gpu):
    """The tiny fixture (T = 16: CUDA-core attention between the persistent pieces, ragged 32-row problem):
    ten AdamW steps inside the step kernel against the reference's PyTorch model, 3xTF32."""
    z = golden("llm_train_tiny.npz")
    m, params, tok, tgt, steps = build(gpu, z, 1)
    losses, info = run_steps(gpu, m, tok, tgt, steps, z["hyper"], False)
    assert np.abs(losses - z["losses"]).max() <= 1e-3, losses - z["losses"]
    m.close()


def test_gpt2_small_20_steps_through_the_step(gpu):
    """GPT-2 small (124M), B=4, T=64, 20 AdamW steps, every step one call of gpt2_megakernel_step: per-step
    loss within 1e-3 of the reference's PyTorch model (3xTF32)."""
    z = golden("llm_train_124M.npz")
    m, params, tok, tgt, steps = build(gpu, z, 1)
    losses, info = run_steps(gpu, m, tok, tgt, steps, z["hyper"], False)
    assert np.abs(losses - z["losses"]).max() <= 1e-3, (losses, z["losses"])
    after = np.empty_like(params)
    m.get_params(after)
    C, Vp, V = 768, 50304, 50257
    assert np.all(after[: C * Vp].reshape(C, Vp)[:, V:] == 0)  # pad columns of wte stay zero through AdamW
    m.close()


@pytest.mark.parametrize("in_kernel", IN_KERNEL)
def test_sequence_length_1024_through_the_step(gpu, in_kernel):
    """T = 1024 (the benchmarked sequence length), TF32 GEMMs and fused attention, six AdamW steps with the
    benchmarked hyper-parameters: same bounds as the separate-launch step (5e-3 on the loss)."""
    z = golden("llm_train_t1024.npz")
    m, params, tok, tgt, steps = build(gpu, z, 0)
    losses, info = run_steps(gpu, m, tok, tgt, steps, z["hyper"], in_kernel)
    diff = np.abs(losses - z["losses"])
    print(f"step T=1024 in_kernel={in_kernel}: max loss diff {diff.max():.2e}, {info}")
    assert diff.max() <= 5e-3, (losses, z["losses"])
    m.close()


def test_step_with_unsatisfiable_dependency_ends_cleanly(gpu):
    """Host-side fault injection: one op of the first persistent piece is told to wait for more arrivals than
    its producer publishes. The step must end by itself, report the timeout, and the device must stay
    usable (a fresh step object on the same model runs)."""
    z = golden("llm_train_tiny.npz")
    m, params, tok, tgt, steps = build(gpu, z, 1)
    st = gpu.Step(m, tok, tgt, with_update=False)
    assert st.debug_set_expected(0, 1, 0, 1 << 30, 200) == 0  # piece 0, op 1 (layernorm), dependency 0
    t0 = time.time()
    assert st.run() == 0
    torch.cuda.synchronize()
    assert time.time() - t0 < 10.0
    assert st.status() == gpu.DEV_TIMEOUT
    st.close()
    assert gpu.last_status()[0] == gpu.DEV_TIMEOUT  # the host-visible flag; reading clears it
    st2 = gpu.Step(m, tok, tgt, with_update=False)
    assert st2.run() == 0
    torch.cuda.synchronize()
    assert st2.status() == 0
    assert abs(m.mean_loss() - z["losses"][0]) <= 1e-4
    st2.close()
    m.close()
