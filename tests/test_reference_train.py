"""The reference's own training step (src/train.cu and its layer kernels, compiled unmodified behind
oracle/ref_train_shim.cu) against this build's model on the same parameters and tokens, at the shape
the reference ships (GPT-2 small, B=4, T=64): the loss of the first forward pass must agree.

Only the first loss is compared: the reference's Path-A cross-entropy backward covers ceil(M/256) rows only
(src/train.cu:402 of the reference) and its embedding backward indexes g_wte inconsistently
(src/layers/embedding.cu:93), so its later steps are not a training oracle."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_first_loss_matches_the_reference_forward(gpu, orc):
    L = orc.ref_train_lib()
    if L is None:
        pytest.skip("oracle/_ref/libref_train.so was not built (no reference tree at build time)")
    B, T, C, V, Vp, NL = 4, 64, 768, 50257, 50304, 12
    assert L.ref_train_create(B, T, 7) == 0
    n_ref = L.ref_train_num_params()
    m = gpu.Model(V, Vp, NL, 12, C, 1024, B, T, mode=gpu.MODE_TF32X3)
    assert n_ref == m.num_params - C * (Vp - V)
    rng = np.random.default_rng(11)
    flat = (rng.standard_normal(n_ref) * 0.02).astype(np.float32)   # the reference's order, wte [C][V]
    # layernorm weights 1: tensors 2 + 12 l, 8 + 12 l and the last but one, found through the padded offsets
    offs = m.offsets()
    shift = C * (Vp - V)
    for i in [2 + 12 * l + k for l in range(NL) for k in (0, 6)] + [2 + 12 * NL]:
        flat[offs[i] - shift: offs[i] - shift + C] = 1.0
    assert L.ref_train_set_params(flat.ctypes.data, n_ref) == 0
    padded = np.zeros(m.num_params, np.float32)
    padded[: C * Vp].reshape(C, Vp)[:, :V] = flat[: C * V].reshape(C, V)
    padded[C * Vp:] = flat[C * V:]
    m.set_params(padded)
    gen = torch.Generator(device="cuda").manual_seed(5)
    tok = torch.randint(0, V, (B * T,), dtype=torch.int32, device="cuda", generator=gen)
    tgt = torch.randint(0, V, (B * T,), dtype=torch.int32, device="cuda", generator=gen)
    ref_loss = L.ref_train_step(tok.data_ptr(), tgt.data_ptr())
    assert L.ref_train_sync() == 0
    assert m.forward(tok, tgt) == 0
    loss = m.mean_loss()
    assert np.isfinite(ref_loss) and np.isfinite(loss)
    assert abs(loss - ref_loss) <= 1e-3, (loss, ref_loss)   # reference builds with --use_fast_math
    m.close()
