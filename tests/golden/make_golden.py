"""Generates the golden fixtures of the linear-layer GEMMs from the reference's own PyTorch model.

    python tests/golden/make_golden.py /path/to/reference

Imports scripts/llm.py of vnnm404/gpt2.cu (from the tree given on the command line), builds two tiny
GPT models with the reference's seeded init, runs one fp32 forward + backward on CPU with seeded
tokens, and records, for each of the five linear layers of the hot path (QKV, attention output
projection, MLP fc, MLP fc-proj of block 0, and the tied lm_head), what went in and what the
reference produced:

    x [M,K]   w [K,N] (the nn.Linear weight transposed to the reference's C layout)   b [N] or absent
    y [M,N] = the module's own output          dy [M,N] = the gradient autograd handed the module
    dx [M,K] = the module's own input gradient  dw [K,N], db [N] = its parameter gradients

The lm_head shares its weight with the embedding, so its weight gradient is taken from
torch.autograd.grad of the same F.linear call replayed on the recorded x and dy (the embedding's
contribution would otherwise be mixed in).

Only this script needs the reference tree; the tests read the .npz files it wrote.
"""
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def capture(ref_root, name, n_embd, n_head, vocab, B, T, seed):
    sys.path.insert(0, os.path.join(ref_root, "scripts"))
    import llm  # the reference's model file

    torch.manual_seed(seed)
    cfg = llm.GPTConfig(block_size=max(T, 16), vocab_size=vocab, n_layer=2, n_head=n_head, n_embd=n_embd)
    model = llm.GPT(cfg).float()
    # the reference initialises biases to zero; give them seeded values so the bias path is exercised
    g = torch.Generator().manual_seed(seed + 1)
    with torch.no_grad():
        for m in model.modules():
            if isinstance(m, torch.nn.Linear) and m.bias is not None:
                m.bias.copy_(torch.randn(m.bias.shape, generator=g) * 0.02)
    rng = np.random.default_rng(seed)
    idx = torch.from_numpy(rng.integers(0, vocab, size=(B, T), dtype=np.int64))
    tgt = torch.from_numpy(rng.integers(0, vocab, size=(B, T), dtype=np.int64))

    blk = model.transformer.h[0]
    layers = {
        "qkv": blk.attn.c_attn,
        "attn_proj": blk.attn.c_proj,
        "fc": blk.mlp.c_fc,
        "fc_proj": blk.mlp.c_proj,
        "lm_head": model.lm_head,
    }
    rec = {k: {} for k in layers}

    def fwd_hook(key):
        def h(mod, inp, out):
            rec[key]["x"] = inp[0].detach().clone()
            rec[key]["y"] = out.detach().clone()
        return h

    def bwd_hook(key):
        def h(mod, gin, gout):
            rec[key]["dy"] = gout[0].detach().clone()
            rec[key]["dx"] = gin[0].detach().clone()
        return h

    for k, m in layers.items():
        m.register_forward_hook(fwd_hook(k))
        m.register_full_backward_hook(bwd_hook(k))

    _, loss = model(idx, tgt)
    loss.backward()

    out = {}
    for k, m in layers.items():
        r = rec[k]
        K = m.in_features
        N = m.out_features
        x = r["x"].reshape(-1, K)
        dy = r["dy"].reshape(-1, N)
        out[f"{k}.x"] = x.numpy()
        out[f"{k}.w"] = m.weight.detach().t().contiguous().numpy()  # [K,N]
        out[f"{k}.y"] = r["y"].reshape(-1, N).numpy()
        out[f"{k}.dy"] = dy.numpy()
        out[f"{k}.dx"] = r["dx"].reshape(-1, K).numpy()
        if k == "lm_head":
            xr = x.clone().requires_grad_(True)
            wr = m.weight.detach().clone().requires_grad_(True)
            (dw,) = torch.autograd.grad(F.linear(xr, wr), wr, grad_outputs=dy)
            out[f"{k}.dw"] = dw.t().contiguous().numpy()
        else:
            out[f"{k}.dw"] = m.weight.grad.detach().t().contiguous().numpy()
            out[f"{k}.b"] = m.bias.detach().numpy()
            out[f"{k}.db"] = m.bias.grad.detach().numpy()
    out["meta"] = np.array([B, T, n_embd, n_head, vocab, seed], dtype=np.int64)
    out["loss"] = np.array([loss.item()], dtype=np.float64)
    path = os.path.join(HERE, name)
    np.savez_compressed(path, **{k: np.ascontiguousarray(v) for k, v in out.items()})
    print(name, "loss", loss.item(), "bytes", os.path.getsize(path))
    sys.path.pop(0)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    ref = sys.argv[1]
    # every dimension a multiple of 4: the TMA + tcgen05 path
    capture(ref, "llm_tiny_aligned.npz", n_embd=64, n_head=2, vocab=96, B=2, T=24, seed=11)
    # vocabulary 101 and width 36: ragged k-blocks, and an lm_head the TMA path cannot address
    capture(ref, "llm_tiny_ragged.npz", n_embd=36, n_head=2, vocab=101, B=3, T=7, seed=12)
