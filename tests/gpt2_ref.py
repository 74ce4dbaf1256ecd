"""Test infrastructure: the seeded parameter initialisation of the reference's PyTorch model
(scripts/llm.py:126-143 of vnnm404/gpt2.cu) restated without importing it, and the conversion of a
set of named tensors to the reference's flat parameter order (src/gpt2.cu:48-198) with the padded
vocabulary this library uses.

llm.py draws every weight with torch.nn.init.normal_ from one torch.Generator seeded with 42, in the
order nn.Module.apply visits the modules (children first): wte, wpe, then per block c_attn, attention
c_proj, c_fc, MLP c_proj; std 0.02, residual projections 0.02 / sqrt(2 * n_layer); biases zero,
layernorm weights one; lm_head shares wte. tests/golden/make_golden_train.py asserts that this
restatement reproduces llm.py's tensors bit for bit."""
import math

import numpy as np
import torch


def init_params(vocab_size, block_size, n_layer, n_head, n_embd, seed=42):
    """Returns a dict of torch tensors named as in llm.py's state_dict (nn.Linear weights are [out, in])."""
    g = torch.Generator()
    g.manual_seed(seed)
    C = n_embd
    p = {}

    def normal(shape, std):
        t = torch.empty(shape, dtype=torch.float32)
        torch.nn.init.normal_(t, mean=0.0, std=std, generator=g)
        return t

    p["wte"] = normal((vocab_size, C), 0.02)
    p["wpe"] = normal((block_size, C), 0.02)
    rs = 0.02 / math.sqrt(2 * n_layer)
    for l in range(n_layer):
        p[f"h.{l}.ln_1.weight"] = torch.ones(C)
        p[f"h.{l}.ln_1.bias"] = torch.zeros(C)
        p[f"h.{l}.attn.c_attn.weight"] = normal((3 * C, C), 0.02)
        p[f"h.{l}.attn.c_attn.bias"] = torch.zeros(3 * C)
        p[f"h.{l}.attn.c_proj.weight"] = normal((C, C), rs)
        p[f"h.{l}.attn.c_proj.bias"] = torch.zeros(C)
        p[f"h.{l}.ln_2.weight"] = torch.ones(C)
        p[f"h.{l}.ln_2.bias"] = torch.zeros(C)
        p[f"h.{l}.mlp.c_fc.weight"] = normal((4 * C, C), 0.02)
        p[f"h.{l}.mlp.c_fc.bias"] = torch.zeros(4 * C)
        p[f"h.{l}.mlp.c_proj.weight"] = normal((C, 4 * C), rs)
        p[f"h.{l}.mlp.c_proj.bias"] = torch.zeros(C)
    p["ln_f.weight"] = torch.ones(C)
    p["ln_f.bias"] = torch.zeros(C)
    return p


def to_flat(p, n_layer, padded_vocab):
    """Named tensors -> one float32 numpy vector in the reference's parameter order: wte as [C][Vp]
    (transposed, pad columns zero), every nn.Linear weight transposed to [in][out]."""
    V, C = p["wte"].shape
    parts = []
    wte = torch.zeros((C, padded_vocab), dtype=torch.float32)
    wte[:, :V] = p["wte"].t()
    parts.append(wte)
    parts.append(p["wpe"])
    for l in range(n_layer):
        h = f"h.{l}."
        parts += [p[h + "ln_1.weight"], p[h + "ln_1.bias"], p[h + "attn.c_attn.weight"].t(), p[h + "attn.c_attn.bias"],
                  p[h + "attn.c_proj.weight"].t(), p[h + "attn.c_proj.bias"], p[h + "ln_2.weight"], p[h + "ln_2.bias"],
                  p[h + "mlp.c_fc.weight"].t(), p[h + "mlp.c_fc.bias"], p[h + "mlp.c_proj.weight"].t(),
                  p[h + "mlp.c_proj.bias"]]
    parts += [p["ln_f.weight"], p["ln_f.bias"]]
    return np.concatenate([t.contiguous().reshape(-1).numpy() for t in parts]).astype(np.float32)


def named_from_llm_model(model):
    """llm.py GPT instance -> the same naming as init_params (values or gradients via `attr`)."""
    sd = {}
    for k, v in model.named_parameters():
        k = k.replace("transformer.", "")
        if k == "lm_head.weight":
            continue
        sd[k.replace("wte.weight", "wte").replace("wpe.weight", "wpe")] = v
    return sd
