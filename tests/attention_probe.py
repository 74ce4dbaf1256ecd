"""Small driver for profiling the attention kernels on their own: one (or a few) forward + backward
passes of gpt2_attention_* on seeded inputs, B sequences of 12 heads, T = 1024.

    python tests/attention_probe.py [B] [repetitions] [flash|gemm|simt]
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import __graft_entry__ as ge  # noqa: E402


def main():
    B = int(sys.argv[1]) if len(sys.argv) > 1 else 4
    reps = int(sys.argv[2]) if len(sys.argv) > 2 else 1
    impl = sys.argv[3] if len(sys.argv) > 3 else "flash"
    g = ge.load_package()
    g.init(0)
    code = {"flash": g.ATT_FLASH, "gemm": g.ATT_GEMM, "simt": g.ATT_SIMT}[impl]
    NH, T = 12, 1024
    C = NH * 64
    gen = torch.Generator(device="cuda").manual_seed(1)
    qkv = torch.randn(B * T, 3 * C, device="cuda", generator=gen)
    dout = torch.randn(B * T, C, device="cuda", generator=gen) * 0.1
    out = torch.empty(B * T, C, device="cuda")
    lse = torch.empty(B, NH, T, device="cuda")
    row = torch.empty_like(lse)
    probs = torch.empty(B, NH, T, T, device="cuda") if impl == "gemm" else None
    tt = torch.empty(B, NH, T, T, device="cuda") if impl == "gemm" else None
    gq = torch.empty_like(qkv)
    for _ in range(reps):
        assert g.attention_forward(out, lse, probs, qkv, B, T, NH, C, code, 0) == 0
        assert g.attention_backward(gq, dout, qkv, out, lse, probs, row, tt, B, T, C, NH, code, 0) == 0
    torch.cuda.synchronize()
    print("status", g.lib.gpt2_attention_status(), "finite", bool(torch.isfinite(gq).all()))


if __name__ == "__main__":
    main()
