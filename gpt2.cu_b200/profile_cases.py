"""Reduced cases of the library's workloads for profiler captures (`ncu -k ... -c ...`): each case sets up
seeded operands, runs a few launches of one kernel family and exits. The measured numbers come from
bench.py; these cases exist so that a capture stays small (one kernel, a few launches, a few GB).

    python gpt2.cu_b200/profile_cases.py gemm --only qkv.fwd,qkv.wgrad --rows 8192 --steps 2 --warmup 3
    python gpt2.cu_b200/profile_cases.py gemm --only lm_head.fwd --rows 2048 --steps 1 --warmup 3
    python gpt2.cu_b200/profile_cases.py attention --batch 8 --reps 2 [--impl flash|gemm|simt]
    python gpt2.cu_b200/profile_cases.py train --shape 16x1024 --model small --steps 1 --warmup 2 [--path launches|step]

`--mode tf32|tf32x3` selects the arithmetic of the GEMMs. Every case prints one JSON line."""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("case", choices=["gemm", "attention", "train"])
    ap.add_argument("--mode", default="tf32", choices=["tf32", "tf32x3"])
    ap.add_argument("--only", default="", help="gemm: comma list like lm_head.fwd,qkv.wgrad (default: all 15)")
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=8, help="attention: sequences")
    ap.add_argument("--reps", type=int, default=2, help="attention: forward + backward repetitions")
    ap.add_argument("--impl", default="flash", choices=["flash", "gemm", "simt"])
    ap.add_argument("--shape", default="16x1024", help="train: BxT")
    ap.add_argument("--model", default="small", choices=["small", "medium", "large"])
    ap.add_argument("--path", default="launches", choices=["launches", "step"])
    args = ap.parse_args()

    import torch

    import __graft_entry__ as ge

    g = ge.load_package()
    wl = ge._load_module("gpt2cu_b200_workloads", os.path.join(ROOT, "gpt2.cu_b200", "workloads.py"))
    dp = ge._load_module("gpt2cu_b200_dp", os.path.join(ROOT, "gpt2.cu_b200", "dp.py"))
    torch.cuda.set_device(0)
    g.init(0)
    mode = g.MODE_TF32X3 if args.mode == "tf32x3" else g.MODE_TF32
    stream = torch.cuda.current_stream().cuda_stream
    if args.case == "gemm":
        only = set(args.only.split(",")) if args.only else None
        gs = wl.GemmSet(g, torch, args.rows, mode, 1234, only)
        for _ in range(args.warmup):
            gs.step(stream)
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(args.steps):
            gs.step(stream)
        e.record()
        torch.cuda.synchronize()
        ms = s.elapsed_time(e) / args.steps
        st, rec = g.last_status()
        out = {"case": "gemm", "only": sorted(only) if only else None, "rows": args.rows, "ms_per_step": ms,
               "tflops": gs.flops() / (ms * 1e-3) / 1e12, "status": st}
    elif args.case == "attention":
        out = {"case": "attention", "batch": args.batch, **wl.attention_case(g, torch, args.batch, args.reps, args.impl)}
    else:
        tb, tt = (int(v) for v in args.shape.lower().split("x"))

        def barrier():
            torch.cuda.synchronize()
        out = {"case": "train", **wl.measure_train(g, dp, torch, 0, 0, 1, barrier, None, mode, B=tb, T=tt, steps=args.steps,
                                                   warmup=args.warmup, model_name=args.model, path=args.path)}
    print(json.dumps(out), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
