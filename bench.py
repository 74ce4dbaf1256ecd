"""Benchmark of the linear-layer GEMM path (GPT-2 small layer set, forward + backward_input +
backward_weight of QKV, attention projection, MLP fc, MLP fc-proj and the tied lm_head at
M = B*T = 8*1024 rows, fp32 in HBM, TF32 tensor-core math).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--mode tf32|tf32x3]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

A step is one pass over the 15 GEMMs on one batch of seeded synthetic operands
(X ~ N(0,1), W ~ N(0,0.02), dY ~ N(0,1e-2)). With N > 1 every rank runs the same set on its own
batch (weak scaling) and the weight/bias gradients are averaged with NCCL on a side stream under
the remaining GEMMs. Rank 0 prints ONE JSON line.

Keys beyond the usual ones:
  value      whole-job GEMM TFLOP/s (2*M*N*K per GEMM, 3xTF32 still counted once), operands
             resident in HBM, CUDA-event time, max over ranks.
  e2e        the same set through the host-buffer entry points of the C ABI (pinned host operands,
             H2D and D2H copies inside the timed region).
  roofline   the tcgen05 kernel alone: algorithmic flops / summed CUDA-event time of its launches in
             the timed region, against the measured dense tensor peak (MEASURED_PEAKS.json: bf16
             sustained figure halved, TF32 runs at half the bf16 rate on this part).
  cpu_baseline  the CPU restatement of the reference's GEMMs (oracle/) on the host cores, on a
             bounded row sample of the same set. A reported baseline, not the target.
`--impl reference` times that CPU restatement alone (the reference's path has no CPU
implementation of its own to run; its CUDA kernels, compiled unmodified into oracle/_ref, are timed
beside it on the same GPU when that library is present).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M_ROWS = 8192
BATCH, SEQ = 8, 1024
LAYERS = [("qkv", 768, 2304), ("attn_proj", 768, 768), ("fc", 768, 3072), ("fc_proj", 3072, 768),
          ("lm_head", 768, 50304)]
KINDS = ["fwd", "dgrad", "wgrad"]
L2_BYTES = 126 << 20


def step_flops(rows=M_ROWS):
    return sum(3 * 2.0 * rows * K * N for _, K, N in LAYERS)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_burst": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []  # (wall-clock time the sample was read, csv line)

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "25"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t_begin=None, t_end=None):
        """Summary of the samples read inside [t_begin, t_end] (all samples when not given)."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, ln in self.lines:
            if t_begin is not None and not (t_begin <= ts <= t_end + 0.05):
                continue
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                mhz.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for nm, val in zip(names, f[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


# ------------------------------------------------------------------------------------------
# CPU baseline (oracle port) and the reference arm
# ------------------------------------------------------------------------------------------
def cpu_pass(orc, rows, np):
    """One pass of the 15 GEMMs at `rows` rows with the CPU restatement; returns seconds."""
    rng = np.random.default_rng(7)
    total = 0.0
    for _, K, N in LAYERS:
        x = rng.standard_normal((rows, K), dtype=np.float32)
        w = (rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.02))
        dy = (rng.standard_normal((rows, N), dtype=np.float32) * np.float32(0.01))
        t0 = time.perf_counter()
        orc.forward(x, w, None)
        orc.backward_input(dy, w)
        orc.backward_weight(dy, x, want_bias=True)
        total += time.perf_counter() - t0
    return total


def cpu_baseline(rows=None):
    import numpy as np
    import __graft_entry__ as ge

    orc = ge.load_oracle()
    cores = os.cpu_count() or 1
    orc.set_threads(cores)
    if rows is None:
        # size the sample for roughly 12 s of CPU work: two probes give fixed cost and cost per row
        t_a, t_b = cpu_pass(orc, 8, np), cpu_pass(orc, 72, np)
        per_row = max((t_b - t_a) / 64.0, 1e-6)
        fixed = max(t_a - 8 * per_row, 0.0)
        rows = int(max(8, min(M_ROWS, (12.0 - fixed) / per_row)))
        rows = max(8, rows // 8 * 8)
    sec = cpu_pass(orc, rows, np)
    return {"value": step_flops(rows) / sec / 1e12, "unit": "TFLOP/s", "cores": orc.get_threads(), "kind": "port",
            "sample": f"the 15-GEMM set at {rows} of {M_ROWS} rows (all K, N), fp32 sequential-k FMA order, "
                      f"{sec:.1f} s", "rows": rows, "seconds": sec}


def reference_gpu_baseline(torch, steps=3):
    """The reference's own CUDA kernels (mlp.h, compiled unmodified) on this GPU, same set."""
    import __graft_entry__ as ge

    L = ge.load_oracle().ref_lib()
    if L is None or not torch.cuda.is_available():
        return None
    total_ms = 0.0
    per = {}
    for name, K, N in LAYERS:
        x = torch.randn((M_ROWS, K), device="cuda")
        w = torch.randn((K, N), device="cuda") * 0.02
        dy = torch.randn((M_ROWS, N), device="cuda") * 0.01
        y = torch.empty((M_ROWS, N), device="cuda")
        dx = torch.empty((M_ROWS, K), device="cuda")
        dw = torch.empty((K, N), device="cuda")
        db = torch.empty((N,), device="cuda")
        calls = [
            lambda: L.ref_mlp_forward(y.data_ptr(), x.data_ptr(), w.data_ptr(), None, BATCH, SEQ, K, N, None),
            lambda: L.ref_mlp_backward_input(dx.data_ptr(), dy.data_ptr(), w.data_ptr(), BATCH, SEQ, K, N, None),
            lambda: L.ref_mlp_backward_weight(dw.data_ptr(), db.data_ptr(), dy.data_ptr(), x.data_ptr(), BATCH,
                                              SEQ, K, N, None),
        ]
        for kind, fn in zip(KINDS, calls):
            fn()
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(steps):
                fn()
            e.record()
            torch.cuda.synchronize()
            ms = s.elapsed_time(e) / steps
            per[f"{name}.{kind}"] = round(ms, 3)
            total_ms += ms
        del x, w, dy, y, dx, dw, db
    return {"value": step_flops() / (total_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": total_ms,
            "what": "reference mlp.h kernels recompiled for sm_100a (fp32 CUDA cores), same GPU, same set",
            "per_gemm_ms": per}


def reference_train_baseline(torch, steps=10, warmup=2):
    """The reference's own training step (src/train.cu + its layer kernels, compiled unmodified) at the
    shape it ships, B=4, T=64, GPT-2 small, seeded weights, on this GPU. Its loop reads the loss back
    every step (tests/test_train.cu:283-301 of the reference), so that is inside the timing too."""
    import __graft_entry__ as ge

    L = ge.load_oracle().ref_train_lib()
    if L is None or not torch.cuda.is_available():
        return None
    B, T = 4, 64
    rc = L.ref_train_create(B, T, 1234)
    if rc != 0:
        return {"unavailable": f"ref_train_create returned {rc}"}
    gen = torch.Generator(device="cuda").manual_seed(100)
    tok = torch.randint(0, 50257, (B * T,), dtype=torch.int32, device="cuda", generator=gen)
    tgt = torch.randint(0, 50257, (B * T,), dtype=torch.int32, device="cuda", generator=gen)
    loss = None
    for _ in range(warmup):
        loss = L.ref_train_step(tok.data_ptr(), tgt.data_ptr())
    L.ref_train_sync()
    t0 = time.perf_counter()
    for _ in range(steps):
        loss = L.ref_train_step(tok.data_ptr(), tgt.data_ptr())
    L.ref_train_sync()
    sec = time.perf_counter() - t0
    return {"tokens_per_s": B * T * steps / sec, "ms_per_step": sec / steps * 1e3, "steps": steps, "B": B, "T": T,
            "loss_last": float(loss),
            "what": "reference src/train.cu step (forward, cross_entropy, backward, gpt2_update: separate kernel "
                    "launches, fp32 CUDA cores) recompiled for sm_100a, same GPU"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    import numpy as np  # noqa: F401

    base = cpu_baseline()
    rows = base["rows"]
    # K timed steps of the same bounded sample (W warm-ups), all host threads
    import __graft_entry__ as ge
    orc = ge.load_oracle()
    for _ in range(min(args.warmup, 1)):
        cpu_pass(orc, rows, np)
    times = [cpu_pass(orc, rows, np) for _ in range(max(1, min(args.steps, 3)))]
    sec = statistics.mean(times)
    value = step_flops(rows) / sec / 1e12
    line = {
        "impl": "reference", "metric": "gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": len(times), "warmup": min(args.warmup, 1), "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, rows=rows),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": base["cores"], "kind": "port",
                         "sample": base["sample"]},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    try:
        import torch
        ref_gpu = reference_gpu_baseline(torch)
        if ref_gpu:
            line["reference_gpu"] = ref_gpu
    except Exception as exc:  # the CPU number above stands on its own
        line["reference_gpu"] = {"unavailable": str(exc)[:200]}
    try:
        ref_train = reference_train_baseline(torch)
        if ref_train:
            line["reference_train"] = ref_train
    except Exception as exc:
        line["reference_train"] = {"unavailable": str(exc)[:200]}
    print(json.dumps(line), flush=True)
    return 0


def workload_config(args, rows=M_ROWS):
    return {"workload": "GPT-2 small linear-layer GEMM set (QKV, attn-proj, fc, fc-proj, lm_head; fwd+dgrad+wgrad)",
            "rows_per_gpu": rows, "B": BATCH, "T": SEQ, "layers": {n: [K, N] for n, K, N in LAYERS},
            "mode": args.mode, "parallelism": f"dp{args.gpus}",
            "l2": "operands of one step total > 7 GB per GPU, far beyond the 126 MB L2; no explicit flush"}


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    import __graft_entry__ as ge

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the GEMM path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"  # keep stdout to the one JSON line
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    g = ge.load_package()
    g.init(local_rank)
    dp = ge._load_module("gpt2cu_b200_dp", os.path.join(ROOT, "gpt2.cu_b200", "dp.py"))
    if args.only_train:
        def barrier0():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
        mode0 = g.MODE_TF32X3 if args.mode == "tf32x3" else g.MODE_TF32
        tb, tt = (int(v) for v in args.train_shape.lower().split("x"))
        train = measure_train(g, dp, torch, local_rank, rank, world, barrier0, dist if world > 1 else None, mode0,
                              B=tb, T=tt, steps=args.steps, warmup=args.warmup, model_name=args.train_model)
        if rank == 0:
            print(json.dumps({"partial": True, "train": train}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return 0
    exch = dp.GradientExchange()
    mode = g.MODE_TF32X3 if args.mode == "tf32x3" else g.MODE_TF32
    opts = g.make_opts(mode=mode)

    rows = args.rows
    seq = SEQ if rows % SEQ == 0 else rows
    batch = rows // seq
    only = set(args.only.split(",")) if args.only else None
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    bufs = []
    for name, K, N in LAYERS:
        if only and not any(o.startswith(name + ".") for o in only):
            continue
        d = {
            "x": torch.randn((rows, K), device="cuda", generator=gen),
            "w": torch.randn((K, N), device="cuda", generator=gen) * 0.02,
            "b": None if name == "lm_head" else torch.randn((N,), device="cuda", generator=gen) * 0.02,
            "dy": torch.randn((rows, N), device="cuda", generator=gen) * 0.01,
            "y": torch.empty((rows, N), device="cuda"),
            "dx": torch.empty((rows, K), device="cuda"),
            "dw": torch.empty((K, N), device="cuda"),
            "db": None if name == "lm_head" else torch.empty((N,), device="cuda"),
        }
        bufs.append((name, K, N, d))
    stream = torch.cuda.current_stream().cuda_stream

    ev_pairs = []

    def one_step(timed_events=None):
        for name, K, N, d in bufs:
            calls = (
                ("fwd", lambda: g.forward(d["y"], d["x"], d["w"], d["b"], batch, seq, K, N, opts, stream)),
                ("dgrad", lambda: g.backward_input(d["dx"], d["dy"], d["w"], batch, seq, K, N, opts, stream)),
                ("wgrad", lambda: g.backward_weight(d["dw"], d["db"], d["dy"], d["x"], batch, seq, K, N, opts,
                                                    stream)),
            )
            for kind, fn in calls:
                if only and f"{name}.{kind}" not in only:
                    continue
                if timed_events is not None:
                    s = torch.cuda.Event(enable_timing=True)
                    e = torch.cuda.Event(enable_timing=True)
                    s.record()
                    rc = fn()
                    e.record()
                    timed_events.append((s, e))
                else:
                    rc = fn()
                if rc != 0:
                    raise SystemExit(f"GEMM call failed with code {rc}")
            exch.exchange([d["dw"], d["db"]])  # this layer's gradients travel under the next GEMMs
        exch.finish()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # nvidia-smi needs a moment to start: launched before the warm-up
    for _ in range(args.warmup):
        one_step()
    barrier()
    launches0 = g.lib.gpt2_linear_launch_count()
    t_start = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    barrier()
    wall0 = time.time()
    t_start.record()
    for _ in range(args.steps):
        one_step(ev_pairs)
    t_end.record()
    barrier()
    wall1 = time.time()
    launches = g.lib.gpt2_linear_launch_count() - launches0
    clocks = sampler.stop(wall0, wall1) if rank == 0 else None
    elapsed_ms = t_start.elapsed_time(t_end)
    kernel_ms = sum(s.elapsed_time(e) for s, e in ev_pairs)
    st, rec = g.last_status()
    if st != 0:
        raise SystemExit(f"device status {rec}")
    if world > 1:
        tt = torch.tensor([elapsed_ms, kernel_ms], device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        elapsed_ms, kernel_ms = tt.tolist()
    ms_per_step = elapsed_ms / args.steps
    if only:
        flops_step = sum(2.0 * rows * K * N for n_, K, N in LAYERS for k_ in KINDS if f"{n_}.{k_}" in only)
    else:
        flops_step = step_flops(rows)
    value = flops_step * world / (ms_per_step * 1e-3) / 1e12
    if only or args.no_e2e or rows != M_ROWS:
        # reduced run (profiling aid): kernel-only numbers, no end-to-end / CPU legs
        if rank == 0:
            print(json.dumps({"partial": True, "only": sorted(only) if only else None, "rows": rows,
                              "value": value, "unit": "TFLOP/s", "ms_per_step": ms_per_step,
                              "kernel_ms_per_step": kernel_ms / args.steps, "gpu_launches": int(launches),
                              "clocks": clocks}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return 0

    # ---- end to end through the host-buffer entry points (rank-local, all ranks in parallel)
    e2e = measure_e2e(g, torch, opts, stream, world, barrier, dist if world > 1 else None,
                      steps=max(1, min(args.steps, 2)))

    # ---- the set as one persistent launch (rank 0 only: a single-GPU comparison)
    mega = None
    if rank == 0 and not args.no_train:
        try:
            mega = measure_megakernel(g, torch, mode)
        except Exception as exc:  # a reported extra, never the headline
            mega = {"unavailable": str(exc)[:200]}
    barrier()

    # ---- the GEMM path inside a whole training step (GPT-2 small, B=16 per GPU, T=1024)
    train = None if args.no_train else measure_train(g, dp, torch, local_rank, rank, world, barrier,
                                                      dist if world > 1 else None, mode)
    # ---- and at the shape the reference ships (B=4, T=64), where its own step can run beside it
    train_small = None if args.no_train else measure_train(g, dp, torch, local_rank, rank, world, barrier,
                                                            dist if world > 1 else None, mode, B=4, T=64,
                                                            steps=20, warmup=3)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0

    peaks = load_peaks()
    peak_tf32 = peaks["bf16_sustained"] / 2.0
    n_launch = len(ev_pairs)
    achieved = flops_step * args.steps / (kernel_ms * 1e-3) / 1e12 if kernel_ms > 0 else None
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": peak_tf32, "unit": "TFLOP/s",
        "frac": (achieved / peak_tf32) if achieved else None,
        "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
        "kernel": "gpt2_linear_tcgen05_kernel", "launches_timed": n_launch,
        "avg_launch_ms": kernel_ms / n_launch if n_launch else None,
        "flops_per_launch": flops_step / 15.0,
        "peak_source": f"MEASURED_PEAKS.json bf16 sustained {peaks['bf16_sustained']} TF/s / 2 (TF32 rate), of "
                       f"{peaks['source']}; burst figure would be {peaks['bf16_burst'] / 2.0}",
    }
    base = cpu_baseline() if world == 1 else None
    line = {
        "metric": "gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "tf32" if mode == g.MODE_TF32 else "3xtf32", "data": "synthetic",
        "config": workload_config(args), "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches),
        "roofline": roofline,
    }
    if base:
        line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
    if train:
        line["train"] = train
    if train_small is not None:
        line["train_small"] = train_small
    if mega is not None:
        line["megakernel"] = mega
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, averaged over the
# 15 launches of one step, from the ncu capture summarised under profiles/.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 485.5e6  # profiles/tcgen05_kernel_gemm_set_launch_list_and_traffic.md


MODELS = {"small": (768, 12, 12), "medium": (1024, 24, 16), "large": (1280, 36, 20)}  # width, layers, heads


def measure_train(g, dp, torch, local_rank, rank, world, barrier, dist, mode, B=16, T=1024, steps=5, warmup=2,
                  model_name="small"):
    """Tokens/s of whole training steps (forward, backward, gradient all-reduce over NCCL overlapped
    with the backward pass, AdamW) of GPT-2 small at B sequences of T tokens per GPU, random-init
    weights and uniform random tokens: the configuration BASELINE.json calls the megakernel step."""
    import numpy as np

    C, L, NH = MODELS[model_name]
    V, Vp = 50257, 50304
    model = g.Model(V, Vp, L, NH, C, 1024, B, T, mode=mode)
    rng = np.random.default_rng(42)  # same weights on every rank
    params = rng.standard_normal(model.num_params, dtype=np.float32) * np.float32(0.02)
    offs = model.offsets()
    params[: C * Vp].reshape(C, Vp)[:, V:] = 0
    for i in [2 + 12 * l + k for l in range(L) for k in (0, 6)] + [2 + 12 * L]:
        params[offs[i]: offs[i] + C] = 1.0  # layernorm weights
    model.set_params(params)
    gen = torch.Generator(device="cuda").manual_seed(100 + rank)
    tok = torch.randint(0, V, (B * T,), dtype=torch.int32, device="cuda", generator=gen)
    tgt = torch.randint(0, V, (B * T,), dtype=torch.int32, device="cuda", generator=gen)
    step = dp.DataParallelStep(model, torch.device("cuda", local_rank), use_graph=(world == 1))
    stream = torch.cuda.current_stream().cuda_stream
    hyper = (3e-4, 0.9, 0.95, 1e-8, 0.1)
    t = 0
    for _ in range(warmup):
        t += 1
        if step(tok, tgt, *hyper, t, stream) != 0:
            raise SystemExit("training step failed")
    barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        t += 1
        step(tok, tgt, *hyper, t, stream)
    e.record()
    barrier()
    ms = s.elapsed_time(e)
    loss = model.mean_loss()
    if dist is not None:
        tt = torch.tensor([ms], device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = tt.item()
    out = {"tokens_per_s": B * T * world * steps / (ms * 1e-3), "ms_per_step": ms / steps, "steps": steps,
           "config": f"GPT-2 {model_name} ({L} layers, {C} wide, vocabulary 50257 padded to 50304), B={B} per GPU, T={T}, "
                     f"AdamW lr 3e-4 betas 0.9/0.95 wd 0.1, fp32 master weights, {'3xTF32' if mode else 'TF32'} GEMMs, "
                     + ("attention as batched causal GEMMs on the linear-layer kernel" if (mode or T % 128) else
                        "fused causal attention on the tensor cores (no T x T tensors)")
                     + "; residual adds and GELU backward in GEMM epilogues", "loss_after": loss,
           "gradient_exchange": "none (1 GPU; forward + backward replayed from a CUDA graph)" if world == 1
           else "NCCL average, one bucket per block, overlapped"}
    model.close()
    return out


def measure_megakernel(g, torch, mode, steps=20, warmup=3):
    """The same 15 GEMMs as ONE persistent launch (gpt2_schedule_create + gpt2_megakernel_run): tile lists of
    all ops walked by 148 resident CTAs, outputs published on the dependency counters. The ops of the set
    are independent, so no counter is waited for; what shows is the cost of launch boundaries."""
    o = g.make_opts(mode=mode)
    gen = torch.Generator(device="cuda").manual_seed(11)
    ops, keep = [], []
    for name, K, N in LAYERS:
        x = torch.randn((M_ROWS, K), device="cuda", generator=gen)
        w = torch.randn((K, N), device="cuda", generator=gen) * 0.02
        b = None if name == "lm_head" else torch.randn((N,), device="cuda", generator=gen) * 0.02
        dy = torch.randn((M_ROWS, N), device="cuda", generator=gen) * 0.01
        y = torch.empty((M_ROWS, N), device="cuda")
        dx = torch.empty((M_ROWS, K), device="cuda")
        dw = torch.empty((K, N), device="cuda")
        db = None if name == "lm_head" else torch.empty((N,), device="cuda")
        ops += [g.make_op(g.OP_FORWARD, BATCH, SEQ, K, N, y, x, w, bias=b, opts=o),
                g.make_op(g.OP_BACKWARD_INPUT, BATCH, SEQ, K, N, dx, dy, w, opts=o),
                g.make_op(g.OP_BACKWARD_WEIGHT, BATCH, SEQ, K, N, dw, x, dy, out_bias=db, opts=o)]
        keep.append((x, w, b, dy, y, dx, dw, db))
    sched = g.Schedule(ops)
    for _ in range(warmup):
        if sched.run() != 0:
            raise SystemExit("megakernel run failed")
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        sched.run()
    e.record()
    torch.cuda.synchronize()
    st = sched.status()
    ms = s.elapsed_time(e) / steps
    sched.close()
    del keep
    if st != 0:
        return {"unavailable": f"device status {st}"}
    return {"value": step_flops() / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms, "steps": steps,
            "launches_per_step": 1,
            "what": "the 15 GEMMs of the set as one persistent launch (gpt2_megakernel_run); lm_head weight gradient "
                    "without the transposed-activation path of the per-call entry point"}


def measure_e2e(g, torch, opts, stream, world, barrier, dist, steps):
    """Same 15 GEMMs through gpt2_linear_*_host with pinned host operands: every step copies the
    operands host->device and the results device->host inside the timed region."""
    h2d = d2h = 0
    host = []
    for name, K, N in LAYERS:
        hx = torch.randn((M_ROWS, K)).pin_memory()
        hw = (torch.randn((K, N)) * 0.02).pin_memory()
        hb = None if name == "lm_head" else (torch.randn((N,)) * 0.02).pin_memory()
        hdy = (torch.randn((M_ROWS, N)) * 0.01).pin_memory()
        hy = torch.empty((M_ROWS, N)).pin_memory()
        hdx = torch.empty((M_ROWS, K)).pin_memory()
        hdw = torch.empty((K, N)).pin_memory()
        hdb = None if name == "lm_head" else torch.empty((N,)).pin_memory()
        host.append((name, K, N, hx, hw, hb, hdy, hy, hdx, hdw, hdb))
        nb = N if hb is not None else 0
        # bytes that actually cross PCIe: every distinct input once per step (x, w, b, dy: the pipelined
        # calls upload a host buffer once per synchronisation window), every output once
        h2d += 4 * (M_ROWS * K + K * N + nb + M_ROWS * N)
        d2h += 4 * (M_ROWS * N + M_ROWS * K + K * N + nb)

    def one():
        # the pipelined host-buffer calls: every call copies its own operands in and its results out;
        # the step ends with the synchronise that makes the 15 results valid in host memory
        for name, K, N, hx, hw, hb, hdy, hy, hdx, hdw, hdb in host:
            rc = g.forward_host_async(hy, hx, hw, hb, BATCH, SEQ, K, N, opts)
            rc |= g.backward_input_host_async(hdx, hdy, hw, BATCH, SEQ, K, N, opts)
            rc |= g.backward_weight_host_async(hdw, hdb, hdy, hx, BATCH, SEQ, K, N, opts)
            if rc != 0:
                raise SystemExit(f"host-buffer GEMM call failed with code {rc}")
        rc = g.host_synchronize()
        if rc != 0:
            raise SystemExit(f"host-buffer GEMM step failed with code {rc}")

    one()  # warm-up: staging buffers get allocated here
    barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        one()
    e.record()
    barrier()
    ms = s.elapsed_time(e)
    if dist is not None:
        tt = torch.tensor([ms], device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = tt.item()
    return {"value": step_flops() * world * steps / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": steps, "ms_per_step": ms / steps,
            "api": "gpt2_linear_{forward,backward_input,backward_weight}_host_async + gpt2_linear_host_synchronize "
                   "once per step (pinned host buffers; copies in, kernels and copies out on three streams; each input "
                   "buffer uploaded once per step, each result copied out)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", default="tf32", choices=["tf32", "tf32x3"])
    ap.add_argument("--rows", type=int, default=M_ROWS, help="rows per GPU (profiling aid; default is the workload)")
    ap.add_argument("--only", default="", help="comma list like lm_head.fwd,qkv.wgrad (profiling aid)")
    ap.add_argument("--no-e2e", dest="no_e2e", action="store_true", help="kernel-only run (profiling aid)")
    ap.add_argument("--no-train", dest="no_train", action="store_true", help="skip the whole-training-step leg")
    ap.add_argument("--train-shape", dest="train_shape", default="16x1024",
                    help="BxT of the --only-train leg (profiling aid; default 16x1024)")
    ap.add_argument("--train-model", dest="train_model", default="small", choices=sorted(MODELS),
                    help="model of the --only-train leg (profiling aid; default small = GPT-2 124M)")
    ap.add_argument("--only-train", dest="only_train", action="store_true",
                    help="run only the whole-training-step leg (profiling aid)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    args.warmup = max(args.warmup, 3)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
