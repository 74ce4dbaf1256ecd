"""Seeded synthetic workloads of the linear-layer path, shared by bench.py (the measured lines) and
profile_cases.py (reduced cases for ncu captures): the GPT-2 small GEMM set, the training step made of
separate launches, the same step as a schedule of the persistent kernel, and the attention layer alone.

Everything here drives the C ABI through the ctypes binding with torch tensors as device memory; nothing
computes on the CPU."""
import os
import statistics
import subprocess
import threading
import time

M_ROWS = 8192
BATCH, SEQ = 8, 1024
# forward weights [K][N] of the five linear layers of GPT-2 small
LAYERS = [("qkv", 768, 2304), ("attn_proj", 768, 768), ("fc", 768, 3072), ("fc_proj", 3072, 768),
          ("lm_head", 768, 50304)]
KINDS = ["fwd", "dgrad", "wgrad"]
MODELS = {"small": (768, 12, 12), "medium": (1024, 24, 16), "large": (1280, 36, 20)}  # width, layers, heads
VOCAB, PADDED_VOCAB = 50257, 50304
TRAIN_HYPER = (3e-4, 0.9, 0.95, 1e-8, 0.1)  # lr, beta1, beta2, eps, weight decay


def step_flops(rows=M_ROWS):
    return sum(3 * 2.0 * rows * K * N for _, K, N in LAYERS)


def train_gemm_flops(model_name, tokens):
    """2*M*N*K over the linear-layer GEMMs (forward, input gradient, weight gradient) of one training step."""
    C, L, _ = MODELS[model_name]
    return 6.0 * tokens * (L * 12 * C * C + C * PADDED_VOCAB)


class ClockSampler:
    """nvidia-smi clocks / throttle reasons of one GPU while a timed region runs."""
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


class GemmSet:
    """Device operands of the 15 GEMMs at `rows` rows and one pass over them in the order a backward pass
    produces gradients last-layer-first: lm_head, fc_proj, fc, attn_proj, qkv, each forward, backward_input,
    backward_weight. With an exchange object, each layer's weight / bias gradients are handed to it right
    after their GEMM, so that the largest gradient (lm_head, 154.5 MB) travels under the twelve GEMMs behind it."""

    def __init__(self, g, torch, rows, mode, seed, only=None):
        self.g, self.torch = g, torch
        self.rows = rows
        self.seq = SEQ if rows % SEQ == 0 else rows
        self.batch = rows // self.seq
        self.opts = g.make_opts(mode=mode)
        self.only = only
        gen = torch.Generator(device="cuda").manual_seed(seed)
        self.bufs = []
        for name, K, N in reversed(LAYERS):
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
            self.bufs.append((name, K, N, d))

    def flops(self):
        if self.only:
            return sum(2.0 * self.rows * K * N for n_, K, N in LAYERS for k_ in KINDS if f"{n_}.{k_}" in self.only)
        return step_flops(self.rows)

    def step(self, stream, exchange=None, events=None):
        """events: dict name -> list of (start, end) CUDA events, filled when given"""
        g, torch = self.g, self.torch
        for name, K, N, d in self.bufs:
            calls = (
                ("fwd", lambda: g.forward(d["y"], d["x"], d["w"], d["b"], self.batch, self.seq, K, N, self.opts, stream)),
                ("dgrad", lambda: g.backward_input(d["dx"], d["dy"], d["w"], self.batch, self.seq, K, N, self.opts, stream)),
                ("wgrad", lambda: g.backward_weight(d["dw"], d["db"], d["dy"], d["x"], self.batch, self.seq, K, N,
                                                    self.opts, stream)),
            )
            for kind, fn in calls:
                if self.only and f"{name}.{kind}" not in self.only:
                    continue
                if events is not None:
                    s = torch.cuda.Event(enable_timing=True)
                    e = torch.cuda.Event(enable_timing=True)
                    s.record()
                    rc = fn()
                    e.record()
                    events.setdefault(f"{name}.{kind}", []).append((s, e))
                else:
                    rc = fn()
                if rc != 0:
                    raise SystemExit(f"GEMM call {name}.{kind} failed with code {rc}")
            if exchange is not None:
                exchange.exchange([d["dw"], d["db"]])  # this layer's gradients travel under the next GEMMs
        if exchange is not None:
            exchange.finish()


def seeded_model(g, model_name, B, T, mode):
    """A Model with the same seeded random weights on every rank (normal 0.02, layernorm weights one, pad
    columns of wte zero)."""
    import numpy as np

    C, L, NH = MODELS[model_name]
    model = g.Model(VOCAB, PADDED_VOCAB, L, NH, C, 1024, B, T, mode=mode)
    rng = np.random.default_rng(42)
    params = rng.standard_normal(model.num_params, dtype=np.float32) * np.float32(0.02)
    offs = model.offsets()
    params[: C * PADDED_VOCAB].reshape(C, PADDED_VOCAB)[:, VOCAB:] = 0
    for i in [2 + 12 * l + k for l in range(L) for k in (0, 6)] + [2 + 12 * L]:
        params[offs[i]: offs[i] + C] = 1.0
    model.set_params(params)
    return model


def measure_train(g, dp, torch, local_rank, rank, world, barrier, dist, mode, B=16, T=1024, steps=5, warmup=3,
                  model_name="small", path="launches", graph=None):
    """Tokens/s of whole training steps (forward, backward, gradient all-reduce over NCCL overlapped with the
    backward pass, AdamW) at B sequences of T tokens per GPU, random-init weights and uniform random tokens.

    path = "launches": one launch per layer call; with one rank, forward + backward are replayed from a CUDA
    graph (graph=False keeps the eager launches that more than one rank uses, for a like-with-like scaling
    curve). path = "step": the whole step as a schedule of the persistent kernel (one rank only: AdamW is
    part of the launch). Returns tokens/s, ms per step, the last loss, and a checksum of the parameters that all
    ranks must share."""
    C, L, NH = MODELS[model_name]
    model = seeded_model(g, model_name, B, T, mode)
    gen = torch.Generator(device="cuda").manual_seed(100 + rank)
    tok = torch.randint(0, VOCAB, (B * T,), dtype=torch.int32, device="cuda", generator=gen)
    tgt = torch.randint(0, VOCAB, (B * T,), dtype=torch.int32, device="cuda", generator=gen)
    stream = torch.cuda.current_stream().cuda_stream
    hyper = TRAIN_HYPER
    info = None
    if path == "step":
        if world != 1:
            raise SystemExit("the single-launch step includes AdamW: one rank only")
        # attention runs as tiles of the same launch where the fused tensor-core attention applies (T % 128 == 0);
        # otherwise its kernels are launched between pieces of the schedule
        sched = g.Step(model, tok, tgt, with_update=True, attention_in_kernel=(T % 128 == 0))
        info = sched.info()

        def one(t):
            return sched.run(*hyper, t, stream)
    else:
        use_graph = (world == 1) if graph is None else (graph and world == 1)
        runner = dp.DataParallelStep(model, torch.device("cuda", local_rank), use_graph=use_graph)

        def one(t):
            return runner(tok, tgt, *hyper, t, stream)
    t = 0
    for _ in range(warmup):
        t += 1
        if one(t) != 0:
            raise SystemExit("training step failed")
    barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        t += 1
        one(t)
    e.record()
    barrier()
    ms = s.elapsed_time(e)
    loss = model.mean_loss()
    if path == "step" and sched.status() != 0:
        raise SystemExit("the persistent step reported a device timeout")
    # every rank must hold the same parameters after the same number of averaged updates
    ptr = dp.device_tensor(model.params_ptr(), model.num_params, torch.device("cuda", local_rank))
    checksum = ptr.double().sum()
    agree, spread = True, 0.0
    if dist is not None:
        tt = torch.tensor([ms], device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = tt.item()
        hi, lo = checksum.clone(), checksum.clone()
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        spread = float(hi - lo)
        agree = spread == 0.0
    tokens = B * T * world * steps
    out = {"tokens_per_s": tokens / (ms * 1e-3), "ms_per_step": ms / steps, "steps": steps, "path": path,
           "config": f"GPT-2 {model_name} ({L} layers, {C} wide, vocabulary 50257 padded to 50304), B={B} per GPU, T={T}, "
                     f"AdamW lr 3e-4 betas 0.9/0.95 wd 0.1, fp32 master weights, {'3xTF32' if mode else 'TF32'} GEMMs, "
                     + ("attention as batched causal GEMMs on the linear-layer kernel" if (mode or T % 128) else
                        "fused causal attention on the tensor cores (no T x T tensors)")
                     + "; residual adds and GELU backward in GEMM epilogues", "loss_after": loss,
           "gemm_tflops": train_gemm_flops(model_name, B * T) * world * steps / (ms * 1e-3) / 1e12,
           "param_checksum": float(checksum), "ranks_agree": agree, "checksum_spread": spread,
           "gradient_exchange": ("none (1 GPU)" if world == 1 else
                                 "NCCL average, one bucket per block, overlapped; AdamW per bucket as it lands")}
    if info:
        out["launches_per_step"] = info["launches"]
        out["ops"] = info["ops"]
        out["tiles"] = info["tiles"]
    elif world == 1:
        out["launches_per_step"] = ("forward + backward replayed from a CUDA graph" if use_graph else
                                    "separate launches, eager (the path more than one rank uses)")
    if path == "step":
        sched.close()
    model.close()
    return out


def measure_gemm_list(g, torch, mode, steps=20, warmup=3):
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
            "what": "the 15 GEMMs of the set as one persistent launch (gpt2_megakernel_run)"}


def attention_case(g, torch, B, reps, impl="flash", T=1024, NH=12):
    """`reps` forward + backward passes of gpt2_attention_* on seeded inputs, B sequences of NH heads."""
    code = {"flash": g.ATT_FLASH, "gemm": g.ATT_GEMM, "simt": g.ATT_SIMT}[impl]
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
    return {"status": g.lib.gpt2_attention_status(), "finite": bool(torch.isfinite(gq).all())}
