"""GPU tests of the persistent multi-GEMM launch: dependent GEMMs ordered by the tile dependency
counters inside ONE kernel launch give the same results as one call per GEMM, and a dependency
that can never be satisfied ends the launch with a timeout status instead of hanging."""
import time

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def mlp_block(g, B, S, C, mode, seed=0, det=1, pair=0):
    """x -> h = x.W1+b1 -> y = h.W2+b2, then the backward of both GEMMs (no GELU: a linear
    chain keeps every intermediate checkable by GEMMs alone)."""
    M = B * S
    gen = torch.Generator(device="cuda").manual_seed(seed)
    t = {
        "x": torch.randn((M, C), device="cuda", generator=gen),
        "w1": torch.randn((C, 4 * C), device="cuda", generator=gen) * 0.02,
        "b1": torch.randn((4 * C,), device="cuda", generator=gen) * 0.02,
        "w2": torch.randn((4 * C, C), device="cuda", generator=gen) * 0.02,
        "b2": torch.randn((C,), device="cuda", generator=gen) * 0.02,
        "dy": torch.randn((M, C), device="cuda", generator=gen) * 0.01,
    }
    for name, shape in (("h", (M, 4 * C)), ("y", (M, C)), ("dh", (M, 4 * C)), ("dw2", (4 * C, C)),
                        ("db2", (C,)), ("dx", (M, C)), ("dw1", (C, 4 * C)), ("db1", (4 * C,))):
        t[name] = torch.full(shape, float("nan"), device="cuda")
    o = g.make_opts(mode=mode, deterministic=det, cta_pair=pair)
    ops = [
        g.make_op(g.OP_FORWARD, B, S, C, 4 * C, t["h"], t["x"], t["w1"], bias=t["b1"], opts=o),
        g.make_op(g.OP_FORWARD, B, S, 4 * C, C, t["y"], t["h"], t["w2"], bias=t["b2"], opts=o,
                  deps=[(0, g.DEP_ROWBLOCK)]),
        g.make_op(g.OP_BACKWARD_INPUT, B, S, 4 * C, C, t["dh"], t["dy"], t["w2"], opts=o),
        g.make_op(g.OP_BACKWARD_WEIGHT, B, S, 4 * C, C, t["dw2"], t["h"], t["dy"], out_bias=t["db2"], opts=o,
                  deps=[(0, g.DEP_WHOLE_OP)]),
        g.make_op(g.OP_BACKWARD_INPUT, B, S, C, 4 * C, t["dx"], t["dh"], t["w1"], opts=o,
                  deps=[(2, g.DEP_ROWBLOCK)]),
        g.make_op(g.OP_BACKWARD_WEIGHT, B, S, C, 4 * C, t["dw1"], t["x"], t["dh"], out_bias=t["db1"], opts=o,
                  deps=[(2, g.DEP_WHOLE_OP)]),
    ]
    return t, ops, o


def separate_calls(g, t, B, S, C, o):
    r = {k: torch.full_like(t[k], float("nan")) for k in ("h", "y", "dh", "dw2", "db2", "dx", "dw1", "db1")}
    g.check("f", g.forward(r["h"], t["x"], t["w1"], t["b1"], B, S, C, 4 * C, o))
    g.check("f", g.forward(r["y"], r["h"], t["w2"], t["b2"], B, S, 4 * C, C, o))
    g.check("bi", g.backward_input(r["dh"], t["dy"], t["w2"], B, S, 4 * C, C, o))
    g.check("bw", g.backward_weight(r["dw2"], r["db2"], t["dy"], r["h"], B, S, 4 * C, C, o))
    g.check("bi", g.backward_input(r["dx"], r["dh"], t["w1"], B, S, C, 4 * C, o))
    g.check("bw", g.backward_weight(r["dw1"], r["db1"], r["dh"], t["x"], B, S, C, 4 * C, o))
    torch.cuda.synchronize()
    return r


@pytest.mark.parametrize("pair", [0, 2])  # 0: single CTAs (default); 2: CTA pairs, 256-row tiles
@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("B,S,C", [(2, 256, 64), (4, 1024, 256), (3, 100, 96), (1, 300, 160)])
def test_dependent_chain_in_one_launch(gpu, orc, B, S, C, mode, pair):
    t, ops, o = mlp_block(gpu, B, S, C, mode, seed=C, pair=pair)
    sched = gpu.Schedule(ops)
    launches0 = gpu.lib.gpt2_linear_launch_count()
    for _ in range(3):  # counters are re-armed on every run
        assert sched.run() == 0
    torch.cuda.synchronize()
    assert sched.status() == 0
    assert gpu.lib.gpt2_linear_launch_count() - launches0 == 3  # one kernel launch per run
    r = separate_calls(gpu, t, B, S, C, o)
    tol = {0: 2e-3, 1: 2e-5}[mode]
    for k in ("h", "y", "dh", "dx", "dw1", "dw2"):
        a, b = t[k], r[k]
        assert torch.isfinite(a).all(), k
        assert ((a - b).abs().max() / b.abs().max()).item() <= tol, k
    # against the float64 oracle, end of the chain
    x, w1, b1, w2, b2 = (t[k].cpu().numpy() for k in ("x", "w1", "b1", "w2", "b2"))
    h64 = orc.forward(x, w1, b1, f64=True)
    y64 = h64 @ w2.astype(np.float64) + b2
    assert orc.max_rel_err(t["y"].cpu().numpy(), y64) <= {0: 4e-3, 1: 2e-5}[mode]
    sched.close()


def test_whole_gemm_set_in_one_launch(gpu):
    """The five layer shapes x forward/backward_input/backward_weight as 15 independent ops."""
    B, S, C, V = 4, 64, 768, 50304
    M = B * S
    o = gpu.make_opts(mode=0, deterministic=1)
    gen = torch.Generator(device="cuda").manual_seed(3)
    ops, outs, refs, keep = [], [], [], []
    for (K, N) in [(C, 3 * C), (C, C), (C, 4 * C), (4 * C, C), (C, V)]:
        x = torch.randn((M, K), device="cuda", generator=gen)
        w = torch.randn((K, N), device="cuda", generator=gen) * 0.02
        b = torch.randn((N,), device="cuda", generator=gen) * 0.02
        dy = torch.randn((M, N), device="cuda", generator=gen) * 0.01
        y, dx, dw, db = (torch.empty(s, device="cuda") for s in ((M, N), (M, K), (K, N), (N,)))
        ops += [gpu.make_op(gpu.OP_FORWARD, B, S, K, N, y, x, w, bias=b, opts=o),
                gpu.make_op(gpu.OP_BACKWARD_INPUT, B, S, K, N, dx, dy, w, opts=o),
                gpu.make_op(gpu.OP_BACKWARD_WEIGHT, B, S, K, N, dw, x, dy, out_bias=db, opts=o)]
        outs.append((y, dx, dw, db))
        keep.append((x, w, b, dy))  # the schedule holds raw pointers: the operands must stay allocated
        refs.append((x @ w + b, dy @ w.t(), x.t() @ dy, dy.sum(0)))
    torch.backends.cuda.matmul.allow_tf32 = False
    sched = gpu.Schedule(ops)
    assert sched.run() == 0
    torch.cuda.synchronize()
    assert sched.status() == 0
    for got, want in zip(outs, refs):
        for a, b in zip(got, want):
            assert ((a - b).abs().max() / b.abs().max()).item() <= 2e-3
    sched.close()


def test_unsatisfiable_dependency_times_out_cleanly(gpu):
    """Host-side fault injection: the consumer is told to wait for more arrivals than its
    producer will ever publish. The launch must end by itself with the timeout status, name the
    op and counter, and leave the device usable."""
    t, ops, o = mlp_block(gpu, 2, 256, 64, 0)
    sched = gpu.Schedule(ops)
    assert sched.debug_set_expected(1, 0, 1 << 30, 200) == 0  # op 1, dependency 0, 200 ms limit
    t0 = time.time()
    assert sched.run() == 0
    torch.cuda.synchronize()
    assert time.time() - t0 < 10.0
    assert sched.status() == gpu.DEV_TIMEOUT
    sched.close()
    # the timeout raised the host-visible flag: the next device-pointer call refuses to launch and
    # returns the status, until gpt2_linear_last_status() has read (and cleared) it
    x = torch.randn((128, 64), device="cuda")
    w = torch.randn((64, 64), device="cuda")
    y = torch.empty((128, 64), device="cuda")
    assert gpu.forward(y, x, w, None, 1, 128, 64, 64, o) == gpu.DEV_TIMEOUT
    st, _ = gpu.last_status()
    assert st == gpu.DEV_TIMEOUT
    assert gpu.last_status()[0] == 0
    assert gpu.forward(y, x, w, None, 1, 128, 64, 64, o) == 0
    torch.cuda.synchronize()
    # the device is still usable: a fresh schedule of the same chain runs to completion
    t2, ops2, o2 = mlp_block(gpu, 2, 256, 64, 0)
    s2 = gpu.Schedule(ops2)
    assert s2.run() == 0
    torch.cuda.synchronize()
    assert s2.status() == 0
    assert torch.isfinite(t2["y"]).all()
    s2.close()
