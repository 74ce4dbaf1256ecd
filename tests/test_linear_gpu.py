"""GPU parity tests: the three linear-layer calls through the C ABI against the CPU oracle
(float64 truth), on the same seeded inputs.

Tolerances are the ones the specification of this path states: max relative error
(max|y - y_ref| / max|y_ref|) <= 1e-2 in TF32 mode and <= 2e-3 in 3xTF32 mode.
"""
import numpy as np
import pytest
import torch

from conftest import LAYERS, golden

pytestmark = pytest.mark.gpu

TOL = {0: 1e-2, 1: 2e-3}
# what the modes actually deliver on N(0,1) x N(0,0.02) data (checked, so regressions show)
TIGHT = {0: 2e-3, 1: 2e-5}


def dev(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def run_all(g, x, w, b, dy, mode, want_bias=True, **okw):
    """Runs forward / backward_input / backward_weight on the device; returns numpy outputs."""
    M, K = x.shape
    N = w.shape[1]
    xd, wd, bd, dyd = dev(x), dev(w), dev(b), dev(dy)
    y = torch.full((M, N), float("nan"), device="cuda")
    dx = torch.full((M, K), float("nan"), device="cuda")
    dw = torch.full((K, N), float("nan"), device="cuda")
    db = torch.full((N,), float("nan"), device="cuda") if want_bias else None
    o = g.make_opts(mode=mode, **okw)
    g.check("forward", g.forward(y, xd, wd, bd, 1, M, K, N, o))
    g.check("backward_input", g.backward_input(dx, dyd, wd, 1, M, K, N, o))
    g.check("backward_weight", g.backward_weight(dw, db, dyd, xd, 1, M, K, N, o))
    torch.cuda.synchronize()
    st, rec = g.last_status()
    assert st == 0, f"device status record {rec}"
    return y.cpu().numpy(), dx.cpu().numpy(), dw.cpu().numpy(), None if db is None else db.cpu().numpy()


def check_all(orc, outs, x, w, b, dy, tol):
    y, dx, dw, db = outs
    errs = {
        "y": orc.max_rel_err(y, orc.forward(x, w, b, f64=True)),
        "dx": orc.max_rel_err(dx, orc.backward_input(dy, w, f64=True)),
    }
    dw_t, db_t = orc.backward_weight(dy, x, want_bias=db is not None, f64=True)
    errs["dw"] = orc.max_rel_err(dw, dw_t)
    if db is not None:
        errs["db"] = orc.max_rel_err(db, db_t)
    for k, v in errs.items():
        assert np.isfinite(v) and v <= tol, (k, v, errs)
    return errs


def seeded(M, K, N, seed=0):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K), dtype=np.float32)
    w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    b = (rng.standard_normal(N) * 0.02).astype(np.float32)
    dy = (rng.standard_normal((M, N)) * 0.01).astype(np.float32)
    return x, w, b, dy


# shapes: aligned multiples of the tile, ragged in every dimension (still 16-byte strides),
# tiny, one k-block, many k-blocks, and the B=4,T=64 GPT-2 small layer shapes
SHAPES = [
    (128, 32, 64), (128, 128, 256), (256, 768, 768), (384, 96, 320),
    (4, 4, 4), (1, 8, 12), (129, 36, 68), (200, 100, 52), (130, 260, 516),
    (256, 768, 2304), (256, 3072, 768), (256, 768, 3072),
]


@pytest.mark.parametrize("pair", [1, 2])  # 1: one CTA per 128-row tile; 2: CTA pairs, 256-row tiles
@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("M,K,N", SHAPES)
def test_parity_against_oracle(gpu, orc, M, K, N, mode, pair):
    x, w, b, dy = seeded(M, K, N, seed=M + K + N)
    outs = run_all(gpu, x, w, b, dy, mode, cta_pair=pair)
    check_all(orc, outs, x, w, b, dy, TIGHT[mode])


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("fx", ["llm_tiny_aligned.npz", "llm_tiny_ragged.npz"])
@pytest.mark.parametrize("layer", LAYERS)
def test_parity_against_reference_model_fixtures(gpu, orc, fx, layer, mode):
    """Same inputs the reference's PyTorch model saw; outputs compared with what it produced.
    The ragged fixture's lm_head (vocabulary 101) exercises the CUDA-core kernel for shapes
    TMA cannot address."""
    z = golden(fx)
    x, w, y, dy, dx, dw = (z[f"{layer}.{k}"] for k in ("x", "w", "y", "dy", "dx", "dw"))
    b = z[f"{layer}.b"] if f"{layer}.b" in z else None
    got = run_all(gpu, x, w, b, dy, mode, want_bias=b is not None)
    assert orc.max_rel_err(got[0], y) <= TOL[mode]
    assert orc.max_rel_err(got[1], dx) <= TOL[mode]
    assert orc.max_rel_err(got[2], dw) <= TOL[mode]
    if b is not None:
        assert orc.max_rel_err(got[3], z[f"{layer}.db"]) <= TOL[mode]


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("M,K,N", [(256, 64, 8192), (132, 36, 8196)])
def test_wide_weight_gradient_uses_transposed_activations(gpu, orc, M, K, N, mode):
    """N >= 8192 and N >= 8 K: backward_weight transposes `in` into scratch and runs with a K-major A
    operand (the lm_head case); the bias gradient is still the fused column sum."""
    x, w, b, dy = seeded(M, K, N, seed=N)
    outs = run_all(gpu, x, w, b, dy, mode)
    check_all(orc, outs, x, w, b, dy, TIGHT[mode])
    outs = run_all(gpu, x, w, b, dy, mode, deterministic=1, split_k=3)
    check_all(orc, outs, x, w, b, dy, TIGHT[mode])


def test_null_bias_and_null_bias_grad(gpu, orc):
    x, w, b, dy = seeded(256, 64, 128, seed=3)
    y, dx, dw, db = run_all(gpu, x, w, None, dy, 0, want_bias=False)
    assert db is None
    assert orc.max_rel_err(y, orc.forward(x, w, None, f64=True)) <= TIGHT[0]


def test_unaligned_shapes_use_cuda_core_kernel(gpu, orc):
    """K or N not a multiple of 4 floats: no TMA; results are fp32-exact-ish."""
    for (M, K, N) in [(70, 33, 50), (64, 64, 50257 % 1000), (5, 7, 9)]:
        x, w, b, dy = seeded(M, K, N, seed=K)
        outs = run_all(gpu, x, w, b, dy, 0)
        check_all(orc, outs, x, w, b, dy, 1e-5)


def test_force_simt_matches(gpu, orc):
    x, w, b, dy = seeded(256, 128, 192, seed=9)
    outs = run_all(gpu, x, w, b, dy, 0, force_simt=1)
    check_all(orc, outs, x, w, b, dy, 1e-5)


@pytest.mark.parametrize("pair", [1, 2])
@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("det", [0, 1])
@pytest.mark.parametrize("splits", [2, 5])
def test_split_k_weight_gradient(gpu, orc, splits, det, mode, pair):
    x, w, b, dy = seeded(1024, 384, 256, seed=splits)
    outs = run_all(gpu, x, w, b, dy, mode, split_k=splits, deterministic=det, cta_pair=pair)
    check_all(orc, outs, x, w, b, dy, TIGHT[mode])


def test_deterministic_split_is_bitwise_repeatable(gpu):
    x, w, b, dy = seeded(2048, 128, 256, seed=21)
    a = run_all(gpu, x, w, b, dy, 0, split_k=4, deterministic=1)
    for _ in range(3):
        c = run_all(gpu, x, w, b, dy, 0, split_k=4, deterministic=1)
        assert np.array_equal(a[2], c[2]) and np.array_equal(a[3], c[3])


def test_small_m_long_reduction_picks_splits(gpu, orc):
    """lm_head-like backward_input at tiny M: few tiles, long reduction -> automatic split."""
    x, w, b, dy = seeded(64, 128, 8192, seed=4)
    outs = run_all(gpu, x, w, b, dy, 0)
    check_all(orc, outs, x, w, b, dy, TIGHT[0])


@pytest.mark.parametrize("pair", [1, 2])
def test_gelu_dual_store(gpu, orc, pair):
    x, w, b, dy = seeded(300, 64, 256, seed=6)
    M, K = x.shape
    N = w.shape[1]
    y = torch.empty((M, N), device="cuda")
    y2 = torch.empty((M, N), device="cuda")
    o = gpu.make_opts(mode=1, flags=gpu.EPI_GELU_DUAL, out2=y2.data_ptr(), cta_pair=pair)
    gpu.check("forward", gpu.forward(y, dev(x), dev(w), dev(b), 1, M, K, N, o))
    torch.cuda.synchronize()
    pre = y.cpu().numpy()
    assert orc.max_rel_err(pre, orc.forward(x, w, b, f64=True)) <= TIGHT[1]
    assert np.allclose(y2.cpu().numpy(), orc.gelu(pre), atol=2e-6)


@pytest.mark.parametrize("pair", [1, 2])
@pytest.mark.parametrize("M,K,N,split", [(300, 64, 256, 0), (256, 768, 768, 0), (129, 36, 68, 0), (128, 1024, 128, 4)])
def test_residual_add_in_the_epilogue(gpu, orc, M, K, N, split, pair):
    """forward with GPT2L_AUX_ADD: out = x.w + b + residual (the reference runs residual_forward after
    the projection); with an atomic split the residual must be added exactly once"""
    x, w, b, dy = seeded(M, K, N, seed=21)
    res = np.random.default_rng(5).standard_normal((M, N), dtype=np.float32)
    resd = dev(res)
    y = torch.full((M, N), float("nan"), device="cuda")
    o = gpu.make_opts(mode=1, aux=resd.data_ptr(), aux_op=gpu.AUX_ADD, split_k=split, cta_pair=pair)
    gpu.check("forward", gpu.forward(y, dev(x), dev(w), dev(b), 1, M, K, N, o))
    torch.cuda.synchronize()
    truth = orc.forward(x, w, b, f64=True) + res.astype(np.float64)
    assert orc.max_rel_err(y.cpu().numpy(), truth) <= TIGHT[1]
    assert np.array_equal(resd.cpu().numpy(), res)  # the operand is read-only


@pytest.mark.parametrize("pair", [1, 2])
@pytest.mark.parametrize("M,K,N", [(300, 256, 64), (256, 3072, 768), (130, 516, 260)])
def test_gelu_backward_in_the_epilogue(gpu, orc, M, K, N, pair):
    """backward_input with GPT2L_AUX_GELU_GRAD: dx = (dy.w^T) * gelu'(pre), pre shaped like dx (the
    reference runs gelu_backward on the result); a requested split must be ignored, not misapplied"""
    x, w, b, dy = seeded(M, K, N, seed=22)
    pre = (np.random.default_rng(6).standard_normal((M, K)) * 2).astype(np.float32)
    dx = torch.full((M, K), float("nan"), device="cuda")
    pred = dev(pre)
    for split in (0, 3):
        o = gpu.make_opts(mode=1, aux=pred.data_ptr(), aux_op=gpu.AUX_GELU_GRAD, split_k=split, cta_pair=pair)
        gpu.check("backward_input", gpu.backward_input(dx, dev(dy), dev(w), 1, M, K, N, o))
        torch.cuda.synchronize()
        truth = orc.gelu_grad_mul(pre, orc.backward_input(dy, w, f64=True))
        assert orc.max_rel_err(dx.cpu().numpy(), truth) <= TIGHT[1]


def test_epilogue_operand_argument_checks(gpu):
    x, w, b, dy = seeded(128, 64, 64, seed=23)
    y = torch.empty((128, 64), device="cuda")
    aux = torch.zeros((128, 64), device="cuda")
    dw = torch.empty((64, 64), device="cuda")
    bad = gpu.make_opts(mode=1, aux=None, aux_op=gpu.AUX_ADD)
    assert gpu.forward(y, dev(x), dev(w), dev(b), 1, 128, 64, 64, bad) == gpu.ERR_BAD_ARG
    bad = gpu.make_opts(mode=1, aux=aux.data_ptr(), aux_op=7)
    assert gpu.forward(y, dev(x), dev(w), dev(b), 1, 128, 64, 64, bad) == gpu.ERR_BAD_ARG
    bad = gpu.make_opts(mode=1, aux=aux.data_ptr(), aux_op=gpu.AUX_ADD)
    assert gpu.backward_weight(dw, None, dev(dy), dev(x), 1, 128, 64, 64, bad) == gpu.ERR_BAD_ARG
    bad = gpu.make_opts(mode=1, aux=aux.data_ptr(), aux_op=gpu.AUX_ADD, force_simt=1)
    assert gpu.forward(y, dev(x), dev(w), dev(b), 1, 128, 64, 64, bad) == gpu.ERR_BAD_ARG


def test_outputs_are_overwritten_not_accumulated(gpu, orc):
    x, w, b, dy = seeded(256, 64, 128, seed=8)
    # deterministic=1: the default split-K combine uses floating-point atomics, whose order varies
    first = run_all(gpu, x, w, b, dy, 1, deterministic=1)
    second = run_all(gpu, x, w, b, dy, 1, deterministic=1)  # buffers pre-filled with NaN inside run_all
    for a, c in zip(first, second):
        assert np.array_equal(a, c)


def test_host_buffer_entry_points(gpu, orc):
    x, w, b, dy = seeded(512, 96, 160, seed=12)
    M, K = x.shape
    N = w.shape[1]
    y = np.empty((M, N), np.float32)
    dx = np.empty((M, K), np.float32)
    dw = np.empty((K, N), np.float32)
    db = np.empty((N,), np.float32)
    o = gpu.make_opts(mode=1)
    assert gpu.forward(y, x, w, b, 1, M, K, N, o, host=True) == 0
    assert gpu.backward_input(dx, dy, w, 1, M, K, N, o, host=True) == 0
    assert gpu.backward_weight(dw, db, dy, x, 1, M, K, N, o, host=True) == 0
    check_all(orc, (y, dx, dw, db), x, w, b, dy, TIGHT[1])


def test_pipelined_host_calls_match_the_blocking_ones(gpu, orc):
    """six calls in flight over two staging sets (the third and later calls reuse a set; shapes grow so
    that a set is re-allocated while the pipeline is busy), results read only after the synchronise"""
    import torch as _t

    o = gpu.make_opts(mode=1, deterministic=1)
    jobs = []
    for i, (M, K, N) in enumerate([(256, 64, 96), (384, 96, 160), (512, 128, 192)]):
        x, w, b, dy = seeded(M, K, N, seed=40 + i)
        pin = lambda a: _t.from_numpy(a).pin_memory()
        hx, hw, hb, hdy = pin(x), pin(w), pin(b), pin(dy)
        hy = _t.empty((M, N)).pin_memory()
        hdx = _t.empty((M, K)).pin_memory()
        hdw = _t.empty((K, N)).pin_memory()
        hdb = _t.empty((N,)).pin_memory()
        assert gpu.forward_host_async(hy, hx, hw, hb, 1, M, K, N, o) == 0
        assert gpu.backward_input_host_async(hdx, hdy, hw, 1, M, K, N, o) == 0
        assert gpu.backward_weight_host_async(hdw, hdb, hdy, hx, 1, M, K, N, o) == 0
        # inputs stay alive (and unchanged) until the synchronise, as the contract of the calls demands
        jobs.append((x, w, b, dy, hy, hdx, hdw, hdb, (hx, hw, hb, hdy)))
    assert gpu.host_synchronize() == 0
    for x, w, b, dy, hy, hdx, hdw, hdb, _inputs in jobs:
        check_all(orc, (hy.numpy(), hdx.numpy(), hdw.numpy(), hdb.numpy()), x, w, b, dy, TIGHT[1])
    assert gpu.host_synchronize() == 0  # nothing pending: returns at once
    # no bias / no bias gradient (the lm_head case), through a staging set that has held larger operands
    x, w, b, dy = seeded(130, 36, 68, seed=77)
    pin = lambda a: _t.from_numpy(a).pin_memory()
    hx, hw, hdy = pin(x), pin(w), pin(dy)
    hy, hdw = _t.empty((130, 68)).pin_memory(), _t.empty((36, 68)).pin_memory()
    assert gpu.forward_host_async(hy, hx, hw, None, 1, 130, 36, 68, o) == 0
    assert gpu.backward_weight_host_async(hdw, None, hdy, hx, 1, 130, 36, 68, o) == 0
    assert gpu.host_synchronize() == 0
    assert orc.max_rel_err(hy.numpy(), orc.forward(x, w, None, f64=True)) <= TIGHT[1]
    assert orc.max_rel_err(hdw.numpy(), orc.backward_weight(dy, x, want_bias=False, f64=True)[0]) <= TIGHT[1]
    # an input is uploaded once per window; after the synchronise it may change, and the next window sees it
    hx.mul_(2.0)
    assert gpu.forward_host_async(hy, hx, hw, None, 1, 130, 36, 68, o) == 0
    assert gpu.host_synchronize() == 0
    assert orc.max_rel_err(hy.numpy(), orc.forward(2.0 * x, w, None, f64=True)) <= TIGHT[1]
    hx, hw, hb = pin(seeded(512, 128, 192, seed=42)[0]), pin(seeded(512, 128, 192, seed=42)[1]), pin(seeded(512, 128, 192, seed=42)[2])
    hy = _t.empty((512, 192)).pin_memory()
    bad = gpu.make_opts(mode=1, aux=1 << 20, aux_op=gpu.AUX_ADD)
    assert gpu.forward_host_async(hy, hx, hw, hb, 1, 512, 128, 192, bad) == gpu.ERR_BAD_ARG


def test_linearity_at_full_size(gpu):
    """Size-independent property at the benchmark's QKV shape (M = 8192): the forward is linear
    in x, so f(x1) + f(x2) - f(0) == f(x1 + x2) up to TF32 rounding; 3xTF32 makes it tight."""
    M, K, N = 8192, 768, 2304
    gen = torch.Generator(device="cuda").manual_seed(1)
    x1 = torch.randn((M, K), device="cuda", generator=gen)
    x2 = torch.randn((M, K), device="cuda", generator=gen)
    w = torch.randn((K, N), device="cuda", generator=gen) * 0.02
    b = torch.randn((N,), device="cuda", generator=gen) * 0.02
    o = gpu.make_opts(mode=1)
    outs = []
    for xin in (x1, x2, x1 + x2, torch.zeros_like(x1)):
        y = torch.empty((M, N), device="cuda")
        gpu.check("forward", gpu.forward(y, xin, w, b, 8, 1024, K, N, o))
        outs.append(y)
    torch.cuda.synchronize()
    lhs = outs[0] + outs[1] - outs[3]
    rel = (lhs - outs[2]).abs().max().item() / outs[2].abs().max().item()
    assert rel <= 1e-5, rel
    assert torch.equal(outs[3], b.expand(M, N))  # x = 0 leaves exactly the bias


def test_epilogue_on_the_load_store_path_gives_the_same_results(gpu, orc):
    """GPT2L_EPI_TMA=0 keeps the epilogue's staged boxes on the load/store path (read back and stored by the
    warps) instead of handing them to the copy engine. The switch is read once per process, so the three
    calls run in a child process with it set; ragged and aligned shapes, plain and split-K."""
    import os
    import subprocess
    import sys

    from conftest import ROOT

    code = r"""
import os, sys
import numpy as np, torch
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
import __graft_entry__ as ge
import test_linear_gpu as t
g = ge.load_package(); g.init(0)
orc = ge.load_oracle()
for (M, K, N), sk in (((256, 768, 768), 0), ((129, 36, 68), 0), ((384, 96, 320), 3), ((256, 768, 50304), 0)):
    x, w, b, dy = t.seeded(M, K, N, seed=5)
    for pair in (1, 2):
        outs = t.run_all(g, x, w, b, dy, 0, split_k=sk, cta_pair=pair)
        t.check_all(orc, outs, x, w, b, dy, t.TIGHT[0])
print("ok")
"""
    env = dict(os.environ, GPT2L_EPI_TMA="0")
    res = subprocess.run([sys.executable, "-c", code, ROOT], env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and res.stdout.strip().endswith("ok"), res.stdout[-2000:] + res.stderr[-2000:]
