"""GPU test of gpt2_linear_backward_weight_noalloc — the weight gradient for callers that are not
allowed to allocate device memory (code running inside a server that owns all GPU memory through
its own pool, or inside loops that cannot take cudaMalloc's device-wide synchronisation).

It is called through the C ABI twice in a row, on different shapes, and each result is compared
with the regular entry point (deterministic split-K, cudaMalloc'ed workspace) on the same inputs.
The two calls share the library's fixed scratch array, so the second call also proves that stale
contents of the first do no harm. Free device memory is read before and after: the calls must not
change it. This file sorts last on purpose: a run that stops at the first failure has then already
run every other test."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = {0: 2e-3, 1: 2e-5}  # the tolerances the other parity tests use for TF32 / 3xTF32


def operands(M, K, N, seed):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn((M, K), device="cuda", generator=gen)
    dy = torch.randn((M, N), device="cuda", generator=gen) * 0.01
    return x, dy


def rel(a, b):
    return ((a - b).abs().max() / b.abs().max()).item()


@pytest.mark.parametrize("mode", [0, 1])
def test_noalloc_weight_gradient_matches_regular_entry_point(gpu, mode):
    shapes = [(2048, 256, 384, 4), (1000, 96, 160, 0)]  # (M, K, N, forced split count; 0 = automatic)
    prepared = []
    for i, (M, K, N, sk) in enumerate(shapes):
        x, dy = operands(M, K, N, seed=40 + i)
        want_w = torch.empty((K, N), device="cuda")
        want_b = torch.empty((N,), device="cuda")
        o = gpu.make_opts(mode=mode, split_k=sk, deterministic=1)
        gpu.check("backward_weight", gpu.backward_weight(want_w, want_b, dy, x, 1, M, K, N, o))
        got_w = torch.full((K, N), float("nan"), device="cuda")
        got_b = torch.full((N,), float("nan"), device="cuda")
        prepared.append((M, K, N, o, x, dy, want_w, want_b, got_w, got_b))
    torch.cuda.synchronize()
    # first call on this device happens here at the latest (set-up), outside the measured pair
    M, K, N, o, x, dy, _, _, got_w, got_b = prepared[0]
    assert gpu.backward_weight_noalloc(got_w, got_b, dy, x, 1, M, K, N, o) == 0
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for (M, K, N, o, x, dy, want_w, want_b, got_w, got_b) in prepared:  # two calls in a row
        got_w.fill_(float("nan"))
        got_b.fill_(float("nan"))
        assert gpu.backward_weight_noalloc(got_w, got_b, dy, x, 1, M, K, N, o) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "the no-allocation entry point changed the amount of free device memory"
    st, rec = gpu.noalloc_last_status()
    assert st == 0, rec  # no wait gave up in any of the three calls
    for i, (M, K, N, o, x, dy, want_w, want_b, got_w, got_b) in enumerate(prepared):
        if shapes[i][3] > 0:
            # forced split count: same tiling, same fixed combination order as the regular call
            assert torch.equal(got_w, want_w)
        assert torch.isfinite(got_w).all() and torch.isfinite(got_b).all()
        assert rel(got_w, want_w) <= TOL[mode]
        assert rel(got_b, want_b) <= TOL[mode]
        # and against an independent fp64 product
        truth = (x.double().t() @ dy.double())
        assert rel(got_w.double(), truth) <= TOL[mode]


def test_noalloc_rejects_what_does_not_fit(gpu):
    """768 x 3072 output with 16 forced splits needs 16 x 9 MiB of partial tiles: more than the
    fixed array holds. The call must refuse, not allocate."""
    M, K, N = 4096, 768, 3072
    x, dy = operands(M, K, N, seed=50)
    gw = torch.zeros((K, N), device="cuda")
    o = gpu.make_opts(mode=0, split_k=16)
    assert gpu.backward_weight_noalloc(gw, None, dy, x, 1, M, K, N, o) == gpu.ERR_TOO_LARGE
    # the same problem with an automatic split count runs (the count is lowered to fit)
    o = gpu.make_opts(mode=0)
    assert gpu.backward_weight_noalloc(gw, None, dy, x, 1, M, K, N, o) == 0
    torch.cuda.synchronize()
    truth = x.double().t() @ dy.double()
    assert rel(gw.double(), truth) <= TOL[0]
    assert gpu.backward_weight_noalloc(None, None, dy, x, 1, M, K, N, o) == gpu.ERR_BAD_ARG


def test_noalloc_status_record_is_kept_until_read(gpu):
    """A timeout record of this path must survive later calls and be cleared only by its reader. The
    record is planted from the host (no kernel is made to give up); two calls follow, then the reader
    must still return it, and a second read must return 0."""
    M, K, N = 512, 128, 256
    x, dy = operands(M, K, N, seed=60)
    gw = torch.empty((K, N), device="cuda")
    assert gpu.backward_weight_noalloc(gw, None, dy, x, 1, M, K, N, gpu.make_opts(mode=0)) == 0
    torch.cuda.synchronize()
    assert gpu.noalloc_last_status()[0] == 0
    planted = [gpu.DEV_TIMEOUT, 3, 17, 5, 8, 7]
    assert gpu.noalloc_debug_set_status(planted) == 0
    for _ in range(2):
        assert gpu.backward_weight_noalloc(gw, None, dy, x, 1, M, K, N, gpu.make_opts(mode=0, split_k=2)) == 0
    torch.cuda.synchronize()
    truth = x.double().t() @ dy.double()
    assert rel(gw.double(), truth) <= TOL[0]  # the planted record did not disturb the calls
    st, rec = gpu.noalloc_last_status()
    assert st == gpu.DEV_TIMEOUT and rec == planted
    assert gpu.noalloc_last_status()[0] == 0
