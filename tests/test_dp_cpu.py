"""CPU tests of the data-parallel host logic: bucket planning, and a world_size-2 gloo run of the
gradient exchange (two ranks with different gradients end up with the same average)."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _dp():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as ge
    return ge._load_module("gpt2cu_b200_dp", os.path.join(ROOT, "gpt2.cu_b200", "dp.py"))


def test_bucket_plan_keeps_order_and_limits_size():
    dp = _dp()
    sizes = [("ln_f", 1536), ("blk1", 7_087_872), ("blk0", 7_087_872), ("wte", 38_633_472), ("wpe", 786_432)]
    buckets = dp.plan_buckets(sizes, 32 << 20)
    assert [n for b in buckets for n in b] == [n for n, _ in sizes]
    assert buckets == [["ln_f", "blk1"], ["blk0"], ["wte"], ["wpe"]]
    assert dp.plan_buckets([], 1024) == []


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    dp = _dp()
    ex = dp.GradientExchange()
    g = torch.Generator().manual_seed(100 + rank)
    dw = torch.randn(48, 32, generator=g)
    db = torch.randn(32, generator=g)
    ex.exchange([dw, db, None])
    ex.finish()
    # every rank must now hold the mean of the per-rank gradients
    want_w = sum(torch.randn(48, 32, generator=torch.Generator().manual_seed(100 + r)) for r in range(world)) / world
    ok = torch.allclose(dw, want_w, atol=1e-6) and ex.calls == 1
    gathered = [torch.zeros_like(db) for _ in range(world)]
    dist.all_gather(gathered, db)
    ok = ok and all(torch.equal(gathered[0], t) for t in gathered)
    out[rank] = bool(ok)
    dist.destroy_process_group()


def test_gradient_exchange_world_size_2_gloo():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    assert dict(out) == {0: True, 1: True}


def test_single_process_is_a_noop():
    dp = _dp()
    ex = dp.GradientExchange()
    t = torch.ones(4)
    ex.exchange([t])
    ex.finish()
    assert ex.calls == 0 and torch.equal(t, torch.ones(4))


def test_shard_bounds():
    dp = _dp()
    assert dp.shard_bounds(10, 10 + 17, 4) == (4, 26)
    assert dp.shard_bounds(0, 3, 8) == (0, 0)   # smaller than the world: wholly replicated
    assert dp.shard_bounds(5, 5 + 16, 2) == (8, 21)


def _sharded_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    dp = _dp()
    n = 1000
    ranges = [(601, 1000), (600, 601), (37, 600), (0, 37)]  # odd sizes, one smaller than the world, reverse order
    params0 = torch.randn(n, generator=torch.Generator().manual_seed(7))
    grads_of = lambda r: torch.randn(n, generator=torch.Generator().manual_seed(50 + r))
    params, grads = params0.clone(), grads_of(rank)
    sx = dp.ShardedExchange(grads, params)
    for lo, hi in ranges:
        sx.reduce(lo, hi)
    sx.finish()
    owned = sx.owned()
    touched = torch.zeros(n, dtype=torch.bool)
    for first, count in owned:          # stand-in for gpt2_model_update_range: plain SGD on the owned floats only
        params[first:first + count] -= 0.1 * grads[first:first + count]
        touched[first:first + count] = True
    sx.gather()
    mean = sum(grads_of(r) for r in range(world)) / world
    ok = torch.allclose(params, params0 - 0.1 * mean, atol=1e-6)
    # this rank updated its share only: about 1/world of the floats plus the small remainders
    ok = ok and int(touched.sum()) <= n // world + world * len(ranges)
    ok = ok and sx.calls == len(ranges) and sx.ranges == []
    out[rank] = bool(ok)
    dist.destroy_process_group()


def test_sharded_optimizer_exchange_world_size_2_gloo():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    port = 31500 + (os.getpid() % 2000)
    mp.spawn(_sharded_worker, args=(world, port, out), nprocs=world, join=True)
    assert dict(out) == {0: True, 1: True}


def test_sharded_exchange_single_process_owns_everything():
    dp = _dp()
    g, p = torch.ones(10), torch.zeros(10)
    sx = dp.ShardedExchange(g, p)
    sx.reduce(4, 10)
    sx.reduce(0, 4)
    sx.finish()
    assert sx.owned() == [(4, 6), (0, 4)]
    sx.gather()
    assert sx.ranges == []
