"""Two-GPU test of the data-parallel training step: two ranks, each with half of a batch, must end
up with the gradients (and, after AdamW, the parameters) that one GPU computes on the whole batch.
Needs two GPUs; on a one-GPU machine it is skipped (the host logic is covered by the gloo tests)."""
import os
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT, golden

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out, shard):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch.distributed as dist

    import __graft_entry__ as ge
    import gpt2_ref

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    g = ge.load_package()
    g.init(rank)
    dp = ge._load_module("gpt2cu_b200_dp", os.path.join(ROOT, "gpt2.cu_b200", "dp.py"))
    z = golden("llm_train_tiny.npz")
    n_layer, n_head, n_embd, vocab, padded, block, B, T, steps = (int(v) for v in z["meta"])
    params = gpt2_ref.to_flat(gpt2_ref.init_params(vocab, block, n_layer, n_head, n_embd), n_layer, padded)
    tokens, targets = z["tokens"], z["targets"]  # [B, T] with B = 2: one sequence per rank
    hyper = tuple(float(v) for v in z["hyper"])
    per = B // world
    m = g.Model(vocab, padded, n_layer, n_head, n_embd, block, per, T, mode=g.MODE_TF32X3)
    m.set_params(params)
    tok = torch.from_numpy(tokens[rank * per:(rank + 1) * per].reshape(-1).copy()).cuda()
    tgt = torch.from_numpy(targets[rank * per:(rank + 1) * per].reshape(-1).copy()).cuda()
    step = dp.DataParallelStep(m, torch.device("cuda", rank), shard_optimizer=shard)
    assert step(tok, tgt, *hyper, 1) == 0
    torch.cuda.synchronize()
    grads = np.empty_like(params)
    m.get_grads(grads)
    after = np.empty_like(params)
    m.get_params(after)
    ok = True
    if rank == 0:
        full = g.Model(vocab, padded, n_layer, n_head, n_embd, block, B, T, mode=g.MODE_TF32X3)
        full.set_params(params)
        ft = torch.from_numpy(tokens.reshape(-1).copy()).cuda()
        fg = torch.from_numpy(targets.reshape(-1).copy()).cuda()
        assert full.forward(ft, fg) == 0 and full.backward() == 0 and full.update(*hyper, 1) == 0
        torch.cuda.synchronize()
        want_g = np.empty_like(params)
        full.get_grads(want_g)
        want_p = np.empty_like(params)
        full.get_params(want_p)
        eg = np.abs(grads - want_g).max() / np.abs(want_g).max()
        # AdamW's first step moves a weight by lr * g / (|g| + eps) + lr * wd * p: almost independent of |g|,
        # so wherever the gradient is clearly non-zero (above 1e-4 of the largest, ten times the bound on the
        # gradient error itself) the two runs must land on the same parameter to 1e-6. Only where g is within
        # rounding of zero may the runs disagree on its sign, and there the parameters are within 2 * lr.
        gmax = np.abs(want_g).max()
        clear = np.abs(want_g) > 1e-4 * gmax
        ep_clear = np.abs(after - want_p)[clear].max()
        ep_rest = np.abs(after - want_p)[~clear].max() if (~clear).any() else 0.0
        ep = max(ep_clear, ep_rest)
        out["clear_fraction"] = float(clear.mean())
        calls = step.sharded.calls if shard else step.exchange.calls
        if shard:
            # only this rank's slices hold averaged gradients: compare those
            mask = np.zeros(params.size, bool)
            sx = dp.ShardedExchange(torch.zeros(1), torch.zeros(1))
            sx.world, sx.rank = world, rank
            sx.ranges = [step.block[l] for l in range(n_layer)] + [step.lnf, step.embed]
            for first, count in sx.owned():
                mask[first:first + count] = True
            eg = np.abs(grads - want_g)[mask].max() / np.abs(want_g).max()
        ok = bool(eg <= 1e-5 and ep_clear <= 1e-6 and ep_rest <= 2 * hyper[0] and clear.mean() > 0.5
                  and calls == n_layer + (2 if shard else 1))
        out["err"] = (float(eg), float(ep_clear), float(ep_rest), calls)
    # the update really ran over every range this rank is responsible for (all of them when replicated)
    moved = after != params
    if shard:
        sx = dp.ShardedExchange(torch.zeros(1), torch.zeros(1))
        sx.world, sx.rank = world, rank
        sx.ranges = [step.block[l] for l in range(n_layer)] + [step.lnf, step.embed]
        mine = sx.owned()
    else:
        mine = [(lo, hi - lo) for lo, hi in [step.block[l] for l in range(n_layer)] + [step.lnf, step.embed]]
    for first, count in mine:
        if count > 0 and np.any(params[first:first + count] != 0):
            ok = ok and bool(moved[first:first + count].any())
    # every rank holds the same parameters (and, with the all-reduce, the same averaged gradients)
    t = torch.from_numpy(after if shard else grads).cuda()
    ref = t.clone()
    dist.broadcast(ref, 0)
    ok = ok and bool(torch.equal(t, ref))
    out[rank] = ok
    dist.destroy_process_group()


@pytest.mark.parametrize("shard", [False, True])  # all-reduce + replicated AdamW / reduce-scatter + sharded AdamW
def test_two_gpu_step_equals_one_gpu_step_on_the_whole_batch(gpu, shard):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(2, 29600 + os.getpid() % 1000 + int(shard), out, shard), nprocs=2, join=True)
    print("two-GPU step vs one-GPU step:", dict(out))
    assert out.get(0) and out.get(1), dict(out)
