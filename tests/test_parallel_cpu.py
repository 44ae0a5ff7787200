"""Expert-parallel dispatch / combine plumbing on CPU ranks (gloo, world_size 2): the
all-to-all bookkeeping of parallel.py with a stand-in for the local expert computation."""
import importlib
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PKG, ROOT


class FakeMoE:
    """experts_forward stand-in: out = rows * (expert id + 1) * weight (int64, wrapping)"""
    n_routed_experts = 8

    def experts_forward(self, start_pos, rows, weights, indices, base=None):
        assert indices.shape == (rows.shape[0], 1) and weights.shape == indices.shape
        lo = self.n_routed_experts // dist.get_world_size() * dist.get_rank()
        hi = lo + self.n_routed_experts // dist.get_world_size()
        assert bool(((indices >= lo) & (indices < hi)).all()), "a row reached a rank that does not own its expert"
        return rows * (indices + 1) * weights


def _worker(rank, world, port, T, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        par = importlib.import_module(PKG + ".parallel")
        g = torch.Generator().manual_seed(100 + rank)
        k, dim = 3, 6
        x = torch.randint(-1000, 1000, (T[rank], dim), generator=g, dtype=torch.int64)
        indices = torch.stack([torch.randperm(FakeMoE.n_routed_experts, generator=g)[:k] for _ in range(T[rank])]) \
            if T[rank] else torch.zeros((0, k), dtype=torch.int64)
        weights = torch.randint(1, 50, (T[rank], k), generator=g, dtype=torch.int64)
        y = par.expert_parallel_forward(FakeMoE(), 0, x, weights, indices)
        want = (x[:, None, :] * (indices + 1)[:, :, None] * weights[:, :, None]).sum(1)
        out[rank] = bool(torch.equal(y, want))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("T", [(5, 9), (0, 4), (16, 16)])
def test_expert_parallel_dispatch_and_combine(T):
    mgr = mp.Manager()
    out = mgr.dict()
    port = 29600 + (os.getpid() + sum(T)) % 300
    mp.spawn(_worker, args=(2, port, T, out), nprocs=2, join=True)
    assert dict(out) == {0: True, 1: True}


def test_dispatch_plan_orders_rows_by_destination():
    sys.path.insert(0, ROOT)
    par = importlib.import_module(PKG + ".parallel")
    idx = torch.tensor([[0, 5], [7, 2], [3, 4]])
    order, counts = par.dispatch_plan(idx, 8, 2)
    assert counts.tolist() == [3, 3]
    dest = (idx.flatten() // 4)[order]
    assert dest.tolist() == sorted(dest.tolist())
