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
    """experts_forward stand-in: out = rows * sum over the row's local experts of (expert id + 1) * weight
    (int64, wrapping); a row arrives once per owner rank with the other ranks' experts set to -1"""
    n_routed_experts = 8

    def experts_forward(self, start_pos, rows, weights, indices, base=None, max_pairs=None):
        assert max_pairs is not None and int(((indices >= 0)).sum()) == max_pairs
        assert indices.shape == weights.shape and indices.shape[0] == rows.shape[0]
        lo = self.n_routed_experts // dist.get_world_size() * dist.get_rank()
        hi = lo + self.n_routed_experts // dist.get_world_size()
        local = (indices >= lo) & (indices < hi)
        assert bool((local | (indices == -1)).all()), "an expert id of another rank was not masked"
        assert bool(local.any(1).all()), "a row reached a rank that owns none of its experts"
        return rows * ((indices + 1) * weights * local).sum(1, keepdim=True)


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
        # no GPUs for the ranks of this group: the peer-memory exchange must declare itself unavailable, so that
        # MoE.forward takes the collective path below
        assert not par.peer_available()
        y, side = par.expert_parallel_forward(FakeMoE(), 0, x, weights, indices, before_sync=lambda: 7)
        assert side == 7
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
    idx = torch.tensor([[0, 5], [7, 6], [3, 4], [1, 2]])          # tokens 1 and 3 keep both experts on one rank
    order, counts, dest = par.dispatch_plan(idx, 8, 2)
    assert counts.tolist() == [[3, 4], [3, 4]]                      # rows (one per token and owner rank), pairs
    assert dest.tolist() == [[0, 1], [1, 1], [0, 1], [0, 0]]
    pairs = order[:6].tolist()                                      # r * T + t, by rank then token
    assert pairs == [0 * 4 + 0, 0 * 4 + 2, 0 * 4 + 3, 1 * 4 + 0, 1 * 4 + 1, 1 * 4 + 2]


def _vocab_worker(rank, world, port, out):
    """vocabulary-parallel embedding (masked lookup + all_reduce, model.py:104-150) and the gather of the
    logits' vocabulary slices (model.py:1577-1580) on CPU ranks"""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M = importlib.import_module(PKG + ".model")
        M.world_size, M.rank = world, rank
        vocab, dim, B = 64, 12, 5
        g = torch.Generator().manual_seed(7)                      # the same table and tokens on every rank
        table = torch.randint(-2**40, 2**40, (vocab, dim), generator=g, dtype=torch.int64)
        tokens = torch.randint(0, vocab, (B, 9), generator=g)
        emb = M.ParallelEmbedding(vocab, dim)
        assert emb.weight.shape == (vocab // world, dim)
        emb.weight = table[rank * (vocab // world):(rank + 1) * (vocab // world)].clone()
        got = emb(tokens.clone())
        ok = bool(torch.equal(got, torch.nn.functional.embedding(tokens, table)))
        # logits: every rank holds the columns of its vocabulary slice; gathered in rank order
        logits_full = torch.randint(-2**30, 2**30, (1, B, vocab), generator=g, dtype=torch.int64)
        part = logits_full[..., rank * (vocab // world):(rank + 1) * (vocab // world)].contiguous()
        gathered = M._all_gather_last(part)
        ok = ok and bool(torch.equal(gathered, logits_full))
        ok = ok and bool(torch.equal(gathered.argmax(-1), logits_full.argmax(-1)))
        out[rank] = ok
    finally:
        dist.destroy_process_group()


def test_vocab_parallel_embedding_and_logits_gather():
    mgr = mp.Manager()
    out = mgr.dict()
    port = 29900 + os.getpid() % 90
    mp.spawn(_vocab_worker, args=(2, port, out), nprocs=2, join=True)
    assert dict(out) == {0: True, 1: True}
