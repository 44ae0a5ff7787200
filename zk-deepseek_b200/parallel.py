"""Multi-GPU pieces of the integer forward pass: one process per GPU, NCCL through
torch.distributed (gloo on CPU in the tests of the index logic).

Expert parallelism (replaces the reference's full-tensor all_reduce, model.py:1381-1382):
each rank holds the tokens it gated and `n_routed_experts / world_size` experts.  A token row
travels ONCE to every rank that owns at least one of its experts (with DeepSeek-V3's grouped
routing, 4 of 8 groups, that is at most four ranks for eight experts), together with the ids and
weights of the token's experts on that rank.  The owner runs its grouped expert GEMMs on the rows
it received, sums each row's weighted expert outputs, and the sums come back with a second
all-to-all.  Exact: every expert output is complete on its owner, `* w // 2^23` is applied per
(token, expert) before the order-free integer sums.

Collectives per layer: one small all-to-all of row counts, one of packed rows
(`dim + 2 k` words: the row, k expert ids, k weights), one of result rows.  NCCL wants the split
sizes on the host: the counts are copied to pinned memory right after the gate, `before_sync`
(the shared expert) is launched, and only then does the host wait for the copy, so the GPU never
idles on that read-back.
"""
import torch
import torch.distributed as dist


def dispatch_plan(indices, n_experts, world):
    """Device-side bookkeeping of the dispatch, no host synchronisation.  indices [T, k] global
    expert ids.  Returns
      pair_order [world * T]: (rank, token) pairs as r * T + t, those that exist first, ordered by
                              destination rank then token (stable);
      send_counts [world, 2]: rows and (token, expert) pairs per destination rank;
      dest [T, k]:            owner rank of every (token, slot)."""
    T, k = indices.shape
    per_rank = n_experts // world
    dest = (indices // per_rank).to(torch.int64)
    member = torch.zeros((T, world), dtype=torch.bool, device=indices.device)
    member.scatter_(1, dest, torch.ones_like(dest, dtype=torch.bool))
    flat = member.t().reshape(-1)                       # rank-major: index r * T + t
    pair_order = torch.argsort(flat.to(torch.int8), descending=True, stable=True)
    # rows per destination, and (token, expert) pairs per destination: the owner sizes its grouped GEMMs by them
    send_counts = torch.stack([member.sum(0).to(torch.int64),
                               torch.zeros(world, dtype=torch.int64, device=indices.device).index_add_(
                                   0, dest.flatten(), torch.ones(T * k, dtype=torch.int64, device=indices.device))], dim=1)
    return pair_order, send_counts, dest


class _HostCounts:
    """send / receive counts on their way to the host: a pinned buffer and the event of its copy"""

    def __init__(self, send_counts, group):
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts.contiguous(), group=group)
        both = torch.stack([send_counts, recv_counts])
        if both.is_cuda:
            self.host = torch.empty(both.shape, dtype=both.dtype, pin_memory=True)
            self.host.copy_(both, non_blocking=True)
            self.event = torch.cuda.Event()
            self.event.record()
        else:
            self.host, self.event = both, None

    def wait(self):
        if self.event is not None:
            self.event.synchronize()
        return (self.host[0, :, 0].tolist(), self.host[1, :, 0].tolist(), int(self.host[1, :, 1].sum()))


def expert_parallel_forward(moe, start_pos, x, weights, indices, group=None, before_sync=None):
    """sum over ALL experts of expert(x) * w // 2^23 for this rank's tokens x [T, dim].
    before_sync: optional callable run after the counts are on their way to the host and before the
    host waits for them (work that needs neither); its result is returned as the second value."""
    world = dist.get_world_size(group)
    T, k = indices.shape
    dim = x.shape[1]
    pair_order, send_counts, dest = dispatch_plan(indices, moe.n_routed_experts, world)
    counts = _HostCounts(send_counts, group)
    side = before_sync() if before_sync is not None else None
    sc, rc, local_pairs = counts.wait()
    n_send, n_recv = sum(sc), sum(rc)

    pairs = pair_order[:n_send]
    rank_of = pairs // T if T else pairs
    tok = pairs - rank_of * T
    # one packed row per (token, destination): the row, then the token's k expert ids with those owned
    # by other ranks replaced by -1, then its k weights
    packed = torch.empty((n_send, dim + 2 * k), dtype=torch.int64, device=x.device)
    packed[:, :dim] = x[tok]
    here = dest[tok] == rank_of[:, None]
    packed[:, dim:dim + k] = torch.where(here, indices[tok], torch.full_like(indices[tok], -1))
    packed[:, dim + k:] = weights[tok]
    recv = torch.empty((n_recv, dim + 2 * k), dtype=torch.int64, device=x.device)
    dist.all_to_all_single(recv, packed, output_split_sizes=rc, input_split_sizes=sc, group=group)
    del packed

    # the owner: every received row with its (up to k) local experts; rows come back already weighted
    # and summed over this rank's experts
    if n_recv:
        out = moe.experts_forward(start_pos, recv[:, :dim].contiguous(), recv[:, dim + k:].contiguous(),
                                  recv[:, dim:dim + k].contiguous(), max_pairs=local_pairs)
    else:
        out = recv[:, :dim]
    del recv
    back = torch.empty((n_send, dim), dtype=torch.int64, device=x.device)
    dist.all_to_all_single(back, out.contiguous(), output_split_sizes=sc, input_split_sizes=rc, group=group)
    y = torch.zeros_like(x)
    y.index_add_(0, tok, back)                      # at most `world` (in practice <= 4) rows per token
    return y, side
