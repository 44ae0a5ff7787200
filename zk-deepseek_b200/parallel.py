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

On GPUs of one node the rows do not travel through a collective at all (`PeerExchange`,
`expert_parallel_forward_peer`): every rank publishes its token rows in a symmetric buffer that the other
processes have mapped, the owner's limb split reads the rows it needs in place over NVLink (the dispatch
is part of the first expert GEMM's operand preparation), and the owner's combine kernel writes each
token's weighted sum straight into a slot of the token's home GPU, which adds the slots it expects.  The
only collective left is an all-gather of the routing tables (ids and weights, 16 k bytes per token); two
bounded flag barriers in peer memory order one layer call after the other.  The NCCL all-to-all path above stays for CPU
(gloo) runs and for process groups without symmetric memory.
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


class PeerExchange:
    """Symmetric buffers of one process group for expert parallelism over peer memory: token rows
    `[capacity, dim]`, result slots `[capacity, world, dim]`, `world` barrier flags.  Every rank must create it
    and call it with the same capacity (the bench and the model split the tokens evenly); fewer tokens than
    the capacity are fine."""

    def __init__(self, group, capacity, dim, device):
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 16:
            raise ValueError("PeerExchange handles up to 16 GPUs of one node")
        self.capacity, self.dim, self.device = int(capacity), int(dim), device
        n_x, n_slots = self.capacity * dim, self.capacity * self.world * dim
        self.buf = symm.empty((n_x + n_slots + self.world,), dtype=torch.int64, device=device)
        self.buf[n_x + n_slots:].zero_()
        self.handle = symm.rendezvous(self.buf, self.group)
        base = [int(p) for p in self.handle.buffer_ptrs]
        self.x_ptrs = base
        self.slot_ptrs = [b + 8 * n_x for b in base]
        self.flag_ptrs = [b + 8 * (n_x + n_slots) for b in base]
        self.x_local = self.buf[:n_x].view(self.capacity, dim)
        self.slots_local = self.buf[n_x:n_x + n_slots].view(self.capacity, self.world, dim)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.epoch = 0
        torch.cuda.synchronize(device)
        dist.barrier(group=group)            # every rank's flags are zero before anyone announces an epoch

    def barrier(self, K):
        self.epoch += 1
        K.peer_barrier(self.flag_ptrs, self.rank, self.epoch, self.status)

    def raise_if_timed_out(self):
        """host check (synchronises the stream): a barrier's bounded wait ran out on this rank"""
        if int(self.status.item()):
            raise RuntimeError("peer barrier timed out on rank %d: a rank did not reach the barrier" % self.rank)


_exchanges = {}
_peer_ok = None


def peer_available(group=None):
    """True when the peer-memory exchange can serve this process group: torch's symmetric memory is present,
    at most 16 ranks, all of them on this node (one GPU each), an NCCL group.  Decided once; the same on every
    rank."""
    global _peer_ok
    if _peer_ok is None:
        import os
        try:
            import torch.distributed._symmetric_memory  # noqa: F401
            world = dist.get_world_size(group)
            local = int(os.environ.get("LOCAL_WORLD_SIZE", world))
            _peer_ok = (world <= 16 and local == world and torch.cuda.device_count() >= world
                        and "nccl" in str(dist.get_backend(group)))
        except Exception:
            _peer_ok = False
    return _peer_ok


def peer_exchange(group, tokens, dim, device):
    """the PeerExchange of this group, created (collectively) on first use or when more tokens are needed"""
    key = id(group) if group is not None else 0
    ex = _exchanges.get(key)
    if ex is None or ex.capacity < tokens or ex.dim != dim:
        if ex is not None:
            torch.cuda.synchronize(device)
            dist.barrier(group=group)        # nobody still reads the old buffers
        ex = _exchanges[key] = PeerExchange(group, tokens, dim, device)
    return ex


def expert_parallel_forward_peer(moe, K, start_pos, x, weights, indices, group=None, before_sync=None, base=None):
    """expert_parallel_forward over peer memory (GPUs of one node).  `before_sync` as there; `base` (or the result
    of before_sync, when it is a [T, dim] tensor) is added to the sum.  Returns (y, side)."""
    T, k = indices.shape
    dim = x.shape[1]
    ex = peer_exchange(group, T, dim, x.device)
    world, rank, cap = ex.world, ex.rank, ex.capacity
    per_rank = moe.n_routed_experts // world
    # publish: rows into the symmetric buffer, routing tables to every rank
    ex.x_local[:T].copy_(x)
    meta = torch.empty((cap, 2 * k), dtype=torch.int64, device=x.device)
    meta[:T, :k] = indices
    meta[:T, k:] = weights
    if T < cap:
        meta[T:, :k] = -1
        meta[T:, k:] = 0
    meta_all = torch.empty((world * cap, 2 * k), dtype=torch.int64, device=x.device)
    dist.all_gather_into_tensor(meta_all, meta, group=group)
    idx_all = meta_all[:, :k].contiguous()
    w_all = meta_all[:, k:].contiguous()
    # pairs this rank owns, on their way to the host behind the shared expert (sizes the grouped GEMMs)
    mine = (idx_all >= rank * per_rank) & (idx_all < (rank + 1) * per_rank)
    n_mine = mine.sum().to(torch.int64).reshape(1)
    host = torch.empty(1, dtype=torch.int64, pin_memory=True)
    host.copy_(n_mine, non_blocking=True)
    ev = torch.cuda.Event()
    ev.record()
    ex.barrier(K)                       # every rank's rows are in place; the previous call's slots have been read
    side = before_sync() if before_sync is not None else None
    ev.synchronize()
    local_pairs = int(host[0])
    if local_pairs:
        moe.experts_forward(start_pos, None, w_all, idx_all, max_pairs=local_pairs,
                            parts=(ex.x_ptrs, cap), combine=lambda out, pos: K.moe_combine_peer(
                                out, pos, w_all, cap, ex.slot_ptrs, rank))
    ex.barrier(K)                       # every owner's slots have arrived
    if base is None and torch.is_tensor(side):
        base = side.reshape(T, dim)
    y = K.moe_sum_slots(base, ex.slots_local[:T], indices.contiguous(), per_rank)
    return y, side
