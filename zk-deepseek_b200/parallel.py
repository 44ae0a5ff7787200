"""Multi-GPU pieces of the integer forward pass: one process per GPU, NCCL through
torch.distributed (gloo on CPU in the tests of the index logic).

Expert parallelism (replaces the reference's full-tensor all_reduce, model.py:1381-1382):
each rank holds the tokens it gated and `n_routed_experts / world_size` experts.  Token rows
go to the ranks owning their experts with one all-to-all, the owners run the grouped expert
GEMMs, and the weighted results come back with a second all-to-all.  Exact: every expert output
is complete on its owner, the `* w // 2^23` is applied per (token, expert) before the order-free
integer sum.
"""
import torch
import torch.distributed as dist


def dispatch_plan(indices, n_experts, world):
    """Host-free bookkeeping of the dispatch.  indices [T, k] global expert ids.
    Returns (order, send_counts) where order sorts the T*k (token, slot) pairs by destination
    rank (stable), and send_counts [world] counts the pairs per destination."""
    per_rank = n_experts // world
    dest = (indices.flatten() // per_rank).to(torch.int64)
    order = torch.argsort(dest, stable=True)
    send_counts = torch.bincount(dest, minlength=world)
    return order, send_counts


def exchange_counts(send_counts, group=None):
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    return recv_counts


def all_to_all_rows(rows, send_counts, recv_counts, group=None):
    """rows [sum(send_counts), C] sorted by destination -> [sum(recv_counts), C] grouped by source"""
    out = rows.new_empty((int(sum(recv_counts)),) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=list(recv_counts),
                           input_split_sizes=list(send_counts), group=group)
    return out


def expert_parallel_forward(moe, start_pos, x, weights, indices, group=None):
    """sum over ALL experts of expert(x) * w // 2^23 for this rank's tokens x [T, dim]."""
    world = dist.get_world_size(group)
    T, k = indices.shape
    order, send_counts = dispatch_plan(indices, moe.n_routed_experts, world)
    recv_counts = exchange_counts(send_counts, group)
    sc, rc = send_counts.tolist(), recv_counts.tolist()     # split sizes are host arguments of NCCL
    tok = order // k
    rows = x[tok]                                            # [T*k, dim] sorted by destination
    ids = indices.flatten()[order].contiguous()
    wts = weights.flatten()[order].contiguous()
    r_rows = all_to_all_rows(rows, sc, rc, group)
    r_ids = all_to_all_rows(ids[:, None], sc, rc, group)
    r_wts = all_to_all_rows(wts[:, None], sc, rc, group)
    # every received row is one (token, expert) pair: k = 1 routing on the owner
    out = moe.experts_forward(start_pos, r_rows, r_wts, r_ids)
    back = all_to_all_rows(out, rc, sc, group)               # weighted expert outputs, sender order
    y = torch.zeros_like(x)
    y.index_add_(0, tok, back)
    return y
