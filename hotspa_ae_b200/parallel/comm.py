"""Differentiable collectives on local shards (the executor's baseline communication path).

Each Function pairs a forward collective with its dual in backward, the way a CommOp's gradient is
again a CommOp in the reference (hetu/graph/ops/Communication.cc:586-621):
all-gather <-> reduce-scatter, all-reduce <-> identity, identity <-> all-reduce, slice <-> all-gather.
NCCL on GPUs; gloo fall-backs (all_reduce / all_gather lists) keep the same code testable on CPU.
The fused compute+collective kernels replace these on the hot path (see parallel/symm.py).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _world(group) -> int:
    return dist.get_world_size(group) if group is not None else 1


def _rank(group) -> int:
    return dist.get_rank(group) if group is not None else 0


def all_gather_dim0(x: torch.Tensor, group) -> torch.Tensor:
    n = _world(group)
    if n == 1:
        return x
    x = x.contiguous()
    out = torch.empty((n * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    if x.is_cuda:
        dist.all_gather_into_tensor(out, x, group=group)
    else:
        dist.all_gather(list(out.chunk(n, dim=0)), x, group=group)
    return out


def reduce_scatter_dim0(x: torch.Tensor, group) -> torch.Tensor:
    n = _world(group)
    if n == 1:
        return x
    x = x.contiguous()
    if x.is_cuda:
        out = torch.empty((x.shape[0] // n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x, group=group)
        return out
    y = x.clone()
    dist.all_reduce(y, group=group)
    return y.chunk(n, dim=0)[_rank(group)].contiguous()


def all_reduce(x: torch.Tensor, group) -> torch.Tensor:
    if _world(group) == 1:
        return x
    y = x.contiguous().clone()
    dist.all_reduce(y, group=group)
    return y


def _move(x, dim):
    return x if dim == 0 else x.transpose(0, dim)


class AllGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, dim):
        ctx.group, ctx.dim = group, dim
        return _move(all_gather_dim0(_move(x, dim).contiguous(), group), dim)

    @staticmethod
    def backward(ctx, g):
        return _move(reduce_scatter_dim0(_move(g, ctx.dim).contiguous(), ctx.group), ctx.dim), None, None


class ReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, dim):
        ctx.group, ctx.dim = group, dim
        return _move(reduce_scatter_dim0(_move(x, dim).contiguous(), group), dim)

    @staticmethod
    def backward(ctx, g):
        return _move(all_gather_dim0(_move(g, ctx.dim).contiguous(), ctx.group), ctx.dim), None, None


class AllReduce(torch.autograd.Function):
    """partial -> duplicate; the gradient of a duplicated sum flows back unchanged."""

    @staticmethod
    def forward(ctx, x, group):
        return all_reduce(x, group)

    @staticmethod
    def backward(ctx, g):
        return g, None


class CopyToGroup(torch.autograd.Function):
    """duplicate consumed by differently-sharded weights: identity forward, all-reduce backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return all_reduce(g, ctx.group), None


class SplitLocal(torch.autograd.Function):
    """duplicate -> split along `dim`: keep the local slice forward, all-gather backward."""

    @staticmethod
    def forward(ctx, x, group, dim, index, count):
        ctx.group, ctx.dim = group, dim
        return x.chunk(count, dim=dim)[index].contiguous()

    @staticmethod
    def backward(ctx, g):
        return _move(all_gather_dim0(_move(g, ctx.dim).contiguous(), ctx.group), ctx.dim), None, None, None, None


# ---------------------------------------------------------------------------------------------------------------
# Heterogeneous ("split") collectives: the members of a DS union shard the tensor with different counts, so a rank's
# shard is cut into micro-blocks of the finest granularity and every micro-block runs its collective over the group
# of its holders, one per member (reference: hetu/graph/ops/Communication.cc:990-1202; group construction :248-392,
# here `_core.split_comm_groups`).  `groups[i]` is the list of process groups of micro-block i that contain this
# rank; holders that duplicate a block carry identical data (the local pre-collective ran before), so when a
# micro-block has several groups the last result stands.
# ---------------------------------------------------------------------------------------------------------------

def split_collective_groups(local_ds_list, rank_groups, rank=None):
    """Plan of the split collectives for `rank`: (split_dim, micro_blocks, [[ranks...] per group] per micro-block)."""
    from .. import core as _core
    from . import mesh as M
    rank = M.mesh().rank if rank is None else rank
    plan = _core.split_comm_groups(list(local_ds_list), [list(g) for g in rank_groups], int(rank))
    return plan.split_dim, plan.micro_blocks, [[tuple(g) for g in gs] for gs in plan.groups]


def ensure_split_groups(local_ds_list, rank_groups):
    """Create, collectively and in one order on all ranks, every process group any member rank will use."""
    from . import mesh as M
    every = set()
    for g in rank_groups:
        for r in g:
            for gs in split_collective_groups(local_ds_list, rank_groups, r)[2]:
                every.update(gs)
    M.mesh().ensure_groups(sorted(every))


def _resolve(groups):
    from . import mesh as M
    return [[M.mesh().group(g) if isinstance(g, (tuple, list)) else g for g in gs] for gs in groups]


def _split_apply(x, groups, dim, fn):
    groups = _resolve(groups)
    parts = _move(x, dim).contiguous().chunk(len(groups), dim=0)
    outs = []
    for part, gs in zip(parts, groups):
        res = part
        for g in gs:
            res = fn(part.contiguous(), g)
        outs.append(res)
    return _move(torch.cat(outs, dim=0), dim).contiguous()


def split_all_reduce(x, groups, dim=0):
    return _split_apply(x, groups, dim, all_reduce)


def split_all_gather(x, groups, dim=0):
    return _split_apply(x, groups, dim, all_gather_dim0)


def split_reduce_scatter(x, groups, dim=0):
    return _split_apply(x, groups, dim, reduce_scatter_dim0)


class SplitAllReduce(torch.autograd.Function):
    """partial over the union -> duplicate; micro-block i is summed over groups[i]."""

    @staticmethod
    def forward(ctx, x, groups, dim):
        return split_all_reduce(x, groups, dim)

    @staticmethod
    def backward(ctx, g):
        return g, None, None


class SplitAllGather(torch.autograd.Function):
    """split over the union -> duplicate; micro-block i grows by the size of its group along `dim`."""

    @staticmethod
    def forward(ctx, x, groups, dim):
        ctx.groups, ctx.dim = groups, dim
        return split_all_gather(x, groups, dim)

    @staticmethod
    def backward(ctx, g):
        return split_reduce_scatter(g, ctx.groups, ctx.dim), None, None


class SplitReduceScatter(torch.autograd.Function):
    """partial over the union -> split; micro-block i is summed and scattered over groups[i] along `dim`."""

    @staticmethod
    def forward(ctx, x, groups, dim):
        ctx.groups, ctx.dim = groups, dim
        return split_reduce_scatter(x, groups, dim)

    @staticmethod
    def backward(ctx, g):
        return split_all_gather(g, ctx.groups, ctx.dim), None, None


def combine_ce_stats(stats: torch.Tensor, group) -> torch.Tensor:
    """(max, sum-exp, target) per row of every vocab shard -> global (max, sum-exp, target).
    One small all-gather instead of the reference's three all-reduces
    (hetu/graph/ops/VocabParallelCrossEntropyLoss.cc:61-101)."""
    n = _world(group)
    if n == 1:
        return stats
    allst = all_gather_dim0(stats.contiguous()[None], group)          # [n, rows, 3]
    m = allst[:, :, 0]
    gmax = m.max(dim=0).values
    gsum = (allst[:, :, 1] * (m - gmax[None]).exp()).sum(dim=0)
    gtgt = allst[:, :, 2].sum(dim=0)
    return torch.stack([gmax, gsum, gtgt], dim=1)


def p2p_exchange(sends, recvs):
    """sends: [(tensor, peer_rank)], recvs: [(shape, dtype, device, peer_rank)] -> received tensors.
    All transfers are posted as one group (ncclGroupStart/End) so opposite directions cannot deadlock."""
    ops, outs = [], []
    for t, peer in sends:
        ops.append(dist.P2POp(dist.isend, t.contiguous(), peer))
    for shape, dtype, device, peer in recvs:
        buf = torch.empty(shape, dtype=dtype, device=device)
        outs.append(buf)
        ops.append(dist.P2POp(dist.irecv, buf, peer))
    if ops:
        for r in dist.batch_isend_irecv(ops):
            r.wait()
    return outs
