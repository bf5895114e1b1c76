"""Communication groups with the full verb set of the reference's NCCL backend
(hetu/impl/communication/nccl_comm_group.cu:139-717, base class hetu/impl/communication/comm_group.h:23-181):
Broadcast, AllReduce, AllReduceCoalesce, AlltoAll, Reduce, AllGather, ReduceScatter, Gather, Scatter, Send, Recv,
ISend/IRecv handed back as tasks, BatchedISendIRecv, Barrier, Sync.

One `CommunicationGroup` per ordered rank list, cached process-wide (`get_or_create`, `empty_cache`); ranks are world
ranks, `group.rank` is the position inside the group.  Transport is `torch.distributed` (NCCL on GPUs, gloo on CPU);
collectives run on the caller's current stream, so passing work to a named stream is a `with torch.cuda.stream(...)`
around the call.  Gloo lacks a few verbs (reduce_scatter, all_to_all, gather/scatter on some builds); those fall back
to compositions of the verbs it has, which keeps every path testable on CPU ranks.
"""
from __future__ import annotations

from typing import Sequence

import torch
import torch.distributed as dist

from . import mesh as M

_REDUCE = {
    "sum": dist.ReduceOp.SUM, "mean": dist.ReduceOp.SUM, "avg": dist.ReduceOp.SUM,
    "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN, "prod": dist.ReduceOp.PRODUCT,
}

_CACHE: dict[tuple, "CommunicationGroup"] = {}


class Task:
    """Handle of a non-blocking send/receive (or a list of them)."""

    def __init__(self, works):
        self._works = [w for w in works if w is not None]

    def wait(self) -> None:
        for w in self._works:
            w.wait()
        self._works = []

    def is_completed(self) -> bool:
        return all(w.is_completed() for w in self._works)


class CommunicationGroup:
    def __init__(self, world_ranks: Sequence[int]):
        self.world_ranks = tuple(int(r) for r in world_ranks)
        if len(set(self.world_ranks)) != len(self.world_ranks):
            raise ValueError(f"duplicate ranks in {self.world_ranks}")
        mesh = M.mesh()
        self.size = len(self.world_ranks)
        self.rank = self.world_ranks.index(mesh.rank) if mesh.rank in self.world_ranks else -1
        self._pg = mesh.group(self.world_ranks)
        self._gloo = (not mesh.use_cuda)

    # ------------------------------------------------------------------ construction / cache
    @staticmethod
    def get_or_create(world_ranks: Sequence[int]) -> "CommunicationGroup":
        """Collective over the whole job the first time a rank list is seen (process groups are created by all)."""
        key = tuple(int(r) for r in world_ranks)
        if key not in _CACHE:
            M.mesh().ensure_groups([key])
            _CACHE[key] = CommunicationGroup(key)
        return _CACHE[key]

    @staticmethod
    def empty_cache() -> None:
        _CACHE.clear()

    def world_rank(self, group_rank: int) -> int:
        return self.world_ranks[group_rank]

    def _check(self) -> bool:
        if self.rank < 0:
            raise RuntimeError(f"rank {M.mesh().rank} is not a member of {self.world_ranks}")
        return self.size > 1

    # ------------------------------------------------------------------ collectives
    def broadcast(self, x: torch.Tensor, root: int = 0) -> torch.Tensor:
        if self._check():
            dist.broadcast(x, src=self.world_ranks[root], group=self._pg)
        return x

    def all_reduce(self, x: torch.Tensor, op: str = "sum") -> torch.Tensor:
        if self._check():
            dist.all_reduce(x, op=_REDUCE[op], group=self._pg)
        if op in ("mean", "avg"):
            x.div_(self.size)
        return x

    def all_reduce_coalesce(self, xs: Sequence[torch.Tensor], op: str = "sum") -> Sequence[torch.Tensor]:
        """One all-reduce over a flat copy of all tensors (same dtype), then scattered back in place."""
        xs = list(xs)
        if not xs:
            return xs
        if not self._check():
            return xs
        if len({x.dtype for x in xs}) != 1:
            raise TypeError("all_reduce_coalesce needs tensors of one dtype")
        flat = torch.cat([x.reshape(-1) for x in xs])
        self.all_reduce(flat, op)
        off = 0
        for x in xs:
            x.copy_(flat[off:off + x.numel()].view_as(x))
            off += x.numel()
        return xs

    def reduce(self, x: torch.Tensor, root: int = 0, op: str = "sum") -> torch.Tensor:
        if self._check():
            dist.reduce(x, dst=self.world_ranks[root], op=_REDUCE[op], group=self._pg)
        if op in ("mean", "avg") and self.rank == root:
            x.div_(self.size)
        return x

    def all_gather(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """Concatenate every member's `x` along dim 0."""
        x = x.contiguous()
        if out is None:
            out = torch.empty((self.size * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        if not self._check():
            out.copy_(x)
            return out
        if x.is_cuda:
            dist.all_gather_into_tensor(out, x, group=self._pg)
        else:
            dist.all_gather(list(out.chunk(self.size, dim=0)), x, group=self._pg)
        return out

    def reduce_scatter(self, x: torch.Tensor, out: torch.Tensor | None = None, op: str = "sum") -> torch.Tensor:
        """Reduce over the group and keep chunk `rank` of dim 0."""
        x = x.contiguous()
        if x.shape[0] % self.size:
            raise ValueError(f"reduce_scatter: dim 0 of {tuple(x.shape)} does not divide by {self.size}")
        if out is None:
            out = torch.empty((x.shape[0] // self.size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        if not self._check():
            out.copy_(x)
            return out
        if x.is_cuda:
            dist.reduce_scatter_tensor(out, x, op=_REDUCE[op], group=self._pg)
        else:
            y = x.clone()
            dist.all_reduce(y, op=_REDUCE[op], group=self._pg)
            out.copy_(y.chunk(self.size, dim=0)[self.rank])
        if op in ("mean", "avg"):
            out.div_(self.size)
        return out

    def all_to_all(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """Chunk j of dim 0 goes to member j; chunk i of the result came from member i."""
        x = x.contiguous()
        if x.shape[0] % self.size:
            raise ValueError(f"all_to_all: dim 0 of {tuple(x.shape)} does not divide by {self.size}")
        if out is None:
            out = torch.empty_like(x)
        if not self._check():
            out.copy_(x)
            return out
        if x.is_cuda:
            dist.all_to_all_single(out, x, group=self._pg)
            return out
        # gloo: the send/recv loop the reference uses for every backend
        sends, recvs = x.chunk(self.size, dim=0), out.chunk(self.size, dim=0)
        recvs[self.rank].copy_(sends[self.rank])
        ops = []
        for j in range(self.size):
            if j == self.rank:
                continue
            ops.append(dist.P2POp(dist.isend, sends[j].contiguous(), self.world_ranks[j], group=self._pg))
            ops.append(dist.P2POp(dist.irecv, recvs[j], self.world_ranks[j], group=self._pg))
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        return out

    def gather(self, x: torch.Tensor, root: int = 0) -> torch.Tensor | None:
        """Root receives the concatenation along dim 0; the others get None."""
        if not self._check():
            return x.clone()
        x = x.contiguous()
        if self.rank == root:
            out = torch.empty((self.size * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
            parts = list(out.chunk(self.size, dim=0))
            dist.gather(x, gather_list=parts, dst=self.world_ranks[root], group=self._pg)
            return out
        dist.gather(x, gather_list=None, dst=self.world_ranks[root], group=self._pg)
        return None

    def scatter(self, x: torch.Tensor | None, out: torch.Tensor, root: int = 0) -> torch.Tensor:
        """Member i receives chunk i of root's `x` (dim 0) into `out`."""
        if not self._check():
            out.copy_(x)
            return out
        if self.rank == root:
            parts = [c.contiguous() for c in x.chunk(self.size, dim=0)]
            dist.scatter(out, scatter_list=parts, src=self.world_ranks[root], group=self._pg)
        else:
            dist.scatter(out, scatter_list=None, src=self.world_ranks[root], group=self._pg)
        return out

    # ------------------------------------------------------------------ point to point
    def send(self, x: torch.Tensor, receiver: int) -> None:
        dist.send(x.contiguous(), dst=self.world_ranks[receiver], group=self._pg)

    def recv(self, out: torch.Tensor, sender: int) -> torch.Tensor:
        dist.recv(out, src=self.world_ranks[sender], group=self._pg)
        return out

    def isend(self, x: torch.Tensor, receiver: int) -> Task:
        return Task([dist.isend(x.contiguous(), dst=self.world_ranks[receiver], group=self._pg)])

    def irecv(self, out: torch.Tensor, sender: int) -> Task:
        return Task([dist.irecv(out, src=self.world_ranks[sender], group=self._pg)])

    def batched_isend_irecv(self, sends: Sequence[tuple], recvs: Sequence[tuple]) -> Task:
        """sends: (tensor, receiver group rank); recvs: (buffer, sender group rank).  Issued as one group of
        operations so that opposite-direction transfers between two members cannot deadlock."""
        ops = [dist.P2POp(dist.isend, t.contiguous(), self.world_ranks[r], group=self._pg) for t, r in sends]
        ops += [dist.P2POp(dist.irecv, t, self.world_ranks[r], group=self._pg) for t, r in recvs]
        return Task(dist.batch_isend_irecv(ops) if ops else [])

    # ------------------------------------------------------------------ synchronisation
    def barrier(self, sync: bool = True) -> None:
        """A one-element all-reduce, like the reference; `sync` also waits for the device."""
        if self._check():
            flag = torch.zeros(1, dtype=torch.int32, device=M.mesh().torch_device)
            dist.all_reduce(flag, group=self._pg)
            if sync:
                self.sync()

    def sync(self) -> None:
        if M.mesh().use_cuda:
            torch.cuda.current_stream().synchronize()

    def __repr__(self) -> str:
        return f"CommunicationGroup(ranks={list(self.world_ranks)}, rank={self.rank})"


def get_world_group() -> CommunicationGroup:
    return CommunicationGroup.get_or_create(range(M.mesh().world_size))
