"""Worker (4 gloo ranks): every verb of CommunicationGroup on the world group and on a 2-rank subgroup."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import hetu as ht  # noqa: E402
from hotspa_ae_b200.parallel.comm_group import CommunicationGroup, get_world_group  # noqa: E402


def main():
    ht.init_comm_group(8)
    rank = int(os.environ["RANK"])
    w = get_world_group()
    n = w.size
    assert n == 4 and w.rank == rank
    f = lambda r: torch.arange(8, dtype=torch.float32).reshape(4, 2) + 100 * r

    x = f(rank)
    w.broadcast(x, root=2)
    assert torch.equal(x, f(2))
    assert torch.equal(w.all_reduce(f(rank)), sum(f(r) for r in range(n)))
    assert torch.equal(w.all_reduce(f(rank), "max"), f(3))
    assert torch.allclose(w.all_reduce(f(rank), "mean"), sum(f(r) for r in range(n)) / n)
    a, b = f(rank), torch.ones(3) * rank
    w.all_reduce_coalesce([a, b])
    assert torch.equal(a, sum(f(r) for r in range(n))) and torch.equal(b, torch.ones(3) * 6)
    y = w.reduce(f(rank), root=1)
    if rank == 1:
        assert torch.equal(y, sum(f(r) for r in range(n)))
    assert torch.equal(w.all_gather(f(rank)), torch.cat([f(r) for r in range(n)]))
    assert torch.equal(w.reduce_scatter(f(rank)), sum(f(r) for r in range(n))[rank:rank + 1])
    got = w.all_to_all(f(rank))
    assert torch.equal(got, torch.cat([f(r)[rank:rank + 1] for r in range(n)])), got
    g = w.gather(f(rank), root=3)
    assert (g is None) == (rank != 3)
    if rank == 3:
        assert torch.equal(g, torch.cat([f(r) for r in range(n)]))
    out = torch.empty(1, 2)
    w.scatter(f(0) if rank == 0 else None, out, root=0)
    assert torch.equal(out, f(0)[rank:rank + 1])

    # ring exchange with the batched verb, then blocking and task-style point to point on a subgroup
    buf = torch.empty(4, 2)
    w.batched_isend_irecv([(f(rank), (rank + 1) % n)], [(buf, (rank - 1) % n)]).wait()
    assert torch.equal(buf, f((rank - 1) % n))
    sub = CommunicationGroup.get_or_create([1, 3])
    other = CommunicationGroup.get_or_create([0, 2])
    mine = sub if rank in (1, 3) else other
    assert mine.size == 2 and mine.world_rank(mine.rank) == rank
    peer = 1 - mine.rank
    if mine.rank == 0:
        mine.send(f(rank), peer)
        t = mine.irecv(buf, peer)
    else:
        mine.recv(buf, peer)
        assert torch.equal(buf, f(mine.world_rank(peer)))
        t = mine.isend(f(rank) * 2, peer)
    t.wait()
    if mine.rank == 0:
        assert torch.equal(buf, f(mine.world_rank(peer)) * 2)
    assert torch.equal(mine.all_reduce(torch.ones(2) * rank), torch.ones(2) * (4 if rank in (1, 3) else 2))
    try:
        (other if rank in (1, 3) else sub).all_reduce(torch.ones(1))
        raise AssertionError("a non-member must not be able to use the group")
    except RuntimeError:
        pass
    assert CommunicationGroup.get_or_create([1, 3]) is sub
    w.barrier()
    if rank == 0:
        print("COMM_GROUP_OK")


if __name__ == "__main__":
    main()
