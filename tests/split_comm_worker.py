"""Worker (4 gloo ranks): heterogeneous collectives between a member that duplicates a tensor on ranks 0, 1 and a
member that splits its rows over ranks 2, 3; and between a 2-way and a 1-way split."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import hetu as ht  # noqa: E402
from hotspa_ae_b200.parallel import comm as C  # noqa: E402

DS = ht.DistributedStates


def main():
    ht.init_comm_group(8)
    rank = int(os.environ["RANK"])
    rows, cols = 8, 3
    base = torch.arange(rows * cols, dtype=torch.float32).reshape(rows, cols)

    # --- union A: member 0 = ranks (0, 1) duplicate, member 1 = ranks (2, 3) split rows 2-way -------------------
    local = [DS(2, {-1: 2}, [-1]), DS(2, {0: 2}, [0])]
    rgroups = [[0, 1], [2, 3]]
    C.ensure_split_groups(local, rgroups)
    dim, micro, groups = C.split_collective_groups(local, rgroups)
    assert dim == 0
    if rank < 2:
        assert micro == 2 and groups == [[(rank, 2)], [(rank, 3)]], groups
        mine = base * 10                                   # member 0's partial value (same on both duplicates)
    else:
        assert micro == 1 and groups == [[(0, rank), (1, rank)]], groups
        mine = (base * 1).chunk(2, dim=0)[rank - 2]        # member 1's partial value, this rank's rows
    x = mine.clone().requires_grad_(True)
    y = C.SplitAllReduce.apply(x, groups, 0)
    want = base * 11
    want = want if rank < 2 else want.chunk(2, dim=0)[rank - 2]
    assert torch.equal(y.detach(), want), (rank, y, want)
    y.sum().backward()
    assert torch.equal(x.grad, torch.ones_like(x))

    # --- union B: member 0 = rank 0 holds all rows, member 1 = ranks (2, 3) split rows; rank 1 idle ---------------
    local = [DS(1, {}, []), DS(2, {0: 2}, [0])]
    rgroups = [[0], [2, 3]]
    C.ensure_split_groups(local, rgroups)
    if rank != 1:
        dim, micro, groups = C.split_collective_groups(local, rgroups)
        part = base if rank == 0 else base.chunk(2, dim=0)[rank - 2]
        part = part * (rank + 1)
        # reduce-scatter: every micro-block is summed over (rank 0, holder) and split between the two
        x = part.clone().requires_grad_(True)
        y = C.SplitReduceScatter.apply(x, groups, 0)
        if rank == 0:
            assert micro == 2 and y.shape == (rows // 2, cols)
            want = torch.cat([base[0:2] * (1 + 3), base[4:6] * (1 + 4)])
        else:
            assert micro == 1 and y.shape == (rows // 4, cols)
            lo = (rank - 2) * 4 + 2
            want = base[lo:lo + 2] * (1 + rank + 1)
        assert torch.equal(y.detach(), want), (rank, y, want)
        # all-gather is its dual: gradient of the gather is the reduce-scatter of the incoming gradient
        z = C.SplitAllGather.apply(y, groups, 0)
        assert z.shape == part.shape
        z.sum().backward()
        assert torch.equal(x.grad, torch.full_like(x, 2.0)), x.grad
    torch.distributed.barrier()
    if rank == 0:
        print("SPLIT_COMM_OK")


if __name__ == "__main__":
    main()
