"""Worker (3 gloo ranks): a comm op that changes the hetero dimension of a union.  Member A = ranks (0, 1), member B =
rank 2.  (1) partial over the members AND over A's two ranks -> duplicate everywhere: an all-reduce inside A, then a
split all-reduce across the members.  (2) rows split over the members -> duplicate: a split all-gather."""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import hetu as ht  # noqa: E402
from hotspa_ae_b200 import core as C  # noqa: E402

DS, DSU, DG = ht.DistributedStates, ht.DistributedStatesUnion, ht.DeviceGroup


def main():
    ht.init_comm_group(8)
    rank = int(os.environ["RANK"])
    member = 0 if rank < 2 else 1
    groups = [[DG([0, 1]), DG([2])]]
    # reference convention: a member's DS counts its devices times the number of members
    partial = [DSU([DS(4, {-2: 4}, [-2]), DS(2, {-2: 2}, [-2])], -2)]
    dup = [DSU([DS(4, {-1: 4}, [-1]), DS(2, {-1: 2}, [-1])], -1)]
    rows = [DSU([DS(4, {0: 2, -1: 2}, [0, -1]), DS(2, {0: 2}, [0])], 0)]
    with ht.graph("define_and_run", num_strategy=1) as g:
        x = ht.parallel_placeholder(ht.float32, [4, 3], partial, groups, name="x")
        y = ht.comm(x, dup, groups, name="sum_everything")
        r = ht.parallel_placeholder(ht.float32, [4, 3], rows, groups, name="r")
        z = ht.comm(r, dup, groups, name="gather_rows")
    base = np.arange(12, dtype=np.float32).reshape(4, 3)
    mine = base * (rank + 1)                                   # every rank holds a different partial value
    half = (base + 100 * member)[:2]                           # each member feeds its own 2 rows
    out = g.run(None, [y, z], {x: mine, r: half}, 1, 0, ht.run_level("grad"))
    plan = g.executor.plan(0)
    infos = {op.name: plan.comm[op.id] for op in g.ops if op.type == "comm"}
    a = infos["sum_everything"]
    assert C.comm_type_name(a.kind) == "SPLIT_ALL_REDUCE" and (a.pre is not None) == (member == 0), (a, member)
    if member == 0:
        assert C.comm_type_name(a.pre.kind) == "ALL_REDUCE" and tuple(a.pre.group_ranks) == (0, 1)
    assert C.comm_type_name(infos["gather_rows"].kind) == "SPLIT_ALL_GATHER"
    ok = np.allclose(np.asarray(out[0]), base * 6)            # 1 + 2 + 3
    want_rows = np.concatenate([base[:2], (base + 100)[:2]])
    ok = ok and np.allclose(np.asarray(out[1]), want_rows)
    print(f"rank {rank}: ok={ok}", flush=True)
    t = torch.tensor([0 if ok else 1])
    torch.distributed.all_reduce(t)
    if rank == 0 and int(t.item()) == 0:
        print("SPLIT_COMM_GRAPH_OK")
    sys.exit(0 if int(t.item()) == 0 else 3)


if __name__ == "__main__":
    main()
