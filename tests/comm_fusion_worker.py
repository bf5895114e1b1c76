"""Worker (2 gloo ranks): collectives back to back are planned as one.  partial -> duplicate -> split rows is a
reduce-scatter, and gathering and re-splitting the rows after it adds nothing: the whole chain runs as one
reduce-scatter.  Values and gradients stay those of the step-by-step program."""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import hetu as ht  # noqa: E402
from hotspa_ae_b200 import core as C  # noqa: E402
from hotspa_ae_b200.graph import init as I  # noqa: E402

DS, DSU, DG = ht.DistributedStates, ht.DistributedStatesUnion, ht.DeviceGroup


def main():
    ht.init_comm_group(8)
    rank = int(os.environ["RANK"])
    grp = [[DG([0, 1])]]
    split0 = [DSU([DS(2, {0: 2}, [0])])]
    split1 = [DSU([DS(2, {1: 2}, [1])])]
    dup = [DSU([DS(2, {-1: 2}, [-1])])]
    rows, k, n = 4, 6, 4
    with ht.graph("define_and_run", num_strategy=1) as g:
        x = ht.parallel_placeholder(ht.float32, [rows, k], split1, grp, name="x")       # columns split
        w = ht.parallel_parameter(I.normal_initializer(0.0, 0.4), [k, n], split0, None, device_group_hierarchy=grp,
                                  name="w")                                            # rows split -> partial product
        y = ht.matmul(x, w)                                    # partial over the two ranks
        y = ht.comm(y, dup, grp, name="all_reduce")
        y = ht.comm(y, split0, grp, name="take_rows")          # together: a reduce-scatter
        z = ht.comm(y, dup, grp, name="gather_rows")
        z = ht.comm(z, split0, grp, name="take_rows_again")    # together: nothing
        loss = ht.reduce_sum(z * z)
        train_op = ht.SGDOptimizer(lr=0.1).minimize(loss)
    xs = np.random.default_rng(0).standard_normal((rows, k)).astype(np.float32)
    g.run(loss, [loss, train_op], {x: xs[:, rank * 3:(rank + 1) * 3]}, 1, 0, ht.run_level("alloc"))
    plan = g.executor.plan(0)
    kinds = {op.name: C.comm_type_name(plan.comm[op.id].kind) for op in g.ops if op.type == "comm"}
    # the chain partial -> dup -> rows -> dup -> rows collapses into one reduce-scatter, carried by the last op
    assert kinds["all_reduce"] == kinds["take_rows"] == kinds["gather_rows"] == "UNUSED", kinds
    assert kinds["take_rows_again"] == "REDUCE_SCATTER", kinds
    w_local = torch.tensor(np.array(w.get_data()))
    parts = [torch.zeros_like(w_local), torch.zeros_like(w_local)]
    torch.distributed.all_gather(parts, w_local)
    W = torch.cat(parts, 0).requires_grad_(True)
    out = g.run(loss, [loss, train_op], {x: xs[:, rank * 3:(rank + 1) * 3]}, 1, 0, ht.run_level("update"))
    ref = ((torch.tensor(xs) @ W) ** 2).sum()
    ref.backward()
    mine = torch.tensor(float(np.asarray(out[0]).reshape(-1)[0]))
    torch.distributed.all_reduce(mine)                          # each rank's loss covers its rows
    want = (W - 0.1 * W.grad).detach()[rank * 3:(rank + 1) * 3]
    got = torch.tensor(np.array(w.get_data()))
    ok = abs(float(mine) - float(ref)) < 1e-3 * abs(float(ref)) and torch.allclose(got, want, rtol=1e-4, atol=1e-5)
    print(f"rank {rank}: loss {float(mine):.4f} vs {float(ref):.4f}; weight diff {float((got - want).abs().max()):.2e} ok={ok}",
          flush=True)
    t = torch.tensor([0 if ok else 1])
    torch.distributed.all_reduce(t)
    if rank == 0 and int(t.item()) == 0:
        print("COMM_FUSION_OK")
    sys.exit(0 if int(t.item()) == 0 else 3)


if __name__ == "__main__":
    main()
