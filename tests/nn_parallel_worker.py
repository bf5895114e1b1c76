"""Worker (2 gloo ranks): the device-group parallel layers - column-parallel linear (output kept split) feeding a
row-parallel linear, plus a vocab-parallel embedding; forward value and one SGD step against single-process math."""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import hetu as ht  # noqa: E402
from hotspa_ae_b200.utils import checkpoint as CK  # noqa: E402


def main():
    ht.init_comm_group(8)
    rank = int(os.environ["RANK"])
    rng = np.random.default_rng(0)
    ids = rng.integers(0, 12, size=(6,))
    with ht.graph("define_and_run") as g:
        i = ht.placeholder(ht.int64, [6], name="ids")
        emb = ht.nn.VocabParallelEmbedding(12, 8, [0, 1], name="vemb")
        col = ht.nn.ColumnParallelLinear(8, 10, [0, 1], gather_output=False, name="col")
        row = ht.nn.RowParallelLinear(10, 4, [0, 1], input_is_parallel=True, name="row")
        y = row(ht.relu(col(emb(i))))
        loss = ht.reduce_sum(y * y)
        train_op = ht.SGDOptimizer(lr=0.01).minimize(loss)
    g.run(loss, [loss, train_op], {i: ids}, 1, 0, ht.run_level("alloc"))
    params = {"emb": emb.weight, "w1": col.weight, "b1": col.bias, "w2": row.weight, "b2": row.bias}
    before = {k: CK.gather_global(g, p).clone() for k, p in params.items()}
    out = g.run(loss, [loss, train_op], {i: ids}, 1, 0, ht.run_level("update"))
    after = {k: CK.gather_global(g, p) for k, p in params.items()}
    ref = {k: v.clone().requires_grad_(True) for k, v in before.items()}
    h = torch.relu(ref["emb"][torch.tensor(ids)] @ ref["w1"].T + ref["b1"])
    yr = h @ ref["w2"].T + ref["b2"]
    lr_ = (yr * yr).sum()
    lr_.backward()
    got = float(np.asarray(out[0]).reshape(-1)[0])
    ok = abs(got - float(lr_)) < 1e-3 * max(1.0, abs(float(lr_)))
    worst = 0.0
    for k in params:
        want = before[k] - 0.01 * ref[k].grad
        worst = max(worst, float((after[k] - want).abs().max()))
    ok = ok and worst < 1e-4
    print(f"rank {rank}: loss {got:.5f} vs {float(lr_):.5f}, worst weight diff {worst:.2e} ok={ok}", flush=True)
    t = torch.tensor([0 if ok else 1])
    torch.distributed.all_reduce(t)
    if rank == 0 and int(t.item()) == 0:
        print("NN_PARALLEL_OK")
    sys.exit(0 if int(t.item()) == 0 else 3)


if __name__ == "__main__":
    main()
