"""Worker (2 gloo ranks): Megatron tensor parallelism WITHOUT sequence parallelism - RMSNorm on replicated
activations, column-parallel then row-parallel linear with an all-reduce and a replicated bias.  The replicated
parameters see the same activations on both ranks, so their (identical) gradients must count once."""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import hetu as ht  # noqa: E402
from hotspa_ae_b200.parallel.strategy_config import find_config, generate_llama_3d_config, propagate_zero  # noqa: E402
from hotspa_ae_b200.utils import checkpoint as CK  # noqa: E402


def main():
    ht.init_comm_group(8)
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    dp = world // 2                                   # 2 ranks: tp2; 4 ranks: dp2 x tp2 (ranks (0, 1) and (2, 3))
    cfg = propagate_zero(generate_llama_3d_config(1, world, dp, 2, 1, False))
    h, f, rows = 8, 12, 6 * dp
    x_u, x_g = ht.nn.config2ds(cfg["input"])
    with ht.graph("define_and_run", num_strategy=1) as g:
        x = ht.parallel_placeholder(ht.float32, [rows, h], [x_u], [x_g], name="x")
        norm = ht.nn.HtMultiParallelRMSNorm(h, [find_config(cfg, "layernorm1", 0)], sp=False, name="norm")
        col = ht.nn.HtMultiColumnParallelLinear(h, f, [find_config(cfg, "dense_h_to_4h", 0)], bias=True,
                                                gather_output=False, name="col")
        row = ht.nn.HtMultiRowParallelLinear(f, h, [find_config(cfg, "dense_4h_to_h", 0)], sp=False, bias=True,
                                             name="row")
        y = row(ht.relu(col(norm(x))))
        loss = ht.reduce_sum(y * y)
        train_op = ht.SGDOptimizer(lr=0.01).minimize(loss)
    xs = np.random.default_rng(0).standard_normal((rows, h)).astype(np.float32)
    full_xs = xs
    xs = np.split(xs, dp)[rank // 2]                  # this replica's rows
    g.run(loss, [loss, train_op], {x: xs}, 1, 0, ht.run_level("alloc"))
    params = {"g": norm.weight, "w1": col.weight, "b1": col.bias, "w2": row.weight, "b2": row.bias}
    # give the biases and the norm weight non-trivial values
    for k, scale in (("b1", 0.1), ("b2", 0.2), ("g", 1.0)):
        p = params[k]
        p.reset_data(np.asarray(scale + 0.05 * np.arange(p.global_shape[0]), dtype=np.float32))
    before = {k: CK.gather_global(g, p).clone() for k, p in params.items()}
    out = g.run(loss, [loss, train_op], {x: xs}, 1, 0, ht.run_level("update"))
    after = {k: CK.gather_global(g, p) for k, p in params.items()}
    ref = {k: v.clone().requires_grad_(True) for k, v in before.items()}
    X = torch.tensor(full_xs)
    n = X * torch.rsqrt(X.pow(2).mean(-1, keepdim=True) + 1e-6) * ref["g"]
    hmid = torch.relu(n @ ref["w1"].T + ref["b1"])
    yr = hmid @ ref["w2"] + ref["b2"]                # the row-parallel weight is stored [in, out]
    lr_ = (yr * yr).sum()
    lr_.backward()
    mine = torch.tensor(float(np.asarray(out[0]).reshape(-1)[0]) if rank % 2 == 0 else 0.0)   # one rank per replica
    torch.distributed.all_reduce(mine)
    got = float(mine)
    ok = abs(got - float(lr_)) < 1e-3 * max(1.0, abs(float(lr_)))
    worst, where = 0.0, ""
    for k in params:
        d = float((after[k] - (before[k] - 0.01 * ref[k].grad)).abs().max())
        if d > worst:
            worst, where = d, k
    ok = ok and worst < 1e-4
    print(f"rank {rank}: loss {got:.5f} vs {float(lr_):.5f}, worst weight diff {worst:.2e} ({where}) ok={ok}", flush=True)
    t = torch.tensor([0 if ok else 1])
    torch.distributed.all_reduce(t)
    if rank == 0 and int(t.item()) == 0:
        print("NONSP_TP_OK")
    sys.exit(0 if int(t.item()) == 0 else 3)


if __name__ == "__main__":
    main()
