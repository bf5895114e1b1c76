"""Worker: an activation crosses from a 2-rank group where it is split by rows to another 2-rank group where it is
replicated (the layouts differ, so the transfer is planner-driven); parameters on both sides must receive the
gradients of a single-process run."""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import hetu as ht  # noqa: E402
from hotspa_ae_b200.graph import init as I  # noqa: E402

DS, DSU, DG = ht.DistributedStates, ht.DistributedStatesUnion, ht.DeviceGroup


def main():
    ht.init_comm_group(8)
    rank = int(os.environ["RANK"])
    g0, g1 = [DG([0, 1])], [DG([2, 3])]
    rows, h, out = 8, 16, 8
    with ht.graph("define_and_run", num_strategy=1) as g:
        x = ht.parallel_placeholder(ht.float32, [rows, h], [DSU([DS(2, {0: 2}, [0])])], [g0], name="x")
        w0 = ht.parallel_parameter(I.normal_initializer(0.0, 0.3), [h, h], [DSU([DS(2, {-1: 2}, [-1])])], None,
                                   device_group_hierarchy=[g0], name="w0")
        w1 = ht.parallel_parameter(I.normal_initializer(0.0, 0.3), [out, h], [DSU([DS(2, {0: 2}, [0])])], None,
                                   device_group_hierarchy=[g1], name="w1")
        hmid = ht.linear(x, w0, trans_b=True)                                   # rows split over ranks 0, 1
        h2 = ht.comm(hmid, [DSU([DS(2, {-1: 2}, [-1])])], [g1], name="repartition")   # replicated on ranks 2, 3
        y = ht.linear(h2, w1, trans_b=True, device_group_hierarchy=[g1])        # columns split over ranks 2, 3
        loss = ht.reduce_sum(y * y)
        train_op = ht.SGDOptimizer(lr=0.1).minimize(loss)
    kind = g.executor.plan(0).comm[h2.producer.id]
    assert kind.repartition, kind
    xs = np.random.default_rng(0).standard_normal((rows, h)).astype(np.float32)
    g.run(loss, [loss, train_op], {}, 0, 0, ht.run_level("alloc"))
    store = g.executor.store
    w0_full = w1_full = None
    gen = torch.Generator().manual_seed(store.seed + 7919 * 0)
    w0_full = g.param_inits[w0.id].fill([h, h], gen, "cpu").requires_grad_(True)
    gen = torch.Generator().manual_seed(store.seed + 7919 * 1)
    w1_full = g.param_inits[w1.id].fill([out, h], gen, "cpu").requires_grad_(True)
    feed = {x: xs[(rank % 2) * 4:(rank % 2) * 4 + 4]} if rank < 2 else {}
    g.run(loss, [loss, train_op], feed, 1, 0, ht.run_level("update"))
    ref = ((torch.from_numpy(xs) @ w0_full.t()) @ w1_full.t()).pow(2).sum()
    ref.backward()
    ok = True
    if rank < 2:
        got = torch.from_numpy(w0.get_data())
        want = (w0_full - 0.1 * w0_full.grad).detach()
        ok = torch.allclose(got, want, rtol=1e-4, atol=1e-5)
    else:
        got = torch.from_numpy(w1.get_data())
        want = (w1_full - 0.1 * w1_full.grad).detach()[(rank - 2) * 4:(rank - 2) * 4 + 4]
        ok = torch.allclose(got, want, rtol=1e-4, atol=1e-5)
    if not ok:
        gw = (w1_full if rank >= 2 else w0_full)
        init = gw.detach()[(rank - 2) * 4:(rank - 2) * 4 + 4] if rank >= 2 else gw.detach()
        gr = gw.grad[(rank - 2) * 4:(rank - 2) * 4 + 4] if rank >= 2 else gw.grad
        upd = (init - got) / 0.1
        print(f"rank {rank}: update/grad ratio {(upd / gr).flatten()[:6].tolist()} init match {torch.allclose(init, got + 0.1 * upd)}", flush=True)
    print(f"rank {rank}: repartition ok={ok} max diff {(got - want).abs().max().item():.2e}", flush=True)
    t = torch.tensor([0 if ok else 1])
    torch.distributed.all_reduce(t)
    sys.exit(0 if int(t.item()) == 0 else 3)


if __name__ == "__main__":
    main()
