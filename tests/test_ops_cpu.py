"""The long tail of graph ops against plain PyTorch on one CPU process."""
import numpy as np
import torch

import hetu as ht


def _run(build, feeds):
    ht.init_comm_group(8)
    with ht.graph("define_and_run", num_strategy=1) as g:
        phs = {k: ht.placeholder(torch.from_numpy(v).dtype, list(v.shape), name=k) for k, v in feeds.items()}
        outs = build(**phs)
        outs = list(outs) if isinstance(outs, (tuple, list)) else [outs]
    res = g.run(None, outs, {phs[k]: v for k, v in feeds.items()}, 1, 0, ht.run_level("update"))
    return [r.numpy() for r in res]


def test_shape_and_index_ops():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((4, 6)).astype(np.float32)
    idx = rng.integers(0, 6, size=(4, 3)).astype(np.int64)
    got = _run(lambda x, idx: (ht.pad(x, [1, 2], "constant", 0.5), ht.triu(x), ht.roll(x, [1], [1]),
                               ht.repeat(x, [2, 1]), ht.gather(x, 1, idx), ht.masked_fill(x, ht.range_mask(x, 0.0, 9.0), -1.0),
                               ht.diagonal(x), ht.norm(x, 2, 1), ht.broadcast(ht.reduce_sum(x, [1]), [6, 4])),
               {"x": x, "idx": idx})
    t = torch.from_numpy(x)
    want = [torch.nn.functional.pad(t, [1, 2], value=0.5), torch.triu(t), torch.roll(t, [1], [1]), t.repeat(2, 1),
            torch.gather(t, 1, torch.from_numpy(idx)), t.masked_fill((t >= 0) & (t <= 9), -1.0), torch.diagonal(t),
            torch.linalg.vector_norm(t, 2, 1), t.sum(1).expand(6, 4)]
    for a, b in zip(got, want):
        np.testing.assert_allclose(a, b.numpy(), rtol=1e-5, atol=1e-6)


def test_losses_and_einsum():
    rng = np.random.default_rng(1)
    p = rng.random((8, 5)).astype(np.float32) * 0.9 + 0.05
    y = (rng.random((8, 5)) > 0.5).astype(np.float32)
    lab = rng.integers(0, 5, size=(8,)).astype(np.int64)
    got = _run(lambda p, y, lab: (ht.binary_cross_entropy(p, y, "mean"), ht.nll_loss(ht.log(p), lab, "sum"),
                                  ht.kl_div(ht.log(p), y, "sum"), ht.softmax_cross_entropy(p, y, "mean"),
                                  ht.einsum("ij,kj->ik", p, y), ht.onehot(lab, 5), ht.mse_loss(p, y)),
               {"p": p, "y": y, "lab": lab})
    tp, ty, tl = torch.from_numpy(p), torch.from_numpy(y), torch.from_numpy(lab)
    F = torch.nn.functional
    want = [F.binary_cross_entropy(tp, ty), F.nll_loss(tp.log(), tl, reduction="sum"),
            F.kl_div(tp.log(), ty, reduction="sum"), (-(F.log_softmax(tp, -1) * ty).sum(-1)).mean(), tp @ ty.t(),
            F.one_hot(tl, 5).float(), F.mse_loss(tp, ty)]
    for a, b in zip(got, want):
        np.testing.assert_allclose(a.reshape(-1), b.numpy().reshape(-1), rtol=1e-5, atol=1e-6)


def test_cnn_ops():
    rng = np.random.default_rng(2)
    x = rng.standard_normal((2, 3, 8, 8)).astype(np.float32)
    w = rng.standard_normal((4, 3, 3, 3)).astype(np.float32)
    b = rng.standard_normal((4,)).astype(np.float32)
    got = _run(lambda x, w, b: (ht.conv2d(x, w, b, 1, 1), ht.maxpool(x, 2, 2, 0, 2), ht.avgpool(x, 2, 2, 0, 2),
                                ht.instance_norm(x), ht.interpolate(x, [16, 16])), {"x": x, "w": w, "b": b})
    F = torch.nn.functional
    tx, tw, tb = torch.from_numpy(x), torch.from_numpy(w), torch.from_numpy(b)
    want = [F.conv2d(tx, tw, tb, 1, 1), F.max_pool2d(tx, 2, 2), F.avg_pool2d(tx, 2, 2), F.instance_norm(tx, eps=1e-7),
            F.interpolate(tx, size=[16, 16], mode="bicubic")]
    for a, b_ in zip(got, want):
        np.testing.assert_allclose(a, b_.numpy(), rtol=1e-4, atol=1e-5)
