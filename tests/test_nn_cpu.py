"""hetu.nn: the torch-like module set and the device-group parallel layers, one CPU process, against torch."""
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import hetu as ht
from hotspa_ae_b200.parallel import mesh as M


def _run(build, feeds):
    """build(g) -> (placeholders, fetch tensors); returns the fetched values as numpy arrays."""
    M.reset_mesh()
    ht.init_comm_group(8)
    with ht.graph("define_and_run") as g:
        phs, outs, extra = build()
    vals = g.run(None, list(outs), dict(zip(phs, feeds)), 1, 0, ht.run_level("grad"))
    return [np.asarray(v.float() if torch.is_tensor(v) else v) for v in vals], extra


def test_activations_and_containers():
    x = np.random.default_rng(0).standard_normal((4, 6)).astype(np.float32)

    def build():
        p = ht.placeholder(ht.float32, [4, 6], name="x")
        d = ht.nn.ModuleDict({"a": ht.nn.LeakyReLU(0.2), "b": ht.nn.NewGeLU()})
        assert len(d) == 2 and "a" in d and d.keys() == ["a", "b"] and [k for k in d] == ["a", "b"]
        assert len(list(d.values())) == 2 and d.items()[1][0] == "b"
        with pytest.raises(KeyError):
            d["c"]
        return [p], [d["a"](p), d["b"](p)], None

    (lr, ng), _ = _run(build, [x])
    t = torch.tensor(x)
    np.testing.assert_allclose(lr, F.leaky_relu(t, 0.2).numpy(), rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(ng, F.gelu(t, approximate="tanh").numpy(), rtol=1e-5, atol=1e-6)


def test_cnn_stack_matches_torch():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((2, 3, 8, 8)).astype(np.float32)

    def build():
        p = ht.placeholder(ht.float32, [2, 3, 8, 8], name="img")
        conv = ht.nn.Conv2d(3, 4, 3, stride=1, padding=1, name="c1")
        bn = ht.nn.BatchNorm(4, name="bn1")
        y = ht.nn.ZeroPad2d(1)(p)
        y1 = conv(p)
        y2 = bn(y1)
        y3 = ht.nn.MaxPool2d(2)(y2)
        y4 = ht.nn.AvgPool2d(2)(y2)
        y5 = ht.nn.InstanceNorm()(y1)
        return [p], [y, y1, y2, y3, y4, y5], (conv, bn)

    (pad, y1, y2, y3, y4, y5), (conv, bn) = _run(build, [x])
    t = torch.tensor(x)
    w, b = torch.tensor(np.array(conv.weight.get_data())), torch.tensor(np.array(conv.bias.get_data()))
    assert pad.shape == (2, 3, 10, 10) and pad[0, 0, 0, 0] == 0
    r1 = F.conv2d(t, w, b, 1, 1)
    np.testing.assert_allclose(y1, r1.numpy(), rtol=1e-4, atol=1e-5)
    r2 = F.batch_norm(r1, torch.zeros(4), torch.ones(4), torch.ones(4), torch.zeros(4), True, 0.1, 1e-5)
    np.testing.assert_allclose(y2, r2.numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(y3, F.max_pool2d(r2, 2).numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(y4, F.avg_pool2d(r2, 2).numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(y5, F.instance_norm(r1, eps=1e-7).numpy(), rtol=1e-4, atol=1e-4)


def test_losses_match_torch():
    rng = np.random.default_rng(2)
    logp = np.log(rng.dirichlet(np.ones(5), size=6)).astype(np.float32)
    lab = rng.integers(0, 5, size=6)
    prob = rng.uniform(0.05, 0.95, size=(6, 5)).astype(np.float32)
    tgt = rng.uniform(0.0, 1.0, size=(6, 5)).astype(np.float32)

    def build():
        a = ht.placeholder(ht.float32, [6, 5], name="logp")
        l = ht.placeholder(ht.int64, [6], name="lab")
        p = ht.placeholder(ht.float32, [6, 5], name="prob")
        t = ht.placeholder(ht.float32, [6, 5], name="tgt")
        return [a, l, p, t], [ht.nn.NLLLoss()(a, l), ht.nn.BCELoss("sum")(p, t), ht.nn.KLDivLoss("sum")(a, t)], None

    (nll, bce, kl), _ = _run(build, [logp, lab, prob, tgt])
    np.testing.assert_allclose(nll.reshape(-1)[0], F.nll_loss(torch.tensor(logp), torch.tensor(lab)).item(), rtol=1e-5)
    np.testing.assert_allclose(bce.reshape(-1)[0],
                               F.binary_cross_entropy(torch.tensor(prob), torch.tensor(tgt), reduction="sum").item(),
                               rtol=1e-5)
    np.testing.assert_allclose(kl.reshape(-1)[0],
                               F.kl_div(torch.tensor(logp), torch.tensor(tgt), reduction="sum").item(), rtol=1e-4)


def test_functional_constructors_and_parameter():
    M.reset_mesh()
    ht.init_comm_group(8)
    with ht.graph("define_and_run") as g:
        a = ht.nn.functional.xavier_uniform_([64, 32], requires_grad=True, name="xa")
        b = ht.nn.init.kaiming_normal_([256, 128], nonlinearity="relu", name="kn")
        c = ht.nn.functional.constant_([3], 2.5, name="c")
        p = ht.nn.Parameter(np.arange(6, dtype=np.float32).reshape(2, 3), name="from_np")
        q = ht.nn.Parameter(c, requires_grad=True)
        x = ht.placeholder(ht.float32, [1], name="x")
    g.run(None, [x], {x: np.zeros(1, np.float32)}, 1, 0, ht.run_level("alloc"))
    av, bv = np.array(a.get_data()), np.array(b.get_data())
    lim = math.sqrt(3.0 / ((64 + 32) / 2))
    assert a.requires_grad and not b.requires_grad and q is c and c.requires_grad
    assert np.abs(av).max() <= lim + 1e-6 and np.abs(av).max() > 0.8 * lim
    assert abs(bv.std() - math.sqrt(2.0 / 128)) < 0.01
    assert np.allclose(np.array(c.get_data()), 2.5) and np.array(p.get_data())[1, 2] == 5.0
    assert ht.nn.functional.calculate_gain("tanh") == 5.0 / 3
    with pytest.raises(TypeError):
        ht.nn.Parameter(None)


def test_device_group_parallel_layers_single_device():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((4, 8)).astype(np.float32)
    ids = rng.integers(0, 10, size=(4,))

    def build():
        p = ht.placeholder(ht.float32, [4, 8], name="x")
        i = ht.placeholder(ht.int64, [4], name="ids")
        col = ht.nn.ColumnParallelLinear(8, 6, [0], name="col")
        row = ht.nn.RowParallelLinear(6, 8, [0], name="row")
        emb = ht.nn.VocabParallelEmbedding(10, 8, [0], name="vemb")
        ln = ht.nn.ParallelLayerNorm(8, [0], name="pln")
        assert ht.nn.get_device_index(ht.DeviceGroup([0])) == 0 and ht.nn.get_device_index([5]) == -1
        return [p, i], [row(col(p)), ln(emb(i) + ht.nn.ParallelEmbedding(10, 8, [0], name="pemb")(i))], (col, row)

    (y, e), (col, row) = _run(build, [x, ids])
    w1, b1 = np.array(col.weight.get_data()), np.array(col.bias.get_data())
    w2, b2 = np.array(row.weight.get_data()), np.array(row.bias.get_data())
    np.testing.assert_allclose(y, (x @ w1.T + b1) @ w2.T + b2, rtol=1e-4, atol=1e-5)
    assert e.shape == (4, 8) and abs(float(e.mean())) < 1e-5
