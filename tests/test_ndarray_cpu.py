"""ht.NDArray: construction, conversions and the static op set against numpy / torch."""
import numpy as np
import pytest
import torch

import hetu as ht

ND = ht.NDArray


def test_construction_and_conversion():
    a = ND([[1.0, 2.0], [3.0, 4.0]])
    assert a.dtype == torch.float32 and a.shape == [2, 2] and a.numel() == 4 and a.ndim == 2
    assert ND([1, 2, 3]).dtype == torch.int64
    src = np.arange(6, dtype=np.float32).reshape(2, 3)
    b = ND(src)
    src[0, 0] = 99                                  # the constructor copies
    assert b.numpy()[0, 0] == 0
    shared = ht.numpy_to_NDArray(src)
    src[0, 1] = 77                                  # the wrapper shares
    assert shared.numpy()[0, 1] == 77
    c = b.to(dtype="bfloat16")
    assert c.dtype == torch.bfloat16
    with pytest.raises(TypeError):
        c.numpy()
    assert c.numpy(force=True).dtype == np.float32
    assert ND(b, dtype=ht.int32).dtype == torch.int32
    assert np.asarray(b).shape == (2, 3) and len(b) == 2 and b[1].shape == [3]
    assert str(b.device) == "cpu"


def test_arithmetic_and_unary_ops():
    x = np.random.default_rng(0).standard_normal((3, 4)).astype(np.float32)
    y = np.random.default_rng(1).standard_normal((3, 4)).astype(np.float32)
    a, b = ND(x), ND(y)
    np.testing.assert_allclose((a + b).numpy(), x + y)
    np.testing.assert_allclose((2 - a).numpy(), 2 - x, rtol=1e-6)
    np.testing.assert_allclose((a * 3).numpy(), x * 3)
    np.testing.assert_allclose((1 / (a * a + 1)).numpy(), 1 / (x * x + 1), rtol=1e-6)
    np.testing.assert_allclose(ND.sub(a, b).numpy(), x - y)
    np.testing.assert_allclose(ND.div(a, 2.0).numpy(), x / 2)
    np.testing.assert_allclose(ND.pow(ND.abs(a), 1.5).numpy(), np.abs(x) ** 1.5, rtol=1e-5)
    for name, ref in [("exp", np.exp), ("sin", np.sin), ("cos", np.cos), ("tanh", np.tanh), ("floor", np.floor),
                      ("ceil", np.ceil), ("neg", np.negative)]:
        np.testing.assert_allclose(getattr(ND, name)(a).numpy(), ref(x), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(ND.relu(a).numpy(), np.maximum(x, 0))
    np.testing.assert_allclose(ND.sigmoid(a).numpy(), 1 / (1 + np.exp(-x)), rtol=1e-5)
    np.testing.assert_allclose(ND.where(ND(x > 0), a, b).numpy(), np.where(x > 0, x, y))
    packed = ND(np.concatenate([x, y], axis=1))
    np.testing.assert_allclose(ND.swiglu(packed).numpy(), x / (1 + np.exp(-x)) * y, rtol=1e-5, atol=1e-6)
    assert ND.toInt32(a).dtype == torch.int32 and ND.toFloat64(a).dtype == torch.float64


def test_reductions_linear_algebra_and_shapes():
    x = np.random.default_rng(2).standard_normal((2, 3, 4)).astype(np.float32)
    a = ND(x)
    np.testing.assert_allclose(ND.sum(a, [0, 2]).numpy(), x.sum((0, 2)), rtol=1e-5)
    np.testing.assert_allclose(ND.mean(a, 1, keepdims=True).numpy(), x.mean(1, keepdims=True), rtol=1e-5)
    np.testing.assert_allclose(ND.max(a).numpy(), x.max())
    np.testing.assert_allclose(ND.prod(a, [2]).numpy(), x.prod(2), rtol=1e-5)
    np.testing.assert_allclose(ND.softmax(a, -1).numpy().sum(-1), np.ones((2, 3)), rtol=1e-5)
    w = np.random.default_rng(3).standard_normal((5, 4)).astype(np.float32)
    np.testing.assert_allclose(ND.linear(a, ND(w)).numpy(), x @ w.T, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(ND.matmul(a, ND(w), trans_right=True).numpy(), x @ w.T, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose((a @ ND(w.T.copy())).numpy(), x @ w.T, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(ND.dot(a, a).numpy(), (x * x).sum(), rtol=1e-5)
    assert ND.reshape(a, [6, 4]).shape == [6, 4] and ND.permute(a, [2, 0, 1]).shape == [4, 2, 3]
    assert ND.flatten(a, 1).shape == [2, 12] and ND.unsqueeze(a, 0).shape == [1, 2, 3, 4]
    assert ND.adddim(ND(x[0]), 0, 5).shape == [5, 3, 4]
    np.testing.assert_array_equal(ND.slice(a, [0, 1, 1], [2, 2, 2]).numpy(), x[:, 1:3, 1:3])
    parts = ND.split(a, 2, axis=2)
    assert len(parts) == 2 and parts[0].shape == [2, 3, 2]
    np.testing.assert_array_equal(ND.cat(parts, axis=2).numpy(), x)
    assert [p.shape[1] for p in ND.split(a, [1, 2], axis=1)] == [1, 2]
    np.testing.assert_array_equal(ND.roll(a, 1, 2).numpy(), np.roll(x, 1, 2))
    np.testing.assert_array_equal(ND.triu(ND(x[0])).numpy(), np.triu(x[0]))
    assert ND.pad(ND(x[0]), [1, 1]).shape == [3, 6] and ND.repeat(ND(x[0]), [2, 1]).shape == [6, 4]
    assert ND.broadcast(ND(x[0, 0]), [3, 4]).shape == [3, 4]


def test_creation_indexing_and_losses():
    z = ND.zeros([2, 3])
    assert z.numpy().sum() == 0 and ND.ones_like(z).numpy().sum() == 6 and ND.full([2], 7, dtype="int64").numpy()[1] == 7
    r1, r2 = ND.rand([1000], seed=5), ND.rand([1000], seed=5)
    np.testing.assert_array_equal(r1.numpy(), r2.numpy())
    assert 0 <= r1.numpy().min() and r1.numpy().max() <= 1
    g = ND.randn([4000], mean=1.0, stddev=2.0, seed=1).numpy()
    assert abs(g.mean() - 1.0) < 0.15 and abs(g.std() - 2.0) < 0.15
    t = ND.truncated_normal_(ND.empty([1000]), 0.0, 1.0, -1.0, 1.0, seed=3).numpy()
    assert t.min() >= -1.0 and t.max() <= 1.0
    table = ND(np.arange(12, dtype=np.float32).reshape(4, 3))
    np.testing.assert_array_equal(ND.embedding(table, ND([3, 0])).numpy(), table.numpy()[[3, 0]])
    np.testing.assert_array_equal(ND.onehot(ND([1, 0]), 3).numpy(), np.eye(3, dtype=np.float32)[[1, 0]])
    np.testing.assert_array_equal(ND.gather(table, 1, ND([[2], [0], [1], [1]])).numpy()[:, 0], [2, 3, 7, 10])
    logits = np.random.default_rng(4).standard_normal((5, 7)).astype(np.float32)
    lab = np.array([1, 0, 6, 3, 3])
    lse = np.log(np.exp(logits).sum(-1))
    np.testing.assert_allclose(ND.sceloss(ND(logits), ND(lab), "mean").numpy(),
                               (lse - logits[np.arange(5), lab]).mean(), rtol=1e-5)
    np.testing.assert_allclose(ND.mseloss(ND(logits), ND(logits * 0), "sum").numpy(), (logits ** 2).sum(), rtol=1e-5)
    x = np.random.default_rng(6).standard_normal((2, 8)).astype(np.float32)
    ln = ND.layernorm(ND(x), ND.ones([8]), ND.zeros([8]), [8]).numpy()
    np.testing.assert_allclose(ln.mean(-1), 0, atol=1e-5)


def test_ndarray_as_a_graph_feed():
    with ht.graph("define_and_run") as g:
        x = ht.placeholder(ht.float32, [2, 3], name="x")
        y = ht.reduce_sum(x * x)
    val = ND(np.ones((2, 3), dtype=np.float32) * 2)
    out = g.run(y, [y], {x: val})
    assert float(np.asarray(out[0]).reshape(-1)[0]) == 24.0
