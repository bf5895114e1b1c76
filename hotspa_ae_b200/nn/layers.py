"""Plain (replicated) layers and the single-strategy spellings of the parallel layers.

* ``Linear``, ``Embedding``, ``LayerNorm``, ``RMSNorm``, ``ReLU``/``GELU``/``SiLU``/``Tanh``/``Sigmoid``, ``MSELoss``,
  ``CrossEntropyLoss``: torch-like modules over graph tensors replicated on every device
  (reference: python_refactor/hetu/nn/modules/{linear,normalization,activation,loss}.py).
* ``HtColumnParallelLinear`` ... : the earlier generations of the parallel-layer API that take one strategy
  description instead of a list (reference: python_refactor/hetu/nn/modules/parallel_ds.py); they wrap the
  multi-strategy layers with a one-element list.
"""
from __future__ import annotations

from ..core import DistributedStates, DistributedStatesUnion
from ..graph import graph as G
from ..graph import init as I
from ..graph import ops as O
from ..graph.tensor import float32
from ..parallel import mesh as M
from .module import Module
from .parallel_layers import (HtMultiColumnParallelLinear, HtMultiParallelEmbedding, HtMultiParallelLayerNorm,
                              HtMultiParallelRMSNorm, HtMultiRowParallelLinear, HtMultiVocabParallelEmbedding)


def _dup_hierarchy():
    g = G.current_graph()
    n = M.mesh().world_size
    return [DistributedStatesUnion([DistributedStates(n, {-1: n}, [-1])]) for _ in range(g.num_strategy)]


def _param(init, shape, name):
    return G.parallel_parameter(init, shape, _dup_hierarchy(), None, dtype=float32, requires_grad=True, name=name)


class Linear(Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, name: str = "linear"):
        super().__init__()
        self.weight = _param(I.he_uniform_initializer(), [out_features, in_features], f"{name}_weight")
        self.bias = _param(I.zeros_initializer(), [out_features], f"{name}_bias") if bias else None

    def forward(self, x):
        return O.linear(x, self.weight, self.bias, trans_b=True)


class Embedding(Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, name: str = "embedding"):
        super().__init__()
        self.weight = _param(I.normal_initializer(0.0, 1.0), [num_embeddings, embedding_dim], f"{name}_table")

    def forward(self, ids):
        return O.embedding_lookup(self.weight, ids)


class LayerNorm(Module):
    def __init__(self, normalized_shape: int, eps: float = 1e-5, name: str = "ln"):
        super().__init__()
        self.eps = eps
        self.weight = _param(I.ones_initializer(), [normalized_shape], f"{name}_weight")
        self.bias = _param(I.zeros_initializer(), [normalized_shape], f"{name}_bias")

    def forward(self, x):
        out = O.fused_layernorm(x, self.weight, self.bias, None, self.eps)
        return out[0] if isinstance(out, (tuple, list)) else out


class RMSNorm(Module):
    def __init__(self, normalized_shape: int, eps: float = 1e-6, name: str = "rmsnorm"):
        super().__init__()
        self.eps = eps
        self.weight = _param(I.ones_initializer(), [normalized_shape], f"{name}_weight")

    def forward(self, x):
        out = O.rms_norm(x, None, self.weight, None, True, self.eps)
        return out[0] if isinstance(out, (tuple, list)) else out


def _act(fn_name):
    class _A(Module):
        def forward(self, x):
            return getattr(O, fn_name)(x)
    _A.__name__ = fn_name
    return _A


ReLU, GELU, SiLU, Tanh, Sigmoid = _act("relu"), _act("gelu"), _act("silu"), _act("tanh"), _act("sigmoid")


class MSELoss(Module):
    def __init__(self, reduction: str = "mean"):
        super().__init__()
        self.reduction = reduction

    def forward(self, pred, target):
        return O.mse_loss(pred, target, self.reduction)


class CrossEntropyLoss(Module):
    def __init__(self, ignored_index: int = -1, reduction: str = "mean"):
        super().__init__()
        self.ignored_index, self.reduction = ignored_index, reduction

    def forward(self, logits, labels):
        return O.vocab_parallel_cross_entropy(logits, labels, self.ignored_index, self.reduction)


# ---- single-strategy spellings -------------------------------------------------------------------------------
def _single(cls):
    class _One(cls):
        def __init__(self, *args, **kwargs):
            args = list(args)
            if "ds_parallel_config" in kwargs:
                kwargs["multi_ds_parallel_config"] = [kwargs.pop("ds_parallel_config")]
            else:
                for i, a in enumerate(args):
                    if isinstance(a, dict):
                        args[i] = [a]
                        break
            super().__init__(*args, **kwargs)
    _One.__name__ = cls.__name__.replace("HtMulti", "Ht")
    return _One


HtColumnParallelLinear = _single(HtMultiColumnParallelLinear)
HtRowParallelLinear = _single(HtMultiRowParallelLinear)
HtParallelEmbedding = _single(HtMultiParallelEmbedding)
HtVocabParallelEmbedding = _single(HtMultiVocabParallelEmbedding)
HtParallelLayerNorm = _single(HtMultiParallelLayerNorm)
HtParallelRMSNorm = _single(HtMultiParallelRMSNorm)
