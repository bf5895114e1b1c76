"""The rest of the torch-like module set (reference: python_refactor/hetu/nn/modules/{activation,batchnorm,conv,
dropout,instancenorm,loss,padding,pooling,container}.py) and the first generation of the parallel layers, which take
a device group instead of a strategy description (reference: python_refactor/hetu/nn/modules/parallel.py).

These modules are replicated (or, for the parallel ones, Megatron-style sharded over one device group); the CNN
layers run on the library kernels behind the graph ops of the same name.
"""
from __future__ import annotations

from ..core import DistributedStates, DistributedStatesUnion
from ..graph import graph as G
from ..graph import init as I
from ..graph import ops as O
from ..graph import ops_extra as OX
from ..graph.tensor import float32
from ..parallel import mesh as M
from .layers import _param
from .module import Module


# ---- activations -------------------------------------------------------------------------------------------------
class LeakyReLU(Module):
    def __init__(self, negative_slope: float = 0.1):
        super().__init__()
        self.negative_slope = negative_slope

    def forward(self, x):
        # max(x, slope * x) for slopes below one
        return O.relu(x) * (1.0 - self.negative_slope) + x * self.negative_slope


class NewGeLU(Module):
    """The tanh approximation of GELU used by GPT-2."""

    def forward(self, x):
        return 0.5 * x * (1.0 + O.tanh(0.7978845608028654 * (x + 0.044715 * (x * x * x))))


# ---- containers ----------------------------------------------------------------------------------------------------
class ModuleDict(Module):
    def __init__(self, modules: dict | None = None):
        super().__init__()
        self._keys: list[str] = []
        for k, m in (modules or {}).items():
            self[k] = m

    def __setitem__(self, key: str, module: Module) -> None:
        if key not in self._keys:
            self._keys.append(key)
        setattr(self, key, module)

    def __getitem__(self, key: str) -> Module:
        if key not in self._keys:
            raise KeyError(key)
        return getattr(self, key)

    def __contains__(self, key: str) -> bool:
        return key in self._keys

    def __len__(self) -> int:
        return len(self._keys)

    def __iter__(self):
        return iter(self._keys)

    def keys(self):
        return list(self._keys)

    def values(self):
        return [getattr(self, k) for k in self._keys]

    def items(self):
        return [(k, getattr(self, k)) for k in self._keys]


# ---- CNN layers ----------------------------------------------------------------------------------------------------
class Conv2d(Module):
    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride: int = 1, padding: int = 0,
                 bias: bool = True, name: str = "conv"):
        super().__init__()
        kh, kw = (kernel_size, kernel_size) if isinstance(kernel_size, int) else kernel_size
        self.stride, self.padding = stride, padding
        self.weight = _param(I.he_uniform_initializer(), [out_channels, in_channels, kh, kw], f"{name}_weight")
        self.bias = _param(I.zeros_initializer(), [out_channels], f"{name}_bias") if bias else None

    def forward(self, x):
        return OX.conv2d(x, self.weight, self.bias, self.padding, self.stride)


class MaxPool2d(Module):
    def __init__(self, kernel_size, stride: int | None = None, padding: int = 0):
        super().__init__()
        self.kh, self.kw = (kernel_size, kernel_size) if isinstance(kernel_size, int) else kernel_size
        self.stride, self.padding = stride if stride is not None else self.kh, padding

    def forward(self, x):
        return OX.maxpool(x, kernel_H=self.kh, kernel_W=self.kw, padding=self.padding, stride=self.stride)


class AvgPool2d(MaxPool2d):
    def forward(self, x):
        return OX.avgpool(x, kernel_H=self.kh, kernel_W=self.kw, padding=self.padding, stride=self.stride)


class BatchNorm(Module):
    """Batch normalisation over the channel dimension of [N, C, H, W]; the running statistics are buffers (parameters
    without gradient) updated by the library kernel in training mode."""

    def __init__(self, num_features: int, eps: float = 1e-5, momentum: float = 0.1, name: str = "bn"):
        super().__init__()
        self.eps, self.momentum = eps, momentum
        self.weight = _param(I.ones_initializer(), [num_features], f"{name}_weight")
        self.bias = _param(I.zeros_initializer(), [num_features], f"{name}_bias")
        dup = _dup()
        self.running_mean = G.parallel_parameter(I.zeros_initializer(), [num_features], dup, None, dtype=float32,
                                                 requires_grad=False, name=f"{name}_running_mean")
        self.running_var = G.parallel_parameter(I.ones_initializer(), [num_features], dup, None, dtype=float32,
                                                requires_grad=False, name=f"{name}_running_var")

    def forward(self, x):
        return OX.batch_norm(x, self.weight, self.bias, self.running_mean, self.running_var, self.momentum, self.eps)


class InstanceNorm(Module):
    def __init__(self, num_features: int | None = None, eps: float = 1e-7):
        super().__init__()
        self.eps = eps

    def forward(self, x):
        return OX.instance_norm(x, eps=self.eps)


class Dropout2d(Module):
    def __init__(self, p: float = 0.5):
        super().__init__()
        self.p = p

    def forward(self, x):
        return OX.dropout2d(x, p=self.p) if self.training and self.p > 0 else x


class ConstantPad2d(Module):
    """padding = (left, right, top, bottom), like torch."""

    def __init__(self, padding, value: float = 0.0):
        super().__init__()
        self.padding = [padding] * 4 if isinstance(padding, int) else list(padding)
        self.value = value

    def forward(self, x):
        return OX.pad(x, pads=self.padding, mode="constant", constant=self.value)


class ZeroPad2d(ConstantPad2d):
    def __init__(self, padding):
        super().__init__(padding, 0.0)


# ---- losses --------------------------------------------------------------------------------------------------------
class _Loss(Module):
    def __init__(self, reduction: str = "mean"):
        super().__init__()
        self.reduction = reduction


class NLLLoss(_Loss):
    def forward(self, log_probs, target):
        return OX.nll_loss(log_probs, target, reduction=self.reduction)


class BCELoss(_Loss):
    def forward(self, probs, target):
        return OX.binary_cross_entropy(probs, target, reduction=self.reduction)


class KLDivLoss(_Loss):
    def forward(self, log_probs, target):
        return OX.kl_div(log_probs, target, reduction=self.reduction)


# ---- first-generation parallel layers (one device group, Megatron layout) ------------------------------------------
def _dup():
    g = G.current_graph()
    n = M.mesh().world_size
    return [DistributedStatesUnion([DistributedStates(n, {-1: n}, [-1])]) for _ in range(g.num_strategy)]


def get_device_index(device_group) -> int:
    """Position of this process in `device_group` (-1 when it is not a member)."""
    me = M.mesh().rank
    ranks = device_group.ranks() if hasattr(device_group, "ranks") else list(device_group)
    return ranks.index(me) if me in ranks else -1


def _group_hierarchy(device_group, states: dict, order: list):
    g = G.current_graph()
    group = device_group if isinstance(device_group, M.DeviceGroup) else M.DeviceGroup(list(device_group))
    n = group.num_devices
    ds = DistributedStates(n, states(n) if callable(states) else states, order)
    return [DistributedStatesUnion([ds]) for _ in range(g.num_strategy)], [[group] for _ in range(g.num_strategy)]


class ColumnParallelLinear(Module):
    """y = x W^T with W's output features split over the device group; `gather_output` all-gathers the columns."""

    def __init__(self, in_features: int, out_features: int, device_group, bias: bool = True,
                 gather_output: bool = True, name: str = "colp"):
        super().__init__()
        self.gather_output = gather_output
        self.group = device_group if isinstance(device_group, M.DeviceGroup) else M.DeviceGroup(list(device_group))
        n = self.group.num_devices
        dsh, dgh = _group_hierarchy(self.group, {0: n}, [0])
        self.weight = G.parallel_parameter(I.he_uniform_initializer(), [out_features, in_features], dsh, None,
                                           dtype=float32, requires_grad=True, device_group_hierarchy=dgh,
                                           name=f"{name}_weight")
        self.bias = G.parallel_parameter(I.zeros_initializer(), [out_features], dsh, None, dtype=float32,
                                         requires_grad=True, device_group_hierarchy=dgh,
                                         name=f"{name}_bias") if bias else None
        self._dup, self._dgh = _group_hierarchy(self.group, {-1: n}, [-1])

    def forward(self, x):
        y = O.linear(x, self.weight, self.bias, trans_b=True)
        if self.gather_output and self.group.num_devices > 1:
            y = O.comm(y, self._dup, self._dgh)
        return y


class RowParallelLinear(Module):
    """y = x W^T with W's input features split over the device group: x arrives split along its last dimension
    (or is split here when `input_is_parallel` is False), partial results are all-reduced."""

    def __init__(self, in_features: int, out_features: int, device_group, bias: bool = True,
                 input_is_parallel: bool = True, name: str = "rowp"):
        super().__init__()
        self.input_is_parallel = input_is_parallel
        self.group = device_group if isinstance(device_group, M.DeviceGroup) else M.DeviceGroup(list(device_group))
        n = self.group.num_devices
        dsh, dgh = _group_hierarchy(self.group, {1: n}, [1])
        self.weight = G.parallel_parameter(I.he_uniform_initializer(), [out_features, in_features], dsh, None,
                                           dtype=float32, requires_grad=True, device_group_hierarchy=dgh,
                                           name=f"{name}_weight")
        self._dup, self._dgh = _group_hierarchy(self.group, {-1: n}, [-1])
        self._split_last = lambda ndim: _group_hierarchy(self.group, {ndim - 1: n}, [ndim - 1])[0]
        self.bias = G.parallel_parameter(I.zeros_initializer(), [out_features], self._dup, None, dtype=float32,
                                         requires_grad=True, device_group_hierarchy=self._dgh,
                                         name=f"{name}_bias") if bias else None

    def forward(self, x):
        if not self.input_is_parallel and self.group.num_devices > 1:
            x = O.comm(x, self._split_last(x.ndim), self._dgh)
        y = O.linear(x, self.weight, None, trans_b=True)
        if self.group.num_devices > 1:
            y = O.comm(y, self._dup, self._dgh)
        return y + self.bias if self.bias is not None else y


class ParallelEmbedding(Module):
    """Embedding table replicated over the device group."""

    def __init__(self, num_embeddings: int, embedding_dim: int, device_group, name: str = "pemb"):
        super().__init__()
        group = device_group if isinstance(device_group, M.DeviceGroup) else M.DeviceGroup(list(device_group))
        dsh, dgh = _group_hierarchy(group, {-1: group.num_devices}, [-1])
        self.weight = G.parallel_parameter(I.normal_initializer(0.0, 1.0), [num_embeddings, embedding_dim], dsh, None,
                                           dtype=float32, requires_grad=True, device_group_hierarchy=dgh,
                                           name=f"{name}_table")

    def forward(self, ids):
        return O.embedding_lookup(self.weight, ids)


class VocabParallelEmbedding(Module):
    """Embedding table split by vocabulary rows over the device group; rows outside a shard contribute zeros and the
    partial lookups are all-reduced."""

    def __init__(self, num_embeddings: int, embedding_dim: int, device_group, name: str = "vpemb"):
        super().__init__()
        self.group = device_group if isinstance(device_group, M.DeviceGroup) else M.DeviceGroup(list(device_group))
        n = self.group.num_devices
        dsh, dgh = _group_hierarchy(self.group, {0: n}, [0])
        self.weight = G.parallel_parameter(I.normal_initializer(0.0, 1.0), [num_embeddings, embedding_dim], dsh, None,
                                           dtype=float32, requires_grad=True, device_group_hierarchy=dgh,
                                           name=f"{name}_table")
        self._dup, self._dgh = _group_hierarchy(self.group, {-1: n}, [-1])

    def forward(self, ids):
        y = O.embedding_lookup(self.weight, ids)
        if self.group.num_devices > 1:
            y = O.comm(y, self._dup, self._dgh)
        return y


class ParallelLayerNorm(Module):
    """LayerNorm whose weights are replicated over the device group."""

    def __init__(self, normalized_shape: int, device_group, eps: float = 1e-5, name: str = "pln"):
        super().__init__()
        self.eps = eps
        group = device_group if isinstance(device_group, M.DeviceGroup) else M.DeviceGroup(list(device_group))
        dsh, dgh = _group_hierarchy(group, {-1: group.num_devices}, [-1])
        mk = lambda init, nm: G.parallel_parameter(init, [normalized_shape], dsh, None, dtype=float32,  # noqa: E731
                                                   requires_grad=True, device_group_hierarchy=dgh, name=nm)
        self.weight, self.bias = mk(I.ones_initializer(), f"{name}_weight"), mk(I.zeros_initializer(), f"{name}_bias")

    def forward(self, x):
        out = O.fused_layernorm(x, self.weight, self.bias, None, self.eps)
        return out[0] if isinstance(out, (tuple, list)) else out
