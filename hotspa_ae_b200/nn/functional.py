"""Weight constructors of `hetu.nn.functional` (reference: python_refactor/hetu/nn/functional.py): each returns a new
replicated parameter tensor of the given shape filled by the named scheme.  `hetu.nn.init` is the same module."""
from __future__ import annotations

import math

from ..graph import init as I
from ..graph.tensor import float32
from .layers import _param

_counter = [0]


def _new(init, shape, requires_grad, name):
    _counter[0] += 1
    t = _param(init, list(shape), name or f"functional_param_{_counter[0]}")
    t.requires_grad = bool(requires_grad)
    return t


def calculate_gain(nonlinearity: str, param: float | None = None) -> float:
    if nonlinearity in ("linear", "conv1d", "conv2d", "conv3d", "sigmoid"):
        return 1.0
    if nonlinearity == "tanh":
        return 5.0 / 3
    if nonlinearity == "relu":
        return math.sqrt(2.0)
    if nonlinearity == "leaky_relu":
        slope = 0.01 if param is None else float(param)
        return math.sqrt(2.0 / (1 + slope ** 2))
    raise ValueError(f"unsupported nonlinearity {nonlinearity}")


def generalized_xavier_(tshape, dist: str, mode: str, gain: float, requires_grad: bool = False, dtype=float32,
                        device_group=None, name=None):
    """normal: std = sqrt(gain / fan); uniform: limit = sqrt(gain / fan) (callers fold the factor 3 into `gain`,
    like the reference's)."""
    init = I.GeneralizedXavierInitializer(gain / 3.0 if dist == "uniform" else gain, mode, dist)
    return _new(init, tshape, requires_grad, name)


def xavier_uniform_(tshape, gain: float = 1.0, requires_grad: bool = False, device_group=None, name=None):
    return generalized_xavier_(tshape, "uniform", "avg", gain * 3, requires_grad, name=name)


def xavier_normal_(tshape, gain: float = 1.0, requires_grad: bool = False, device_group=None, name=None):
    return generalized_xavier_(tshape, "normal", "avg", gain, requires_grad, name=name)


def kaiming_uniform_(tshape, a: float = 0.0, mode: str = "fan_in", nonlinearity: str = "leaky_relu",
                     requires_grad: bool = False, dtype=float32, device_group=None, name=None):
    gain = calculate_gain(nonlinearity, a)
    return generalized_xavier_(tshape, "uniform", mode, gain ** 2 * 3, requires_grad, name=name)


def kaiming_normal_(tshape, a: float = 0.0, mode: str = "fan_in", nonlinearity: str = "leaky_relu",
                    requires_grad: bool = False, dtype=float32, device_group=None, name=None):
    gain = calculate_gain(nonlinearity, a)
    return generalized_xavier_(tshape, "normal", mode, gain ** 2, requires_grad, name=name)


he_uniform_, he_normal_ = kaiming_uniform_, kaiming_normal_


def lecun_uniform_(tshape, gain: float = 1.0, requires_grad: bool = False, device_group=None, name=None):
    return generalized_xavier_(tshape, "uniform", "fan_in", gain * 3, requires_grad, name=name)


def lecun_normal_(tshape, gain: float = 1.0, requires_grad: bool = False, device_group=None, name=None):
    return generalized_xavier_(tshape, "normal", "fan_in", gain, requires_grad, name=name)


def zeros_(tshape, requires_grad: bool = False, name=None):
    return _new(I.zeros_initializer(), tshape, requires_grad, name)


def ones_(tshape, requires_grad: bool = False, name=None):
    return _new(I.ones_initializer(), tshape, requires_grad, name)


def constant_(tshape, value: float, requires_grad: bool = False, name=None):
    return _new(I.constant_initializer(value), tshape, requires_grad, name)


def uniform_(tshape, lb: float = 0.0, ub: float = 1.0, requires_grad: bool = False, name=None):
    return _new(I.uniform_initializer(lb, ub), tshape, requires_grad, name)


def normal_(tshape, mean: float = 0.0, std: float = 1.0, requires_grad: bool = False, name=None):
    return _new(I.normal_initializer(mean, std), tshape, requires_grad, name)
