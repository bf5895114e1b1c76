"""Parameter initializers.  An initializer fills the *global* tensor from a seed that depends only on
the parameter (not on the strategy or the rank); each rank then keeps its DS slice, so every
strategy starts from identical weights.  Reference: hetu/graph/init/initializer.h (Constant, Uniform,
Normal, TruncatedNormal, generalized Xavier/He/LeCun, Provided); the reference seeds per shard
(hetu/graph/ops/variable.cc:38-43), which this design replaces on purpose.
"""
from __future__ import annotations

import math

import numpy as np
import torch


class Initializer:
    def fill(self, shape, gen: torch.Generator, device) -> torch.Tensor:  # fp32 global tensor
        raise NotImplementedError


class ConstantInitializer(Initializer):
    def __init__(self, value: float):
        self.value = float(value)

    def fill(self, shape, gen, device):
        return torch.full(shape, self.value, dtype=torch.float32, device=device)


class UniformInitializer(Initializer):
    def __init__(self, lb=-0.05, ub=0.05):
        self.lb, self.ub = lb, ub

    def fill(self, shape, gen, device):
        return torch.empty(shape, dtype=torch.float32, device=device).uniform_(self.lb, self.ub, generator=gen)


class NormalInitializer(Initializer):
    def __init__(self, mean=0.0, stddev=0.02):
        self.mean, self.stddev = mean, stddev

    def fill(self, shape, gen, device):
        return torch.empty(shape, dtype=torch.float32, device=device).normal_(self.mean, self.stddev, generator=gen)


class TruncatedNormalInitializer(NormalInitializer):
    def __init__(self, mean=0.0, stddev=0.02, lb=-2.0, ub=2.0):
        super().__init__(mean, stddev)
        self.lb, self.ub = lb, ub

    def fill(self, shape, gen, device):
        t = super().fill(shape, gen, device)
        lo, hi = self.mean + self.lb * self.stddev, self.mean + self.ub * self.stddev
        return t.clamp_(lo, hi)


class GeneralizedXavierInitializer(Initializer):
    """gain / fan mode / distribution cover Xavier, He and LeCun in their uniform and normal forms."""

    def __init__(self, gain=1.0, mode="avg", dist="normal"):
        self.gain, self.mode, self.dist = gain, mode, dist

    def fill(self, shape, gen, device):
        fan_out, fan_in = (shape[0], shape[1]) if len(shape) >= 2 else (shape[0], shape[0])
        if len(shape) > 2:
            rf = math.prod(shape[2:])
            fan_in, fan_out = fan_in * rf, fan_out * rf
        fan = {"fan_in": fan_in, "fan_out": fan_out, "avg": (fan_in + fan_out) / 2.0}[self.mode]
        if self.dist == "normal":
            return NormalInitializer(0.0, math.sqrt(self.gain / fan)).fill(shape, gen, device)
        lim = math.sqrt(3.0 * self.gain / fan)
        return UniformInitializer(-lim, lim).fill(shape, gen, device)


class ProvidedInitializer(Initializer):
    def __init__(self, data):
        self.data = np.asarray(data)

    def fill(self, shape, gen, device):
        return torch.from_numpy(self.data.astype(np.float32)).reshape(shape).to(device)


def constant_initializer(v): return ConstantInitializer(v)
def zeros_initializer(): return ConstantInitializer(0.0)
def ones_initializer(): return ConstantInitializer(1.0)
def uniform_initializer(lb=-0.05, ub=0.05): return UniformInitializer(lb, ub)
def normal_initializer(mean=0.0, stddev=0.02): return NormalInitializer(mean, stddev)
def truncated_normal_initializer(mean=0.0, stddev=0.02, lb=-2.0, ub=2.0): return TruncatedNormalInitializer(mean, stddev, lb, ub)
def xavier_normal_initializer(gain=1.0): return GeneralizedXavierInitializer(gain, "avg", "normal")
def xavier_uniform_initializer(gain=1.0): return GeneralizedXavierInitializer(gain, "avg", "uniform")
def he_normal_initializer(gain=2.0): return GeneralizedXavierInitializer(gain, "fan_in", "normal")
def he_uniform_initializer(gain=2.0): return GeneralizedXavierInitializer(gain, "fan_in", "uniform")
def lecun_normal_initializer(gain=1.0): return GeneralizedXavierInitializer(gain, "fan_in", "normal")
def lecun_uniform_initializer(gain=1.0): return GeneralizedXavierInitializer(gain, "fan_in", "uniform")
def provided_initializer(data): return ProvidedInitializer(data)


__all__ = sorted(n for n, v in list(globals().items())
                 if not n.startswith("_") and callable(v) and getattr(v, "__module__", None) == __name__)
