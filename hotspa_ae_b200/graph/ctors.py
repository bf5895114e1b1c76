"""Tensor constructors of the package namespace: ``ht.empty / zeros / ones / full / rand / randn / trunc_randn`` and
their ``*_like`` forms (reference: python_refactor/hetu/_binding/graph/tensor_ctor.cc:223-560).  Each makes a variable
tensor in the current graph, filled by the matching initializer; ``ds_hierarchy`` (one union per strategy) gives its
layout, the default is a replica on every device."""
from __future__ import annotations

import itertools

import torch

from ..core import DistributedStates, DistributedStatesUnion
from ..parallel import mesh as M
from . import graph as G
from . import init as I

_ids = itertools.count()


def _make(init, size, dtype, requires_grad, ds_hierarchy, device_group_hierarchy, name, kind):
    g = G.current_graph()
    if ds_hierarchy is None:
        n = M.mesh().world_size
        ds_hierarchy = [DistributedStatesUnion([DistributedStates(n, {-1: n}, [-1])]) for _ in range(g.num_strategy)]
    return G.parallel_parameter(init, [int(s) for s in size], ds_hierarchy, None, dtype=dtype or torch.float32,
                                requires_grad=bool(requires_grad), device_group_hierarchy=device_group_hierarchy,
                                name=name or f"{kind}_{next(_ids)}")


def _like(t, dtype, ds_hierarchy, device_group_hierarchy):
    return (list(t.global_shape), dtype or t.dtype, ds_hierarchy if ds_hierarchy is not None else list(t.ds_hierarchy),
            device_group_hierarchy if device_group_hierarchy is not None else [list(g) for g in t.dg_hierarchy])


def empty(size, dtype=None, requires_grad=False, ds_hierarchy=None, device_group_hierarchy=None, name=None):
    """Uninitialised in the reference; zero-filled here (arenas start cleared)."""
    return _make(I.zeros_initializer(), size, dtype, requires_grad, ds_hierarchy, device_group_hierarchy, name, "empty")


def zeros(size, dtype=None, requires_grad=False, ds_hierarchy=None, device_group_hierarchy=None, name=None):
    return _make(I.zeros_initializer(), size, dtype, requires_grad, ds_hierarchy, device_group_hierarchy, name, "zeros")


def ones(size, dtype=None, requires_grad=False, ds_hierarchy=None, device_group_hierarchy=None, name=None):
    return _make(I.ones_initializer(), size, dtype, requires_grad, ds_hierarchy, device_group_hierarchy, name, "ones")


def full(size, fill_value, dtype=None, requires_grad=False, ds_hierarchy=None, device_group_hierarchy=None, name=None):
    return _make(I.constant_initializer(float(fill_value)), size, dtype, requires_grad, ds_hierarchy,
                 device_group_hierarchy, name, "full")


def rand(size, lb=0.0, ub=1.0, dtype=None, requires_grad=False, ds_hierarchy=None, device_group_hierarchy=None,
         name=None):
    return _make(I.uniform_initializer(float(lb), float(ub)), size, dtype, requires_grad, ds_hierarchy,
                 device_group_hierarchy, name, "rand")


def randn(size, mean=0.0, stddev=1.0, dtype=None, requires_grad=False, ds_hierarchy=None,
          device_group_hierarchy=None, name=None):
    return _make(I.normal_initializer(float(mean), float(stddev)), size, dtype, requires_grad, ds_hierarchy,
                 device_group_hierarchy, name, "randn")


def trunc_randn(size, mean=0.0, stddev=1.0, lb=-2.0, ub=2.0, dtype=None, requires_grad=False, ds_hierarchy=None,
                device_group_hierarchy=None, name=None):
    return _make(I.truncated_normal_initializer(float(mean), float(stddev), float(lb), float(ub)), size, dtype,
                 requires_grad, ds_hierarchy, device_group_hierarchy, name, "trunc_randn")


def empty_like(tensor, dtype=None, requires_grad=False, ds_hierarchy=None, device_group_hierarchy=None, name=None):
    s, d, h, dg = _like(tensor, dtype, ds_hierarchy, device_group_hierarchy)
    return empty(s, d, requires_grad, h, dg, name)


def full_like(tensor, fill_value, dtype=None, requires_grad=False, ds_hierarchy=None, device_group_hierarchy=None,
              name=None):
    s, d, h, dg = _like(tensor, dtype, ds_hierarchy, device_group_hierarchy)
    return full(s, fill_value, d, requires_grad, h, dg, name)


def rand_like(tensor, lb=0.0, ub=1.0, dtype=None, requires_grad=False, ds_hierarchy=None, device_group_hierarchy=None,
              name=None):
    s, d, h, dg = _like(tensor, dtype, ds_hierarchy, device_group_hierarchy)
    return rand(s, lb, ub, d, requires_grad, h, dg, name)


def randn_like(tensor, mean=0.0, stddev=1.0, dtype=None, requires_grad=False, ds_hierarchy=None,
               device_group_hierarchy=None, name=None):
    s, d, h, dg = _like(tensor, dtype, ds_hierarchy, device_group_hierarchy)
    return randn(s, mean, stddev, d, requires_grad, h, dg, name)


def trunc_randn_like(tensor, mean=0.0, stddev=1.0, lb=-2.0, ub=2.0, dtype=None, requires_grad=False,
                     ds_hierarchy=None, device_group_hierarchy=None, name=None):
    s, d, h, dg = _like(tensor, dtype, ds_hierarchy, device_group_hierarchy)
    return trunc_randn(s, mean, stddev, lb, ub, d, requires_grad, h, dg, name)
