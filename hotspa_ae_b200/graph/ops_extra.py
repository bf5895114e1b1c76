"""Long tail of the op library: shape/view ops, classic losses, CNN ops, masks and index ops.

These ops are off the LLM hot path; their compute is the matching PyTorch expression on the local shard, with
the same three hooks as the ops of :mod:`ops` (infer / deduce / compute).  Output shapes are inferred by running
the expression on meta tensors of the current global shapes.  Distributed states: the batch (first) dimension
may be split (data parallel); any other split must be resolved with ``ht.comm`` first.
Reference counterparts: the ops bound in python_refactor/hetu/_binding/codegen/ops.yml that are not in
:mod:`ops` (Broadcast, Pad, Diagonal, Einsum, Conv2d, pooling, BatchNorm, InstanceNorm, classic losses, Gather,
Interpolate, RangeMask, MaskedFill, Norm, AsStrided, Repeat, Roll, Onehot, Triu, Arange, Dot, in-place variants).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..core import DistributedStates, IntSymbol
from . import ops as O
from .ops import make_op_front, register


def _batch_only_ds(ds: DistributedStates, out_ndim: int) -> DistributedStates:
    n = ds.device_num
    for d, c in ds.states.items():
        if d > 0 and c > 1:
            raise ValueError(f"this op needs its non-batch dimensions unsplit, got {ds}; reshard with ht.comm first")
    if ds.get_dim(-2) > 1:
        raise ValueError("this op cannot consume a partial tensor; reduce it with ht.comm first")
    b = ds.get_dim(0) if out_ndim > 0 else 1
    states = {-1: n // b}
    if b > 1:
        states[0] = b
    order = [o for o in ds.order if o in (0, -1) and states.get(o, 1) > 1]
    for o in (0, -1):
        if states.get(o, 1) > 1 and o not in order:
            order.append(o)
    return DistributedStates(n, states, order)


def _register_local(name: str, fn, n_out: int = 1, keep_batch: bool = True):
    """`fn(*tensors, **attrs)` -> tensor or tuple; shape inference runs it on meta tensors."""

    @register(name)
    class _Local:
        @staticmethod
        def infer(inputs, attrs):
            metas = [torch.empty(t.global_shape, dtype=t.dtype, device="meta") for t in inputs]
            outs = fn(*metas, **attrs)
            outs = outs if isinstance(outs, (tuple, list)) else [outs]
            return [([IntSymbol(int(s)) for s in o.shape] or [IntSymbol(1)], o.dtype) for o in outs]

        @staticmethod
        def deduce(in_ds, attrs, inputs):
            metas = [torch.empty(t.global_shape, dtype=t.dtype, device="meta") for t in inputs]
            outs = fn(*metas, **attrs)
            outs = outs if isinstance(outs, (tuple, list)) else [outs]
            res = []
            for o in outs:
                keeps = keep_batch and o.dim() > 0 and inputs and inputs[0].ndim > 0 and \
                    o.shape[0] == inputs[0].global_shape[0]
                ds = _batch_only_ds(in_ds[0], o.dim()) if in_ds else DistributedStates(1, {-1: 1}, [-1])
                if not keeps and ds.get_dim(0) > 1:
                    raise ValueError(f"{name}: the batch split does not survive this op; reshard first")
                res.append(ds)
            return res

        @staticmethod
        def compute(rt, op, vals):
            outs = fn(*vals, **op.attrs)
            return list(outs) if isinstance(outs, (tuple, list)) else [outs]
    return _Local


def _front(name, n_in, **defaults):
    def f(*args, name_=None, **kw):
        tensors = [a for a in args[:n_in] if a is not None]
        attrs = dict(defaults)
        keys = list(defaults)
        for k, v in zip(keys, args[n_in:]):
            attrs[k] = v
        attrs.update(kw)
        outs = make_op_front(name, tensors, attrs, name_)
        return outs[0] if len(outs) == 1 else tuple(outs)
    f.__name__ = name
    return f


# ---- shape / view / index -------------------------------------------------------------------------------
def _expand_shape(x, shape, add_axes):
    if not add_axes:
        return [1] * (len(shape) - x.dim()) + list(x.shape)
    it = iter(x.shape)
    return [1 if i in set(add_axes) else next(it) for i in range(len(shape))]


_register_local("broadcast", lambda x, shape, add_axes=(): x.reshape(_expand_shape(x, shape, add_axes)).expand(*shape),
                keep_batch=False)
broadcast = _front("broadcast", 1, shape=None, add_axes=())

_register_local("pad", lambda x, pads, mode="constant", constant=0.0: F.pad(x, list(pads), mode=mode.lower(),
                                                                            value=constant if mode.lower() == "constant" else None))
pad = _front("pad", 1, pads=None, mode="constant", constant=0.0)

_register_local("diagonal", lambda x, offset=0, dim1=0, dim2=1: torch.diagonal(x, offset, dim1, dim2), keep_batch=False)
diagonal = _front("diagonal", 1, offset=0, dim1=0, dim2=1)

_register_local("triu", lambda x, lower=False, diagonal=0: torch.tril(x, diagonal) if lower else torch.triu(x, diagonal))
triu = _front("triu", 1, lower=False, diagonal=0)

_register_local("repeat", lambda x, repeats: x.repeat(*repeats), keep_batch=False)
repeat = _front("repeat", 1, repeats=None)

_register_local("roll", lambda x, shifts, dims: torch.roll(x, list(shifts), list(dims)))
roll = _front("roll", 1, shifts=None, dims=None)

_register_local("as_strided", lambda x, outshape, stride, storage_offset=0: torch.as_strided(
    x.contiguous(), list(outshape), list(stride), storage_offset).clone(), keep_batch=False)
as_strided = _front("as_strided", 1, outshape=None, stride=None, storage_offset=0)

_register_local("gather", lambda x, index, dim=0: torch.gather(x, dim, index.long()))
gather = lambda x, dim, index, name=None: make_op_front("gather", [x, index], {"dim": dim}, name)[0]  # noqa: E731

_register_local("onehot", lambda x, num_classes: F.one_hot(x.long(), num_classes).float())
onehot = _front("onehot", 1, num_classes=None)

_register_local("masked_fill", lambda x, mask, val=0.0: x.masked_fill(mask.bool(), val))
masked_fill = lambda x, mask, val, name=None: make_op_front("masked_fill", [x, mask], {"val": val}, name)[0]  # noqa: E731

_register_local("range_mask", lambda x, min=0, max=0: ((x >= min) & (x <= max)).to(x.dtype))  # noqa: A002
range_mask = _front("range_mask", 1, min=0, max=0)

_register_local("dynamic_concat", lambda *xs, axis=0: torch.cat(xs, dim=axis), keep_batch=False)


def dynamic_concat(xs, axis=0, name=None):
    return make_op_front("dynamic_concat", list(xs), {"axis": axis}, name)[0]


@register("arange")
class _Arange:
    @staticmethod
    def infer(inputs, attrs):
        n = len(range(int(attrs["start"]), int(attrs["end"]), int(attrs["step"])))
        return [([IntSymbol(n)], torch.int64 if all(float(attrs[k]).is_integer() for k in ("start", "end", "step"))
                 else torch.float32)]

    @staticmethod
    def deduce(in_ds, attrs, inputs):
        from ..parallel import mesh as M
        n = M.mesh().world_size
        return [DistributedStates(n, {-1: n}, [-1])]

    @staticmethod
    def compute(rt, op, vals):
        a = op.attrs
        return [torch.arange(a["start"], a["end"], a["step"], device=rt.mesh.torch_device)]


def arange(start, end=None, step=1, name=None):
    if end is None:
        start, end = 0, start
    return make_op_front("arange", [], {"start": start, "end": end, "step": step}, name)[0]


# ---- math ------------------------------------------------------------------------------------------------
_register_local("einsum", lambda *xs, equation="": torch.einsum(equation, *xs), keep_batch=False)


def einsum(equation, *xs, name=None):
    xs = xs[0] if len(xs) == 1 and isinstance(xs[0], (list, tuple)) else xs
    return make_op_front("einsum", list(xs), {"equation": equation}, name)[0]


_register_local("dot", lambda a, b: (a * b).sum().reshape(1) if a.dim() == 1 else a @ b, keep_batch=False)
dot = _front("dot", 2)

_register_local("norm", lambda x, p=2, dim=0, keepdim=False: torch.linalg.vector_norm(x.float(), ord=p, dim=dim,
                                                                                      keepdim=keepdim).to(x.dtype))
norm = _front("norm", 1, p=2, dim=0, keepdim=False)

_register_local("interpolate", lambda x, outshape=None, align_corners=False, scale_factor=0.0: F.interpolate(
    x, size=list(outshape) if outshape else None, scale_factor=scale_factor or None, mode="bicubic",
    align_corners=align_corners))
interpolate = _front("interpolate", 1, outshape=None, align_corners=False, scale_factor=0.0)

_register_local("dropout2d", lambda x, p=0.5: F.dropout2d(x, p, True))
dropout2d = _front("dropout2d", 1, p=0.5)

# ---- classic losses ----------------------------------------------------------------------------------------
_RED = {"mean": "mean", "sum": "sum", "none": "none"}


def _reduce1(v):
    return v.reshape(1) if v.dim() == 0 else v


_register_local("binary_cross_entropy", lambda p, y, reduction="mean": _reduce1(
    F.binary_cross_entropy(p.float(), y.float(), reduction=_RED[reduction.lower()])), keep_batch=False)
binary_cross_entropy = _front("binary_cross_entropy", 2, reduction="mean")

_register_local("nll_loss", lambda p, y, reduction="mean": _reduce1(
    F.nll_loss(p.float(), y.long(), reduction=_RED[reduction.lower()])), keep_batch=False)
nll_loss = _front("nll_loss", 2, reduction="mean")

_register_local("kl_div", lambda p, y, reduction="mean": _reduce1(
    F.kl_div(p.float(), y.float(), reduction=_RED[reduction.lower()])), keep_batch=False)
kl_div = _front("kl_div", 2, reduction="mean")

_register_local("softmax_cross_entropy", lambda p, y, reduction="mean": _reduce1(
    (-(F.log_softmax(p.float(), -1) * y.float()).sum(-1)) if reduction.lower() == "none" else
    getattr(-(F.log_softmax(p.float(), -1) * y.float()).sum(-1), reduction.lower())()), keep_batch=False)
softmax_cross_entropy = _front("softmax_cross_entropy", 2, reduction="mean")

# ---- CNN ----------------------------------------------------------------------------------------------------
_register_local("conv2d", lambda x, w, b=None, padding=0, stride=1: F.conv2d(x, w.to(x.dtype), None if b is None else
                                                                              b.to(x.dtype), stride, padding))


def conv2d(x, weight, bias=None, padding=0, stride=1, name=None):
    ins = [x, weight] + ([bias] if bias is not None else [])
    return make_op_front("conv2d", ins, {"padding": padding, "stride": stride}, name)[0]


_register_local("avgpool", lambda x, kernel_H=2, kernel_W=2, padding=0, stride=1: F.avg_pool2d(
    x, (kernel_H, kernel_W), stride, padding))
avgpool = _front("avgpool", 1, kernel_H=2, kernel_W=2, padding=0, stride=1)

_register_local("maxpool", lambda x, kernel_H=2, kernel_W=2, padding=0, stride=1: F.max_pool2d(
    x, (kernel_H, kernel_W), stride, padding))
maxpool = _front("maxpool", 1, kernel_H=2, kernel_W=2, padding=0, stride=1)


def _batch_norm(x, scale, bias, running_mean, running_var, momentum=0.1, eps=1e-5):
    return F.batch_norm(x, running_mean, running_var, scale, bias, True, momentum, eps)


_register_local("batch_norm", _batch_norm)


def batch_norm(x, scale, bias, running_mean, running_var, momentum=0.1, eps=1e-5, name=None):
    return make_op_front("batch_norm", [x, scale, bias, running_mean, running_var],
                         {"momentum": momentum, "eps": eps}, name)[0]


_register_local("instance_norm", lambda x, eps=1e-7: F.instance_norm(x, eps=eps))
instance_norm = _front("instance_norm", 1, eps=1e-7)

_register_local("layer_norm_plain", lambda x, w, b, normalized_shape=None, eps=1e-5: F.layer_norm(
    x, list(normalized_shape) if normalized_shape else list(x.shape[-1:]), w.to(x.dtype), b.to(x.dtype), eps))


def layer_norm(x, weight, bias, normalized_shape=None, eps=1e-5, name=None):
    return make_op_front("layer_norm_plain", [x, weight, bias], {"normalized_shape": normalized_shape, "eps": eps},
                         name)[0]


# ---- in-place spellings ------------------------------------------------------------------------------------
# The graph is functional: an in-place op returns a new tensor that replaces its first operand downstream.
add_, sub_, mul_, div_ = O.add, O.sub, O.mul, O.div
neg_, sqrt_, rsqrt_, reciprocal_, pow_ = O.neg, O.sqrt, O.rsqrt, O.reciprocal, O.pow
ceil_, floor_, round_, relu_, sigmoid_, sin_, abs_, exp_, log_, tanh_ = (O.ceil, O.floor, O.round, O.relu, O.sigmoid,
                                                                          O.sin, O.abs, O.exp, O.log, O.tanh)
leakyrelu = leakyrelu_ = O.leaky_relu
dropout_ = O.dropout
dropout2d_ = dropout2d
where_ = O.where
sum = O.reduce_sum  # noqa: A001
mean = O.reduce_mean

__all__ = ["broadcast", "pad", "diagonal", "triu", "repeat", "roll", "as_strided", "gather", "onehot", "masked_fill",
           "range_mask", "dynamic_concat", "arange", "einsum", "dot", "norm", "interpolate", "dropout2d",
           "binary_cross_entropy", "nll_loss", "kl_div", "softmax_cross_entropy", "conv2d", "avgpool", "maxpool",
           "batch_norm", "instance_norm", "layer_norm", "add_", "sub_", "mul_", "div_", "neg_", "sqrt_", "rsqrt_",
           "reciprocal_", "pow_", "ceil_", "floor_", "round_", "relu_", "sigmoid_", "sin_", "abs_", "exp_", "log_",
           "tanh_", "leakyrelu", "leakyrelu_", "dropout_", "dropout2d_", "where_", "sum", "mean"]
