"""`ht.NDArray`: the imperative array type (reference: hetu/core/ndarray.h:17-550 and its Python binding
python_refactor/hetu/_binding/core/ndarray.cc: constructor from arrays / sequences / numpy, `numpy()`, `numel()`,
`to(dtype=, device=)`, `device`, `dtype`, plus ~100 static ops).

Storage, strides and the caching allocator are PyTorch's: an NDArray owns one `torch.Tensor` (`.data`) and every
static op forwards to the matching torch call or, for the LLM ops, to this package's kernels through
`ops.functional`.  The class exists so that code written against the reference's imperative API (feeds, state
dicts, checkpoint helpers, quick experiments) runs unchanged; the training path never goes through it.
"""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch
import torch.nn.functional as F

_DTYPES = {
    "uint8": torch.uint8, "int8": torch.int8, "int16": torch.int16, "int32": torch.int32, "int64": torch.int64,
    "float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32, "float64": torch.float64,
    "bool": torch.bool,
}


def _dtype(d):
    if d is None or isinstance(d, torch.dtype):
        return d
    if isinstance(d, str):
        return _DTYPES[d]
    name = getattr(d, "name", None) or str(d).split(".")[-1]
    return _DTYPES[name]


def _device(d):
    if d is None or isinstance(d, torch.device):
        return d
    if isinstance(d, str):
        return torch.device(d.replace("gpu", "cuda"))
    kind = getattr(d, "type", "cpu")
    idx = getattr(d, "local_index", getattr(d, "index", 0))
    return torch.device("cuda", idx) if kind in ("cuda", "gpu") else torch.device("cpu")


def _t(x):
    return x.data if isinstance(x, NDArray) else x


def _wrap(x):
    if isinstance(x, torch.Tensor):
        return NDArray(x, _share=True)
    if isinstance(x, (tuple, list)):
        return [_wrap(v) for v in x]
    return x


class NDArray:
    __slots__ = ("data",)

    def __init__(self, data, dtype=None, device=None, _share: bool = False):
        dtype, device = _dtype(dtype), _device(device)
        if isinstance(data, NDArray):
            t = data.data if _share else data.data.clone()
        elif isinstance(data, torch.Tensor):
            t = data if _share else data.clone()
        elif isinstance(data, np.ndarray):
            t = torch.from_numpy(np.ascontiguousarray(data)).clone()
        else:
            arr = np.asarray(data)
            if arr.dtype == np.float64 and dtype is None:      # python floats become float32, ints stay int64
                arr = arr.astype(np.float32)
            t = torch.from_numpy(arr)
        if dtype is not None or device is not None:
            t = t.to(device=device, dtype=dtype)
        self.data = t

    # ----------------------------------------------------------------- properties / conversions
    @property
    def dtype(self):
        return self.data.dtype

    @property
    def device(self):
        return self.data.device

    @property
    def shape(self):
        return list(self.data.shape)

    @property
    def ndim(self):
        return self.data.dim()

    def stride(self):
        return list(self.data.stride())

    def numel(self) -> int:
        return self.data.numel()

    def is_contiguous(self) -> bool:
        return self.data.is_contiguous()

    def numpy(self, force: bool = False) -> np.ndarray:
        t = self.data.detach()
        if t.dtype == torch.bfloat16:
            if not force:
                raise TypeError("numpy has no bfloat16; pass force=True to get float32")
            t = t.float()
        return t.cpu().numpy()

    def to(self, dtype=None, device=None) -> "NDArray":
        return NDArray.to_(self, device, dtype)

    def __repr__(self) -> str:
        return f"NDArray({self.data!r})"

    def __len__(self) -> int:
        return self.data.shape[0]

    def __getitem__(self, idx):
        return _wrap(self.data[idx])

    def __array__(self, dtype=None):
        a = self.numpy(force=True)
        return a.astype(dtype) if dtype is not None else a

    # ----------------------------------------------------------------- movement / casts
    @staticmethod
    def to_(x, device=None, dtype=None) -> "NDArray":
        return _wrap(_t(x).to(device=_device(device), dtype=_dtype(dtype)))

    @staticmethod
    def cuda(x, dev_id: int = 0):
        return _wrap(_t(x).to(torch.device("cuda", dev_id)))

    @staticmethod
    def cpu(x):
        return _wrap(_t(x).cpu())

    @staticmethod
    def copy(x):
        return _wrap(_t(x).clone())

    @staticmethod
    def contiguous(x):
        return _wrap(_t(x).contiguous())

    # ----------------------------------------------------------------- creation
    @staticmethod
    def empty(shape, device=None, dtype="float32"):
        return _wrap(torch.empty(tuple(shape), device=_device(device), dtype=_dtype(dtype)))

    @staticmethod
    def full(shape, value, device=None, dtype="float32"):
        return _wrap(torch.full(tuple(shape), value, device=_device(device), dtype=_dtype(dtype)))

    @staticmethod
    def zeros(shape, device=None, dtype="float32"):
        return NDArray.full(shape, 0, device, dtype)

    @staticmethod
    def ones(shape, device=None, dtype="float32"):
        return NDArray.full(shape, 1, device, dtype)

    @staticmethod
    def rand(shape, lb=0.0, ub=1.0, seed=None, device=None, dtype="float32"):
        return NDArray.uniform_(NDArray.empty(shape, device, dtype), lb, ub, seed)

    @staticmethod
    def randn(shape, mean=0.0, stddev=1.0, seed=None, device=None, dtype="float32"):
        return NDArray.normal_(NDArray.empty(shape, device, dtype), mean, stddev, seed)

    @staticmethod
    def empty_like(x):
        return _wrap(torch.empty_like(_t(x)))

    @staticmethod
    def full_like(x, value):
        return _wrap(torch.full_like(_t(x), value))

    @staticmethod
    def zeros_like(x):
        return _wrap(torch.zeros_like(_t(x)))

    @staticmethod
    def ones_like(x):
        return _wrap(torch.ones_like(_t(x)))

    @staticmethod
    def _gen(x, seed):
        if seed is None:
            return None
        return torch.Generator(device=_t(x).device).manual_seed(int(seed))

    @staticmethod
    def full_(x, value):
        _t(x).fill_(value)
        return x

    @staticmethod
    def zeros_(x):
        return NDArray.full_(x, 0)

    @staticmethod
    def ones_(x):
        return NDArray.full_(x, 1)

    @staticmethod
    def uniform_(x, lb=0.0, ub=1.0, seed=None):
        _t(x).uniform_(lb, ub, generator=NDArray._gen(x, seed))
        return x

    @staticmethod
    def normal_(x, mean=0.0, stddev=1.0, seed=None):
        _t(x).normal_(mean, stddev, generator=NDArray._gen(x, seed))
        return x

    @staticmethod
    def truncated_normal_(x, mean=0.0, stddev=1.0, lb=-2.0, ub=2.0, seed=None):
        torch.nn.init.trunc_normal_(_t(x), mean, stddev, lb, ub, generator=NDArray._gen(x, seed))
        return x

    # ----------------------------------------------------------------- elementwise
    @staticmethod
    def add(x, y):
        return _wrap(_t(x) + _t(y))

    @staticmethod
    def sub(x, y):
        return _wrap(_t(x) - _t(y))

    @staticmethod
    def mul(x, y):
        return _wrap(_t(x) * _t(y))

    @staticmethod
    def div(x, y):
        return _wrap(_t(x) / _t(y))

    @staticmethod
    def pow(x, exponent):
        return _wrap(torch.pow(_t(x), exponent))

    @staticmethod
    def where(cond, x, y):
        return _wrap(torch.where(_t(cond).bool(), _t(x), _t(y)))

    @staticmethod
    def leakyrelu(x, alpha=0.01):
        return _wrap(F.leaky_relu(_t(x), alpha))

    @staticmethod
    def gelu(x):
        return _wrap(F.gelu(_t(x)))

    @staticmethod
    def swiglu(x):
        """silu(x[..., :h]) * x[..., h:] on the packed gate/up tensor."""
        a, b = _t(x).chunk(2, dim=-1)
        return _wrap(F.silu(a) * b)

    # ----------------------------------------------------------------- reductions
    @staticmethod
    def reduce(x, kind: str, axes=None, keepdims: bool = False):
        t = _t(x)
        axes = list(range(t.dim())) if axes is None else ([axes] if isinstance(axes, int) else list(axes))
        if kind in ("sum", "mean"):
            return _wrap(getattr(torch, kind)(t, dim=axes, keepdim=keepdims))
        if kind in ("max", "min"):
            return _wrap(getattr(torch, "a" + kind)(t, dim=axes, keepdim=keepdims))
        if kind == "prod":
            for a in sorted((a % t.dim() for a in axes), reverse=True):
                t = t.prod(dim=a, keepdim=keepdims)
            return _wrap(t)
        raise ValueError(f"unknown reduction {kind}")

    @staticmethod
    def sum(x, axes=None, keepdims=False):
        return NDArray.reduce(x, "sum", axes, keepdims)

    @staticmethod
    def mean(x, axes=None, keepdims=False):
        return NDArray.reduce(x, "mean", axes, keepdims)

    @staticmethod
    def max(x, axes=None, keepdims=False):
        return NDArray.reduce(x, "max", axes, keepdims)

    @staticmethod
    def min(x, axes=None, keepdims=False):
        return NDArray.reduce(x, "min", axes, keepdims)

    @staticmethod
    def prod(x, axes=None, keepdims=False):
        return NDArray.reduce(x, "prod", axes, keepdims)

    @staticmethod
    def norm(x, p=2, dim=0, keepdim=False):
        return _wrap(torch.linalg.vector_norm(_t(x).float(), ord=p, dim=dim, keepdim=keepdim).to(_t(x).dtype))

    @staticmethod
    def softmax(x, dim=-1):
        return _wrap(torch.softmax(_t(x), dim=dim))

    # ----------------------------------------------------------------- linear algebra
    @staticmethod
    def matmul(x, y, trans_left=False, trans_right=False):
        a, b = _t(x), _t(y)
        return _wrap((a.transpose(-1, -2) if trans_left else a) @ (b.transpose(-1, -2) if trans_right else b))

    @staticmethod
    def bmm(x, y, trans_left=False, trans_right=False):
        return NDArray.matmul(x, y, trans_left, trans_right)

    @staticmethod
    def dot(x, y):
        return _wrap(torch.dot(_t(x).reshape(-1), _t(y).reshape(-1)))

    @staticmethod
    def linear(a, b, bias=None, trans_a=False, trans_b=True):
        a, b = _t(a), _t(b)
        out = (a.transpose(-1, -2) if trans_a else a) @ (b.transpose(-1, -2) if trans_b else b)
        return _wrap(out if bias is None else out + _t(bias))

    # ----------------------------------------------------------------- shape / view
    @staticmethod
    def reshape(x, shape):
        return _wrap(_t(x).reshape(tuple(shape)))

    @staticmethod
    def view(x, shape):
        return _wrap(_t(x).view(tuple(shape)))

    @staticmethod
    def flatten(x, start_dim=0, end_dim=-1):
        return _wrap(_t(x).flatten(start_dim, end_dim))

    @staticmethod
    def squeeze(x, dim=None):
        return _wrap(_t(x).squeeze() if dim is None else _t(x).squeeze(dim))

    @staticmethod
    def unsqueeze(x, dim):
        return _wrap(_t(x).unsqueeze(dim))

    @staticmethod
    def permute(x, dims):
        return _wrap(_t(x).permute(*dims))

    @staticmethod
    def movedim(x, src, dst):
        return _wrap(_t(x).movedim(src, dst))

    @staticmethod
    def adddim(x, dim, size):
        """Insert a dimension at `dim` and repeat the array `size` times along it."""
        return _wrap(_t(x).unsqueeze(dim).expand(*_t(x).shape[:dim], size, *_t(x).shape[dim:]).contiguous())

    @staticmethod
    def as_strided(x, shape, stride, storage_offset=0):
        return _wrap(torch.as_strided(_t(x), tuple(shape), tuple(stride), storage_offset))

    @staticmethod
    def broadcast(x, shape, add_axes: Sequence[int] = ()):
        t = _t(x)
        for a in sorted(add_axes):
            t = t.unsqueeze(a)
        return _wrap(t.expand(tuple(shape)).contiguous())

    @staticmethod
    def slice(x, begin, size):
        t = _t(x)
        idx = tuple(slice(b, b + s) for b, s in zip(begin, size))
        return _wrap(t[idx])

    @staticmethod
    def split(x, parts, axis=0):
        """`parts`: a count (equal chunks) or a list of sizes."""
        t = _t(x)
        if isinstance(parts, int):
            return _wrap(list(t.chunk(parts, dim=axis)))
        return _wrap(list(t.split(list(parts), dim=axis)))

    @staticmethod
    def cat(xs, axis=0):
        return _wrap(torch.cat([_t(v) for v in xs], dim=axis))

    @staticmethod
    def repeat(x, repeats):
        return _wrap(_t(x).repeat(*repeats))

    @staticmethod
    def roll(x, shifts, dims):
        return _wrap(torch.roll(_t(x), shifts, dims))

    @staticmethod
    def pad(x, paddings, mode="constant", value=0.0):
        return _wrap(F.pad(_t(x), list(paddings), mode=mode.lower(), value=value))

    @staticmethod
    def triu(x, lower=False, diagonal=0):
        return _wrap(torch.tril(_t(x), diagonal) if lower else torch.triu(_t(x), diagonal))

    @staticmethod
    def diagonal(x, dim1=0, dim2=1, offset=0):
        return _wrap(torch.diagonal(_t(x), offset, dim1, dim2))

    @staticmethod
    def diagonal_grad(g, dim1=0, dim2=1):
        return _wrap(torch.diag_embed(_t(g), 0, dim1, dim2))

    # ----------------------------------------------------------------- indexing
    @staticmethod
    def gather(x, dim, index):
        return _wrap(torch.gather(_t(x), dim, _t(index).long()))

    @staticmethod
    def onehot(ids, num_classes):
        return _wrap(F.one_hot(_t(ids).long(), num_classes).float())

    @staticmethod
    def embedding(table, ids):
        return _wrap(F.embedding(_t(ids).long(), _t(table)))

    @staticmethod
    def index_add(x, index, source, dim=0):
        return _wrap(_t(x).index_add(dim, _t(index).long(), _t(source)))

    @staticmethod
    def arrayset(x, value):
        return NDArray.full_(x, value)

    # ----------------------------------------------------------------- normalisation / CNN / losses
    @staticmethod
    def layernorm(x, scale, bias, normalized_shape, eps=1e-5):
        return _wrap(F.layer_norm(_t(x), tuple(normalized_shape), _t(scale), _t(bias), eps))

    @staticmethod
    def fused_layernorm(x, scale, bias, normalized_shape, eps=1e-5):
        return NDArray.layernorm(x, scale, bias, normalized_shape, eps)

    @staticmethod
    def instancenorm(x, eps=1e-5):
        return _wrap(F.instance_norm(_t(x), eps=eps))

    @staticmethod
    def batchnorm(x, scale, bias, running_mean, running_var, momentum=0.1, eps=1e-5):
        return _wrap(F.batch_norm(_t(x), _t(running_mean), _t(running_var), _t(scale), _t(bias), True, momentum, eps))

    @staticmethod
    def conv2d(x, w, bias=None, padding=0, stride=1):
        return _wrap(F.conv2d(_t(x), _t(w), None if bias is None else _t(bias), stride, padding))

    @staticmethod
    def maxpool(x, kernel_h, kernel_w, padding=0, stride=1):
        return _wrap(F.max_pool2d(_t(x), (kernel_h, kernel_w), stride, padding))

    @staticmethod
    def avgpool(x, kernel_h, kernel_w, padding=0, stride=1):
        return _wrap(F.avg_pool2d(_t(x), (kernel_h, kernel_w), stride, padding))

    @staticmethod
    def _red(loss, reduction):
        reduction = str(reduction).lower()
        return loss.mean() if reduction == "mean" else loss.sum() if reduction == "sum" else loss

    @staticmethod
    def mseloss(pred, label, reduction="mean"):
        return _wrap(NDArray._red((_t(pred) - _t(label)) ** 2, reduction))

    @staticmethod
    def nllloss(pred, label, reduction="mean"):
        return _wrap(NDArray._red(F.nll_loss(_t(pred), _t(label).long(), reduction="none"), reduction))

    @staticmethod
    def kldiv(pred, label, reduction="mean"):
        return _wrap(NDArray._red(F.kl_div(_t(pred), _t(label), reduction="none"), reduction))

    @staticmethod
    def sceloss(logits, label, reduction="mean"):
        return _wrap(NDArray._red(F.cross_entropy(_t(logits), _t(label).long(), reduction="none"), reduction))


def _unary(name, fn):
    def op(x):
        return _wrap(fn(_t(x)))
    op.__name__ = name
    setattr(NDArray, name, staticmethod(op))


for _n, _f in dict(abs=torch.abs, neg=torch.neg, ceil=torch.ceil, floor=torch.floor, round=torch.round,
                   exp=torch.exp, log=torch.log, sqrt=torch.sqrt, sin=torch.sin, cos=torch.cos,
                   sigmoid=torch.sigmoid, tanh=torch.tanh, relu=torch.relu, reciprocal=torch.reciprocal).items():
    _unary(_n, _f)

for _n, _d in dict(toUInt8="uint8", toInt8="int8", toInt16="int16", toInt32="int32", toInt64="int64",
                   toFloat32="float32", toFloat64="float64").items():
    setattr(NDArray, _n, staticmethod(lambda x, _d=_d: NDArray.to_(x, None, _d)))


def _binop(fn, swap=False):
    def op(self, other):
        a, b = (_t(other), _t(self)) if swap else (_t(self), _t(other))
        return _wrap(fn(a, b))
    return op


NDArray.__add__ = _binop(torch.add)
NDArray.__radd__ = _binop(torch.add, True)
NDArray.__sub__ = _binop(torch.sub)
NDArray.__rsub__ = _binop(lambda a, b: torch.as_tensor(a) - b, True)
NDArray.__mul__ = _binop(torch.mul)
NDArray.__rmul__ = _binop(torch.mul, True)
NDArray.__truediv__ = _binop(torch.div)
NDArray.__rtruediv__ = _binop(lambda a, b: torch.as_tensor(a) / b, True)
NDArray.__matmul__ = _binop(torch.matmul)
NDArray.__neg__ = lambda self: _wrap(-self.data)


def numpy_to_NDArray(array: np.ndarray, dtype=None, device=None) -> NDArray:
    """Shares memory with `array` when no cast or move is asked for (like the reference's zero-copy wrap)."""
    t = torch.from_numpy(np.ascontiguousarray(array))
    return NDArray(t, dtype=dtype, device=device, _share=True)
