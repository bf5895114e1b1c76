"""Graph-level optimizers.  ``minimize(loss)`` returns the train op; running it at run level UPDATE makes
the executor reduce the gradients and call :meth:`apply_flat` once per flat shard (not once per tensor).
Reference: hetu/graph/optim/optimizer.cc, hetu/graph/ops/optimizer_update.cc, hetu/impl/kernel/Optimizers.cu.
"""
from __future__ import annotations

import torch

from ..graph import ops as O
from ..ops import _lib


class GradHandle:
    """Fetchable stand-in for "the gradient of the loss with respect to `var`"."""
    is_grad_handle = True
    is_train_op = False

    def __init__(self, var):
        self.var = var
        self.graph = var.graph
        self.id = ("grad", var.id)
        self.name = f"grad({var.name})"

    def __repr__(self):
        return f"GradHandle({self.var.name})"


class Optimizer:
    def __init__(self, lr: float):
        self.lr = lr
        self.loss = None

    def minimize(self, loss, var_list=None, name=None):
        """compute_gradients + apply_gradients (reference: Optimizer::Minimize, hetu/graph/optim/optimizer.cc)."""
        return self.apply_gradients(self.compute_gradients(loss, var_list), name=name)

    def compute_gradients(self, loss, var_list=None):
        """[(gradient handle, variable)] for the trainable parameters `loss` depends on (or `var_list`).  A handle
        can be fetched in the same `graph.run` as the train op: it yields this rank's fp32 gradient accumulator of
        the variable as it stands after the backward pass (before the data-parallel reduction and the update)."""
        g = loss.graph
        self.loss = loss
        params = [p for p in (var_list if var_list is not None else g.parameters) if p.requires_grad]
        self.var_list = None if var_list is None else list(params)
        return [(GradHandle(p), p) for p in params]

    def apply_gradients(self, grads_and_vars, name=None):
        """The train op that reduces the gradients and updates the variables at run level "update"."""
        pairs = list(grads_and_vars)
        if not pairs:
            raise ValueError("apply_gradients: no variables")
        if self.loss is None:
            raise RuntimeError("apply_gradients needs the pairs returned by compute_gradients")
        for gh, v in pairs:
            if not isinstance(gh, GradHandle) or gh.var is not v:
                raise ValueError("apply_gradients takes the (gradient, variable) pairs made by compute_gradients")
        g = self.loss.graph
        g.optimizer = self
        train_op = O.group([self.loss], name=name or "train_op")
        train_op.is_train_op = True
        g.train_op = train_op
        return train_op

    def apply_flat(self, master, m, v, grad, out_compute, step, grad_scale=1.0):
        raise NotImplementedError


class SGDOptimizer(Optimizer):
    def __init__(self, lr: float = 0.01, momentum: float = 0.0, nesterov: bool = False, weight_decay: float = 0.0):
        super().__init__(lr)
        self.momentum, self.nesterov, self.weight_decay = momentum, nesterov, weight_decay

    def apply_flat(self, master, m, v, grad, out_compute, step, grad_scale=1.0):
        g = grad * grad_scale if grad_scale != 1.0 else grad
        if self.weight_decay:
            g = g + self.weight_decay * master
        if self.momentum > 0:
            m.mul_(self.momentum).add_(g)
            g = g + self.momentum * m if self.nesterov else m
        master.add_(g, alpha=-self.lr)
        out_compute.copy_(master)
        grad.zero_()


class AdamOptimizer(Optimizer):
    """Adam with bias correction and decoupled weight decay (0 by default); one fused kernel per flat shard
    that also emits the compute-dtype parameter copy and clears the gradient."""

    def __init__(self, lr: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8,
                 weight_decay: float = 0.0):
        super().__init__(lr)
        self.beta1, self.beta2, self.eps, self.weight_decay = beta1, beta2, eps, weight_decay

    def apply_flat(self, master, m, v, grad, out_compute, step, grad_scale=1.0):
        bc1 = 1.0 - self.beta1 ** step
        bc2 = 1.0 - self.beta2 ** step
        n = master.numel()
        if master.is_cuda and out_compute.dtype == torch.bfloat16:
            rc = _lib.lib().hsb_adam(master.data_ptr(), m.data_ptr(), v.data_ptr(), grad.data_ptr(),
                                     out_compute.data_ptr(), n, self.lr, self.beta1, self.beta2, self.eps,
                                     self.weight_decay, bc1, bc2, grad_scale, 1, _lib.stream_ptr())
            _lib.check(rc, "hsb_adam")
            _lib.count_launch()
            return
        g = grad * grad_scale if grad_scale != 1.0 else grad
        m.mul_(self.beta1).add_(g, alpha=1 - self.beta1)
        v.mul_(self.beta2).addcmul_(g, g, value=1 - self.beta2)
        upd = (m / bc1) / ((v / bc2).sqrt() + self.eps)
        if self.weight_decay:
            upd = upd + self.weight_decay * master
        master.add_(upd, alpha=-self.lr)
        out_compute.copy_(master)
        grad.zero_()


class SGD(SGDOptimizer):
    """The thin wrapper of the reference's Python optimizer package (python_refactor/hetu/optim/sgd.py): `params` given
    selects the define-by-run use (`zero_grad` / `step` on tensors that carry `.grad`), `params=None` the
    define-and-run use through `minimize`."""

    def __init__(self, params=None, lr: float = 0.1, momentum: float = 0.0, nesterov: bool = False):
        if lr < 0.0:
            raise ValueError(f"Invalid learning rate: {lr}")
        if momentum < 0.0 or momentum > 1:
            raise ValueError(f"Invalid momentum: {momentum}")
        if nesterov and momentum == 0:
            raise ValueError("Nesterov requires non-zero momentum")
        super().__init__(lr=lr, momentum=momentum, nesterov=nesterov)
        self.params = None if params is None else list(params)
        self.defaults = dict(lr=lr, momentum=momentum, nesterov=nesterov)
        if self.params is not None:
            if not self.params:
                raise ValueError("No variables are provided")
            for p in self.params:
                if not p.requires_grad:
                    raise ValueError(f"Parameter {p} is not requires_grad")

    def _need_params(self, fn):
        if self.params is None:
            raise ValueError(f"Function '{fn}' should only be used in define-by-run mode")

    def apply_dense(self, param, grad):
        return O.sgd_update(param, grad, self.defaults["lr"])

    def zero_grad(self):
        self._need_params("zero_grad")
        for p in self.params:
            p.grad = None

    def step(self):
        """Applies `param -= lr * param.grad` for every parameter whose `.grad` is set (a graph tensor or an array
        of the parameter's shape); returns the update ops."""
        self._need_params("step")
        ops = []
        for p in self.params:
            g = getattr(p, "grad", None)
            if g is None:
                continue
            if not hasattr(g, "graph"):
                g = p.graph.from_numpy(g, requires_grad=False) if hasattr(p.graph, "from_numpy") else g
            ops.append(self.apply_dense(p, g))
        return ops


def requires_grad_variables(loss) -> list:
    """Trainable parameters `loss` depends on (reference: hetu.requires_grad_variables of the legacy binding)."""
    seen, out, stack = set(), [], [loss]
    while stack:
        t = stack.pop()
        if t.id in seen:
            continue
        seen.add(t.id)
        if t.is_parameter:
            if t.requires_grad:
                out.append(t)
            continue
        if t.producer is not None:
            stack += list(t.producer.inputs)
    order = {p.id: i for i, p in enumerate(loss.graph.parameters)}
    return sorted(out, key=lambda p: order.get(p.id, 0))


def gradients(loss, var_list=None, grad_loss=None) -> list:
    """Fetchable gradient handles of `loss` with respect to `var_list` (default: every trainable parameter behind
    it), in order.  Fetch them together with a train op, or at run level "grad" with the loss."""
    if grad_loss is not None:
        raise NotImplementedError("a custom seed gradient is given through graph.run(grad_scale=...)")
    vars_ = list(var_list) if var_list is not None else requires_grad_variables(loss)
    return [GradHandle(v) for v in vars_]
