"""Dynamic loss scaling for fp16 training (reference: hetu/graph/autocast/gradscaler.{h,cc}).

``scale(loss)`` multiplies the loss inside the graph; ``minimize(optimizer, loss)`` records the scaled train op;
``step_update(found_inf)`` grows the scale after ``growth_interval`` clean steps and backs off on overflow.
At run time the executor un-scales through ``grad_scale = 1 / scale`` and checks the gradient arena for
non-finite values before the optimizer step (bf16 training needs none of this).
"""
from __future__ import annotations

import torch


class GradScaler:
    def __init__(self, init_scale: float = 65536.0, growth_factor: float = 2.0, backoff_factor: float = 0.5,
                 growth_interval: int = 2000, enabled: bool = True):
        self.scale_value, self.growth_factor, self.backoff_factor = float(init_scale), growth_factor, backoff_factor
        self.growth_interval, self.enabled = growth_interval, enabled
        self._good_steps = 0
        self.found_inf = False

    def scale(self, loss):
        """Graph tensor `loss` times the current scale (a constant captured at definition time is avoided: the
        factor is applied through ``grad_scale`` at run time, so the graph stays valid when the scale changes)."""
        return loss

    def get_scale(self) -> float:
        return self.scale_value if self.enabled else 1.0

    def run_kwargs(self) -> dict:
        """Keyword arguments for ``graph.run``: seeds the backward pass with the scale."""
        return {"grad_scale": self.get_scale()}

    def minimize(self, optimizer, loss, var_list=None, name=None):
        optimizer.grad_scaler = self
        return optimizer.minimize(loss, var_list, name)

    def check_finite(self, grad_arena: torch.Tensor) -> bool:
        self.found_inf = not bool(torch.isfinite(grad_arena).all())
        return not self.found_inf

    def unscale_factor(self) -> float:
        return 1.0 / self.get_scale()

    def step_update(self, found_inf: bool | None = None) -> float:
        found = self.found_inf if found_inf is None else found_inf
        if not self.enabled:
            return 1.0
        if found:
            self.scale_value *= self.backoff_factor
            self._good_steps = 0
        else:
            self._good_steps += 1
            if self._good_steps >= self.growth_interval:
                self.scale_value *= self.growth_factor
                self._good_steps = 0
        self.found_inf = False
        return self.scale_value

    update = step_update
