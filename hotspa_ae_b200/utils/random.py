"""Global random state (reference: hetu/impl/random/*: one seed plus a philox offset counter).

The seed fixes parameter initialisation (``ParamStore.seed`` = seed, every parameter derives its own generator
from it) and dropout; ``step`` counts the random draws that have been handed out, so a resumed run can continue
the sequence instead of repeating it.
"""
from __future__ import annotations

import torch

_state = {"seed": 2023, "step": 0}


def set_random_seed(seed: int) -> None:
    _state["seed"], _state["step"] = int(seed), 0
    torch.manual_seed(int(seed))
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(int(seed))


def get_seed() -> int:
    return _state["seed"]


def get_seed_step() -> int:
    return _state["step"]


def step_seed(n: int = 1) -> int:
    """Reserve `n` draws and return the offset of the first one."""
    s = _state["step"]
    _state["step"] += int(n)
    return s


def get_seed_status() -> tuple:
    return _state["seed"], _state["step"]


def set_seed_status(seed: int, step: int) -> None:
    _state["seed"], _state["step"] = int(seed), int(step)
