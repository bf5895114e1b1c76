from .optimizer import AdamOptimizer, Optimizer, SGDOptimizer  # noqa: F401
