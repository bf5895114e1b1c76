from .optimizer import AdamOptimizer, Optimizer, SGD, SGDOptimizer  # noqa: F401
