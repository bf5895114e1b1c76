from .optimizer import (AdamOptimizer, GradHandle, Optimizer, SGD, SGDOptimizer, gradients,  # noqa: F401
                        requires_grad_variables)
