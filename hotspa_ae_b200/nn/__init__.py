from .module import Dropout, Identity, Module, ModuleList, Sequential  # noqa: F401
from .parallel_layers import (HtMultiColumnParallelLinear, HtMultiParallelEmbedding,  # noqa: F401
                              HtMultiParallelLayerNorm, HtMultiParallelRMSNorm, HtMultiRowParallelLinear,
                              HtMultiVocabParallelEmbedding, config2ds, get_local_index, parallel_data_provider,
                              parallel_multi_data_provider)
from .layers import (CrossEntropyLoss, Embedding, GELU, HtColumnParallelLinear, HtParallelEmbedding,  # noqa: F401
                     HtParallelLayerNorm, HtParallelRMSNorm, HtRowParallelLinear, HtVocabParallelEmbedding, LayerNorm,
                     Linear, MSELoss, ReLU, RMSNorm, SiLU, Sigmoid, Tanh)
from .layers_extra import (AvgPool2d, BatchNorm, BCELoss, ColumnParallelLinear, ConstantPad2d, Conv2d,  # noqa: F401
                           Dropout2d, InstanceNorm, KLDivLoss, LeakyReLU, MaxPool2d, ModuleDict, NewGeLU, NLLLoss,
                           ParallelEmbedding, ParallelLayerNorm, RowParallelLinear, VocabParallelEmbedding, ZeroPad2d,
                           get_device_index)
from . import functional  # noqa: F401
from . import functional as init  # noqa: F401


def Parameter(data, requires_grad: bool = True, name=None):
    """A trainable graph tensor from a tensor that already is a variable, or from array data (reference:
    python_refactor/hetu/nn/parameter.py; there a Tensor subclass, here the parameter tensor itself)."""
    import numpy as np
    from ..graph import graph as G
    from ..graph.tensor import Tensor
    if isinstance(data, Tensor):
        if not data.is_parameter:
            raise TypeError("Parameter(tensor): the tensor must be a variable (made by an initializer or from_numpy)")
        data.requires_grad = bool(requires_grad)
        return data
    if data is None:
        raise TypeError("cannot create a Parameter from None")
    return G.from_numpy(np.asarray(data), requires_grad=requires_grad, name=name)
