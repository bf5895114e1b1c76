from .module import Dropout, Identity, Module, ModuleList, Sequential  # noqa: F401
from .parallel_layers import (HtMultiColumnParallelLinear, HtMultiParallelEmbedding,  # noqa: F401
                              HtMultiParallelLayerNorm, HtMultiParallelRMSNorm, HtMultiRowParallelLinear,
                              HtMultiVocabParallelEmbedding, config2ds, get_local_index, parallel_data_provider,
                              parallel_multi_data_provider)
from .layers import (CrossEntropyLoss, Embedding, GELU, HtColumnParallelLinear, HtParallelEmbedding,  # noqa: F401
                     HtParallelLayerNorm, HtParallelRMSNorm, HtRowParallelLinear, HtVocabParallelEmbedding, LayerNorm,
                     Linear, MSELoss, ReLU, RMSNorm, SiLU, Sigmoid, Tanh)
