"""hotspa_ae_b200: a Blackwell-native (sm_100a) LLM training framework with parallelism hot switching.

Layers: ``csrc`` (CUDA kernels + C++ core) -> ``ops`` -> ``graph``/``parallel`` -> ``nn``/``models`` -> ``train``.
The user-facing Hetu-style API is the top-level ``hetu`` package (``import hetu as ht``).
"""
__version__ = "0.1.0"
