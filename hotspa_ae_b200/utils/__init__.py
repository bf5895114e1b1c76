"""Utilities: checkpoints, data (datasets, loaders, bucketing and packing), logging, profiling, random state,
roofline arithmetic, tokenizer.  `hetu.utils.checkpoint` and `hetu.utils.data` carry the reference's names."""
from . import checkpoint, data, dataset, logging, profiler, random, roofline  # noqa: F401
from .checkpoint import load_checkpoint, save_checkpoint  # noqa: F401
