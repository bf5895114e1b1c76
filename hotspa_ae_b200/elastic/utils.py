"""Argument records of the elastic engine (reference: python_refactor/elastic/engine/utils.py and wrapper.py): what
the trainer is told about the cost model, the dataset position, the current strategy and the experiment switches,
and thin factories for model / optimizer / dataset classes.  Records validate their fields and print as
``Name(field = value, ...)``."""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Any


class Args:
    """Base of the argument records."""

    @staticmethod
    def print_args_list(args_list) -> None:
        for item in args_list:
            print(item)

    def _type_check(self, value, *types):
        if isinstance(value, types):
            return value
        raise TypeError(f"Value {value} must in types {types}.")

    def __str__(self) -> str:
        attrs = ", ".join(f"{k} = {v}" for k, v in vars(self).items())
        return f"{self.__class__.__name__}({attrs})"


@dataclass
class TrainerCtxs(Args):
    """Profiled constants of the cost and memory model the re-planner uses."""
    bf16: bool = True
    hetero_tp_alpha: list = field(default_factory=lambda: [1.0, 1.9, 3.5, 6.2])    # speed-up of tp 1, 2, 4, 8
    hetero_tp_weight: list = field(default_factory=lambda: [1.0, 1.0, 1.0, 1.0])
    normal_layers: int = 32
    normal_mbn: int = 8
    normal_compute_time: float = 1.0
    memory_k: list = field(default_factory=lambda: [1.0, 0.5, 0.25, 0.125])        # GB per layer at tp 1, 2, 4, 8
    memory_embedding: float = 1.0
    memory_extra: float = 4.0
    memory_bound: float = 170.0
    memory_safe_gap: float = 8.0
    straggler_threshold: float = 1.15
    straggler_safe_gap: float = 0.05
    top_k: int = 3

    def __post_init__(self):
        if self.straggler_threshold <= 1.0:
            raise ValueError("straggler_threshold must exceed 1")
        if self.memory_bound <= self.memory_safe_gap:
            raise ValueError("memory_bound must exceed memory_safe_gap")

    def tp_efficiency(self) -> dict:
        """{tp: efficiency} for `StrategyModel`: the measured speed-up over the ideal one."""
        return {t: a / t for t, a in zip((1, 2, 4, 8), self.hetero_tp_alpha)}

    def layer_memory_gb(self, layers: int, tp: int, boundary_stage: bool) -> float:
        k = self.memory_k[(1, 2, 4, 8).index(tp)]
        return layers * k + (self.memory_embedding if boundary_stage else 0.0) + self.memory_extra


@dataclass
class TrainerDatasetArgs(Args):
    dataset: Any = None
    consumed_samples: int = 0
    steps: int = 0
    epochs: int = 1
    step: int = 0
    epoch: int = 0


@dataclass
class TrainerStrategyArgs(Args):
    """One (possibly heterogeneous) strategy in the engine's terms: `hetero_layers[k]` lists the layer count of every
    stage of pipeline k, `hetero_stages[k]` its number of stages; ranks are laid out pipeline by pipeline, stage by
    stage, `tp` wide; `unused_rank_list` drops devices out of their tensor-parallel group."""
    dp: int = 1
    tp: int = 1
    pp: int = 1
    zero: bool = False
    rank_to_device_mapping: dict = field(default_factory=dict)
    suspended_rank_list: list = field(default_factory=list)
    unused_rank_list: list = field(default_factory=list)
    hetero_data: bool = False
    hetero_layers: list = field(default_factory=list)
    hetero_stages: list = field(default_factory=list)
    hetero_micro_batch_num_list: list = field(default_factory=list)

    def __post_init__(self):
        if self.hetero_layers:
            if len(self.hetero_layers) != self.dp:
                raise ValueError("hetero_layers needs one list per pipeline")
            stages = self.hetero_stages or [len(l) for l in self.hetero_layers]
            if [len(l) for l in self.hetero_layers] != list(stages):
                raise ValueError("hetero_stages must give the number of stages of every pipeline")
            self.hetero_stages = list(stages)

    def pipelines(self) -> list:
        """The strategy as the `pipelines` argument of `generate_llama_hetero_3d_config`."""
        layers = self.hetero_layers or [[None] * self.pp for _ in range(self.dp)]
        stages = self.hetero_stages or [self.pp] * self.dp
        mapping = self.rank_to_device_mapping
        out, base = [], 0
        for k in range(self.dp):
            pipe = []
            for s in range(stages[k]):
                ranks = [r for r in range(base, base + self.tp) if r not in self.unused_rank_list]
                pipe.append({"ranks": [mapping.get(r, r) for r in ranks], "layers": layers[k][s]})
                base += self.tp
            out.append(pipe)
        return out

    def to_config(self, num_layers: int) -> dict:
        from ..parallel.strategy_config import generate_llama_3d_config, generate_llama_hetero_3d_config
        pipes = self.pipelines()
        uniform = (not self.hetero_layers and not self.unused_rank_list and not self.rank_to_device_mapping)
        if uniform or self.dp == 1:
            return generate_llama_3d_config(num_layers, self.dp * self.tp * self.pp, self.dp, self.tp, self.pp, self.zero)
        for pipe in pipes:
            for st in pipe:
                if st["layers"] is None:
                    st["layers"] = num_layers // len(pipe)
        return generate_llama_hetero_3d_config(num_layers, pipes, zero=False)


@dataclass
class TrainerEnvs(Args):
    run_straggler_experiment: bool = False
    run_memory_experiment: bool = False
    straggler_file: str = ""
    memory_file: str = ""


class ModelWrapper(Args):
    def __init__(self, model_class, model_config):
        self.model_class, self.model_config = model_class, model_config

    def create_model(self, ds_parallel_configs):
        return self.model_class(self.model_config, ds_parallel_configs)


class OptimizerWrapper(Args):
    def __init__(self, optimizer_class):
        self.optimizer_class = optimizer_class

    def create_optimizer(self, **kwargs):
        return self.optimizer_class(**kwargs)


class DatasetWrapper(Args):
    def __init__(self, dataset_class):
        self.dataset_class = dataset_class

    def create_dataset(self, **kwargs):
        return self.dataset_class(**kwargs)


def record_fields(rec) -> list:
    return [f.name for f in fields(rec)]
