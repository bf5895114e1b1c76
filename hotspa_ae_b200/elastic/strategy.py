"""Re-planning under stragglers: choose (dp, tp, pp), the placement of slow devices, an uneven layer split over
pipeline stages and the share of the batch every data-parallel replica gets, so that the estimated step time
under the measured per-device slow-down ratios is minimal and every device stays under the memory bound.

Cost model (per optimizer step, arbitrary time unit = one layer on one healthy device for one unit of work):
  * a tensor-parallel group runs at the speed of its slowest member; splitting over t devices divides the layer
    time by ``t * tp_efficiency[t]``;
  * a pipeline of s stages with layer counts L_k and group slow-downs r_k processes m micro-batches in
    ``(m + s - 1) * max_k(L_k * r_k)`` (1F1B / GPipe makespan with the slowest stage as the bottleneck);
  * data-parallel replicas run concurrently; the step takes as long as the slowest replica.
The reference solves this with an ILP plus a DFS over heterogeneous stage patterns
(python_refactor/elastic/engine/strategy.py:195-977); here the search is exhaustive over the small (dp, tp, pp)
space of one node with exact dynamic programming for the layer split and proportional work assignment.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

DEFAULT_TP_EFFICIENCY = {1: 1.0, 2: 0.95, 4: 0.88, 8: 0.78}


@dataclass
class Plan:
    dp: int
    tp: int
    pp: int
    rank_order: list                     # physical ranks in dp-major, then stage, then tp order (see to_config_args)
    layers_per_stage: list               # per replica: list of per-stage layer counts
    work_share: list                     # per replica: fraction of the batch
    est_time: float
    unused: list = field(default_factory=list)

    def key(self):
        return (self.dp, self.tp, self.pp, tuple(self.rank_order), tuple(map(tuple, self.layers_per_stage)),
                tuple(round(w, 3) for w in self.work_share))

    def __eq__(self, other):
        return isinstance(other, Plan) and self.key() == other.key()

    def __hash__(self):
        return hash(self.key())


def split_layers(num_layers: int, slow: list) -> tuple:
    """Layer counts per stage minimising max_k(L_k * slow_k), every stage gets at least one layer.
    Returns (counts, bottleneck)."""
    s = len(slow)
    if s > num_layers:
        raise ValueError("more stages than layers")
    # binary search on the bottleneck T: stage k can take floor(T / slow_k) layers
    cands = sorted({l * r for r in slow for l in range(1, num_layers + 1)})
    lo, hi = 0, len(cands) - 1
    while lo < hi:
        mid = (lo + hi) // 2
        cap = sum(min(num_layers, int(cands[mid] / r + 1e-9)) for r in slow)
        ok = cap >= num_layers and all(int(cands[mid] / r + 1e-9) >= 1 for r in slow)
        if ok:
            hi = mid
        else:
            lo = mid + 1
    T = cands[lo]
    caps = [int(T / r + 1e-9) for r in slow]
    counts = [1] * s
    left = num_layers - s
    # hand the remaining layers to the stages with the most head-room first
    while left > 0:
        k = max(range(s), key=lambda i: (caps[i] - counts[i], -slow[i]))
        if caps[k] - counts[k] <= 0:
            k = min(range(s), key=lambda i: (counts[i] + 1) * slow[i])
        counts[k] += 1
        left -= 1
    return counts, max(c * r for c, r in zip(counts, slow))


class StrategyModel:
    def __init__(self, num_layers: int, ranks: list, slowdown: dict | None = None, unused: list | None = None,
                 micro_batches: int = 8, memory_per_layer_gb: float = 0.0, memory_bound_gb: float = 1e9,
                 tp_efficiency: dict | None = None, allowed: list | None = None):
        self.num_layers = num_layers
        self.unused = sorted(set(unused or []))
        self.ranks = [r for r in ranks if r not in self.unused]
        self.slow = {r: float((slowdown or {}).get(r, 1.0)) for r in self.ranks}
        self.micro_batches = micro_batches
        self.mem_layer, self.mem_bound = memory_per_layer_gb, memory_bound_gb
        self.tp_eff = dict(DEFAULT_TP_EFFICIENCY if tp_efficiency is None else tp_efficiency)
        self.allowed = allowed

    def _candidates(self):
        n = len(self.ranks)
        for tp in (1, 2, 4, 8):
            for pp in (1, 2, 4, 8):
                if tp * pp > n or pp > self.num_layers:
                    continue
                dp = n // (tp * pp)
                if dp < 1:
                    continue
                if self.allowed is not None and (dp, tp, pp) not in self.allowed:
                    continue
                yield dp, tp, pp

    def evaluate(self, dp: int, tp: int, pp: int) -> Plan | None:
        used_n = dp * tp * pp
        # slow devices together: sort by slow-down so that a tensor-parallel group (bound by its slowest member)
        # wastes as little healthy capacity as possible; the slowest devices beyond used_n are left out
        order = sorted(self.ranks, key=lambda r: (self.slow[r], r))
        used, spare = order[:used_n], order[used_n:]
        groups = [used[i * tp:(i + 1) * tp] for i in range(dp * pp)]          # fastest groups first
        g_slow = [max(self.slow[r] for r in g) / (tp * self.tp_eff.get(tp, 0.7)) for g in groups]
        # replicas take groups round-robin so that each pipeline mixes fast and slow stages evenly
        replicas = [[] for _ in range(dp)]
        for i, gi in enumerate(sorted(range(len(groups)), key=lambda k: g_slow[k])):
            replicas[i % dp].append(gi)
        layers, bott = [], []
        for rep in replicas:
            counts, b = split_layers(self.num_layers, [g_slow[g] for g in rep])
            if self.mem_layer * max(counts) / tp > self.mem_bound:
                return None
            layers.append(counts)
            bott.append(b)
        inv = np.array([1.0 / b for b in bott])
        share = (inv / inv.sum()).tolist()
        m = max(1, self.micro_batches)
        est = max(sh * dp * (m + pp - 1) / m * b for sh, b in zip(share, bott))
        rank_order = [r for rep in replicas for g in rep for r in groups[g]]
        return Plan(dp, tp, pp, rank_order, layers, share, float(est), unused=sorted(spare + self.unused))

    def make_plans(self, top: int = 1) -> list:
        plans = [p for p in (self.evaluate(*c) for c in self._candidates()) if p is not None]
        if not plans:
            raise RuntimeError("no feasible strategy under the memory bound")
        plans.sort(key=lambda p: (p.est_time, -p.dp))
        return plans[:top]

    def best(self) -> Plan:
        return self.make_plans(1)[0]


def to_config_args(plan: Plan) -> dict:
    """Arguments for ``generate_llama_3d_config`` when the plan is homogeneous across replicas; replicas with
    different layer splits need one config per replica (heterogeneous unions), reported through ``hetero``."""
    same = all(l == plan.layers_per_stage[0] for l in plan.layers_per_stage)
    # generate_llama_3d_config lays ranks out stage-major: stage s owns order[s*width:(s+1)*width] with the
    # tensor-parallel index fastest and the replica index slowest inside a stage
    width = plan.dp * plan.tp
    order = [None] * (plan.pp * width)
    it = iter(plan.rank_order)
    for rep in range(plan.dp):
        for s in range(plan.pp):
            for t in range(plan.tp):
                order[s * width + rep * plan.tp + t] = next(it)
    return {"dp": plan.dp, "tp": plan.tp, "pp": plan.pp, "layers_per_stage": plan.layers_per_stage[0],
            "rank_order": order, "hetero": not same}


def to_hetero_pipelines(plan: Plan) -> list:
    """The plan as the pipelines argument of ``generate_llama_hetero_3d_config``: one pipeline per replica, each a
    list of stages ``{"ranks": tensor-parallel group, "layers": count}`` (replicas may split the layers
    differently, which the homogeneous config form cannot express)."""
    it = iter(plan.rank_order)
    pipes = []
    for rep in range(plan.dp):
        stages = []
        for s in range(plan.pp):
            stages.append({"ranks": [next(it) for _ in range(plan.tp)], "layers": int(plan.layers_per_stage[rep][s])})
        pipes.append(stages)
    return pipes
