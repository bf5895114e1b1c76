"""Strategy description files: one JSON per (gpus, dp, tp, pp) with the distributed-states recipe of every
placeholder and parameter of the Llama/GPT model.

Schema (interchange-compatible with the reference's hotspa/ds_parallel_config/generate_llama_3d_config.py):
top keys ``zero, devices, input, llama{wte, wpe, blocks{blocks<a>-<b>{range, layernorm1, attn{qkv, dense},
layernorm2, mlp{dense_h_to_4h, dense_4h_to_h}}}, layernorm_final}, lm_head, label``; every leaf is
``{split: {dim: [n]}, dup: [n], device_group_union: [[ranks]], type: variable|placeholder[, zero]}`` with one
list entry per member of a heterogeneous union.  Pipeline stage s owns ranks [s*N/pp, (s+1)*N/pp).
"""
from __future__ import annotations

import json
import os


def _leaf(split: dict, dup: int, ranks: list, kind: str) -> dict:
    return {"split": {str(k): [v] for k, v in split.items()}, "dup": [dup], "device_group_union": [list(ranks)],
            "type": kind}


def generate_llama_3d_config(num_layers: int = 32, num_gpus: int = 8, dp: int = 2, tp: int = 2, pp: int = 2,
                             zero: bool = True, device_offset: int = 0, layers_per_stage: list | None = None,
                             rank_order: list | None = None) -> dict:
    """`layers_per_stage` gives an uneven split of the layers over the pipeline stages (slow stages get fewer
    layers); `rank_order` permutes which physical ranks fill the dp x tp x pp grid (e.g. to group slow devices)."""
    if dp * tp * pp != num_gpus:
        raise ValueError(f"dp*tp*pp = {dp * tp * pp} != num_gpus = {num_gpus}")
    if layers_per_stage is None:
        if num_layers % pp:
            raise ValueError("num_layers must be divisible by pp")
        layers_per_stage = [num_layers // pp] * pp
    if len(layers_per_stage) != pp or sum(layers_per_stage) != num_layers or min(layers_per_stage) < 1:
        raise ValueError(f"layers_per_stage {layers_per_stage} does not split {num_layers} layers over {pp} stages")
    zero = bool(zero) and dp > 1
    width = num_gpus // pp
    order = list(rank_order) if rank_order is not None else [device_offset + i for i in range(num_gpus)]
    if sorted(order) != sorted(device_offset + i for i in range(num_gpus)):
        raise ValueError("rank_order must be a permutation of the ranks")
    stage_ranks = [[order[s * width + i] for i in range(width)] for s in range(pp)]
    first, last = stage_ranks[0], stage_ranks[-1]
    var, ph = "variable", "placeholder"
    cfg = {
        "zero": zero,
        "devices": [device_offset + i for i in range(num_gpus)],
        "input": _leaf({0: dp}, tp, first, ph),
        "llama": {
            "wte": _leaf({0: tp}, dp, first, var),
            "wpe": _leaf({}, dp * tp, first, var),
            "blocks": {},
            "layernorm_final": _leaf({}, dp * tp, last, var),
        },
        "lm_head": _leaf({1: tp}, dp, last, var),
        "label": _leaf({0: dp}, tp, last, ph),
    }
    first_layer = 0
    for s, ranks in enumerate(stage_ranks):
        a, b = first_layer, first_layer + layers_per_stage[s] - 1
        first_layer = b + 1
        cfg["llama"]["blocks"][f"blocks{a}-{b}"] = {
            "range": [a, b],
            "layernorm1": _leaf({}, dp * tp, ranks, var),
            "attn": {"qkv": _leaf({1: tp}, dp, ranks, var), "dense": _leaf({0: tp}, dp, ranks, var)},
            "layernorm2": _leaf({}, dp * tp, ranks, var),
            "mlp": {"dense_h_to_4h": _leaf({1: tp}, dp, ranks, var), "dense_4h_to_h": _leaf({0: tp}, dp, ranks, var)},
        }
    return cfg


generate_gpt_3d_config = generate_llama_3d_config


def generate_llama_hetero_3d_config(num_layers: int, pipelines: list, zero: bool = False) -> dict:
    """Heterogeneous strategy: the data-parallel replicas are pipelines of different shape.

    ``pipelines`` has one entry per replica; an entry lists the replica's stages in order, each stage a dict
    ``{"ranks": [...], "layers": n}``: the ranks are the stage's tensor-parallel group (the degree may differ between
    stages and between replicas), ``layers`` sums to ``num_layers`` inside every replica.  The result uses the
    reference's union form (hotspa/ds_parallel_config/generate_gpt_hetero_3d_config.py:6-112): every list-valued field
    has one element per replica, and blocks are listed one by one because their device groups differ per layer."""
    dp = len(pipelines)
    if dp < 2:
        raise ValueError("a heterogeneous strategy needs at least two pipelines")
    seen: set = set()
    per_layer = []                                  # per pipeline: the tp group of every layer
    for stages in pipelines:
        if sum(int(st["layers"]) for st in stages) != num_layers or any(int(st["layers"]) < 1 for st in stages):
            raise ValueError(f"the stages of every pipeline must split the {num_layers} layers")
        groups = []
        for st in stages:
            ranks = [int(r) for r in st["ranks"]]
            if not ranks or seen & set(ranks):
                raise ValueError("every rank belongs to exactly one stage of one pipeline")
            seen |= set(ranks)
            groups += [ranks] * int(st["layers"])
        per_layer.append(groups)
    var, ph = "variable", "placeholder"
    dp_union = [dp] * dp

    def leaf(split_dim, layer, kind):
        union = [per_layer[k][layer] for k in range(dp)]
        tps = [len(g) for g in union]
        if kind == ph:
            return {"split": {"0": dp_union}, "dup": tps, "device_group_union": union, "type": ph}
        if split_dim is None:
            return {"split": {}, "dup": [t * dp for t in tps], "device_group_union": union, "type": var}
        return {"split": {str(split_dim): tps}, "dup": dp_union, "device_group_union": union, "type": var}

    last = num_layers - 1
    cfg = {
        "zero": bool(zero),
        "devices": sorted(seen),
        "input": leaf(None, 0, ph),
        "llama": {
            "wte": leaf(0, 0, var),
            "wpe": leaf(None, 0, var),
            "blocks": {},
            "layernorm_final": leaf(None, last, var),
        },
        "lm_head": leaf(1, last, var),
        "label": leaf(None, last, ph),
    }
    for i in range(num_layers):
        cfg["llama"]["blocks"][f"blocks{i}"] = {
            "range": [i, i],
            "layernorm1": leaf(None, i, var),
            "attn": {"qkv": leaf(1, i, var), "dense": leaf(0, i, var)},
            "layernorm2": leaf(None, i, var),
            "mlp": {"dense_h_to_4h": leaf(1, i, var), "dense_4h_to_h": leaf(0, i, var)},
        }
    return cfg


generate_gpt_hetero_3d_config = generate_llama_hetero_3d_config


def propagate_zero(cfg: dict) -> dict:
    """Copy the top-level ``zero`` flag onto every variable leaf that does not set its own."""
    zero = cfg.get("zero", False)
    stack = [cfg]
    while stack:
        node = stack.pop()
        for v in node.values():
            if isinstance(v, dict):
                if "type" in v:
                    if v["type"] == "variable" and "zero" not in v:
                        v["zero"] = zero
                else:
                    stack.append(v)
    return cfg


def read_ds_parallel_config(paths) -> list[dict]:
    if isinstance(paths, str):
        paths = paths.split(",") if "," in paths else paths.split()
    return [propagate_zero(json.load(open(p))) for p in paths]


def find_config(cfg: dict, module_name: str, layer_idx: int = -1):
    """The leaf (or sub-dict) called `module_name`, searching nested dicts; a dict with a ``range`` is only
    entered when it contains `layer_idx`."""
    stack = [cfg]
    while stack:
        node = stack.pop(0)
        if module_name in node:
            return node[module_name]
        for v in node.values():
            if isinstance(v, dict):
                if "range" in v and not (v["range"][0] <= layer_idx <= v["range"][-1]):
                    continue
                stack.append(v)
    raise KeyError(f"{module_name} (layer {layer_idx}) not found in the strategy config")


def get_multi_ds_parallel_config(ds_parallel_configs: list[dict], module_name: str, layer_idx: int = -1) -> list:
    return [find_config(c, module_name, layer_idx) for c in ds_parallel_configs]


def write_config(cfg: dict, directory: str, dp: int, tp: int, pp: int) -> str:
    os.makedirs(directory, exist_ok=True)
    path = os.path.join(directory, f"dp{dp}_tp{tp}_pp{pp}.json")
    with open(path, "w") as f:
        json.dump(cfg, f, indent=4)
    return path


def strategy_name(cfg: dict) -> str:
    inp = cfg["input"]
    dp = inp["split"].get("0", [1])[0]
    tp = inp["dup"][0]
    pp = len(cfg["llama"]["blocks"])
    return f"dp{dp}tp{tp}pp{pp}"


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--num_layers", type=int, default=32)
    ap.add_argument("--num_gpus", type=int, default=8)
    ap.add_argument("--dp", type=int, default=2)
    ap.add_argument("--tp", type=int, default=2)
    ap.add_argument("--pp", type=int, default=2)
    ap.add_argument("--zero", action="store_true")
    ap.add_argument("--out_dir", type=str, default="ds_parallel_config")
    a = ap.parse_args()
    print(write_config(generate_llama_3d_config(a.num_layers, a.num_gpus, a.dp, a.tp, a.pp, a.zero), a.out_dir,
                       a.dp, a.tp, a.pp))
