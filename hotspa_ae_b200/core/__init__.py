"""Python handle on the C++ host core (``_hsb_core``): distributed states, planners, symbols.

The extension is built in-tree on first import when it is missing (g++ only, ~20 s).
"""
from __future__ import annotations

import importlib
import os
import sys

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load():
    if _PKG not in sys.path:
        sys.path.insert(0, _PKG)
    try:
        return importlib.import_module("_hsb_core")
    except ImportError:
        from .. import build
        build.build_core()
        importlib.invalidate_caches()
        return importlib.import_module("_hsb_core")


_C = _load()

DistributedStates = _C.DistributedStates
DistributedStatesUnion = _C.DistributedStatesUnion
IntSymbol = _C.IntSymbol
ReshardPlanner = _C.ReshardPlanner
NvmlProfiler = _C.NvmlProfiler
classify_comm = _C.classify_comm
comm_type_name = _C.comm_type_name
split_comm_groups = _C.split_comm_groups
run_barrier_model = _C.run_barrier_model
run_reduce_scatter_model = _C.run_reduce_scatter_model
run_all_gather_model = _C.run_all_gather_model
deduce_linear = _C.deduce_linear
regions_of = _C.regions_of
schedule_1f1b = _C.schedule_1f1b
schedule_gpipe = _C.schedule_gpipe
bucket_and_pack = _C.bucket_and_pack
balance_rows = _C.balance_rows
plan_arena = _C.plan_arena
build_reshard_descriptors = _C.build_reshard_descriptors

NULL_HETERO_DIM = -3


def map_to_local_data(ds, device_index: int) -> dict:
    """{dim: shard index} of device `device_index` under `ds` (reference: hetu.map_to_local_data)."""
    return dict(ds.map_device_to_state_index(device_index))


def sym_value(x) -> int:
    """Concrete value of an int or IntSymbol."""
    return int(x.data) if isinstance(x, IntSymbol) else int(x)
