"""``import hetu as ht`` - the Hetu-style Python API of hotspa_ae_b200.

Graph/context managers, distributed states, parallel placeholders/parameters, the op front-ends,
``ht.nn`` layers and the optimizers, with the names and call signatures of the reference's Python
package (python_refactor/hetu/__init__.py and its bound ops, codegen/ops.yml).
"""
from hotspa_ae_b200.core import (DistributedStates, DistributedStatesUnion, IntSymbol, NULL_HETERO_DIM,  # noqa: F401
                                 map_to_local_data)
from hotspa_ae_b200.graph.graph import (Graph, autocast, from_numpy, from_numpy_parallel, graph,  # noqa: F401
                                        merge_strategy, parallel_parameter, parallel_placeholder, placeholder,
                                        recompute, run_level)
from hotspa_ae_b200.graph.graph import get_autocast, get_default_autocast  # noqa: F401
from hotspa_ae_b200.graph.graph import (delete_graph, get_default_define_and_run_graph,  # noqa: F401
                                        get_default_define_by_run_graph, get_default_eager_graph, get_graph,
                                        make_new_define_and_run_graph, make_new_eager_graph)
from hotspa_ae_b200.graph.gradscaler import GradScaler  # noqa: F401
from hotspa_ae_b200.graph.ctors import (empty, empty_like, full, full_like, ones, rand, rand_like, randn,  # noqa: F401
                                        randn_like, trunc_randn, trunc_randn_like, zeros)
from hotspa_ae_b200.utils.dataset import Dataloader  # noqa: F401
from hotspa_ae_b200.core.stream import Event, Stream, get_stream  # noqa: F401
from hotspa_ae_b200.core.ndarray import NDArray, numpy_to_NDArray  # noqa: F401
from hotspa_ae_b200.utils.random import get_seed_status, set_random_seed, set_seed_status  # noqa: F401
from hotspa_ae_b200.graph.init import *  # noqa: F401,F403
from hotspa_ae_b200.graph.ops import *  # noqa: F401,F403
from hotspa_ae_b200.graph.ops import (abs, bool, pow, reduce, round, slice)  # noqa: F401,A004
from hotspa_ae_b200.graph.ops_extra import *  # noqa: F401,F403
from hotspa_ae_b200.graph.ops_extra import sum  # noqa: F401,A004
from hotspa_ae_b200.graph.tensor import Tensor, bfloat16, bool_, float16, float32, int32, int64  # noqa: F401
from hotspa_ae_b200.optim import AdamOptimizer, Optimizer, SGDOptimizer  # noqa: F401
from hotspa_ae_b200.optim import gradients, requires_grad_variables  # noqa: F401
from hotspa_ae_b200.parallel.mesh import get_local_hostname  # noqa: F401
from hotspa_ae_b200.parallel.mesh import (Device, DeviceGroup, global_comm_barrier, global_device_group,  # noqa: F401
                                          init_comm_group, local_device)
from hotspa_ae_b200 import nn  # noqa: F401
from hotspa_ae_b200 import optim  # noqa: F401
from hotspa_ae_b200 import utils  # noqa: F401

import contextlib as _contextlib


@_contextlib.contextmanager
def context(device_group=None, eager_device=None):
    """Accepted for source compatibility; placement comes from the device-group hierarchies."""
    yield


@_contextlib.contextmanager
def control_dependencies(tensors):
    """Ops run in definition order on one stream, so explicit control edges are a no-op."""
    yield
