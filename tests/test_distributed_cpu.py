"""Parallel strategies and hot switching on CPU ranks (gloo): parity with a single-process PyTorch model."""
import json
import os
import socket
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _torchrun(script, world, args=(), marker=None, timeout=900):
    """Run tests/<script> on `world` gloo ranks.  The rendezvous port is picked by binding port 0 and releasing it, so
    another process can take it before torchrun binds: a failed launch is repeated once on a fresh port, and the
    output of both attempts is shown if the second one fails too."""
    env = dict(os.environ, OMP_NUM_THREADS="1", CUDA_VISIBLE_DEVICES="")
    outputs = []
    for _ in range(2):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HERE, script), *args]
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=timeout, env=env)
        if proc.returncode == 0 and (marker is None or marker in proc.stdout):
            return proc.stdout
        outputs.append(proc.stdout[-3000:])
    raise AssertionError("\n======== second attempt ========\n".join(outputs))


def run_workers(world, strategies, plan, extra=()):
    _torchrun("dist_worker.py", world, ["--strategies", json.dumps(strategies), "--plan", json.dumps(plan), *extra])


@pytest.mark.parametrize("world,strategy", [
    (2, [2, 1, 1, False]),
    (2, [2, 1, 1, True]),
    (2, [1, 2, 1, False]),
    (2, [1, 1, 2, False]),
    (4, [2, 2, 1, True]),
    (8, [2, 2, 2, True]),
])
def test_static_strategy_matches_single_process(world, strategy):
    run_workers(world, [strategy], [[0, "update", 128, 4]])


def test_hot_switch_three_strategies():
    # home = tp2/pp2 (long bucket), then dp4 (short), dp2/tp2 (medium); gradients accumulate across strategies
    strategies = [[1, 2, 2, False], [4, 1, 1, False], [2, 2, 1, True]]
    plan = [[0, "alloc", 256, 2], [1, "grad", 64, 8], [2, "grad", 128, 4], [0, "update", 256, 2]]
    run_workers(4, strategies, plan)


def test_activation_repartition_between_groups_with_different_layouts():
    _torchrun("repartition_worker.py", 4, timeout=600)


def test_heterogeneous_split_collectives():
    _torchrun("split_comm_worker.py", 4, marker="SPLIT_COMM_OK", timeout=600)


def test_communication_group_verbs():
    _torchrun("comm_group_worker.py", 4, marker="COMM_GROUP_OK", timeout=600)


def test_heterogeneous_strategy_mlp_with_gradient_handles():
    # replica A = ranks (0, 1) tensor parallel, replica B = rank 2; split all-reduce of the gradients across them
    _torchrun("hetero_worker.py", 3, marker="HETERO_OK", timeout=600)


@pytest.mark.parametrize("world", [3, 4])
def test_heterogeneous_strategy_tiny_llama(world):
    # 3 ranks: tp2 (+ sequence parallel) replica next to a single-device replica;
    # 4 ranks: a two-stage pipeline replica next to a tp2 replica
    _torchrun("hetero_llama_worker.py", world, marker="HETERO_LLAMA_OK", timeout=900)


def test_hot_switch_between_heterogeneous_home_and_homogeneous_strategy():
    # home = pipeline replica + tp2 replica; a second bucket runs under dp2 x tp2: parameters are copied out of the
    # union (any member may serve a slice), its gradients are added into one holder per cell and then synchronised
    _torchrun("hetero_llama_worker.py", 4, ["--switch"], marker="HETERO_LLAMA_OK", timeout=900)


def test_trainer_under_a_heterogeneous_strategy_matches_the_homogeneous_run():
    _torchrun("hetero_trainer_worker.py", 4, marker="HETERO_TRAINER_OK", timeout=900)
