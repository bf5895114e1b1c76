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


def run_workers(world, strategies, plan, extra=()):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HERE, "dist_worker.py"),
           "--strategies", json.dumps(strategies), "--plan", json.dumps(plan), *extra]
    env = dict(os.environ, OMP_NUM_THREADS="1", CUDA_VISIBLE_DEVICES="")
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=900, env=env)
    assert proc.returncode == 0, proc.stdout[-4000:]


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
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HERE, "repartition_worker.py")]
    env = dict(os.environ, OMP_NUM_THREADS="1", CUDA_VISIBLE_DEVICES="")
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600, env=env)
    assert proc.returncode == 0, proc.stdout[-3000:]


def test_heterogeneous_split_collectives():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HERE, "split_comm_worker.py")]
    env = dict(os.environ, OMP_NUM_THREADS="1", CUDA_VISIBLE_DEVICES="")
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600, env=env)
    assert proc.returncode == 0 and "SPLIT_COMM_OK" in proc.stdout, proc.stdout[-4000:]


def test_communication_group_verbs():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HERE, "comm_group_worker.py")]
    env = dict(os.environ, OMP_NUM_THREADS="1", CUDA_VISIBLE_DEVICES="")
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600, env=env)
    assert proc.returncode == 0 and "COMM_GROUP_OK" in proc.stdout, proc.stdout[-4000:]
