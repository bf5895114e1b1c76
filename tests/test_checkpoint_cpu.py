"""Checkpoint layout (file names, keys, qkv order) and cross-strategy reload on CPU ranks."""
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


@pytest.mark.parametrize("world,src,dst", [(1, [1, 1, 1, False], [1, 1, 1, False]),
                                           (4, [1, 2, 2, False], [2, 2, 1, True])])
def test_checkpoint_roundtrip_across_strategies(tmp_path, world, src, dst):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HERE, "ckpt_worker.py"),
           json.dumps(src), json.dumps(dst), str(tmp_path / "ckpt")]
    env = dict(os.environ, OMP_NUM_THREADS="1", CUDA_VISIBLE_DEVICES="")
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600, env=env)
    assert proc.returncode == 0, proc.stdout[-3000:]
