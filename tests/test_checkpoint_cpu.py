"""Checkpoint layout (file names, keys, qkv order) and cross-strategy reload on CPU ranks."""
import json
import os
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from launch import torchrun_cpu  # noqa: E402


@pytest.mark.parametrize("world,src,dst", [(1, [1, 1, 1, False], [1, 1, 1, False]),
                                           (4, [1, 2, 2, False], [2, 2, 1, True])])
def test_checkpoint_roundtrip_across_strategies(tmp_path, world, src, dst):
    torchrun_cpu("ckpt_worker.py", world, [json.dumps(src), json.dumps(dst), str(tmp_path / "ckpt")], timeout=600)
