"""bench.py's tables and the parts of its contract that need no GPU."""
import json
import os
import subprocess
import sys


ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402

from hotspa_ae_b200.models.llama import llama_config  # noqa: E402
from hotspa_ae_b200.parallel.strategy_config import generate_llama_3d_config  # noqa: E402


def test_plans_are_consistent():
    for model, by_world in bench.PLANS.items():
        layers = llama_config(model).num_layers
        for world, (bounds, strategies, recompute, mb_tokens) in by_world.items():
            assert list(bounds) == sorted(bounds, reverse=True) and bounds[-1] == 0
            assert len(strategies) == len(bounds) - 1 == len(mb_tokens), (model, world)
            assert all(0 <= r < len(strategies) for r in recompute)
            for dp, tp, pp, zero in strategies:
                assert dp * tp * pp == world, (model, world, (dp, tp, pp))
                assert layers % pp == 0
                generate_llama_3d_config(layers, world, dp, tp, pp, zero)        # the layout exists
            # the longest bucket must fit one micro-batch of the strategy that runs it
            assert mb_tokens[0] * strategies[0][1] >= 0
            keep = bench.KEEP_ACTIVATIONS.get(model, {}).get(world, 0)
            if isinstance(keep, list):
                assert len(keep) == len(strategies)
                for k, (dp, tp, pp, _) in zip(keep, strategies):
                    assert 0 <= k <= layers // pp, (model, world, keep)
            else:
                assert 0 <= keep <= layers
    assert set(bench.PLANS["7b"]) == {1, 2, 4, 8}                 # the scaling run needs every one of them


def test_reference_arm_reports_why_it_is_unavailable():
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1",
                           "--steps", "2", "--warmup", "3"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                          text=True, timeout=300, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert proc.returncode == 0, proc.stdout[-2000:]
    line = [l for l in proc.stdout.splitlines() if l.startswith("{")][-1]
    out = json.loads(line)
    assert out["impl"] == "reference" and isinstance(out["unavailable"], str) and out["unavailable"]


def test_without_a_gpu_the_benchmark_refuses_instead_of_falling_back():
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "1", "--warmup", "3"],
                          stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300,
                          env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert proc.returncode != 0 and "needs a GPU" in proc.stdout


def test_run_script_strategy_tables():
    import re
    script = os.path.join(ROOT, "hotspa_ae_b200", "train", "scripts", "llama_hot_switch.sh")
    for model, seq, gpus, data in [("7b", 32768, 8, "synthetic"), ("7b", 16384, 8, "synthetic"), ("7b", 4096, 8, "x"),
                                   ("13b", 32768, 8, "commoncrawl"), ("7b", 32768, 8, "github"), ("3b", 8192, 8, "x"),
                                   ("7b", 32768, 4, "x"), ("7b", 32768, 2, "x"), ("7b", 32768, 1, "x")]:
        proc = subprocess.run(["bash", script, model, str(seq), str(gpus), "3", data], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True, timeout=60, env=dict(os.environ, DRY_RUN="1"))
        assert proc.returncode == 0, proc.stdout
        m = re.search(r"buckets \(([^)]*)\), strategies \(([^)]*)\)", proc.stdout)
        buckets = [int(b) for b in m.group(1).split()]
        strategies = [tuple(int(v) for v in s.split(",")) for s in m.group(2).split()]
        assert buckets[0] == seq and buckets[-1] == 0 and buckets == sorted(buckets, reverse=True)
        assert len(strategies) == len(buckets) - 1, proc.stdout
        assert all(dp * tp * pp == gpus for dp, tp, pp in strategies), proc.stdout
