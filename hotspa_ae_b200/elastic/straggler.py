"""Straggler and failure detection on the host.

* :class:`Straggler` times a fixed matmul workload on this rank's device (the reference's per-device
  micro-benchmark, python_refactor/elastic/engine/straggler.py:66-93) and exchanges profiles either through
  files terminated by an ``EOF`` line (the reference's protocol) or through ``torch.distributed``.
* :class:`StepTimeWindow` keeps a sliding window of per-rank compute times and turns them into slow-down ratios
  against a baseline.
* :class:`Heartbeat` is a host-side liveness protocol over a shared directory or a ``torch.distributed`` store:
  every rank stamps a counter between steps; a rank whose stamp is older than the limit is reported dead, so the
  survivors learn of a failure before their next launch instead of inside a collective.
Nothing here touches a GPU except the benchmark matmul itself.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist

WORKLOAD_ITERS = 10
SLIDING_WINDOW = 5


@dataclass
class WorkloadInfo:
    mbs: int = 1
    seq_len: int = 1024
    hidden_size: int = 1024


class Straggler:
    def __init__(self, local_device, log_file: str | None, workload_info: WorkloadInfo):
        self.local_device = torch.device(local_device) if not isinstance(local_device, torch.device) else local_device
        self.log_file = log_file
        self.workload_info = workload_info
        self.workload_baseline_time: float | None = None

    # ---- file protocol ----------------------------------------------------------------------------
    @staticmethod
    def read_profile(log_file: str, length: int, ignore_first: bool = True, timeout_s: float = 60.0) -> list:
        """Waits (bounded) until the file ends with ``EOF`` and returns its numbers (the first, cold, entry
        dropped)."""
        t0 = time.time()
        while True:
            if os.path.exists(log_file):
                with open(log_file) as f:
                    lines = [ln.strip() for ln in f.readlines() if ln.strip()]
                if lines and lines[-1] == "EOF":
                    vals = [float(x) for x in lines[(1 if ignore_first else 0):-1]]
                    if len(vals) != length:
                        raise ValueError(f"{log_file}: expected {length} entries, found {len(vals)}")
                    return vals
            if time.time() - t0 > timeout_s:
                raise TimeoutError(f"profile {log_file} was not completed within {timeout_s} s")
            time.sleep(0.01)

    def begin_profile(self) -> None:
        os.makedirs(os.path.dirname(os.path.abspath(self.log_file)), exist_ok=True)
        with open(self.log_file, "w") as f:
            f.flush()
            os.fsync(f.fileno())

    def end_profile(self) -> None:
        with open(self.log_file, "a") as f:
            f.write("EOF\n")
            f.flush()
            os.fsync(f.fileno())

    def run_profile(self) -> float:
        t = self.run_workload()
        if self.log_file:
            with open(self.log_file, "a") as f:
                f.write(f"{t}\n")
                f.flush()
                os.fsync(f.fileno())
        return t

    # ---- workload -----------------------------------------------------------------------------------
    def run_workload(self) -> float:
        """Seconds for WORKLOAD_ITERS rounds of x @ Y @ Z with [mbs*seq, h] x [h, 4h] x [4h, h]."""
        w = self.workload_info
        dev = self.local_device
        dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
        g = torch.Generator(device=dev).manual_seed(0)
        x = torch.randn(w.mbs * w.seq_len, w.hidden_size, device=dev, dtype=dtype, generator=g)
        y = torch.randn(4 * w.hidden_size, w.hidden_size, device=dev, dtype=dtype, generator=g) * 0.02
        z = torch.randn(w.hidden_size, 4 * w.hidden_size, device=dev, dtype=dtype, generator=g) * 0.02
        from ..ops.gemm import gemm

        def body(v):
            return gemm(gemm(v, y), z)

        x = body(x)
        if dev.type == "cuda":
            torch.cuda.synchronize(dev)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(WORKLOAD_ITERS):
                x = body(x)
            e1.record()
            torch.cuda.synchronize(dev)
            return e0.elapsed_time(e1) / 1e3
        t0 = time.perf_counter()
        for _ in range(WORKLOAD_ITERS):
            x = body(x)
        return time.perf_counter() - t0

    def calibrate(self, repeats: int = 3) -> float:
        self.run_workload()
        self.workload_baseline_time = float(np.median([self.run_workload() for _ in range(repeats)]))
        return self.workload_baseline_time


def gather_times(value: float, group=None) -> list:
    """Every rank's value, on every rank (host-side exchange over the process group)."""
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return [float(value)]
    out = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, float(value), group=group)
    return [float(v) for v in out]


class StepTimeWindow:
    """Sliding window of compute times per rank -> slow-down ratio per rank against the baseline."""

    def __init__(self, world: int, window: int = SLIDING_WINDOW, threshold: float = 1.15):
        self.world, self.window, self.threshold = world, window, threshold
        self.samples: list = []
        self.baseline: np.ndarray | None = None

    def add(self, per_rank_times) -> None:
        t = np.asarray(per_rank_times, dtype=np.float64)
        if t.shape != (self.world,):
            raise ValueError("one time per rank expected")
        self.samples.append(t)
        self.samples = self.samples[-self.window:]

    def full(self) -> bool:
        return len(self.samples) >= self.window

    def set_baseline(self, per_rank_times=None) -> None:
        self.baseline = np.asarray(per_rank_times, dtype=np.float64) if per_rank_times is not None else \
            np.mean(self.samples, axis=0)

    def ratios(self) -> np.ndarray:
        cur = np.mean(self.samples, axis=0)
        base = self.baseline if self.baseline is not None else np.full(self.world, np.median(cur))
        return cur / np.maximum(base, 1e-12)

    def stragglers(self) -> dict:
        """{rank: slow-down ratio} of the ranks above the threshold."""
        return {int(r): float(x) for r, x in enumerate(self.ratios()) if x > self.threshold}


class Heartbeat:
    """Host-side liveness: ``beat()`` between steps, ``dead_ranks()`` before the next launch.

    Backed by a directory (one small file per rank, works without any process group) or by a
    ``torch.distributed`` store (``store.set`` / ``store.get``)."""

    def __init__(self, rank: int, world: int, directory: str | None = None, store=None, limit_s: float = 30.0):
        if (directory is None) == (store is None):
            raise ValueError("give exactly one of directory / store")
        self.rank, self.world, self.dir, self.store, self.limit_s = rank, world, directory, store, limit_s
        self.count = 0
        if directory is not None:
            os.makedirs(directory, exist_ok=True)

    def _key(self, r: int) -> str:
        return f"heartbeat_{r}"

    def beat(self) -> None:
        self.count += 1
        payload = f"{self.count} {time.time()}"
        if self.dir is not None:
            tmp = os.path.join(self.dir, self._key(self.rank) + ".tmp")
            with open(tmp, "w") as f:
                f.write(payload)
            os.replace(tmp, os.path.join(self.dir, self._key(self.rank)))
        else:
            self.store.set(self._key(self.rank), payload)

    def last_seen(self, r: int):
        try:
            if self.dir is not None:
                with open(os.path.join(self.dir, self._key(r))) as f:
                    payload = f.read()
            else:
                if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                    return None
                payload = self.store.get(self._key(r)).decode()
            c, t = payload.split()
            return int(c), float(t)
        except (OSError, ValueError):
            return None

    def dead_ranks(self, now: float | None = None) -> list:
        now = time.time() if now is None else now
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            seen = self.last_seen(r)
            if seen is None or now - seen[1] > self.limit_s:
                dead.append(r)
        return dead
