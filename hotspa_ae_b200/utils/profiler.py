"""Profiling and observability: memory (allocator + NVML), NVLink per-link counters, per-micro-batch memory
traces, per-step JSONL logs and the hot-switch report.

Environment (names of the reference, hetu/graph/profiler.{h,cc}, executable_graph.cc:1284-1307, 2097-2116,
switch_exec_graph.h:529-546): ``HETU_MEMORY_PROFILE=MICRO_BATCH|INFO|WARN`` with ``HETU_MEMORY_LOG_FILE``,
``HETU_SWITCH_PROFILE=TRACE|MEMORY|NVLINK|TIME|INFO`` with ``HETU_SWITCH_LOG_FILE``, ``HETU_STRAGGLER`` with
``HETU_STRAGGLER_LOG_FILE``.  NVML is only read, never written.
"""
from __future__ import annotations

import json
import os
import time

import torch

from ..core import NvmlProfiler
from . import roofline

_nvml = None


def nvml() -> NvmlProfiler:
    global _nvml
    if _nvml is None:
        _nvml = NvmlProfiler(os.environ.get("HSB_NVML_LIBRARY", ""))
    return _nvml


class CUDAProfiler:
    def __init__(self, device=None):
        self.device = torch.device(device) if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        self._link_base = None

    def memory_info(self) -> dict:
        """Allocator reserved/allocated plus what the driver reports for the whole device (MiB)."""
        out = {"mempool_reserved": 0.0, "mempool_allocated": 0.0, "mempool_peak_reserved": 0.0,
               "all_used": None, "limit": None}
        if self.device.type == "cuda":
            out["mempool_reserved"] = torch.cuda.memory_reserved(self.device) / 2**20
            out["mempool_allocated"] = torch.cuda.memory_allocated(self.device) / 2**20
            out["mempool_peak_reserved"] = torch.cuda.max_memory_reserved(self.device) / 2**20
            m = nvml().memory(self.device.index or 0) if nvml().available() else None
            if m is not None and m.ok:
                out["all_used"], out["limit"] = m.used / 2**20, m.total / 2**20
            else:
                free, total = torch.cuda.mem_get_info(self.device)
                out["all_used"], out["limit"] = (total - free) / 2**20, total / 2**20
        return out

    def nvlink_begin(self) -> None:
        self._link_base = self._links()

    def nvlink_end(self) -> dict:
        """Per-link TX/RX KiB since ``nvlink_begin`` ({} when the counters are unavailable)."""
        now, base = self._links(), self._link_base
        if not now or not base:
            return {}
        return {"tx_kib": [a - b for a, b in zip(now[0], base[0])], "rx_kib": [a - b for a, b in zip(now[1], base[1])]}

    def _links(self):
        if self.device.type != "cuda" or not nvml().available():
            return None
        c = nvml().nvlink(self.device.index or 0)
        return (list(c.tx_kib), list(c.rx_kib)) if c.ok else None


class MemoryTrace:
    """Per-micro-batch memory samples written as one JSON array (``HETU_MEMORY_PROFILE=MICRO_BATCH``)."""

    def __init__(self, path: str | None = None):
        self.enabled = os.environ.get("HETU_MEMORY_PROFILE", "WARN").upper() == "MICRO_BATCH"
        self.path = path or os.environ.get("HETU_MEMORY_LOG_FILE", "")
        self.samples: list = []
        self.prof = CUDAProfiler()

    def sample(self, micro_batch: int, is_forward: bool) -> None:
        if self.enabled:
            d = self.prof.memory_info()
            d.update(micro_batch_id=micro_batch, is_forward=is_forward)
            self.samples.append(d)

    def flush(self) -> None:
        if self.enabled and self.path:
            with open(self.path, "w") as f:
                json.dump(self.samples, f)
                f.flush()
                os.fsync(f.fileno())


class StepLogger:
    """One JSON line per step: tokens, step time, per-bucket times, switch times and bytes."""

    def __init__(self, path: str):
        self.f = open(path, "a")

    def log(self, step: int, result, seconds: float, profile: dict | None = None, config=None,
            n_gpus: int = 1) -> None:
        rec = {"step": step, "time": time.time(), "loss": result.loss, "tokens": result.tokens, "step_s": seconds,
               "tokens_per_s": result.tokens / max(seconds, 1e-9), "buckets": result.buckets}
        if config is not None:
            rec["mfu_of_measured"] = roofline.mfu(rec["tokens_per_s"], config, n_gpus)
        if profile:
            rec["bucket_ms"] = profile.get("bucket_ms")
            rec["switches"] = profile.get("switches")
        self.f.write(json.dumps(rec) + "\n")
        self.f.flush()

    def close(self) -> None:
        self.f.close()


def switch_report(store, file=None) -> list:
    """Hot-switch log of a ParamStore as dicts (device ms, bytes over NVLink, achieved GB/s); printed when
    ``HETU_SWITCH_PROFILE`` is TIME or more verbose, appended to ``HETU_SWITCH_LOG_FILE`` when set."""
    out = []
    for x in store.switch_log:
        e0, e1 = x["events"]
        ms = e0.elapsed_time(e1) if e0 is not None else x["host_ms"]
        nbytes = x["remote_elems"] * (4 if x["kind"] == "grad" else 2)
        esz = 4 if x["kind"] == "grad" else 2
        busiest = x.get("max_recv_elems", 0) * esz
        out.append({"src": x["src"], "dst": x["dst"], "kind": x["kind"], "mode": x["mode"], "ms": ms,
                    "remote_bytes_total": nbytes, "local_elems": x["local_elems"],
                    "busiest_receiver_bytes": busiest,
                    # share of the measured NVLink peer-copy rate on the receiver that takes in the most
                    "link_fraction": roofline.switch_link_fraction(busiest, ms)})
    level = os.environ.get("HETU_SWITCH_PROFILE", "INFO").upper()
    if level in ("TRACE", "MEMORY", "NVLINK", "TIME"):
        for r in out:
            line = f"switch {r['kind']} {r['src']} -> {r['dst']} ({r['mode']}): running time = {r['ms']:.3f} ms"
            print(line, file=file, flush=True)
            path = os.environ.get("HETU_SWITCH_LOG_FILE")
            if path:
                with open(path, "a") as f:
                    f.write(line + "\n")
    return out


def apply_allocator_env() -> None:
    """Maps ``HETU_MAX_SPLIT_SIZE_MB`` onto the caching allocator's ``max_split_size_mb`` (must run before the
    first CUDA allocation).  ``HETU_MAX_INTERNAL_FRAGMENT_SIZE_MB`` has no counterpart and is ignored."""
    v = os.environ.get("HETU_MAX_SPLIT_SIZE_MB")
    if v and int(v) > 0 and "PYTORCH_CUDA_ALLOC_CONF" not in os.environ:
        os.environ["PYTORCH_CUDA_ALLOC_CONF"] = f"max_split_size_mb:{int(v)}"


def empty_cache() -> None:
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
