"""Named streams and events.

The reference gives every device 16 logical streams (hetu/core/stream.h:8-19): Blocking 0, Computing 1,
SwitchComputing 2, H2D 3, D2H 4, P2P 5, Collective 6, SwitchCollective 7, Optimizer 8, Join 15.  Here a logical
stream index maps to one ``torch.cuda.Stream`` per device, created on first use (index 0 is the default stream);
on CPU the handles are inert so the same code runs in tests.  ``Event`` wraps ``torch.cuda.Event`` with the
reference's Record / Sync / Block / TimeSince vocabulary.
"""
from __future__ import annotations

import time

import torch

kBlockingStream, kComputingStream, kSwitchComputingStream, kH2DStream, kD2HStream, kP2PStream, kCollectiveStream, \
    kSwitchCollectiveStream, kOptimizerStream, kJoinStream = 0, 1, 2, 3, 4, 5, 6, 7, 8, 15
NUM_LOGICAL_STREAMS = 16
_streams: dict = {}


class Stream:
    def __init__(self, device, index: int):
        if not 0 <= index < NUM_LOGICAL_STREAMS:
            raise ValueError(f"stream index {index} out of range")
        self.device = torch.device(device)
        self.index = index
        self._cuda = None
        if self.device.type == "cuda":
            self._cuda = torch.cuda.default_stream(self.device) if index in (kBlockingStream, kComputingStream) \
                else torch.cuda.Stream(self.device)

    @property
    def cuda_stream(self):
        return self._cuda

    # spellings of the reference's Stream (hetu/core/stream.h:8-60)
    @property
    def stream_index(self) -> int:
        return self.index

    @property
    def device_type(self) -> str:
        return self.device.type

    @property
    def device_index(self) -> int:
        return self.device.index or 0

    @property
    def is_define(self) -> bool:
        return True

    def __enter__(self):
        if self._cuda is not None:
            self._ctx = torch.cuda.stream(self._cuda)
            self._ctx.__enter__()
        return self

    def __exit__(self, *a):
        if self._cuda is not None:
            self._ctx.__exit__(*a)

    def sync(self) -> None:
        if self._cuda is not None:
            self._cuda.synchronize()

    def wait(self, event: "Event") -> None:
        if self._cuda is not None and event._ev is not None:
            self._cuda.wait_event(event._ev)

    def __repr__(self):
        return f"Stream({self.device}, {self.index})"


def get_stream(device, index: int) -> Stream:
    key = (str(torch.device(device)), index)
    if key not in _streams:
        _streams[key] = Stream(device, index)
    return _streams[key]


class Event:
    def __init__(self, device, enable_timing: bool = True):
        self.device = torch.device(device)
        self._ev = torch.cuda.Event(enable_timing=enable_timing) if self.device.type == "cuda" else None
        self._t = None

    def record(self, stream: Stream | None = None) -> None:
        if self._ev is not None:
            self._ev.record(stream.cuda_stream if stream is not None else None)
        else:
            self._t = time.perf_counter()

    def sync(self) -> None:
        if self._ev is not None:
            self._ev.synchronize()

    def block(self, stream: Stream) -> None:
        stream.wait(self)

    def time_since(self, earlier: "Event") -> float:
        """Milliseconds between `earlier` and this event."""
        if self._ev is not None:
            return earlier._ev.elapsed_time(self._ev)
        return (self._t - earlier._t) * 1e3


def synchronize_all_streams(device) -> None:
    if torch.device(device).type == "cuda":
        torch.cuda.synchronize(device)
