"""Debug-mode memory checks for the peer-memory runtime (host side; nothing here runs in a normal step).

The pool this framework is developed on has no compute-sanitizer, and a stray peer store would corrupt another
rank's arena silently, so the checks that can be made without a tool are made here:

  * **canaries**: with ``HSB_DEBUG_CANARIES=1`` every arena (parameter / gradient arenas, symmetric buffers) is
    allocated with a tail guard filled with a byte pattern; ``check_canaries`` compares the guards on the host and
    names the buffer whose guard changed.  The trainer checks after every step in this mode.
  * **descriptor validation**: before a reshard descriptor table is uploaded, every rectangle is checked against the
    extents of the arena it reads (on the rank it reads from) and of the arena it writes, for alignment, and - for
    copies - for overlap between destination rows.  Enabled by the same variable, or called directly.

The reference has no counterpart (it relies on HT_ASSERTs on buffer state, hetu/graph/switch_exec_graph.cc:923-930).
"""
from __future__ import annotations

import os

import numpy as np
import torch

GUARD_BYTES = 4096
PATTERN = 0xA5


def enabled() -> bool:
    return os.environ.get("HSB_DEBUG_CANARIES", "0") not in ("", "0")


class GuardedAlloc:
    """Registry of (name, guard view) pairs of one owner (a ParamStore or a SymmHeap)."""

    def __init__(self):
        self.guards: list[tuple[str, torch.Tensor]] = []

    def wrap_bytes(self, name: str, raw: torch.Tensor, nbytes: int) -> torch.Tensor:
        """`raw` is a uint8 tensor of nbytes + GUARD_BYTES: paint and register the tail, return the payload."""
        guard = raw[nbytes:nbytes + GUARD_BYTES]
        guard.fill_(PATTERN)
        self.guards.append((name, guard))
        return raw[:nbytes]

    def alloc(self, name: str, numel: int, dtype, device) -> torch.Tensor:
        esz = torch.empty((), dtype=dtype).element_size()
        nbytes = max(numel, 1) * esz
        nbytes = (nbytes + 15) // 16 * 16
        raw = torch.zeros(nbytes + GUARD_BYTES, dtype=torch.uint8, device=device)
        return self.wrap_bytes(name, raw, nbytes)[:max(numel, 1) * esz].view(dtype)

    def check(self) -> None:
        for name, guard in self.guards:
            host = guard.detach().cpu().numpy()
            bad = np.flatnonzero(host != PATTERN)
            if bad.size:
                raise RuntimeError(f"memory guard of {name} was overwritten: {bad.size} bytes, first at +{int(bad[0])} "
                                   f"past the end of the buffer")


def validate_descriptors(descs: np.ndarray, src_extents: dict, dst_extent: tuple, elem_size: int,
                         copy: bool) -> list[str]:
    """descs: int64 [n, 6] rows (src_ptr, dst_ptr, rows, row_bytes, src_ld_bytes, dst_ld_bytes) as the reshard kernel
    takes them (ld = 0 for single-row descriptors).  src_extents: {name: (base, nbytes)} of every arena a source may
    lie in; dst_extent: (base, nbytes) of the arena written.  Returns the list of problems (empty = valid)."""
    errs: list[str] = []
    if descs.size == 0:
        return errs
    d = np.asarray(descs, dtype=np.int64).reshape(-1, 6)
    sp, dp, rows, rb, sld, dld = (d[:, i] for i in range(6))
    bad = np.flatnonzero((rows < 1) | (rb < 1))
    errs += [f"descriptor {i}: empty rectangle (rows {rows[i]}, row bytes {rb[i]})" for i in bad[:8]]
    multi = rows > 1
    bad = np.flatnonzero(multi & ((sld < rb) | (dld < rb)))
    errs += [f"descriptor {i}: leading dimension smaller than the row ({sld[i]}, {dld[i]} < {rb[i]})" for i in bad[:8]]
    mis = (sp | dp | rb | np.where(multi, sld | dld, 0)) % elem_size
    bad = np.flatnonzero(mis != 0)
    errs += [f"descriptor {i}: address, row size or leading dimension not a multiple of {elem_size} bytes"
             for i in bad[:8]]
    s_end = sp + (rows - 1) * np.where(multi, sld, 0) + rb
    d_end = dp + (rows - 1) * np.where(multi, dld, 0) + rb
    inside = np.zeros(len(d), dtype=bool)
    for base, nbytes in src_extents.values():
        inside |= (sp >= base) & (s_end <= base + nbytes)
    bad = np.flatnonzero(~inside)
    errs += [f"descriptor {i}: source [{sp[i]:#x}, {s_end[i]:#x}) lies in no source arena" for i in bad[:8]]
    base, nbytes = dst_extent
    bad = np.flatnonzero((dp < base) | (d_end > base + nbytes))
    errs += [f"descriptor {i}: destination [{dp[i]:#x}, {d_end[i]:#x}) leaves the arena "
             f"[{base:#x}, {base + nbytes:#x})" for i in bad[:8]]
    if copy and not errs:
        # every destination row as an interval; a copy plan writes each byte once
        rep = rows.astype(np.int64)
        idx = np.repeat(np.arange(len(d)), rep)
        within = np.arange(rep.sum()) - np.repeat(np.cumsum(rep) - rep, rep)
        start = dp[idx] + within * np.where(multi, dld, 0)[idx]
        end = start + rb[idx]
        order = np.argsort(start, kind="stable")
        clash = np.flatnonzero(start[order][1:] < end[order][:-1])
        errs += [f"descriptors {idx[order][j]} and {idx[order][j + 1]}: destination rows overlap" for j in clash[:8]]
    return errs
