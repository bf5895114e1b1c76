"""The allocation-free norm-backward entry point against the regular one.

Some callers of the kernel library cannot allocate device memory (a host application owns the memory budget,
or an arena manager reserved everything up front), so ``hsb_norm_bwd_noalloc`` keeps its scratch inside the
library.  This test calls it through its exported C symbol, twice in a row with different shapes (the built-in
scratch still holds the first call's partial sums when the second call starts), and compares every output
with ``hsb_norm_bwd`` run on a scratch buffer that the test allocates.  It also checks that an oversized
request is refused.  The file name sorts last so that a ``-x`` run has finished every other test before it.
"""
import ctypes
import os

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "hotspa_ae_b200", "_hsb_kernels.so")

vp, ci, cl = ctypes.c_void_p, ctypes.c_int, ctypes.c_long


def _load():
    lib = ctypes.CDLL(LIB)
    lib.hsb_norm_bwd_parts.argtypes = [ci, ci]
    lib.hsb_norm_bwd_parts.restype = ci
    lib.hsb_norm_bwd.argtypes = [vp] * 10 + [ci] * 5 + [vp]
    lib.hsb_norm_bwd.restype = ci
    lib.hsb_norm_bwd_noalloc.argtypes = [vp] * 9 + [ci] * 5 + [vp]
    lib.hsb_norm_bwd_noalloc.restype = ci
    lib.hsb_norm_bwd_noalloc_max_floats.argtypes = []
    lib.hsb_norm_bwd_noalloc_max_floats.restype = cl
    return lib


def _case(lib, rows, H, is_rms, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    dev = "cuda"
    dy = torch.randn(rows, H, device=dev, generator=g).bfloat16()
    x = torch.randn(rows, H, device=dev, generator=g).bfloat16()
    w = (1.0 + 0.1 * torch.randn(H, device=dev, generator=g)).bfloat16()
    dres = torch.randn(rows, H, device=dev, generator=g).bfloat16()
    xf = x.float()
    if is_rms:
        mean = None
        rstd = torch.rsqrt(xf.pow(2).mean(-1) + 1e-6)
    else:
        mean = xf.mean(-1)
        rstd = torch.rsqrt(xf.var(-1, unbiased=False) + 1e-5)
    stream = torch.cuda.current_stream().cuda_stream
    ptr = lambda t: 0 if t is None else t.data_ptr()  # noqa: E731
    outs = []
    for noalloc in (False, True):
        dx = torch.empty_like(x)
        dw = torch.full((H,), 0.5, dtype=torch.float32, device=dev)       # accumulate=1 adds onto this
        db = None if is_rms else torch.full((H,), -0.25, dtype=torch.float32, device=dev)
        if noalloc:
            rc = lib.hsb_norm_bwd_noalloc(ptr(dy), ptr(x), ptr(w), ptr(mean), ptr(rstd), ptr(dres), ptr(dx), ptr(dw),
                                          ptr(db), rows, H, int(is_rms), 1, 0, stream)
        else:
            parts = lib.hsb_norm_bwd_parts(rows, 0)
            scratch = torch.empty(parts * 2 * H, dtype=torch.float32, device=dev)
            rc = lib.hsb_norm_bwd(ptr(dy), ptr(x), ptr(w), ptr(mean), ptr(rstd), ptr(dres), ptr(dx), ptr(dw), ptr(db),
                                  ptr(scratch), rows, H, int(is_rms), 1, 0, stream)
        assert rc == 0, f"launcher returned {rc}"
        torch.cuda.synchronize()
        outs.append((dx, dw, db))
    (dx0, dw0, db0), (dx1, dw1, db1) = outs
    torch.testing.assert_close(dx1.float(), dx0.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(dw1, dw0, rtol=1e-4, atol=1e-3)
    if db0 is not None:
        torch.testing.assert_close(db1, db0, rtol=1e-4, atol=1e-3)
    # and against plain fp32 math, so that two equally wrong results cannot pass
    xh = xf * rstd[:, None] if is_rms else (xf - mean[:, None]) * rstd[:, None]
    want_dw = 0.5 + (dy.float() * xh).sum(0)
    torch.testing.assert_close(dw1, want_dw, rtol=2e-3, atol=2e-2)


@pytest.mark.gpu
def test_norm_bwd_noalloc_matches_regular_entry_point_twice():
    lib = _load()
    _case(lib, rows=1000, H=4096, is_rms=True, seed=1)      # first call on the device also does the set-up
    _case(lib, rows=333, H=1024, is_rms=False, seed=2)      # second call: stale partial sums in the scratch
    _case(lib, rows=1000, H=4096, is_rms=True, seed=3)


@pytest.mark.gpu
def test_norm_bwd_noalloc_rejects_oversized_request():
    lib = _load()
    cap = lib.hsb_norm_bwd_noalloc_max_floats()
    rows, H, num_sms = 100000, 8192, 1024               # parts = 2048 -> far beyond the built-in scratch
    assert lib.hsb_norm_bwd_parts(rows, num_sms) * 2 * H > cap
    rc = lib.hsb_norm_bwd_noalloc(0, 0, 0, 0, 0, 0, 0, 0, 0, rows, H, 1, 0, num_sms, 0)
    assert rc == -20
