"""The allocation-free RMSNorm backward entry point, called through its exported C symbol.

Some callers of the kernel library may not allocate device memory at the moment they need the
backward pass (another part of the process is capturing a CUDA graph, a host application gave the
plugin a fixed budget, a latency-critical loop).  ``dcpk_rmsnorm_bwd_noalloc`` serves them: its fp32
weight-gradient accumulator is a fixed array inside the library.  This test calls it twice in a
row - the array is shared between calls and must be cleared by each - and compares both results
with the regular entry point, whose accumulator the caller allocates.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run_both(lib, n_rows, hidden, seed, dev):
    from dcp_b200.ops import _lib
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(n_rows, hidden, device=dev, generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(hidden, device=dev, generator=g)).bfloat16()
    dy = torch.randn(n_rows, hidden, device=dev, generator=g).bfloat16()
    y, rstd = torch.empty_like(x), torch.empty(n_rows, dtype=torch.float32, device=dev)
    s = _lib.stream_handle()
    assert lib.dcpk_rmsnorm_fwd(_lib.ptr(x), _lib.ptr(w), _lib.ptr(y), _lib.ptr(rstd), ctypes.c_int(n_rows),
                                ctypes.c_int(hidden), ctypes.c_float(1e-5), s) == 0
    # regular entry point: the caller provides the zeroed fp32 accumulator
    dx_ref, dw_acc = torch.empty_like(x), torch.zeros(hidden, dtype=torch.float32, device=dev)
    assert lib.dcpk_rmsnorm_bwd(_lib.ptr(x), _lib.ptr(w), _lib.ptr(dy), _lib.ptr(rstd), _lib.ptr(dx_ref),
                                _lib.ptr(dw_acc), ctypes.c_int(n_rows), ctypes.c_int(hidden), s) == 0
    # allocation-free entry point: outputs only
    dx, dw = torch.full_like(x, float("nan")), torch.full((hidden,), float("nan"), dtype=torch.bfloat16, device=dev)
    rc = lib.dcpk_rmsnorm_bwd_noalloc(_lib.ptr(x), _lib.ptr(w), _lib.ptr(dy), _lib.ptr(rstd), _lib.ptr(dx), _lib.ptr(dw),
                                      ctypes.c_int(n_rows), ctypes.c_int(hidden), s)
    assert rc == 0
    torch.cuda.synchronize()
    return dx, dw, dx_ref, dw_acc


def test_no_alloc_entry_point_matches_regular_one_twice():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dcp_b200.ops import _lib
    lib = _lib.load()
    lib.dcpk_rmsnorm_bwd_noalloc.restype = ctypes.c_int
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    # two calls in a row with different data and sizes: the second must not see the first's sums
    for n_rows, hidden, seed in ((300, 4096, 0), (77, 4096, 1), (129, 1024, 2)):
        dx, dw, dx_ref, dw_acc = _run_both(lib, n_rows, hidden, seed, dev)
        assert torch.equal(dx, dx_ref)                       # same kernel, same inputs
        ref = dw_acc.float()
        assert ((dw.float() - ref).abs() / (ref.abs() + 1.0)).max() < 3e-2
    # sizes beyond the built-in accumulator are refused, nothing is launched
    t = torch.zeros(8, device=dev)
    rc = lib.dcpk_rmsnorm_bwd_noalloc(_lib.ptr(t), _lib.ptr(t), _lib.ptr(t), _lib.ptr(t), _lib.ptr(t), _lib.ptr(t),
                                      ctypes.c_int(1), ctypes.c_int(16384), _lib.stream_handle())
    assert rc == -3
