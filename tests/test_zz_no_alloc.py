"""GPU: repdl_b200_sum1d_static, the chain sum whose scratch is a fixed array inside the library.

It exists for callers that may not allocate device memory where they need the sum (inside a
stream capture, in a callback with hard latency bounds, in a process whose device memory is owned
by another component, behind a plugin interface that only hands over inputs and outputs).  The
result must have exactly the bits of repdl_b200_sum1d, which takes its scratch from the caller --
on a first call and on a second call that finds the array dirty from the first.  This file is
collected last on purpose, so that a failure here cannot hide the result of any other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.cpu().view(torch.int32).item() & 0xFFFFFFFF


def _with_scratch(lib, check, x, factor):
    n = x.numel()
    nbytes = lib.repdl_b200_sum1d_scratch_bytes(n)
    scratch = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=x.device)
    out = torch.empty((), dtype=torch.float32, device=x.device)
    check(lib.repdl_b200_sum1d(x.data_ptr(), out.data_ptr(), n, factor, scratch.data_ptr(), nbytes, None),
          "sum1d")
    return out


def _static(lib, check, x, factor):
    out = torch.empty((), dtype=torch.float32, device=x.device)
    check(lib.repdl_b200_sum1d_static(x.data_ptr(), out.data_ptr(), x.numel(), factor, None),
          "sum1d_static")
    return out


def test_static_scratch_sum_matches_caller_scratch_sum_twice_in_a_row():
    from repdl_b200._cabi import check, lib
    g = torch.Generator().manual_seed(77)
    # long enough for the summarised path (several nodes), hovering around 2^20 so that nodes,
    # tiles and leaves all get opened; the second input differs so that the second call really
    # meets a dirty array
    a = torch.randn(700001, generator=g) * 50.0
    a[0] = 1048570.0
    b = (torch.empty(1500000).log_normal_(0, 2, generator=g)
         * (torch.randint(0, 2, (1500000,), generator=g).float() * 2 - 1))
    ad, bd = a.cuda(), b.cuda()
    import oracle
    _static(lib, check, ad, 1.0)  # the set-up call: later calls must not change the device's memory
    torch.cuda.synchronize()
    for x, xc, factor in ((ad, a, 1.0), (bd, b, 0.5), (ad, a, 1.0)):
        want = _with_scratch(lib, check, x, factor)
        torch.cuda.synchronize()
        free0, held0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
        out = torch.empty((), dtype=torch.float32, device=x.device)  # the caller's own output buffer
        held1 = torch.cuda.memory_allocated()
        check(lib.repdl_b200_sum1d_static(x.data_ptr(), out.data_ptr(), x.numel(), factor, None),
              "sum1d_static")
        torch.cuda.synchronize()
        # no allocation behind the caller's back: neither torch's pool nor the device's free memory moved
        assert torch.cuda.memory_allocated() == held1 and torch.cuda.mem_get_info()[0] == free0, (free0, held0)
        assert _bits(out) == _bits(want)
        # ... and both are the reference's chain (the oracle's strict left-to-right sum)
        scaled = oracle.sum1d(xc, False) * factor  # factor 0.5 / 1.0: an exact scaling
        assert _bits(out) == _bits(scaled)
    # a short chain takes the scratch-free path of both entry points
    s = ad[:1000].contiguous()
    assert _bits(_static(lib, check, s, 1.0)) == _bits(_with_scratch(lib, check, s, 1.0))


def test_static_scratch_sum_rejects_chains_beyond_its_maximum():
    from repdl_b200._cabi import lib
    max_n = lib.repdl_b200_sum1d_static_max_n()
    assert max_n == 1 << 28
    x = torch.zeros(16, device="cuda")
    out = torch.zeros((), device="cuda")
    # the size check comes before any memory access, so a small buffer is enough to probe it
    status = lib.repdl_b200_sum1d_static(x.data_ptr(), out.data_ptr(), max_n + 1, 1.0, None)
    assert status == -6  # REPDL_E_STATIC_MAX
    assert b"built-in scratch" in lib.repdl_b200_strerror(status)
