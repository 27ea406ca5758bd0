"""CPU: the host model of the summarised chain sum (tests/sum1d_host_model.cpp) against the oracle.

The model runs the passes of repdl_b200/csrc/sum1d.cu as plain loops with the arithmetic of
repdl_b200/csrc/sum1d_core.cuh, the header the CUDA kernels include.  What is checked here without a
GPU is therefore the algebra itself: leaf summaries, their orientation for negative states, exact
ties, the classification against the predicted state, the item stream with its skip counts, and the
fall-backs (a robust run that does not fit, a node demoted to a raw span, an item buffer that is
too small).
"""
import ctypes
import os
import random
import subprocess
import tempfile

import pytest
import torch

import oracle

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def model():
    out = os.path.join(tempfile.mkdtemp(prefix="repdl_s1_"), "sum1d_host_model.so")
    subprocess.run(["/usr/bin/g++", "-O2", "-ffp-contract=off", "-shared", "-fPIC", "-o", out,
                    os.path.join(HERE, "sum1d_host_model.cpp")], check=True)
    lib = ctypes.CDLL(out)
    lib.s1_model_sum.restype = ctypes.c_float

    def run(x, factor=1.0, cap=0):
        st = (ctypes.c_int64 * 16)()
        r = lib.s1_model_sum(ctypes.c_void_p(x.data_ptr()), ctypes.c_int64(x.numel()),
                             ctypes.c_float(factor), st, ctypes.c_int64(cap))
        return torch.tensor(r), list(st)[:10]
    return run


def bits(t):
    return t.view(torch.int32).item() & 0xFFFFFFFF


def chain_inputs(count, seed):
    """Element distributions that move the running sum through binades in different ways."""
    rnd = random.Random(seed)
    g = torch.Generator().manual_seed(seed)
    for it in range(count):
        n = rnd.randint(1 << 16, 1 << 20)
        kind = it % 8
        if kind == 0:      # zero-mean: the sum hovers around zero and keeps changing binade
            x = torch.randn(n, generator=g)
        elif kind == 1:    # drifting upwards through many binades
            x = torch.rand(n, generator=g) * 10.0 ** rnd.randint(-3, 3)
        elif kind == 2:    # heavy tails
            x = torch.randn(n, generator=g) * torch.exp(3 * torch.randn(n, generator=g))
        elif kind == 3:    # exact ties: halves of the ulp of the running sum
            x = torch.randint(-3, 4, (n,), generator=g).float() * 2.0 ** rnd.randint(-30, -10) + 1e-3
        elif kind == 4:    # a few huge elements among small ones (and a cancellation)
            x = torch.randn(n, generator=g) * 1e-3
            idx = torch.randint(0, n, (8,), generator=g)
            x[idx] = torch.tensor([1e20, -1e20, 3e7, -3e7, 1e30, -1e30, 5e3, -5e3])
        elif kind == 5:    # subnormal and tiny values
            x = torch.randn(n, generator=g) * 1e-40
        elif kind == 6:    # constant: the sum saturates where the element is below half an ulp
            x = torch.full((n,), rnd.choice([1.0, 0.1, 3.0e-5]))
        else:              # sign flips in blocks
            x = torch.rand(n, generator=g) * torch.sign(torch.sin(torch.arange(n) / rnd.randint(50, 50000)))
        yield it, kind, x


def test_model_matches_the_plain_chain(model):
    kinds_with_summaries = 0
    for it, kind, x in chain_inputs(24, 5):
        want = oracle.sum1d(x, False)
        got, st = model(x)
        assert bits(got) == bits(want), (it, kind, x.numel(), st)
        kinds_with_summaries += st[1] > 0
    assert kinds_with_summaries >= 12  # the summaries really carry most chains


def test_model_with_a_tight_item_buffer(model):
    """Nodes that no longer fit into the item buffer become raw spans; the bits stay."""
    for it, kind, x in chain_inputs(8, 6):
        want = oracle.sum1d(x, False)
        nnodes = (x.numel() + 32767) // 32768
        for cap in (nnodes, nnodes + 7, nnodes + 300):
            got, st = model(x, 1.0, cap)
            assert bits(got) == bits(want), (it, kind, cap, st)
            assert st[0] <= cap


def test_model_special_values(model):
    g = torch.Generator().manual_seed(9)
    n = 200000
    base = torch.randn(n, generator=g) * 100
    for special in (float("inf"), float("-inf"), float("nan"), 3.0e38, -3.0e38):
        x = base.clone()
        x[123457] = special
        if special == 3.0e38:
            x[150000] = 3.0e38  # overflows to +inf in the chain
        want, (got, st) = oracle.sum1d(x, False), model(x)
        if want.isnan():
            assert got.isnan()
        else:
            assert bits(got) == bits(want), (special, st)
    # the mean: one rounded multiplication at the end
    x = base[:70001].contiguous()
    f = torch.tensor(1.0 / x.numel(), dtype=torch.float64).float().item()
    assert bits(model(x, f)[0]) == bits(oracle.sum1d(x, True))
    # ragged end inside a leaf, negative running sum throughout
    y = -torch.rand(65536 + 37, generator=g) * 1000
    assert bits(model(y)[0]) == bits(oracle.sum1d(y, False))


def test_model_on_the_config3_stream(model):
    """The first 2^22 elements of config 3's chain against the oracle, and the share of the chain
    that needs real additions (the serial cost the GPU walker pays)."""
    from repdl_b200 import workloads
    x = torch.cat(list(workloads.sum_chunks(1 << 22, 2)))
    got, st = model(x)
    assert bits(got) == bits(oracle.sum1d(x, False))
    leaves = x.numel() // 32
    assert st[7] < leaves // 4, st  # most leaves are applied as summaries
