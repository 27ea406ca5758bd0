"""CPU: pins the C oracle (oracle/repdl_oracle.c) to the reference.

Two independent pins: (1) the committed fixtures in tests/golden/, produced by the reference's own
CPU backend (tests/golden/make_golden.py); (2) when the reference has been built into oracle/_ref
on this machine, a live bit-for-bit comparison against it.
"""
import json
import os

import pytest
import torch

import oracle
from cases import RefAdapter, build_cases, run_case, sha

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
CASES = build_cases()


def golden(name):
    with open(os.path.join(GOLDEN, name)) as f:
        return json.load(f)


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_oracle_matches_golden(case):
    want = golden("small_cases.json")[case[0]]
    got = run_case(oracle, case)
    assert list(got.shape) == want["shape"]
    assert sha(got) == want["sha256"]


@pytest.mark.skipif(oracle.ref() is None, reason="reference not built into oracle/_ref here")
@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_oracle_matches_reference_live(case):
    ref = RefAdapter(oracle.ref())
    a, b = run_case(oracle, case), run_case(ref, case)
    assert a.shape == b.shape
    assert torch.equal(a.contiguous().view(torch.int32), b.contiguous().view(torch.int32))


def test_specials_table():
    """The hand-picked special values: NaN payloads kept, x86 default NaNs, subnormals not flushed."""
    from cases import special_values
    g = golden("small_cases.json")["_specials_hex"]
    x = special_values(0)

    def hx(t):
        return ["%08x" % (v & 0xFFFFFFFF) for v in t.view(torch.int32).tolist()]
    assert hx(x) == g["x"]
    assert hx(oracle.exp(x)) == g["exp"]
    assert hx(oracle.log(x)) == g["log"]
    assert hx(oracle.sqrt(x)) == g["sqrt"]
    assert hx(oracle.div(x, 10.0)) == g["div10"]
    # spot values stated in words: exp(-88) is subnormal, div keeps subnormals, log(-1) = -nan
    i = g["x"].index("c2b00000")
    assert g["exp"][i] == "0041edc4"
    assert g["div10"][g["x"].index("807fffff")] == "800ccccd"
    assert g["log"][g["x"].index("bf800000")] == "ffc00000"
    assert g["sqrt"][g["x"].index("bf800000")] == "7fc00000"
    assert g["exp"][g["x"].index("7f800001")] == "7fc00001"
    # the double-rounding trap: glibc's fp64 log lands exactly on an fp32 midpoint
    assert g["log"][g["x"].index("41178feb")] == "400fe5e8"


def test_sum1d_carry_composes():
    x = torch.randn(100000, generator=torch.Generator().manual_seed(5)) * 1000
    whole = oracle.sum1d(x).item()
    s = 0.0
    for part in x.split(7777):
        s = oracle.sum1d_carry(part, s)
    assert s == whole


def test_config1_hash():
    path = os.path.join(GOLDEN, "configs.json")
    if not os.path.exists(path):
        pytest.skip("configs.json not generated")
    from repdl_b200 import workloads
    a, b = workloads.mm_square(1024, 0)
    assert sha(oracle.mm(a, b)) == golden("configs.json")["c1_mm_1024"]["sha256"]


# ---- optimizer steps: the oracle's restatement of Adam.step (repdl/optim.py:56-83) and the SGD update
@pytest.mark.parametrize("name,wd,ams", [c for c in __import__("cases").OPTIM_CONFIGS],
                         ids=[c[0] for c in __import__("cases").OPTIM_CONFIGS])
def test_oracle_adam_matches_golden(name, wd, ams):
    import cases
    assert cases.run_oracle_adam(oracle, wd, ams) == golden("optim_steps.json")["adam_" + name]


def test_oracle_sgd_matches_golden():
    import cases
    assert cases.run_oracle_sgd(oracle) == golden("optim_steps.json")["sgd"]


@pytest.mark.skipif(oracle.ref_site() is None, reason="reference not built into oracle/_ref here")
def test_oracle_adam_matches_reference_live():
    import sys

    import cases
    sys.path.insert(0, oracle.ref_site())
    import repdl
    for name, wd, ams in cases.OPTIM_CONFIGS:
        want = cases.run_optimizer(lambda ps: repdl.optim.Adam(ps, lr=0.01, weight_decay=wd, amsgrad=ams))
        assert cases.run_oracle_adam(oracle, wd, ams) == want, name
