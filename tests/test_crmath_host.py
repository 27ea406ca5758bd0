"""CPU: repdl_b200/csrc/crmath.cuh compiled for the host (tests/crmath_host_check.cpp).

exp / log against glibc for ALL 2^32 fp32 bit patterns (a few seconds per function on 8 cores; the
same run with every input forced through the slow path, -DCRM_FORCE_SLOW=1, takes minutes and was
done once), and the scalar division of the
streaming kernel against the IEEE quotient: every x whose quotient is subnormal, where rounding
midpoints are reachable (x = 147 * 2^-149, d = 98 is one), plus a strided sweep of the rest.
"""
import os
import subprocess
import tempfile

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def chk():
    out = os.path.join(tempfile.mkdtemp(prefix="repdl_crm_"), "chk")
    subprocess.run(["/usr/bin/g++", "-O2", "-ffp-contract=off", "-mfma", "-fopenmp", "-o", out,
                    os.path.join(HERE, "crmath_host_check.cpp")], check=True)

    def run(*args):
        r = subprocess.run([out, *map(str, args)], capture_output=True, text=True)
        checked, bad = map(int, r.stdout.strip().split("\n")[-1].split()[:2])
        return checked, bad, r.stdout
    return run


@pytest.mark.parametrize("fn", ["exp", "log"])
def test_exp_log_every_input(chk, fn):
    checked, bad, out = chk(fn, 1, 0)
    assert checked == 1 << 32 and bad == 0, out


@pytest.mark.parametrize("d", [98.0, 150.0, 154.0, 182.0, 186.0, 198.0, 10.0, 3.0, -7.0, 1.0e-3, 3.0e38])
def test_scalar_division_equals_the_ieee_quotient(chk, d):
    # stride 1 over the low 2^28 patterns would be the dense sweep of the subnormal quotients; the
    # host loop walks all 2^32 patterns in blocks, so use a small odd stride for everything
    checked, bad, out = chk("div", 13, 5, d)
    assert checked > 300_000_000 and bad == 0, out
