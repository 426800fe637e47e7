"""Host-side exhaustive checks of the float identities behind the GPU requantisation
(megcc_b200/csrc/common.cuh: div_rn_by_const and round_clamp_s8). The C program is compiled
with strict IEEE flags and run in parallel slices; no GPU is involved."""
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def checker(tmp_path_factory):
    exe = str(tmp_path_factory.mktemp("requant_math") / "requant_math_check")
    subprocess.run(["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-o", exe,
                    os.path.join(HERE, "requant_math_check.c"), "-lm"], check=True)
    return exe


def _run_slices(exe, jobs):
    def one(args):
        r = subprocess.run([exe] + [str(a) for a in args], stdout=subprocess.PIPE, text=True)
        return r.returncode, r.stdout.strip()
    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        return list(pool.map(one, jobs))


def test_roundf_identity_holds_for_every_float(checker):
    """trunc(x + copysign(0.49999997f, x)) == roundf(x) on all 2^32 bit patterns below 2^31."""
    out = _run_slices(checker, [("roundf", i << 28, 1 << 28) for i in range(16)])
    assert all(rc == 0 and text.startswith("ok") for rc, text in out), out
    # finite floats below 2^31 in magnitude: exponents 0..157 of both signs
    assert sum(int(text.split()[1]) for _, text in out) == 2 * 158 * (1 << 23)


def test_division_by_constant_is_correctly_rounded(checker):
    """The three-instruction division equals RN(t / d) for the divisor list (34 fixed, 14
    pseudo-random), every mantissa of t at nine exponents, and around every int8 step."""
    out = _run_slices(checker, [("division", i * 4, 4) for i in range(12)])
    assert all(rc == 0 and text.startswith("ok") for rc, text in out), out
