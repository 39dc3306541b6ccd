"""Random programs: every one must lower and JIT-compile, and the oracle must run it (host only)."""
import importlib

import numpy as np
import pytest

import fuzz_programs
from oracle.oracle import OracleDevice

adb = importlib.import_module("autodiff-ir-rust_b200")


class _Both(OracleDevice):
    fused_sums = 0

    def execute(self, proc, dep):
        adb.devices.lower_check(proc, dep)
        # the same program with sums folded into element-wise kernels whatever their size
        plan = adb.devices.lower_check(proc, dep, flags=adb.devices.FLAG_FUSE_SMALL_SUMS)
        _Both.fused_sums += plan.count("    sum v")
        super().execute(proc, dep)


@pytest.mark.parametrize("seed", range(40))
def test_random_program_lowers(seed):
    out = fuzz_programs.build(seed, exact=seed % 2 == 0)(_Both())
    for v in out.values():
        assert not v.is_none


def test_some_random_programs_reach_the_sum_fusion():
    """Runs after the parametrised cases above (same module, collected in order)."""
    assert _Both.fused_sums >= 5
