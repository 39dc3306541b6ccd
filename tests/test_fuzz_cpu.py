"""Random programs: every one must lower and JIT-compile, and the oracle must run it (host only)."""
import importlib

import numpy as np
import pytest

import fuzz_programs
from oracle.oracle import OracleDevice

adb = importlib.import_module("autodiff-ir-rust_b200")


class _Both(OracleDevice):
    def execute(self, proc, dep):
        adb.devices.lower_check(proc, dep)
        super().execute(proc, dep)


@pytest.mark.parametrize("seed", range(40))
def test_random_program_lowers(seed):
    out = fuzz_programs.build(seed, exact=seed % 2 == 0)(_Both())
    for v in out.values():
        assert not v.is_none
