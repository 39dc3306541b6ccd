"""Random programs, B200 against the CPU oracle."""
import numpy as np
import pytest

import fuzz_programs
from helpers import adb, oracle, run_both, assert_exact, assert_rel

pytestmark = pytest.mark.gpu
_small = None


def _fuse_small():
    """A handle that folds sums into element-wise kernels at any size, so that these small programs reach that path."""
    global _small
    if _small is None:
        _small = adb.devices.B200(0, flags=adb.devices.FLAG_FUSE_SMALL_SUMS)
    return _small


@pytest.mark.parametrize("seed", range(60))
def test_exact_programs_agree_bit_for_bit(seed):
    want, got = run_both(fuzz_programs.build(seed, exact=True))
    for k in want:
        assert_exact(k, got[k], want[k])


@pytest.mark.parametrize("seed", range(100, 160))
def test_float_programs_agree(seed):
    with np.errstate(all="ignore"):
        want, got = run_both(fuzz_programs.build(seed, exact=False))
    for k in want:
        w = np.asarray(want[k].data, np.float64)
        if not np.isfinite(w).all():
            continue   # overflow somewhere in the chain: nothing meaningful to compare
        assert_rel(k, got[k], want[k], 1e-4)


@pytest.mark.parametrize("seed", list(range(60)) + list(range(100, 160)))
def test_programs_agree_with_sums_fused_at_any_size(seed):
    exact = seed < 100
    prog = fuzz_programs.build(seed, exact=exact)
    with np.errstate(all="ignore"):
        want, got = prog(oracle()), prog(_fuse_small())
    for k in want:
        if exact:
            assert_exact(k, got[k], want[k])
        elif np.isfinite(np.asarray(want[k].data, np.float64)).all():
            assert_rel(k, got[k], want[k], 1e-4)
