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


_steps = None


def _dot_steps():
    """A handle on which the tiny dot products of these programs stay dot-product steps (by default a product of a few
    multiply-adds is lowered as an element-wise expression and never reaches the dot kernels)."""
    global _steps
    if _steps is None:
        _steps = adb.devices.B200(0, flags=adb.devices.FLAG_NO_TINY_DOT)
    return _steps


@pytest.mark.parametrize("seed", range(60))
def test_exact_programs_agree_bit_for_bit(seed):
    want, got = run_both(fuzz_programs.build(seed, exact=True))
    for k in want:
        assert_exact(k, got[k], want[k])


@pytest.mark.parametrize("seed", list(range(0, 60, 3)) + list(range(100, 160, 3)))
def test_programs_agree_with_tiny_products_as_dot_product_steps(seed):
    exact = seed < 100
    prog = fuzz_programs.build(seed, exact=exact)
    with np.errstate(all="ignore"):
        want, got = prog(oracle()), prog(_dot_steps())
    for k in want:
        if exact:
            assert_exact(k, got[k], want[k])
        elif np.isfinite(np.asarray(want[k].data, np.float64)).all():
            assert_rel(k, got[k], want[k], 1e-4)


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


@pytest.mark.parametrize("seed", list(range(0, 60, 2)) + list(range(100, 160, 2)))
def test_replayed_graphs_agree_with_the_first_execute(seed):
    """The first execute of a program launches its kernels one by one; from the second on the cached plan is captured as
    a CUDA graph in which kernels that do not depend on one another sit on different streams, and replayed.  Every
    execute must give the oracle's result."""
    from helpers import b200
    exact = seed < 100
    prog = fuzz_programs.build(seed, exact=exact)
    with np.errstate(all="ignore"):
        want = prog(oracle())
        for rep in range(3):
            got = prog(b200())
            for k in want:
                if exact:
                    assert_exact(f"{k} (execute {rep})", got[k], want[k])
                elif np.isfinite(np.asarray(want[k].data, np.float64)).all():
                    assert_rel(f"{k} (execute {rep})", got[k], want[k], 1e-4)


@pytest.mark.parametrize("chunk", range(6))
def test_raw_ir_programs_agree_bit_for_bit(chunk):
    """Programs written directly as IR commands (ids reused as results, op-assigns on views, views made inside
    branches, loops that run zero times, products onto their own operands): exact integer arithmetic, so the device
    must reproduce the oracle bit for bit -- or refuse the program with the documented reason."""
    from helpers import b200
    refused = 0
    for seed in range(chunk * 25, chunk * 25 + 25):
        prog = fuzz_programs.build_raw(seed)
        want = prog(oracle())
        try:
            got = prog(b200())
            got_steps = prog(_dot_steps())
        except adb.devices.AdbError as e:
            assert "is a view when control flow joins" in str(e), str(e)
            refused += 1
            continue
        for k in want:
            assert_exact(k, got[k], want[k])
            assert_exact(k + " (dot-product steps)", got_steps[k], want[k])
    assert refused <= 10


@pytest.mark.parametrize("chunk", range(3))
def test_raw_ir_programs_with_sums_rows_and_concats(chunk):
    """The richer raw-IR mix (row sums broadcast back, repeated rows, halves of a concat as alias chains), two executes
    each (the second one replays the captured graph)."""
    from helpers import b200
    refused = 0
    for seed in range(chunk * 25, chunk * 25 + 25):
        prog = fuzz_programs.build_raw(seed, rich=True)
        want = prog(oracle())
        try:
            runs = [prog(b200()), prog(b200())]
        except adb.devices.AdbError as e:
            assert "is a view when control flow joins" in str(e), str(e)
            refused += 1
            continue
        for got in runs:
            for k in want:
                assert_exact(k, got[k], want[k])
    assert refused <= 12


@pytest.mark.parametrize("n", [96, 512])
def test_dot_product_written_onto_its_own_operand(n):
    """`DotProduct v w -> v` with more than one tile per operand (512: tensor-core kernel, 96: CUDA-core kernel), at top
    level and inside a loop."""
    from helpers import b200
    rng = np.random.default_rng(n)
    V = rng.integers(-2, 3, n * n).astype(np.float32)
    W = (rng.integers(0, 3, n * n) == 0).astype(np.float32) * rng.choice([-1.0, 1.0], n * n).astype(np.float32)
    P = adb.ir.IRProcedure
    main = P("main")
    main.push(("CreateMat", V, [n, n], "v"))
    main.push(("CreateMat", W, [n, n], "w"))
    main.push(("CreateMat", np.array([2.0], np.float32), [1], "c"))
    main.push(("CreateConstant", -1.0, "k", [1]))
    main.push(("CreateConstant", 1.0 / n, "s", [n, n]))
    main.push(("DotProduct", "v", "w", "v"))
    body = P("body")
    body.push(("ElwMultiplyEq", "v", "s"))
    body.push(("DotProduct", "w", "v", "v"))
    body.push(("ElwAddEq", "c", "k"))
    main.push(("While", "c", body))
    res = []
    for dev in (oracle(), b200()):
        dev.execute(main, ["v"])
        res.append(dev.get_tensor("v"))
    assert_rel("v", res[1], res[0], 1e-4)
