"""Every element-wise primitive on its own, against the CPU oracle.

Tolerances: + * compare are bit-exact; exp2 / log2 / sin within 2 ulp (fp32), which is the bound stated
for element-wise ops; recip / sqrt within 1 ulp by default (special-function unit) and bit-exact on a handle
created with FLAG_EXACT_DIV.
"""
import numpy as np
import pytest

from helpers import ad, adb, oracle, run_both, assert_exact, assert_ulp

pytestmark = pytest.mark.gpu

N = 1 << 20
RNG = np.random.default_rng(7)


def _special():
    return np.asarray([0.0, -0.0, 1.0, -1.0, 0.5, 2.0, 1e-30, -1e-30, 1e30, -1e30, 3.1415927, 1e-45, 65504.0], np.float32)


def _data(kind):
    if kind == "normal":
        x = RNG.standard_normal(N).astype(np.float32) * 4
    elif kind == "wide":
        x = (RNG.standard_normal(N) * np.exp(RNG.uniform(-20, 20, N))).astype(np.float32)
    elif kind == "positive":
        x = np.exp(RNG.uniform(-40, 40, N)).astype(np.float32)
    elif kind == "exp":
        x = RNG.uniform(-120, 120, N).astype(np.float32)
    elif kind == "angle":
        x = RNG.uniform(-200, 200, N).astype(np.float32)
    s = _special()
    x[:s.size] = s
    return x


def _unary(method, x):
    def prog(dev):
        ad.set_device(dev)
        ad.eager_dep_opt()
        t = ad.tensor(x, [x.size])
        y = getattr(t, method)()
        y.forward()
        y.val().keep()
        ad.execute()
        return {"y": y.val().get()}
    return prog


@pytest.mark.parametrize("method,kind,ulp", [
    ("exp2", "exp", 2), ("log2", "positive", 2), ("sin", "angle", 2), ("sin", "normal", 2),
    ("recip", "wide", 1), ("sqrt", "wide", 1), ("recip", "positive", 1), ("sqrt", "positive", 1),
])
def test_unary(method, kind, ulp):
    x = _data(kind)
    with np.errstate(all="ignore"):
        want, got = run_both(_unary(method, x))
    if ulp == 0:
        assert_exact(method, got["y"], want["y"])
    else:
        assert_ulp(method, got["y"], want["y"], ulp)


@pytest.mark.parametrize("method,kind", [("recip", "wide"), ("sqrt", "wide"), ("recip", "positive")])
def test_division_is_correctly_rounded_on_request(method, kind):
    x = _data(kind)
    dev = adb.devices.B200(0, flags=adb.devices.FLAG_EXACT_DIV)
    try:
        with np.errstate(all="ignore"):
            want, got = _unary(method, x)(oracle()), _unary(method, x)(dev)
    finally:
        dev.close()
    assert_exact(method, got["y"], want["y"])


@pytest.mark.parametrize("op", ["add", "mul"])
def test_binary_bit_exact(op):
    a, b = _data("wide"), _data("normal")

    def prog(dev):
        ad.set_device(dev)
        ad.eager_dep_opt()
        ta, tb = ad.tensor(a, [a.size]), ad.tensor(b, [b.size])
        y = ta + tb if op == "add" else ta * tb
        y.forward()
        y.val().keep()
        ad.execute()
        return {"y": y.val().get()}
    want, got = run_both(prog)
    assert_exact(op, got["y"], want["y"])


@pytest.mark.parametrize("method", ["equal", "more_than", "less_than"])
def test_compare_bit_exact(method):
    a = _data("normal")
    b = a.copy()
    b[::3] += 1.0
    b[1::3] -= 1.0

    def prog(dev):
        ad.set_device(dev)
        ad.eager_dep_opt()
        ta, tb = ad.tensor(a, [a.size]), ad.tensor(b, [b.size])
        y = getattr(ta, method)(tb)
        y.forward()
        y.val().keep()
        ad.execute()
        return {"y": y.val().get()}
    want, got = run_both(prog)
    assert_exact(method, got["y"], want["y"])
    assert set(np.unique(got["y"].data)) <= {0.0, 1.0}


def test_mul_add_is_not_contracted():
    """a*b+c must round twice (the reference's kernels are separate multiplies and adds)."""
    a = RNG.standard_normal(N).astype(np.float32)
    b = RNG.standard_normal(N).astype(np.float32)
    c = (-(a.astype(np.float64) * b.astype(np.float64))).astype(np.float32)  # cancellation exposes an FMA

    def prog(dev):
        ad.set_device(dev)
        ad.eager_dep_opt()
        ta, tb, tc = (ad.tensor(v, [N]) for v in (a, b, c))
        y = ta * tb + tc
        y.forward()
        y.val().keep()
        ad.execute()
        return {"y": y.val().get()}
    want, got = run_both(prog)
    assert_exact("a*b+c", got["y"], want["y"])
    np.testing.assert_array_equal(np.asarray(want["y"].data), (a * b + c).astype(np.float32))
