"""Shared helpers for the parity tests: run one traced program on the CPU oracle and on the B200
backend and compare the kept tensors."""
from __future__ import annotations

import importlib

import numpy as np

adb = importlib.import_module("autodiff-ir-rust_b200")
ad = adb.autodiff
nn = adb.nn

_device = None


def b200():
    """One backend handle per test process (the reference also keeps one global device)."""
    global _device
    if _device is None:
        _device = adb.devices.B200(0)
    return _device


def oracle():
    from oracle.oracle import OracleDevice
    return OracleDevice()


def ulp_distance(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in units of fp32 spacing (monotone integer mapping of the bit patterns)."""
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)

    def key(x):
        i = x.view(np.int32).astype(np.int64)
        return np.where(i < 0, np.int64(-0x80000000) - i, i)
    d = np.abs(key(a) - key(b))
    both_nan = np.isnan(a) & np.isnan(b)
    return np.where(both_nan, 0, d)


def assert_exact(name, got, exp):
    g, e = np.asarray(got.data, np.float32), np.asarray(exp.data, np.float32)
    assert got.dim == exp.dim, f"{name}: dim {got.dim} != {exp.dim}"
    assert np.array_equal(g, e, equal_nan=True), f"{name}: {np.count_nonzero(g != e)} of {g.size} elements differ"


def assert_ulp(name, got, exp, max_ulp):
    g, e = np.asarray(got.data, np.float32), np.asarray(exp.data, np.float32)
    assert got.dim == exp.dim, f"{name}: dim {got.dim} != {exp.dim}"
    d = ulp_distance(g, e)
    worst = int(d.max()) if d.size else 0
    assert worst <= max_ulp, f"{name}: {worst} ulp at {int(d.argmax())}: got {g.flat[int(d.argmax())]!r} want {e.flat[int(d.argmax())]!r}"


def assert_rel(name, got, exp, tol):
    """max |got - exp| relative to the largest magnitude of the expected tensor."""
    g, e = np.asarray(got.data, np.float64), np.asarray(exp.data, np.float64)
    assert got.dim == exp.dim, f"{name}: dim {got.dim} != {exp.dim}"
    if g.size == 0:
        return
    scale = max(float(np.abs(e).max()), 1e-30)
    err = float(np.abs(g - e).max()) / scale
    assert err <= tol, f"{name}: relative error {err:.3e} > {tol:.1e}"


def run_both(program, **kw):
    """program(dev, **kw) -> {name: ValueData}; returns (oracle result, device result)."""
    want = program(oracle(), **kw)
    got = program(b200(), **kw)
    assert set(want) == set(got)
    return want, got
