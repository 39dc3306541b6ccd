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


def c2_float64(inp, rows, cols):
    """Config 2 in float64 with, per element, the scale an fp32 evaluation's error is measured in.

    Returns {"a_grad": (value, sigma), "b_grad": (value, sigma)}.  sigma_i = eps32 x (the magnitude of every term of
    the gradient, each weighted by how much its argument's rounding is amplified): the gradient is a sum of three
    terms that can cancel, exp(-a) is evaluated as exp2(-a log2 e) (its relative error grows with |a|), the sigmoid's
    argument a b + bias + 3 carries an absolute rounding error of eps (|a b| + 4), and cos(x) is evaluated as
    sin(pi/2 - x) (absolute argument error eps (|x| + 4)).  An fp32 chain built from <= 2-ulp primitives stays within a
    small multiple of sigma at EVERY element, including those far below the tensor's maximum."""
    eps = float(np.finfo(np.float32).eps)
    a = np.asarray(inp["a"], np.float64).reshape(rows, cols)
    b = np.asarray(inp["b"], np.float64).reshape(rows, cols)
    z = a * b + np.asarray(inp["bias"], np.float64)[None, :] + 3.0
    S = 1.0 / (1.0 + np.exp(-z))
    dS = S * (1.0 - S)
    E = np.exp(-a)
    R = 1.0 / (1.0 + b * b)
    amp = 8.0 + 2.0 * np.abs(a * b) + 2.0 * np.abs(a)
    a1, a2, a3 = 2.0 * S * dS * b * E, -S * S * E, np.sin(a) * R
    ga = a1 + a2 + a3
    sa = eps * ((np.abs(a1) + np.abs(a2)) * amp + 6.0 * np.abs(a3) + (np.abs(a) + 4.0) * R)
    b1, b2, b3 = 2.0 * S * dS * a * E, np.cos(b), np.cos(a) * 2.0 * b * R * R
    gb = b1 + b2 + b3
    sb = eps * (np.abs(b1) * amp + 4.0 * np.abs(b2) + (np.abs(b) + 4.0) + 8.0 * np.abs(b3) + (np.abs(a) + 4.0) * np.abs(2.0 * b * R * R))
    return {"a_grad": (ga, sa), "b_grad": (gb, sb)}


def assert_chain_per_element(name, got, want, ref64, sigma):
    """Per-element bound for a fused chain: at EVERY element the device's distance from float64 stays within one
    error unit of that element (sigma, see `c2_float64`) and within three times the oracle's own worst distance; the
    oracle (glibc primitives, <= 1 ulp each) sits at about 0.3 units, which also checks the scale."""
    g = np.asarray(got.data, np.float64).reshape(ref64.shape)
    w = np.asarray(want.data, np.float64).reshape(ref64.shape)
    rd, ro = np.abs(g - ref64) / sigma, np.abs(w - ref64) / sigma
    worst_d, worst_o = float(rd.max()), float(ro.max())
    assert worst_o <= 0.6, f"{name}: the oracle itself is {worst_o:.2f} error units from float64 (scale too tight?)"
    assert worst_d <= max(3.0 * worst_o, 1.0), (f"{name}: {worst_d:.2f} error units from float64 at element {int(rd.argmax())} "
                                                f"(oracle: {worst_o:.2f})")
    return worst_d, worst_o
