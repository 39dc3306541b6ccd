"""Full benchmark sizes, checked through properties that do not need the CPU oracle to finish the whole
problem: the element-wise programs are independent per row, so a band of rows run on the oracle must
match the same rows of the full run; x.grad of config 3 is piecewise constant; loop counts are exact."""
import numpy as np
import pytest

from helpers import adb, b200, oracle, assert_rel

pytestmark = pytest.mark.gpu
cfg = adb.configs


def test_c2_full_size_rows_match_oracle_on_a_band():
    rows = cols = 8192
    inp = cfg.c2_inputs(rows, cols)
    got = cfg.c2_fused_elementwise(b200(), rows=rows, cols=cols, inputs=inp)
    band = slice(4000, 4064)
    sub = {"a": inp["a"].reshape(rows, cols)[band].reshape(-1).copy(), "b": inp["b"].reshape(rows, cols)[band].reshape(-1).copy(),
           "bias": inp["bias"]}
    want = cfg.c2_fused_elementwise(oracle(), rows=64, cols=cols, inputs=sub)
    for k in ("a_grad", "b_grad"):
        g = np.asarray(got[k].data).reshape(rows, cols)[band]
        w = np.asarray(want[k].data).reshape(64, cols)
        err = np.abs(g.astype(np.float64) - w).max() / np.abs(w).max()
        assert err < 2e-5, (k, err)
    # the loss is the sum of every element of y; the bias gradient the column sum of one factor of a.grad
    a = inp["a"].astype(np.float64)
    b = inp["b"].astype(np.float64)
    z = a * b + np.tile(inp["bias"].astype(np.float64), rows) + 3.0
    s = 1.0 / (1.0 + np.exp(-z))
    y = s * s * np.exp(-a) + np.sin(b) - np.cos(a) / (1.0 + b * b)
    assert abs(float(got["loss"].data[0]) - y.sum()) / abs(y.sum()) < 1e-4
    dz = 2.0 * s * s * (1.0 - s) * np.exp(-a)
    bias_grad = dz.reshape(rows, cols).sum(0)
    err = np.abs(np.asarray(got["bias_grad"].data, np.float64) - bias_grad).max() / np.abs(bias_grad).max()
    assert err < 1e-4, err


def test_c3_full_size_structure():
    batch, n = 64, 1024
    inp = cfg.c3_inputs(batch, n)
    got = cfg.c3_reduce_movement(b200(), batch=batch, n=n, inputs=inp)
    x = inp["x"].reshape(batch, n, n).astype(np.float64)
    s_ref = x.sum(2)
    s = np.asarray(got["s"].data, np.float32).reshape(batch, n)
    assert np.abs(s - s_ref).max() / np.abs(s_ref).max() < 1e-4
    c = np.concatenate([s, s * np.float32(2)], 0)[batch // 2: batch // 2 + batch]
    np.testing.assert_array_equal(np.asarray(got["slice"].data).reshape(batch, n), c)          # concat + slice: bit-exact
    mask = (c > 0).astype(np.float32)
    np.testing.assert_array_equal(np.asarray(got["mask"].data), mask.reshape(-1))             # compare + view: bit-exact
    np.testing.assert_array_equal(np.asarray(got["row_all"].data), (mask.sum(1) == n).astype(np.float32))
    xg = np.asarray(got["x_grad"].data).reshape(batch, n, n)
    np.testing.assert_array_equal(xg[: batch // 2], np.full((batch // 2, n, n), 2.0, np.float32))   # rows that came through 2*s
    np.testing.assert_array_equal(xg[batch // 2:], np.full((batch // 2, n, n), 1.0, np.float32))
    assert b200().stats()["kernel_launches"] <= 12          # ~26 000 IR commands collapse to a handful of kernels


def test_c5_mid_size_against_float64():
    n, iters = 1024, 6
    inp = cfg.c5_inputs(n)
    got = cfg.c5_dot_loop(b200(), n=n, max_iters=iters, inputs=inp)
    assert float(got["iters"].data[0]) == iters
    a = inp["a"].reshape(n, n).astype(np.float64)
    b = inp["b"].reshape(n, n).astype(np.float64)
    x = np.zeros((n, n))
    for _ in range(iters):
        x = x - 0.01 * (a @ x - b)
    err = np.abs(np.asarray(got["x"].data).reshape(n, n) - x).max() / np.abs(x).max()
    assert err < 1e-4, err
    assert b200().stats()["tc_gemm_launches"] == 3 * iters + 1
