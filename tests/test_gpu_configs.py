"""The five benchmark programs at sizes the CPU oracle finishes in seconds, B200 against oracle.

Tolerances follow the stated bars: comparisons / .all() / indexing / permute / concat bit-exact,
element-wise chains a few ulp per primitive, reductions and dot products 1e-4 relative.
"""
import numpy as np
import pytest

from helpers import adb, run_both, assert_exact, assert_rel, b200

pytestmark = pytest.mark.gpu
cfg = adb.configs


def test_c1_readme_mlp():
    want, got = run_both(cfg.c1_readme_mlp)
    for k in want:
        assert_rel(k, got[k], want[k], 1e-4)


@pytest.mark.parametrize("rows,cols", [(64, 128), (257, 96), (512, 1024)])
def test_c2_fused_elementwise(rows, cols):
    want, got = run_both(cfg.c2_fused_elementwise, rows=rows, cols=cols)
    # gradients are ~60 primitives deep (exp2 / sin at 2 ulp each, amplified by the chain)
    assert_rel("a_grad", got["a_grad"], want["a_grad"], 2e-5)
    assert_rel("b_grad", got["b_grad"], want["b_grad"], 2e-5)
    assert_rel("bias_grad", got["bias_grad"], want["bias_grad"], 1e-4)
    assert_rel("loss", got["loss"], want["loss"], 1e-4)


@pytest.mark.parametrize("batch,n", [(8, 16), (16, 64), (64, 128)])
def test_c3_reduce_movement(batch, n):
    want, got = run_both(cfg.c3_reduce_movement, batch=batch, n=n)
    assert_rel("s", got["s"], want["s"], 1e-4)
    assert_exact("x_grad", got["x_grad"], want["x_grad"])
    # the integer-like stages are exact given the device's own row sums
    s = np.asarray(got["s"].data, np.float32).reshape(batch, n)
    c = np.concatenate([s, s * np.float32(2.0)], 0)[batch // 2: batch // 2 + batch]
    np.testing.assert_array_equal(np.asarray(got["slice"].data).reshape(batch, n), c)
    mask = (c > 0).astype(np.float32)
    np.testing.assert_array_equal(np.asarray(got["mask"].data), mask.reshape(-1))
    np.testing.assert_array_equal(np.asarray(got["row_all"].data), (mask.sum(1) == n).astype(np.float32))
    flips = int(np.count_nonzero(np.asarray(got["mask"].data) != np.asarray(want["mask"].data)))
    assert flips == 0, f"{flips} mask entries differ from the oracle (row sums within 1e-4 of zero?)"


def test_c4_mlp_train_small():
    kw = dict(batch=64, widths=(32, 48, 48, 32, 8), steps=3, lr=1e-2)
    want, got = run_both(cfg.c4_mlp_train, **kw)
    for k in want:
        assert_rel(k, got[k], want[k], 1e-4)
    st = b200().stats()
    assert st["while_iterations"] == 3


@pytest.mark.parametrize("n,iters", [(32, 5), (96, 4)])
def test_c5_dot_loop(n, iters):
    want, got = run_both(cfg.c5_dot_loop, n=n, max_iters=iters)
    assert_exact("iters", got["iters"], want["iters"])
    assert float(got["iters"].data[0]) == iters
    for k in ("x", "a_grad", "x_grad"):
        assert_rel(k, got[k], want[k], 1e-4)
