"""The five benchmark programs at sizes the CPU oracle finishes in seconds, B200 against oracle.

Tolerances follow the stated bars: comparisons / .all() / indexing / permute / concat bit-exact,
element-wise chains a few ulp per primitive, reductions and dot products 1e-4 relative.
"""
import numpy as np
import pytest

from helpers import adb, run_both, assert_exact, assert_rel, b200, oracle, c2_float64, assert_chain_per_element

pytestmark = pytest.mark.gpu
cfg = adb.configs


def test_c1_readme_mlp():
    want, got = run_both(cfg.c1_readme_mlp)
    for k in want:
        assert_rel(k, got[k], want[k], 1e-4)


@pytest.mark.parametrize("rows,cols", [(64, 128), (257, 96), (512, 1024)])
def test_c2_fused_elementwise(rows, cols):
    inp = cfg.c2_inputs(rows, cols)
    want, got = run_both(cfg.c2_fused_elementwise, rows=rows, cols=cols, inputs=inp)
    # gradients are ~60 primitives deep: bounded element by element against float64, in units of each element's own
    # conditioning (not relative to the tensor's maximum, which would say nothing about the small elements)
    ref = c2_float64(inp, rows, cols)
    for k in ("a_grad", "b_grad"):
        assert_chain_per_element(k, got[k], want[k], *ref[k])
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


@pytest.mark.parametrize("lr", [1e-3, 10.0], ids=["lr-of-the-benchmark", "lr-that-moves-the-weights"])
def test_c4_benchmark_widths_against_the_oracle(lr):
    """Config 4 at the benchmark's layer widths (4096-8192-8192-4096-1000; every dot product on the tensor-core
    kernels, N = 1000 ragged tiles included), batch 512, two steps: loss and all eight parameters within 1e-4 of the
    CPU oracle.  At the benchmark's lr of 1e-3 two steps move the first layers by about one ulp, so that run says
    little about their gradients; the second run uses lr 10, where every parameter moves by thousands of ulps, and
    also bounds the UPDATE each parameter received (2e-3 of the largest update)."""
    kw = dict(batch=512, widths=cfg.C4_WIDTHS, steps=2, lr=lr)
    inp = cfg.c4_inputs(batch=512, widths=cfg.C4_WIDTHS)
    want = cfg.c4_mlp_train(oracle(), inputs=inp, **kw)
    got = cfg.c4_mlp_train(b200(), inputs=inp, **kw)
    st = b200().stats()
    assert st["tc_gemm_launches"] == st["gemm_launches"] == 2 * 11, st
    for k in want:
        assert_rel(k, got[k], want[k], 1e-4)
        if k == "loss" or lr < 1.0:
            continue
        w0 = np.asarray(inp[k], np.float64)
        du_w = np.asarray(want[k].data, np.float64) - w0
        du_g = np.asarray(got[k].data, np.float64) - w0
        assert np.abs(du_w).max() > 1000 * 6e-8 * np.abs(w0).max(), k      # the parameter really moved
        err = np.abs(du_g - du_w).max() / np.abs(du_w).max()
        assert err < 2e-3, (k, err)


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
