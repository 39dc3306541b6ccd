"""Row reductions chained with the element-wise work that uses them (one `adb_rows_*` kernel: one block per row, the
input streamed from HBM once): layer normalisation, RMS normalisation, a max-shifted softmax, and the same with the
per-row results kept -- B200 against the CPU oracle, fused against unfused."""
import numpy as np
import pytest

from helpers import ad, adb, nn, b200, oracle, run_both, assert_exact, assert_rel

pytestmark = pytest.mark.gpu
RNG = np.random.default_rng(41)


def _rows_kernels(dev):
    return dev.dump_plan().count("adb_rows_")


def _layernorm(P, Q):
    x = (RNG.standard_normal(P * Q) * 3 + 1).astype(np.float32)

    def prog(dev):
        ad.set_device(dev)
        ad.eager_dep_opt()
        y = nn.LayerNorm(Q).f(ad.tensor(x, [P, Q])).forward()
        y.keep()
        ad.execute()
        return {"y": y.get()}
    return prog


@pytest.mark.parametrize("P,Q", [(4096, 1024), (300, 4096), (1000, 520), (512, 8192)])
def test_layer_norm_is_one_kernel(P, Q):
    want, got = run_both(_layernorm(P, Q))
    assert _rows_kernels(b200()) == 1, b200().dump_plan()
    assert b200().stats()["kernel_launches"] == 1
    assert_rel("y", got["y"], want["y"], 1e-4)


def test_rms_norm_and_softmax_with_row_maximum():
    P, Q = 2048, 768
    x = (RNG.standard_normal(P * Q) * 4).astype(np.float32)

    def prog(dev):
        ad.set_device(dev)
        ad.eager_dep_opt()
        t = ad.tensor(x, [P, Q])
        r = nn.RMS(Q).f(t).forward()
        m = t.max(1)                                            # [P]
        e = (t - m.unsqueeze(-1).broadcast(-1, Q)).exp()
        sm = (e * e.sum(1).recip().unsqueeze(-1).broadcast(-1, Q)).forward()
        r.keep()
        sm.keep()
        ad.execute()
        return {"rms": r.get(), "softmax": sm.get()}
    want, got = run_both(prog)
    # both outputs and all three row reductions (sum of squares, maximum, sum of exponentials) share one kernel
    assert _rows_kernels(b200()) == 1, b200().dump_plan()
    assert_rel("rms", got["rms"], want["rms"], 1e-4)
    assert_rel("softmax", got["softmax"], want["softmax"], 1e-4)
    rows = np.asarray(got["softmax"].data, np.float64).reshape(P, Q).sum(1)
    assert np.abs(rows - 1.0).max() < 1e-4


def test_row_results_are_still_written_and_the_fused_kernel_matches_the_unfused_program():
    P, Q = 1500, 640
    x = RNG.standard_normal(P * Q).astype(np.float32)

    def prog(dev):
        ad.set_device(dev)
        ad.eager_dep_opt()
        t = ad.tensor(x, [P, Q])
        mean = t.mean(1)
        c = t - mean.unsqueeze(-1).broadcast(-1, Q)
        var = c.pow2().mean(1)
        y = (c * (var + 1e-5).sqrt().recip().unsqueeze(-1).broadcast(-1, Q)).forward()
        mv, vv = mean.forward(), var.forward()
        for v in (y, mv, vv):
            v.keep()
        ad.execute()
        return {"y": y.get(), "mean": mv.get(), "var": vv.get()}
    fused = prog(b200())
    assert _rows_kernels(b200()) == 1, b200().dump_plan()
    plain = adb.devices.B200(0, flags=adb.devices.FLAG_NO_FUSION)
    try:
        ref = prog(plain)
    finally:
        plain.close()
    want = prog(oracle())
    for k in ("y", "mean", "var"):
        assert_rel(k, fused[k], want[k], 1e-4)
        assert_rel(k + " (unfused)", fused[k], ref[k], 1e-5)


def test_few_long_rows_keep_the_split_reduce_kernels():
    """64 rows cannot fill the GPU with one block per row: the reductions stay two-pass split kernels."""
    want, got = run_both(_layernorm(64, 16384))
    assert _rows_kernels(b200()) == 0
    assert_rel("y", got["y"], want["y"], 1e-4)


_small = None


def _small_dev():
    global _small
    if _small is None:
        _small = adb.devices.B200(0, flags=adb.devices.FLAG_FUSE_SMALL_SUMS)
    return _small


@pytest.mark.parametrize("seed", range(40))
def test_random_row_chains_at_small_sizes(seed):
    """Random two- and three-stage chains (sum / max along the rows, each stage using the results before it) on
    small, ragged shapes, with the size thresholds of the fusion switched off."""
    rng = np.random.default_rng(1000 + seed)
    P, Q = int(rng.integers(1, 40)), int(rng.integers(1, 70))
    x = rng.standard_normal(P * Q).astype(np.float32)
    w = rng.standard_normal(Q).astype(np.float32)
    kinds = [int(k) for k in rng.integers(0, 2, 3)]
    n_stage = int(rng.integers(2, 4))
    keep_rows = bool(rng.integers(0, 2))

    def prog(dev):
        ad.set_device(dev)
        ad.eager_dep_opt()
        t = ad.tensor(x, [P, Q])
        tw = ad.tensor(w, [Q]).view([1, Q]).broadcast(0, P)
        cur = t * tw
        rows = []
        for s in range(n_stage - 1):
            r = cur.max(1) if kinds[s] else (cur * cur).sum(1)
            rows.append(r)
            b = r.unsqueeze(-1).broadcast(-1, Q)
            cur = (t - b) * 0.5 if kinds[s] else t * (b + 1.0).recip()
        y = (cur + tw).forward()
        y.keep()
        outs = {"y": y}
        if keep_rows:
            for i, r in enumerate(rows):
                v = r.forward()
                v.keep()
                outs[f"r{i}"] = v
        ad.execute()
        return {k: v.get() for k, v in outs.items()}
    want, got = prog(oracle()), prog(_small_dev())
    for k in want:
        assert_rel(k, got[k], want[k], 1e-4)


def test_random_row_chains_do_fuse():
    """(collected after the parametrised cases) the last of them ran on the handle with the thresholds off"""
    assert _small is not None
