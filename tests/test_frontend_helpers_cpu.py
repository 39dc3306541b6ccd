"""The two frontend helpers composed from existing primitives (mean-squared error, abs): values and gradients on the
CPU oracle against numpy, and the programs lower and compile for the B200 backend (host only)."""
import importlib

import numpy as np

from oracle.oracle import OracleDevice

adb = importlib.import_module("autodiff-ir-rust_b200")
ad, nn = adb.autodiff, adb.nn
RNG = np.random.default_rng(3)


def helper_program(dev, y, t, shape):
    ad.set_device(dev)
    ty, tt = ad.tensor(y, shape), ad.tensor(t, shape)
    loss = nn.mse_loss(ty, tt)
    loss.forward()
    loss.backward()
    a = ty.abs().forward()
    a.keep()
    loss.val().keep()
    ad.execute()
    return {"loss": loss.val().get(), "y_grad": ty.grad().get(), "t_grad": tt.grad().get(), "abs": a.get()}


def test_mse_and_abs_on_the_oracle():
    for shape in ([30], [6, 5], [2, 3, 5]):
        y = RNG.standard_normal(30).astype(np.float32)
        t = RNG.standard_normal(30).astype(np.float32)
        out = helper_program(OracleDevice(), y, t, shape)
        assert out["loss"].dim == [1]
        np.testing.assert_allclose(out["loss"].data[0], np.mean((y - t) ** 2), rtol=1e-6)
        np.testing.assert_allclose(out["y_grad"].data, 2 * (y - t) / 30, rtol=1e-5, atol=1e-7)
        np.testing.assert_allclose(out["t_grad"].data, -2 * (y - t) / 30, rtol=1e-5, atol=1e-7)
        np.testing.assert_array_equal(out["abs"].data, np.abs(y))


def test_helpers_lower_for_the_device():
    class LowerOnly(OracleDevice):
        def execute(self, proc, dep):
            self.plan = adb.devices.lower_check(proc, dep)
            super().execute(proc, dep)
    dev = LowerOnly()
    y = RNG.standard_normal(64 * 48).astype(np.float32)
    helper_program(dev, y, y[::-1].copy(), [64, 48])
    assert dev.plan.startswith("plan:")


def test_hash_generator_is_the_same_on_numpy_and_torch_and_keyed_by_global_index():
    """The benchmark's batch generator: integer hashing only, so the numpy version (configs.hash_normal) and the torch
    version (bench.hash_normal_torch) give the same bits, and any slice of a tensor can be drawn on its own -- what lets
    every rank of every N train on the same global batch."""
    import importlib
    import os
    import sys
    import numpy as np
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench
    adb = importlib.import_module("autodiff-ir-rust_b200")
    cfg = adb.configs
    whole = cfg.hash_normal(3, 0, 50_000)
    part = cfg.hash_normal(3, 0, 10_000, start=20_000)
    np.testing.assert_array_equal(whole[20_000:30_000], part)
    t = bench.hash_normal_torch(cfg, 3, 0, 20_000, 10_000, "cpu").numpy()
    np.testing.assert_array_equal(t, part)
    assert not np.array_equal(cfg.hash_normal(3, 1, 1000), cfg.hash_normal(3, 0, 1000))
    big = cfg.hash_normal(7, 2, 1 << 20)
    assert abs(float(big.mean())) < 5e-3 and abs(float(big.std()) - 1.0) < 5e-3
