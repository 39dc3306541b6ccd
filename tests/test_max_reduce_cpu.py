"""Row maximum (`Max`, an IR extension beside `Sum`): the CPU oracle against numpy for every axis, the gradient
mask, and the lowering (generated kernels compile for sm_100a; the data-parallel rewrite keeps a maximum along a
feature axis local and refuses one along the sharded batch)."""
import importlib

import numpy as np
import pytest

from oracle.oracle import OracleDevice

adb = importlib.import_module("autodiff-ir-rust_b200")
ad = adb.autodiff
RNG = np.random.default_rng(17)


def max_program(dev, x, shape, axis):
    ad.set_device(dev)
    t = ad.tensor(x, shape)
    m = t.max(axis)
    total = m
    while len(total.dim()) > 1:
        total = total.sum(len(total.dim()) - 1)
    total = total.sum(0)
    total.forward()
    total.backward()
    mv = m.forward()
    mv.keep()
    ad.execute()
    return {"max": mv.get(), "grad": t.grad().get()}


@pytest.mark.parametrize("shape,axis", [([7], 0), ([4, 6], 0), ([4, 6], 1), ([3, 5, 4], 0), ([3, 5, 4], 1), ([3, 5, 4], -1)])
def test_max_on_the_oracle(shape, axis):
    x = RNG.standard_normal(int(np.prod(shape))).astype(np.float32)
    out = max_program(OracleDevice(), x, shape, axis)
    X = x.reshape(shape)
    want = X.max(axis)
    np.testing.assert_array_equal(np.asarray(out["max"].data).reshape(want.shape), want)
    mask = (X == X.max(axis, keepdims=True)).astype(np.float32)
    np.testing.assert_array_equal(np.asarray(out["grad"].data).reshape(shape), mask)


def test_max_lowers_and_compiles():
    class LowerOnly(OracleDevice):
        def execute(self, proc, dep):
            self.plan = adb.devices.lower_check(proc, dep, with_source=True)
            super().execute(proc, dep)
    dev = LowerOnly()
    x = RNG.standard_normal(64 * 40).astype(np.float32)
    max_program(dev, x, [64, 40], 1)
    assert "reduce(max)" in dev.plan and "fmaxf" in dev.plan


def test_data_parallel_rewrite_keeps_feature_maxima_local_and_refuses_batch_maxima():
    class Capture:
        def ir_callback(self, irb): pass
        def dot_prod_shape(self, a, b): return [a[0], b[1]]
        def execute(self, proc, dep): self.blob = adb.ir.serialize(proc, dep, inline_limit=1 << 30)[0]
        def get_tensor(self, id_): return adb.autodiff.ValueData([1], np.zeros(1, np.float32), id_, False)
    x = RNG.standard_normal(8 * 6).astype(np.float32)

    def trace(axis):
        cap = Capture()
        ad.set_device(cap)
        m = ad.tensor(x, [8, 6]).max(axis).forward()
        m.keep()
        ad.execute()
        return cap.blob
    adb.devices.shard_ir(trace(1), 0, 2, 8)           # per-row maxima of a batch-sharded tensor: fine
    with pytest.raises(adb.devices.AdbError):
        adb.devices.shard_ir(trace(0), 0, 2, 8)       # maximum over the batch axis
