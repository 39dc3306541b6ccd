"""The allocation-free row-sum entry point against the regular path.

Some callers cannot allocate device memory at the point where they need a result (a host callback, a
loop that must not synchronise, a process whose memory is owned by another pool).  For them the
library exports `adb_row_sum_noalloc`, whose scratch is a fixed array inside the library.  This test
calls it through the C-ABI twice in a row -- the second call with a different shape, so stale
scratch contents would show -- and checks both results against `adb_execute` running the same row sum,
within the tolerance used for reductions everywhere else (1e-4 relative).

The file name sorts last on purpose: a run that stops at the first failure has then already run every
other test.
"""
import importlib

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

adb = importlib.import_module("autodiff-ir-rust_b200")
ad = adb.autodiff


def _regular_row_sum(dev, x, rows, length):
    ad.set_device(dev)
    ad.eager_dep_opt()
    t = ad.tensor(x, [rows, length])
    s = t.sum(1)
    s.forward()
    s.val().keep()
    ad.execute()
    return np.asarray(s.val().get().data, np.float32)


def _noalloc_row_sum(x, rows, length):
    import torch
    d_in = torch.from_numpy(x).cuda()
    d_out = torch.full((rows,), float("nan"), device="cuda")
    torch.cuda.synchronize()
    adb.devices.row_sum_noalloc(d_in.data_ptr(), d_out.data_ptr(), rows, length, 0)
    torch.cuda.synchronize()
    return d_out.cpu().numpy()


def test_noalloc_row_sum_matches_regular_path_twice_in_a_row():
    import torch
    torch.cuda.set_device(0)
    dev = adb.devices.B200(0)
    rng = np.random.default_rng(5)
    try:
        for rows, length in [(37, 50000), (1000, 333)]:
            x = rng.standard_normal(rows * length).astype(np.float32)
            want = _regular_row_sum(dev, x, rows, length)
            got = _noalloc_row_sum(x, rows, length)
            scale = float(np.abs(want).max())
            assert np.isfinite(got).all()
            assert float(np.abs(got - want).max()) / scale <= 1e-4, (rows, length)
            ref = x.reshape(rows, length).astype(np.float64).sum(1)
            assert float(np.abs(got - ref).max()) / float(np.abs(ref).max()) <= 1e-4
    finally:
        dev.close()


def test_noalloc_row_sum_rejects_sizes_beyond_its_fixed_scratch():
    import torch
    torch.cuda.set_device(0)
    d = torch.zeros(8, device="cuda")
    with pytest.raises(adb.devices.AdbError) as e:
        adb.devices.row_sum_noalloc(d.data_ptr(), d.data_ptr(), adb.devices.NOALLOC_MAX_PARTIALS + 1, 1, 0)
    assert "exceed" in str(e.value)
