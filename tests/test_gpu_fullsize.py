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
    from helpers import c2_float64, assert_chain_per_element
    ref = c2_float64(sub, 64, cols)
    VD = adb.autodiff.ValueData
    for k in ("a_grad", "b_grad"):
        g = np.asarray(got[k].data).reshape(rows, cols)[band]
        # element by element against float64, in units of each element's conditioning (see helpers.c2_float64)
        assert_chain_per_element(k, VD([64, cols], g.reshape(-1), k, False), want[k], *ref[k])
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


def test_c5_full_size_columns_against_float64():
    """Config 5 at 8192 x 8192, 50 iterations (151 dot products of 8192^3): the iteration count is exact and 64
    columns of X -- the columns evolve independently -- match a float64 recomputation on the host."""
    import torch
    n, iters, cols = 8192, 50, 64
    g = torch.Generator(device="cuda").manual_seed(4)
    a = torch.randn(n * n, device="cuda", generator=g) * n ** -0.5
    b = torch.randn(n * n, device="cuda", generator=g) * n ** -0.5
    DP = adb.ir.DevicePayload
    got = cfg.c5_dot_loop(b200(), n=n, max_iters=iters, inputs={"a": DP(a.data_ptr(), n * n, a), "b": DP(b.data_ptr(), n * n, b)})
    assert float(got["iters"].data[0]) == iters
    assert b200().stats()["tc_gemm_launches"] == 3 * iters + 1
    A = a.view(n, n).double().cpu()
    Bc = b.view(n, n)[:, :cols].double().cpu()
    ref = torch.zeros(n, cols, dtype=torch.float64)
    for _ in range(iters):
        ref = ref - 0.01 * (A @ ref - Bc)
    x = np.asarray(got["x"].data, np.float32).reshape(n, n)[:, :cols].astype(np.float64)
    err = np.abs(x - ref.numpy()).max() / np.abs(ref.numpy()).max()
    assert err < 1e-4, err


@pytest.mark.parametrize("flags", [0, adb.devices.FLAG_NO_FUSION], ids=["fused", "one-kernel-per-command"])
def test_more_than_2_31_elements_use_64_bit_indices(flags):
    """Flat indices beyond 2^31 (the reference's i32 index math, src/kernel/kernel_decl.rs:5, stops there): an in-place
    element-wise update with its column sums inside a loop, then row sums, over 2^31 + 16384 elements, checked
    against torch on the same GPU."""
    import torch
    P, Q = (1 << 20) + 8, 2048
    n = P * Q
    assert n > 1 << 31
    g = torch.Generator(device="cuda").manual_seed(5)
    a = torch.randn(n, device="cuda", generator=g)
    b = torch.randn(n, device="cuda", generator=g)
    DP = adb.ir.DevicePayload
    ad = adb.autodiff
    dev = adb.devices.B200(0, flags=flags)
    try:
        ad.set_device(dev)
        ad.eager_dep_opt()          # read back only what is kept: the [P, Q] tensors stay on the device
        acc = ad.tensor(DP(a.data_ptr(), n, a), [P, Q])
        x = ad.tensor(DP(b.data_ptr(), n, b), [P, Q])
        tot = ad.tensor(np.zeros(Q, np.float32), [Q])

        def body(i):
            nonlocal acc, tot
            acc += x * 0.5
            acc.forward()
            tot += acc.sum(0)
            tot.forward()
        ad.ir_for(range(0, 2), body)
        rows = acc.sum(1).forward()
        rows.keep()
        tot.val().keep()
        ad.execute()
        got_rows = np.asarray(rows.get().data, np.float64)
        got_tot = np.asarray(tot.val().get().data, np.float64)
        fused = dev.dump_plan().count("adb_elwsum_")
    finally:
        dev.close()
    assert fused == (1 if flags == 0 else 0)
    want_rows = (a + b).view(P, Q).sum(1, dtype=torch.float64).cpu().numpy()
    want_tot = ((a + b * 0.5).view(P, Q).sum(0, dtype=torch.float64) + (a + b).view(P, Q).sum(0, dtype=torch.float64)).cpu().numpy()
    assert got_rows.shape == (P,) and got_tot.shape == (Q,)
    # the last rows only come out right when no index wrapped at 2^31 or 2^32
    assert np.abs(got_rows - want_rows).max() / np.abs(want_rows).max() < 1e-4
    assert np.abs(got_rows[-8:] - want_rows[-8:]).max() < 1e-2
    assert np.abs(got_tot - want_tot).max() / np.abs(want_tot).max() < 1e-4


def test_c4_full_size_step_against_float64_on_the_gpu():
    """Config 4 at the benchmark's size (batch 65536, 4096-8192-8192-4096-1000; 5e13 flop), one step at lr 10 (at the
    benchmark's 1e-3 one step moves the first layers by about an ulp): the loss and the update every parameter received
    match a float64 evaluation of the same step (torch autograd on the same GPU, used as a checker only)."""
    import torch
    widths, batch, lr = cfg.C4_WIDTHS, 65536, 10.0
    small = cfg.c4_inputs(batch=0, widths=widths)
    g = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn(batch * widths[0], device="cuda", generator=g)
    t = torch.randn(batch * widths[-1], device="cuda", generator=g)
    w = {k: torch.from_numpy(v).cuda() for k, v in small.items() if k[0] in "wb"}
    DP = adb.ir.DevicePayload
    inputs = {k: DP(v.data_ptr(), v.numel(), v) for k, v in w.items()}
    inputs["x"] = DP(x.data_ptr(), x.numel(), x)
    inputs["t"] = DP(t.data_ptr(), t.numel(), t)
    got = cfg.c4_mlp_train(b200(), batch=batch, widths=widths, steps=1, lr=lr, inputs=inputs)
    st = b200().stats()
    assert st["tc_gemm_launches"] == st["gemm_launches"] == 11, st

    n_layers = len(widths) - 1
    params = {}
    for i in range(n_layers):
        params[f"w{i}"] = w[f"w{i}"].double().view(widths[i], widths[i + 1]).requires_grad_(True)
        params[f"b{i}"] = w[f"b{i}"].double().requires_grad_(True)
    a = x.view(batch, widths[0]).double()
    for i in range(n_layers):
        a = a @ params[f"w{i}"] + params[f"b{i}"]
        if i < n_layers - 1:
            a = torch.sigmoid(a)
    loss = ((a - t.view(batch, widths[-1]).double()) ** 2).sum() / (batch * widths[-1])
    loss.backward()
    del a
    ref_loss = float(loss.detach())
    assert abs(float(got["loss"].data[0]) - ref_loss) / ref_loss < 1e-5
    for k, p in params.items():
        du_ref = (-lr * p.grad).reshape(-1)
        p0 = w[k].double().reshape(-1)
        du_got = torch.from_numpy(np.asarray(got[k].data, np.float32)).cuda().double() - p0
        biggest = float(du_ref.abs().max())
        assert biggest > 100 * 6e-8 * float(p0.abs().max()), k          # the parameter really moved
        err = float((du_got - du_ref).abs().max()) / biggest
        # the fp32 parameter rounds its own update: half an ulp of the parameter on top of the arithmetic error
        floor = 6e-8 * float(p0.abs().max()) / biggest
        assert err < 2e-3 + floor, (k, err)
