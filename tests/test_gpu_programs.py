"""Structure coverage: broadcasts, permutes, views, index/concat, reductions of every launch shape,
dot products with folded transposes, control flow -- B200 against the CPU oracle."""
import numpy as np
import pytest

from helpers import ad, adb, nn, oracle, run_both, assert_exact, assert_rel, assert_ulp, b200

pytestmark = pytest.mark.gpu
RNG = np.random.default_rng(11)


def rnd(*shape):
    return RNG.standard_normal(int(np.prod(shape))).astype(np.float32)


def _run(build, exact=(), rel=(), tol=1e-4):
    """build() -> {name: Tensor}; everything is forwarded, kept, executed and compared."""
    def prog(dev):
        ad.set_device(dev)
        ad.eager_dep_opt()
        outs = build()
        vals = {}
        for k, t in outs.items():
            vals[k] = t.forward() if hasattr(t, "forward") else t
            vals[k].keep()
        ad.execute()
        return {k: v.get() for k, v in vals.items()}
    want, got = run_both(prog)
    for k in want:
        if k in rel:
            assert_rel(k, got[k], want[k], tol)
        else:
            assert_exact(k, got[k], want[k])
    return want, got


@pytest.mark.parametrize("shape", [(7,), (4, 5), (3, 8, 16), (2, 3, 4, 5), (1, 1), (33, 1, 7)])
def test_broadcast_forms(shape):
    a = rnd(*shape)
    inner = shape[-1]
    row = rnd(inner)

    def build():
        ta = ad.tensor(a, list(shape))
        tr = ad.tensor(row, [inner])
        return {"y": ta * tr + 2.0, "z": tr + ta}
    _run(build)


@pytest.mark.parametrize("shape,perm", [((4, 6), [1, 0]), ((3, 4, 5), [0, 2, 1]), ((3, 4, 5), [2, 0, 1]),
                                         ((2, 3, 4, 5), [3, 1, 0, 2]), ((64, 96), [1, 0]), ((8, 128, 64), [0, 2, 1])])
def test_permute_contiguous(shape, perm):
    a = rnd(*shape)

    def build():
        t = ad.tensor(a, list(shape))
        p = t.permute(perm)
        return {"p": p.contigious(), "q": (p * 3.0 + 1.0)}
    want, got = _run(build)
    np.testing.assert_array_equal(np.asarray(got["p"].data).reshape(got["p"].dim), a.reshape(shape).transpose(perm))


@pytest.mark.parametrize("shape,perm", [((512, 768), [1, 0]), ((520, 388), [1, 0]), ((8, 256, 320), [0, 2, 1]), ((128, 64, 96), [2, 0, 1]),
                                         ((6, 132, 4, 100), [0, 3, 2, 1]), ((96, 2048), [1, 0])])
def test_large_permutes_go_through_the_tiled_transpose(shape, perm):
    """Axis swaps of at least 2^16 elements whose source is contiguous along an axis that is not the result's innermost
    one are copied through 64 x 64 shared-memory tiles (adb_transpose_*), with element-wise work on the way: bit-exact,
    ragged tile edges included."""
    from helpers import b200
    a = rnd(*shape)

    def build():
        t = ad.tensor(a, list(shape))
        p = t.permute(perm)
        return {"p": p.contigious(), "q": (p * 3.0 + 1.0)}
    want, got = _run(build)
    assert "adb_transpose_" in b200().dump_plan(), b200().dump_plan()
    np.testing.assert_array_equal(np.asarray(got["p"].data).reshape(got["p"].dim), a.reshape(shape).transpose(perm))
    np.testing.assert_array_equal(np.asarray(got["q"].data).reshape(got["q"].dim),
                                  a.reshape(shape).transpose(perm) * np.float32(3.0) + np.float32(1.0))


def test_view_of_permuted_needs_copy():
    a = rnd(6, 10)

    def build():
        t = ad.tensor(a, [6, 10])
        v = t.t().view([4, 15])          # not expressible as strides of `a`: forces a copy
        w = t.view([3, 2, 10]).permute([1, 0, 2]).view([2, 30])
        return {"v": v * 1.5, "w": w.contigious()}
    want, got = _run(build)
    np.testing.assert_array_equal(np.asarray(got["w"].data).reshape(2, 30), a.reshape(3, 2, 10).transpose(1, 0, 2).reshape(2, 30))


def test_index_and_concat():
    a, b = rnd(5, 8), rnd(3, 8)

    def build():
        ta, tb = ad.tensor(a, [5, 8]), ad.tensor(b, [3, 8])
        c = ad.concat([ta, tb, ta * 2.0], 0)          # [13, 8]
        d = ad.concat([ta.i(2, 0).unsqueeze(0), tb], 0)  # [4, 8]
        e = ad.concat([ta, ta.exp2()], 1)             # [5, 16]
        return {"c": c.contigious(), "rows": c.r(range(3, 11), 0).contigious(), "col": c.i(5, 1).contigious(),
                "d": d * d, "e": e.contigious(), "e_t": e.t().contigious()}
    want, got = _run(build, rel=("e", "e_t"), tol=1e-6)
    full = np.concatenate([a.reshape(5, 8), b.reshape(3, 8), 2 * a.reshape(5, 8)], 0)
    np.testing.assert_array_equal(np.asarray(got["rows"].data).reshape(8, 8), full[3:11])
    np.testing.assert_array_equal(np.asarray(got["col"].data), full[:, 5])


@pytest.mark.parametrize("V,R", [(1, 5), (3, 7), (64, 16), (5, 1000), (300, 33), (2, 40000), (1, 100000), (257, 4096)])
def test_row_sums(V, R):
    a = rnd(V, R)

    def build():
        t = ad.tensor(a, [V, R])
        return {"s": t.sum(1), "m": (t * t + 1.0).sum(1)}
    _run(build, rel=("s", "m"))


@pytest.mark.parametrize("R,V", [(5, 1), (7, 3), (16, 64), (1000, 8), (33, 300), (40000, 4), (4096, 260), (9000, 1024)])
def test_column_sums(R, V):
    a = rnd(R, V)

    def build():
        t = ad.tensor(a, [R, V])
        return {"s": t.sum(0), "m": (t.sin() * 0.5).sum(0)}
    _run(build, rel=("s", "m"))


def test_sum_middle_axis_and_all():
    a = rnd(6, 10, 12)

    def build():
        t = ad.tensor(a, [6, 10, 12])
        ones = ad.tensor(np.ones(24, np.float32), [4, 6])
        almost = np.ones(24, np.float32)
        almost[13] = 0
        return {"mid": t.sum(1), "mean": t.mean(-1), "var": t.var(0, 1), "all1": ones.all(),
                "all0": ad.tensor(almost, [4, 6]).all()}
    want, got = _run(build, rel=("mid", "mean", "var"))
    assert got["all1"].data[0] == 1.0 and got["all0"].data[0] == 0.0


@pytest.mark.parametrize("M,K,N", [(1, 1, 1), (2, 5, 3), (17, 33, 9), (64, 64, 64), (128, 256, 192), (100, 1000, 7), (300, 70, 130)])
def test_dot_shapes(M, K, N):
    a, b = rnd(M, K), rnd(K, N)
    at, bt = rnd(K, M), rnd(N, K)

    def build():
        ta, tb = ad.tensor(a, [M, K]), ad.tensor(b, [K, N])
        tat, tbt = ad.tensor(at, [K, M]), ad.tensor(bt, [N, K])
        return {"nn": ad.dot(ta, tb), "tn": ad.dot(tat.t(), tb), "nt": ad.dot(ta, tbt.t()), "tt": ad.dot(tat.t(), tbt.t()),
                "fused": ad.dot(ta * 2.0, tb + 1.0)}
    want, got = _run(build, rel=("nn", "tn", "nt", "tt", "fused"))
    ref = a.reshape(M, K).astype(np.float64) @ b.reshape(K, N).astype(np.float64)
    err = np.abs(np.asarray(got["nn"].data).reshape(M, N) - ref).max() / max(np.abs(ref).max(), 1e-30)
    assert err < 1e-4


def test_dot_backward_and_linear_layer():
    x, w, bias = rnd(9, 6), rnd(6, 4), rnd(4)

    def prog(dev):
        ad.set_device(dev)
        tx, tw, tb = ad.tensor(x, [9, 6]), ad.tensor(w, [6, 4]), ad.tensor(bias, [4])
        y = nn.LinearWithWeights(tw, tb).f(tx).sigmoid()
        y.forward()
        y.backward()
        y.val().keep()
        ad.execute()
        return {"y": y.val().get(), "dx": tx.grad().get(), "dw": tw.grad().get(), "db": tb.grad().get()}
    want, got = run_both(prog)
    for k in want:
        assert_rel(k, got[k], want[k], 1e-4)


def test_in_place_through_alias_reads_and_loop_carried_state():
    a = rnd(4, 6)

    def prog(dev):
        ad.set_device(dev)
        t = ad.tensor(a, [4, 6])
        tt = t.t()                      # alias defined before the updates below
        acc = ad.tensor(np.zeros(24, np.float32), [6, 4])

        def body(i):
            nonlocal t, acc
            acc += tt * 1.0             # must see the current contents of t every iteration
            acc.forward()
            t *= 2.0
            t.forward()
        ad.ir_for(range(0, 3), body)
        ad.execute()
        return {"t": t.val().get(), "acc": acc.val().get()}
    want, got = run_both(prog)
    assert_exact("t", got["t"], want["t"])
    assert_exact("acc", got["acc"], want["acc"])
    at = a.reshape(4, 6).T
    ref = (np.float32(0) + at) + at * np.float32(2)
    ref = ref + at * np.float32(4)
    np.testing.assert_array_equal(np.asarray(got["acc"].data).reshape(6, 4), ref)


def test_nested_control_flow_counts():
    def prog(dev):
        ad.set_device(dev)
        total = ad.scalar(0.0)
        evens = ad.scalar(0.0)

        def outer(i):
            nonlocal total

            def inner(j):
                nonlocal total
                total += 1.0
                total.forward()
            ad.ir_for(range(0, 4), inner)

            def even():
                nonlocal evens
                evens += 1.0
                evens.forward()
            half = i.clone() * 0.5
            ad.ir_if(lambda: (half.sin() * 0.0 + half).equal(ad.constant(1.0, [1])), even)   # only i == 2
        ad.ir_for(range(0, 5), outer)
        ad.execute()
        return {"total": total.val().get(), "evens": evens.val().get()}
    want, got = run_both(prog)
    assert_exact("total", got["total"], want["total"])
    assert_exact("evens", got["evens"], want["evens"])
    assert got["total"].data[0] == 20.0 and got["evens"].data[0] == 1.0


def test_plan_is_cached_and_payloads_rebound():
    dev = b200()

    def run(scale):
        ad.set_device(dev)
        ad.eager_dep_opt()
        x = ad.tensor(np.arange(8, dtype=np.float32) * scale, [8])
        y = (x * 3.0 + 1.0).exp2().sum(0)
        y.forward()
        y.val().keep()
        ad.execute()
        return float(y.val().get().data[0]), dev.stats()
    v1, s1 = run(0.25)
    v2, s2 = run(0.5)
    assert s2["jit_compiles"] == 0 and s2["lower_ms"] == 0.0      # same structure: plan and kernels reused
    assert abs(v1 - float(np.exp2(np.arange(8) * 0.75 + 1).sum())) < 1e-2
    assert abs(v2 - float(np.exp2(np.arange(8) * 1.5 + 1).sum())) / v2 < 1e-5


def test_malformed_blob_is_rejected_without_killing_the_context():
    dev = b200()
    with pytest.raises(Exception):
        dev.execute_blob(b"ADIRgarbage")
    ad.set_device(dev)
    x = ad.tensor([1.0, 2.0], [2])
    bad = ad.dot(x.view([1, 2]), x.view([1, 2]))   # inner dimensions disagree
    with pytest.raises(AssertionError):
        bad.forward()
    y = x + 1.0
    y.forward()
    y.val().keep()
    ad.execute()
    np.testing.assert_array_equal(y.val().get().data, [2.0, 3.0])


def test_pinned_payload_uploaded_inside_a_loop_is_prefetched_correctly():
    """A CreateMat inside a loop body re-uploads on every iteration (src/devices/opencl/kernels/alloc.rs:5-12);
    from pinned memory the backend double-buffers that copy on a second stream."""
    import torch
    n = 512 * 1024                      # 2 MiB: above the prefetch threshold
    host = torch.empty(n, pin_memory=True)
    host.copy_(torch.from_numpy(rnd(n)))
    data = host.numpy()

    def prog(dev):
        ad.set_device(dev)
        acc = ad.tensor(np.zeros(n, np.float32), [512, 1024])

        def body(i):
            nonlocal acc
            x = ad.tensor(data, [512, 1024])
            acc += x * (i.clone() + 1.0).broadcast(0, 512 * 1024).view([512, 1024])
            acc.forward()
        ad.ir_for(range(0, 5), body)
        ad.execute()
        return {"acc": acc.val().get()}
    want, got = run_both(prog)
    assert_exact("acc", got["acc"], want["acc"])
    assert b200().stats()["h2d_bytes"] >= 5 * n * 4


def test_device_payload_in_a_captured_loop_then_a_new_program_with_a_dot():
    """A device-resident CreateMat inside a loop body is copied inside the replayed CUDA graph; the next
    execute (a different program, launched kernel by kernel) must not see any error left behind by it."""
    import torch
    n = 256 * 512
    x_dev = torch.from_numpy(rnd(n)).cuda()
    x_host = x_dev.cpu().numpy()

    def loop_prog(dev, payload):
        ad.set_device(dev)
        acc = ad.tensor(np.zeros(n, np.float32), [256, 512])

        def body(i):
            nonlocal acc
            x = ad.tensor(payload, [256, 512])
            acc += x * 0.5
            acc.forward()
        ad.ir_for(range(0, 4), body)
        ad.execute()
        return {"acc": acc.val().get()}

    def dot_prog(dev):
        ad.set_device(dev)
        a = ad.tensor(x_host[:128 * 256].copy(), [128, 256])
        b = ad.tensor(x_host[128 * 256:128 * 256 + 256 * 64].copy(), [256, 64])
        y = ad.dot(a, b).forward()
        y.keep()
        ad.execute()
        return {"y": y.get()}

    want = loop_prog(oracle(), x_host)
    for _ in range(2):
        got = loop_prog(b200(), adb.ir.DevicePayload(x_dev.data_ptr(), n, x_dev))
        assert_exact("acc", got["acc"], want["acc"])
        want_y, got_y = dot_prog(oracle()), dot_prog(b200())
        assert_rel("y", got_y["y"], want_y["y"], 1e-4)


@pytest.mark.parametrize("shape", [[4096], [64, 48], [8, 16, 32]])
def test_mse_loss_and_abs_helpers(shape):
    n = int(np.prod(shape))
    y, t = rnd(n), rnd(n)

    def prog(dev):
        ad.set_device(dev)
        ty, tt = ad.tensor(y, shape), ad.tensor(t, shape)
        loss = nn.mse_loss(ty, tt)
        loss.forward()
        loss.backward()
        a = ty.abs().forward()
        a.keep()
        loss.val().keep()
        ad.execute()
        return {"loss": loss.val().get(), "y_grad": ty.grad().get(), "abs": a.get()}
    want, got = run_both(prog)
    assert_rel("loss", got["loss"], want["loss"], 1e-4)
    assert_ulp("y_grad", got["y_grad"], want["y_grad"], 2)
    assert_ulp("abs", got["abs"], want["abs"], 1)


def test_arena_that_does_not_fit_is_refused_and_the_handle_stays_usable():
    """A program whose buffers need more memory than the GPU has: `adb_execute` reports ADB_ERR_OOM before anything
    runs (the arena size is known after lowering); the next program on the same handle works."""
    n = 1 << 18
    x = rnd(n)
    dev = b200()
    ad.set_device(dev)
    ad.eager_dep_opt()
    t = ad.tensor(x, [1, n])
    big = (t.broadcast(0, n) * 2.0 + 1.0).forward()       # 2^36 elements = 256 GiB
    big.keep()
    with pytest.raises(adb.devices.AdbError) as e:
        ad.execute()
    assert "does not fit" in str(e.value)
    want, got = run_both(lambda d: _tiny(d, x))
    assert_exact("y", got["y"], want["y"])


def _tiny(dev, x):
    ad.set_device(dev)
    ad.eager_dep_opt()
    y = (ad.tensor(x[:1024].copy(), [1024]) * 3.0).forward()
    y.keep()
    ad.execute()
    return {"y": y.get()}


def test_plan_cache_is_bounded_and_evicted_programs_still_run():
    """More distinct programs than the cache holds (256): every one is right, and the first one, whose plan was
    dropped in the meantime, is lowered again and right again."""
    dev = adb.devices.B200(0)
    try:
        def run(n):
            ad.set_device(dev)
            ad.eager_dep_opt()
            x = np.arange(n, dtype=np.float32)
            y = (ad.tensor(x, [n]) * 2.0 + float(n)).forward()
            y.keep()
            ad.execute()
            np.testing.assert_array_equal(y.get().data, x * 2.0 + float(n))
            return dev.stats()["lower_ms"]
        for n in range(1, 271):
            run(n)
        assert run(270) == 0.0      # still cached: no lowering
        assert run(1) > 0.0         # evicted: lowered again
    finally:
        dev.close()


@pytest.mark.parametrize("shape,axis", [([4096], 0), ([300, 33], 1), ([300, 33], 0), ([2, 40000], 1), ([9000, 64], 0),
                                        ([8, 16, 32], 1), ([257, 4096], 1)])
def test_max_reduce_every_launch_shape(shape, axis):
    """Row / column launch shapes and the two-pass split of the reduce kernels, with maximum instead of sum:
    bit-exact against the oracle (a maximum involves no rounding), gradient mask included."""
    n = int(np.prod(shape))
    x = rnd(n)

    def prog(dev):
        ad.set_device(dev)
        t = ad.tensor(x, shape)
        m = (t * 1.5).max(axis)
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
    want, got = run_both(prog)
    assert_exact("max", got["max"], want["max"])
    assert_exact("grad", got["grad"], want["grad"])


def test_kept_tensor_can_stay_on_the_device():
    """`adb_get_tensor_device`: address and shape of a kept tensor in HBM (valid until the next execute), for callers
    that feed the result to other GPU code instead of reading it back."""
    import torch
    from cuda.bindings import runtime as cudart
    n = 3 * 1000
    x = rnd(n)
    dev = b200()
    ad.set_device(dev)
    ad.eager_dep_opt()
    y = (ad.tensor(x, [3, 1000]) * 2.0 + 1.0).forward()
    y.keep()
    ad.execute()
    ptr, shape = dev.get_tensor_device(y.id)
    assert shape == [3, 1000] and ptr
    out = torch.empty(n, device="cuda")
    (err,) = cudart.cudaMemcpy(out.data_ptr(), ptr, n * 4, cudart.cudaMemcpyKind.cudaMemcpyDeviceToDevice)
    assert int(err) == 0
    np.testing.assert_array_equal(out.cpu().numpy(), x * np.float32(2.0) + np.float32(1.0))
    assert dev.get_tensor_device("no-such-id") is None


def test_checkpoint_of_kept_tensors_round_trips(tmp_path):
    """`B200.save_tensors`: kept tensors of the last execute into one .npz; loading them as payloads resumes the run."""
    w0 = rnd(64 * 32)
    x = rnd(16 * 64)

    def step(dev, w_init):
        ad.set_device(dev)
        ad.eager_dep_opt()
        w = ad.tensor(w_init, [64, 32])
        y = ad.dot(ad.tensor(x, [16, 64]), w)
        loss = nn.mse_loss(y, ad.tensor(np.zeros(16 * 32, np.float32), [16, 32]))
        loss.forward()
        loss.backward()
        nn.SGD([w], 0.1).step()
        w.val().keep()
        ad.execute()
        return w
    dev = b200()
    w = step(dev, w0)
    path = str(tmp_path / "ckpt.npz")
    assert dev.save_tensors(path, [w]) == [w.val().id]
    saved = np.load(path)[w.val().id]
    np.testing.assert_array_equal(saved.reshape(-1), w.val().get().data)
    # two steps in a row == one step, checkpoint, one step from the checkpoint
    w2 = step(dev, saved.reshape(-1).copy())
    ref = step(oracle(), np.asarray(step(oracle(), w0).val().get().data, np.float32))
    assert_rel("w after resume", w2.val().get(), ref.val().get(), 1e-5)


def test_tensors_without_elements():
    """A [0, 4] tensor through element-wise work, a sum and a concat with a non-empty tensor, executed twice (the second
    time from the cached plan): shapes and values as the oracle has them."""
    E = np.zeros(0, np.float32)

    def prog(dev):
        main = adb.ir.IRProcedure("main")
        for c in [("CreateMat", E, [0, 4], "a"), ("CreateMat", np.arange(4, dtype=np.float32), [1, 4], "b"),
                  ("ElwAdd", "a", "a", "c"), ("Sum", "a", "s"), ("ElwAdd", "b", "b", "d"),
                  ("Concat", "a", "b", 0, "e"), ("Contigious", "e", "f"),
                  ("CreateMat", E, [3, 0], "p"), ("CreateMat", E, [0, 4], "q"), ("DotProduct", "p", "q", "pq"),
                  ("CreateMat", np.ones(8, np.float32), [4, 2], "w"), ("DotProduct", "a", "w", "aw"),
                  ("Sum", "p", "ps"), ("Max", "p", "pm")]:
            main.push(c)
        dep = ["c", "s", "d", "f", "pq", "aw", "ps", "pm"]
        dev.execute(main, dep)
        return {k: dev.get_tensor(k) for k in dep}
    want = prog(oracle())
    for _ in range(2):
        got = prog(b200())
        for k in want:
            assert got[k].dim == want[k].dim, k
            assert_exact(k, got[k], want[k])
