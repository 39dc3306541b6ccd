"""The data-parallel rewrite, checked on CPU: world_size-2 gloo ranks run the rewritten IR on the CPU
oracle (its AllReduce hook calls torch.distributed) and must reproduce the single-process result."""
import importlib
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
adb = importlib.import_module("autodiff-ir-rust_b200")
cfg = adb.configs

KW = dict(batch=32, widths=(16, 24, 24, 16, 8), steps=3, lr=1e-2)


class _Capture:
    """Device stand-in that records the blob the frontend hands over."""

    def ir_callback(self, irb):
        pass

    def execute(self, proc, dep):
        self.blob, self.keep = adb.ir.serialize(proc, dep)
        self.ids = sorted(dep)

    def get_tensor(self, id_):
        return adb.autodiff.ValueData([1], np.zeros(1, np.float32), id_, False)


def _traced_c4(kw=None):
    kw = kw or KW
    cap = _Capture()
    inputs = cfg.c4_inputs(batch=kw["batch"], widths=kw["widths"])
    handles = cfg.c4_mlp_train(cap, inputs=inputs, execute=False, **kw)
    adb.autodiff.execute()
    return cap, handles, inputs


def _batch_ids(kw):
    """ids of x and t: `c4_mlp_train` creates the weights, then the biases, then x and t"""
    mats = [c[3] for c in adb.autodiff.current_ir().main if c[0] == "CreateMat"]
    n_layers = len(kw["widths"]) - 1
    return mats[2 * n_layers: 2 * n_layers + 2]


def test_rewrite_places_one_allreduce_per_parameter_and_one_for_the_loss():
    cap, handles, _ = _traced_c4()
    plan = adb.devices.lower_check(adb.autodiff.current_ir(), set(cap.ids), rank=0, world=2, shard_batch=KW["batch"],
                                   flags=adb.devices.FLAG_NO_BUCKETS)
    lines = [l for l in plan.splitlines() if " allreduce " in l]
    assert len(lines) == 9, plan   # 4 weights + 4 biases + the kept loss
    assert all("  #" in l for l in lines), "collectives belong inside the training loop"
    # by default the eight gradients, which nothing reads before the optimiser step, share one collective over buffers
    # that the arena keeps side by side; the kept loss stays on its own
    plan = adb.devices.lower_check(adb.autodiff.current_ir(), set(cap.ids), rank=0, world=2, shard_batch=KW["batch"])
    lines = [l for l in plan.splitlines() if " allreduce " in l]
    assert len(lines) == 2 and sum(l.count(" + ") for l in lines) == 7, plan
    assert all("  #" in l for l in lines)
    sharded = adb.devices.shard_ir(cap.blob, 1, 2, KW["batch"])
    assert sharded != cap.blob


def _worker(rank, world, port, out_dir, kw=None, with_ids=False):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle.oracle import OracleDevice
    kw = kw or KW
    cap, handles, _ = _traced_c4(kw)
    blob = adb.devices.shard_ir(cap.blob, rank, world, kw["batch"], _batch_ids(kw) if with_ids else None)

    def allreduce(arr):
        t = torch.from_numpy(arr)
        dist.all_reduce(t)

    dev = OracleDevice(allreduce=allreduce)
    dev.execute_blob(blob)
    out = {k: dev.get_tensor(v.id).numpy() for k, v in handles.items()}
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), **out)
    dist.destroy_process_group()


def test_two_gloo_ranks_match_one_process(tmp_path):
    import torch.multiprocessing as mp
    from oracle.oracle import OracleDevice
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    want = cfg.c4_mlp_train(OracleDevice(), inputs=cfg.c4_inputs(batch=KW["batch"], widths=KW["widths"]), **KW)
    for r in range(2):
        got = np.load(tmp_path / f"rank{r}.npz")
        for k, v in want.items():
            ref = v.numpy()
            err = np.abs(got[k] - ref).max() / max(np.abs(ref).max(), 1e-30)
            # only the order of the batch summation differs
            assert err < 1e-5, (r, k, err)


def test_rewrite_rejects_programs_it_cannot_split():
    ad = adb.autodiff
    cap = _Capture()
    ad.set_device(cap)
    x = ad.tensor(np.ones(32 * 4, np.float32), [32, 4])
    w = ad.tensor(np.ones(32 * 4, np.float32) * 2, [32, 4])      # same leading size as the batch but used as a parameter
    y = (x * w).i(3, 0)                                           # picks one sample: not expressible per rank
    y.forward()
    y.val().keep()
    ad.execute()
    with pytest.raises(adb.devices.AdbError) as e:
        adb.devices.shard_ir(cap.blob, 0, 2, 32)
    assert "sharded axis" in str(e.value)


@pytest.mark.parametrize("kw,world", [
    (dict(batch=24, widths=(16, 24, 24, 16, 8), steps=3, lr=1e-2), 2),     # batch == hidden widths
    (dict(batch=16, widths=(16, 24, 24, 16, 8), steps=2, lr=1e-2), 2),     # batch == input width (x is square) and a hidden width
    (dict(batch=8, widths=(16, 24, 24, 16, 8), steps=2, lr=1e-2), 2),      # batch == output width (t is square)
    (dict(batch=24, widths=(24, 24, 24, 24, 24), steps=2, lr=1e-2), 4),    # everything is 24 wide, four ranks
])
def test_named_batch_tensors_resolve_a_batch_that_equals_a_layer_width(tmp_path, kw, world):
    """A batch that equals layer widths: by shape alone a weight looks like a batch tensor and the rewrite refuses the
    program; with x and t named, constants and broadcasts that merely look batch-shaped are sorted out where they meet
    tensors, and the gloo ranks reproduce the single-process run."""
    import torch.multiprocessing as mp
    from oracle.oracle import OracleDevice
    cap, _, _ = _traced_c4(kw)
    ids = _batch_ids(kw)
    assert len(ids) == 2
    with pytest.raises(adb.devices.AdbError):
        adb.devices.shard_ir(cap.blob, 0, world, kw["batch"])
    port = 31500 + (os.getpid() % 2000) + world * 7 + kw["batch"]
    mp.spawn(_worker, args=(world, port, str(tmp_path), kw, True), nprocs=world, join=True)
    want = cfg.c4_mlp_train(OracleDevice(), inputs=cfg.c4_inputs(batch=kw["batch"], widths=kw["widths"]), **kw)
    for r in range(world):
        got = np.load(tmp_path / f"rank{r}.npz")
        for k, v in want.items():
            ref = v.numpy()
            err = np.abs(got[k] - ref).max() / max(np.abs(ref).max(), 1e-30)
            assert err < 1e-5, (r, k, err)


# ---------------------------------------------------------------------------------------------------------------------
# Raw IR through the rewrite, ranks simulated by threads: each rank runs its rewritten program on an oracle of its own
# and the AllReduce hooks meet at a barrier.  (The oracle runs outside the GIL; only the hooks take it.)
def _run_ranks(proc, dep, world, batch):
    import threading
    from oracle.oracle import OracleDevice
    blob, keep = adb.ir.serialize(proc, dep, inline_limit=1 << 40)
    barrier = threading.Barrier(world)
    slots = [None] * world
    results = [None] * world
    errors = []

    def run(rank):
        def allreduce(arr):
            slots[rank] = arr.copy()
            barrier.wait(timeout=60)
            total = np.sum(np.stack(slots), axis=0, dtype=np.float32)
            barrier.wait(timeout=60)
            arr[:] = total
        try:
            dev = OracleDevice(allreduce=allreduce)
            dev.execute_blob(adb.devices.shard_ir(blob, rank, world, batch))
            results[rank] = {d: dev.get_tensor(d).numpy() for d in dep}
        except Exception as e:      # noqa: BLE001 - reported below, and the other ranks must not wait forever
            errors.append(e)
            barrier.abort()

    threads = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    one = OracleDevice()
    one.execute_blob(blob)
    want = {d: one.get_tensor(d).numpy() for d in dep}
    del keep
    return want, results


def _close(want, results, tol=1e-5):
    for got in results:
        for k, ref in want.items():
            err = np.abs(got[k] - ref).max() / max(np.abs(ref).max(), 1e-30)
            assert err < tol, (k, err, got[k], ref)


def _loop_carried_partial(iters):
    """g is replicated when the loop starts and a per-rank partial sum when the body ends: the next pass reads it."""
    B, F = 8, 3
    rng = np.random.default_rng(11)
    P = adb.ir.IRProcedure
    main = P("main")
    main.push(("CreateMat", (rng.standard_normal(B * F) / B).astype(np.float32), [B, F], "x"))
    main.push(("CreateMat", rng.standard_normal(F).astype(np.float32), [F], "g"))
    main.push(("CreateMat", np.zeros(F, np.float32), [F], "acc"))
    main.push(("CreateMat", np.array([float(iters)], np.float32), [1], "cnt"))
    main.push(("CreateConstant", -1.0, "k", [1]))
    main.push(("Permute", "x", [1, 0], "xt"))
    body = P("body")
    body.push(("Exp2", "g", "y"))
    body.push(("ElwAddEq", "acc", "y"))
    body.push(("Sum", "xt", "g"))
    body.push(("ElwAddEq", "cnt", "k"))
    main.push(("While", "cnt", body))
    return main, ["acc"], B      # (g is not kept: a kept partial value is completed where it is produced anyway)


@pytest.mark.parametrize("iters", [0, 1, 3])
def test_partial_value_carried_around_a_loop_is_completed_every_pass(iters):
    proc, dep, B = _loop_carried_partial(iters)
    want, results = _run_ranks(proc, dep, 2, B)
    _close(want, results)


@pytest.mark.parametrize("flag", [0.0, 1.0])
def test_partial_value_from_a_branch_that_may_not_run(flag):
    """`If f {g = Sum(xt)}; out = Exp2(g)`: behind the branch g must be complete whether or not it ran."""
    B, F = 8, 3
    rng = np.random.default_rng(12)
    P = adb.ir.IRProcedure
    main = P("main")
    main.push(("CreateMat", (rng.standard_normal(B * F) / B).astype(np.float32), [B, F], "x"))
    main.push(("CreateMat", rng.standard_normal(F).astype(np.float32), [F], "g"))
    main.push(("CreateMat", np.array([flag], np.float32), [1], "f"))
    main.push(("Permute", "x", [1, 0], "xt"))
    then = P("then")
    then.push(("Sum", "xt", "g"))
    main.push(("If", [("f", then)], None))
    main.push(("Exp2", "g", "out"))
    want, results = _run_ranks(main, ["out"], 2, B)
    _close(want, results)


def test_partial_value_made_before_a_loop_is_not_summed_on_every_pass():
    """g = Sum(xt) in front of the loop, read inside: the AllReduce belongs in front of the loop, once."""
    B, F = 8, 3
    rng = np.random.default_rng(13)
    P = adb.ir.IRProcedure
    main = P("main")
    main.push(("CreateMat", (rng.standard_normal(B * F) / B).astype(np.float32), [B, F], "x"))
    main.push(("CreateMat", np.zeros(F, np.float32), [F], "acc"))
    main.push(("CreateMat", np.array([3.0], np.float32), [1], "cnt"))
    main.push(("CreateConstant", -1.0, "k", [1]))
    main.push(("Permute", "x", [1, 0], "xt"))
    main.push(("Sum", "xt", "g"))
    body = P("body")
    body.push(("Exp2", "g", "y"))
    body.push(("ElwAddEq", "acc", "y"))
    body.push(("ElwAddEq", "cnt", "k"))
    main.push(("While", "cnt", body))
    want, results = _run_ranks(main, ["acc"], 2, B)
    _close(want, results)


def test_reshaped_constant_keeps_its_shape_under_the_rewrite():
    """CreateConstant c[F]; View -> [F, 1]; Broadcast -> [F, 4]; multiplied with a parameter [F, 4]: nothing here has a
    batch dimension, so the rewrite must leave it alone (and not refuse it)."""
    B, F = 8, 3
    rng = np.random.default_rng(14)
    P = adb.ir.IRProcedure
    main = P("main")
    main.push(("CreateMat", rng.standard_normal(B * F).astype(np.float32), [B, F], "x"))
    main.push(("CreateMat", rng.standard_normal(F * 4).astype(np.float32), [F, 4], "w"))
    main.push(("CreateConstant", 0.5, "cv", [F]))
    main.push(("View", "cv", [F, 1], "cv2"))
    main.push(("Broadcast", "cv2", 1, 4, "cv3"))
    main.push(("ElwMultiply", "cv3", "w", "ws"))
    main.push(("DotProduct", "x", "ws", "y"))       # [B, 4], sharded
    main.push(("Permute", "y", [1, 0], "yt"))
    main.push(("Sum", "yt", "s"))                   # partial -> completed because it is kept
    want, results = _run_ranks(main, ["s", "ws"], 2, B)
    _close(want, results)
