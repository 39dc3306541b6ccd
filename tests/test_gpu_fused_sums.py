"""Sums that the lowering moves into an element-wise pass over the same memory (side sums of `adb_elwsum_*`
kernels): row sums, column sums, ragged edges, scalar (vec 1) kernels, a sum of a value the kernel itself
writes, the same inside a loop body -- B200 against the CPU oracle, and fused against unfused."""
import numpy as np
import pytest

from helpers import ad, adb, b200, oracle, run_both, assert_exact, assert_rel

pytestmark = pytest.mark.gpu
cfg = adb.configs
RNG = np.random.default_rng(31)


def _fused_kernels(dev):
    return dev.dump_plan().count("adb_elwsum_")


def _chain(P, Q, keep_y=True):
    x = RNG.standard_normal(P * Q).astype(np.float32)
    w = RNG.standard_normal(Q).astype(np.float32)

    def prog(dev):
        ad.set_device(dev)
        ad.eager_dep_opt()
        tx = ad.tensor(x, [P, Q])
        tw = ad.tensor(w, [Q])
        y = (tx * tw.view([1, Q]).broadcast(0, P) + 0.5).sin() * tx        # streamed once ...
        rows = y.sum(1)                                       # ... with its row sums
        cols = (y * y).sum(0)                                 # ... and the column sums of another value of the pass
        outs = {"rows": rows.forward(), "cols": cols.forward()}
        if keep_y:
            outs["y"] = y.forward()
        for v in outs.values():
            v.keep()
        ad.execute()
        return {k: v.get() for k, v in outs.items()}
    return prog


@pytest.mark.parametrize("P,Q", [(512, 1024), (777, 1000), (1031, 999), (4096, 128), (8, 40000)])
def test_row_and_column_sums_ride_along(P, Q):
    want, got = run_both(_chain(P, Q))
    assert _fused_kernels(b200()) == 1, b200().dump_plan()
    assert_rel("y", got["y"], want["y"], 2e-6)
    assert_rel("rows", got["rows"], want["rows"], 1e-4)
    assert_rel("cols", got["cols"], want["cols"], 1e-4)


def test_fused_equals_unfused():
    """Same program with the fusion switched off (one kernel per IR command): the element-wise output is
    bit-identical, the sums agree to reduction-order accuracy."""
    prog = _chain(640, 768)
    fused = prog(b200())
    assert _fused_kernels(b200()) == 1
    plain = adb.devices.B200(0, flags=adb.devices.FLAG_NO_FUSION)
    try:
        ref = prog(plain)
        assert _fused_kernels(plain) == 0
    finally:
        plain.close()
    assert_exact("y", fused["y"], ref["y"])
    assert_rel("rows", fused["rows"], ref["rows"], 1e-5)
    assert_rel("cols", fused["cols"], ref["cols"], 1e-5)


def test_small_problems_keep_their_own_reduce_kernels():
    _chain(64, 128)(b200())
    assert _fused_kernels(b200()) == 0


def test_config2_is_one_pass_over_its_inputs():
    want, got = run_both(cfg.c2_fused_elementwise, rows=520, cols=1000)
    plan = b200().dump_plan()
    assert plan.count("adb_elwsum_") == 1 and plan.count("sum v") == 2, plan
    assert_rel("a_grad", got["a_grad"], want["a_grad"], 2e-5)
    assert_rel("b_grad", got["b_grad"], want["b_grad"], 2e-5)
    assert_rel("bias_grad", got["bias_grad"], want["bias_grad"], 1e-4)
    assert_rel("loss", got["loss"], want["loss"], 1e-4)


def test_training_loop_with_fused_loss_and_bias_gradients():
    """Activations of 2048 x 512: the loss row sums and every bias gradient (a column sum of a value the backward
    kernel writes) are side sums inside the loop body; three steps against the oracle."""
    kw = dict(batch=2048, widths=(256, 512, 512, 256, 128), steps=3, lr=1e-2)
    want, got = run_both(cfg.c4_mlp_train, **kw)
    assert _fused_kernels(b200()) >= 4, b200().dump_plan()
    for k in want:
        assert_rel(k, got[k], want[k], 1e-4)


def test_sum_of_a_value_written_inside_a_loop_body():
    P, Q = 600, 512
    x = RNG.standard_normal(P * Q).astype(np.float32)

    def prog(dev):
        ad.set_device(dev)
        acc = ad.tensor(np.zeros(P * Q, np.float32), [P, Q])
        tot = ad.tensor(np.zeros(Q, np.float32), [Q])
        tx = ad.tensor(x, [P, Q])

        def body(i):
            nonlocal acc, tot
            acc += tx * 0.25
            acc.forward()
            tot += acc.sum(0)        # column sums of the value the update kernel has just written
            tot.forward()
        ad.ir_for(range(0, 4), body)
        ad.execute()
        return {"acc": acc.val().get(), "tot": tot.val().get()}
    want, got = run_both(prog)
    # the lowering expresses the sum through the operands of the in-place update; the update kernel reads the old
    # element, sums the new value on the side and stores it
    assert _fused_kernels(b200()) == 1, b200().dump_plan()
    assert_rel("acc", got["acc"], want["acc"], 1e-6)
    assert_rel("tot", got["tot"], want["tot"], 1e-4)
