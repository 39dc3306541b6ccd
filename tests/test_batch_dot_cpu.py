"""BatchDot (IR extension, opcode 29): oracle against numpy, lowering through the CPU plan interpreter, gradients,
and the data-parallel rule (slices are independent)."""
import importlib

import numpy as np
import pytest

from oracle.oracle import OracleDevice
from test_plan_interp_cpu import _Both, _interpret, _compare

adb = importlib.import_module("autodiff-ir-rust_b200")
ad = adb.autodiff


def _attention_like(dev, B=6, S=10, D=4, seed=3):
    """softmax-free attention core: (Q K^T) V per slice, with gradients; operands of bmm arrive as permuted views."""
    rng = np.random.default_rng(seed)
    q, k, v = (rng.standard_normal(B * S * D).astype(np.float32) for _ in range(3))
    ad.set_device(dev)
    ad.eager_dep_opt()
    Q, K, V = (ad.tensor(x, [B, S, D]) for x in (q, k, v))
    scores = ad.bmm(Q, K.permute([0, 2, 1])) * (1.0 / np.sqrt(D))
    out = ad.bmm(scores, V)
    loss = (out * out).sum(2).sum(1).sum(0)
    loss.forward()
    loss.backward()
    keep = {"out": out.val(), "loss": loss.val(), "dq": Q.grad(), "dk": K.grad(), "dv": V.grad()}
    for t in keep.values():
        t.keep()
    ad.execute()
    return {n: t.get() for n, t in keep.items()}, (q, k, v)


def test_oracle_matches_numpy():
    got, (q, k, v) = _attention_like(OracleDevice(f64_acc=True))
    B, S, D = 6, 10, 4
    Q, K, V = (x.reshape(B, S, D).astype(np.float64) for x in (q, k, v))
    sc = np.einsum("bsd,btd->bst", Q, K) / np.sqrt(D)
    out = np.einsum("bst,btd->bsd", sc, V)
    np.testing.assert_allclose(got["out"].numpy().reshape(B, S, D), out, rtol=2e-5, atol=1e-5)
    go = 2 * out
    dv = np.einsum("bst,bsd->btd", sc, go)
    dsc = np.einsum("bsd,btd->bst", go, V) / np.sqrt(D)
    dq = np.einsum("bst,btd->bsd", dsc, K)
    dk = np.einsum("bst,bsd->btd", dsc, Q)
    for name, ref in (("dv", dv), ("dq", dq), ("dk", dk)):
        np.testing.assert_allclose(got[name].numpy().reshape(B, S, D), ref, rtol=2e-4, atol=2e-4)


@pytest.mark.parametrize("flags", [0, 1, 2])
def test_lowered_plan_matches_the_oracle(hostcheck, tmp_path, flags):
    dev = _Both()
    kept, _ = _attention_like(dev)
    got = _interpret(hostcheck, tmp_path, dev.blobs[-1], flags, f"bmm{flags}")
    _compare(got, {v.id: v for v in kept.values()}, 1e-4)


def test_permuted_operands_need_no_copy():
    class Rec:
        def ir_callback(self, irb): pass
        def execute(self, proc, dep): self.plan = adb.devices.lower_check(proc, dep)
        def get_tensor(self, id_): return adb.autodiff.ValueData.none()
    r = Rec()
    ad.set_device(r)
    ad.eager_dep_opt()
    rng = np.random.default_rng(9)      # (not constant-filled: those payloads are folded away and never uploaded)
    a = ad.tensor(rng.standard_normal(4 * 8 * 6).astype(np.float32), [4, 8, 6])
    b = ad.tensor(rng.standard_normal(4 * 8 * 5).astype(np.float32), [4, 8, 5])
    y = ad.bmm(a.permute([0, 2, 1]), b).forward()       # [4, 6, 8] x [4, 8, 5]
    y.keep()
    ad.execute()
    assert "gemm x4" in r.plan and " elw " not in r.plan, r.plan


def test_rewrite_keeps_slices_on_their_rank():
    """Both operands cut along the slice axis: every rank multiplies its own slices, no collective."""
    B, S, D = 8, 5, 3
    rng = np.random.default_rng(5)
    P = adb.ir.IRProcedure
    main = P("main")
    main.push(("CreateMat", rng.standard_normal(B * S * D).astype(np.float32), [B, S, D], "a"))
    main.push(("CreateMat", rng.standard_normal(B * D * S).astype(np.float32), [B, D, S], "b"))
    main.push(("BatchDot", "a", "b", "y"))
    blob = adb.ir.serialize(main, ["y"], inline_limit=1 << 40)[0]
    one = OracleDevice()
    one.execute_blob(blob)
    want = one.get_tensor("y").numpy().reshape(B, S, S)
    for rank in range(2):
        dev = OracleDevice()
        dev.execute_blob(adb.devices.shard_ir(blob, rank, 2, B))
        got = dev.get_tensor("y").numpy().reshape(B // 2, S, S)
        np.testing.assert_array_equal(got, want[rank * (B // 2):(rank + 1) * (B // 2)])
