"""Element-wise work folded into the dot product's epilogue (the reference's `DPElwExpr`,
src/kernel/fusion/dp_elw.rs:13-150): bias + activation on the finished sum, the scaled product, and the in-place
`W += c * (A . B)` -- every operand layout, ragged edges, k loops of several accumulation chunks, split k ranges --
against float64, and against the same program with the fusion left out."""
import numpy as np
import pytest

from helpers import ad, adb, b200, oracle, assert_rel

pytestmark = pytest.mark.gpu
RNG = np.random.default_rng(41)
_simt = None


def _device(kind):
    global _simt
    if kind == "tc":
        return b200()
    if _simt is None:
        _simt = adb.devices.B200(0, flags=adb.devices.FLAG_SIMT_DOT)
    return _simt


def _operands(M, K, N, ta, tb):
    a = RNG.standard_normal(M * K).astype(np.float32)
    b = (RNG.standard_normal(K * N) / np.sqrt(K)).astype(np.float32)
    A64 = (a.reshape(K, M).T if ta else a.reshape(M, K)).astype(np.float64)
    B64 = (b.reshape(N, K).T if tb else b.reshape(K, N)).astype(np.float64)
    return a, b, A64, B64


def _tensors(a, b, M, K, N, ta, tb):
    A = ad.tensor(a, [K, M] if ta else [M, K])
    B = ad.tensor(b, [N, K] if tb else [K, N])
    return (A.t() if ta else A), (B.t() if tb else B)


@pytest.mark.parametrize("kind", ["tc", "simt"])
@pytest.mark.parametrize("keep_product", [False, True], ids=["activation-only", "product-kept-too"])
@pytest.mark.parametrize("M,K,N,ta,tb", [(256, 512, 512, False, False), (1536, 4096, 1800, False, False), (2304, 2500, 1000, True, False),
                                         (2048, 3200, 1160, False, True), (128, 1024, 256, False, False), (520, 96, 260, True, True),
                                         (384, 4096, 1000, False, False)])
def test_bias_and_sigmoid_run_in_the_epilogue(M, K, N, ta, tb, keep_product, kind):
    if kind == "simt" and M * K * N > 1 << 28:
        pytest.skip("CUDA-core kernel: small cases only")
    # few tiles and a long k loop: the kernels split k over the SMs instead, which rules out a chain on the finished sum
    split_instead = ((M + 255) // 256) * ((N + 255) // 256) * 4 <= 148 and K >= 2048
    a, b, A64, B64 = _operands(M, K, N, ta, tb)
    bias = RNG.standard_normal(N).astype(np.float32)
    dev = _device(kind)
    ad.set_device(dev)
    ad.eager_dep_opt()
    A, B = _tensors(a, b, M, K, N, ta, tb)
    z = ad.dot(A, B)
    y = (z + ad.tensor(bias, [N])).sigmoid()
    y.forward()
    y.val().keep()
    if keep_product:
        z.val().keep()
    ad.execute()
    plan = dev.dump_plan()
    assert ("epilogue:" in plan and "recip" in plan) == (not split_instead), plan
    assert ("plain product kept" in plan) == (keep_product and not split_instead), plan
    zr = A64 @ B64
    yr = 1.0 / (1.0 + np.exp(-(zr + bias.astype(np.float64))))
    got = np.asarray(y.val().get().data, np.float64).reshape(M, N)
    # the sigmoid's slope is at most 1/4: an error of 1e-4 |z|max in z moves y by less than that
    assert np.abs(got - yr).max() < 1e-4 * max(1.0, np.abs(zr).max())
    if keep_product:
        gz = np.asarray(z.val().get().data, np.float64).reshape(M, N)
        assert np.abs(gz - zr).max() / np.abs(zr).max() < 4.5e-5


def test_epilogue_agrees_with_the_unfused_program_and_the_oracle():
    """relu-like chain with a saved value (x * (x > 0)) and a squared product (x * x): chains that need the running
    value twice."""
    M, K, N = 320, 1536, 200
    a, b, A64, B64 = _operands(M, K, N, False, False)
    bias = RNG.standard_normal(N).astype(np.float32)

    def prog(dev):
        ad.set_device(dev)
        ad.eager_dep_opt()
        A, B = _tensors(a, b, M, K, N, False, False)
        z = ad.dot(A, B) + ad.tensor(bias, [N])
        y = (z * z).forward()
        y.keep()
        ad.execute()
        return {"y": y.get()}
    want = prog(oracle())
    got = prog(b200())
    assert "save" in b200().dump_plan()
    assert_rel("y", got["y"], want["y"], 1e-4)


@pytest.mark.parametrize("kind", ["tc", "simt"])
@pytest.mark.parametrize("B,K2,N", [(512, 640, 520), (1024, 256, 256), (768, 200, 1000), (300, 384, 136)])
def test_sgd_update_runs_in_the_epilogue(B, K2, N, kind):
    """`W += -1 * (lr * dot(x^T, g))` with a k axis of one accumulation chunk (<= 1024): the gradient is never written,
    the product adds its scaled sum straight into W, which must not be cleared first."""
    x = RNG.standard_normal(B * K2).astype(np.float32)
    g = (RNG.standard_normal(B * N) / np.sqrt(B)).astype(np.float32)
    w0 = RNG.standard_normal(K2 * N).astype(np.float32)
    lr = 0.25
    dev = _device(kind)
    ad.set_device(dev)
    ad.eager_dep_opt()
    w = ad.tensor(w0, [K2, N])
    X = ad.tensor(x, [B, K2])
    G = ad.tensor(g, [B, N])
    w += -1.0 * (lr * ad.dot(X.t(), G))
    w.forward()
    w.val().keep()
    ad.execute()
    plan = dev.dump_plan()
    assert "+= product" in plan, plan
    assert dev.stats()["kernel_launches"] <= 2       # the dot product (and the clearing it must NOT do is a memset, not a kernel)
    ref = w0.reshape(K2, N).astype(np.float64) - lr * (x.reshape(B, K2).astype(np.float64).T @ g.reshape(B, N).astype(np.float64))
    got = np.asarray(w.val().get().data, np.float64).reshape(K2, N)
    assert np.abs(got - ref).max() / np.abs(ref).max() < 4.5e-5


@pytest.mark.parametrize("lr", [0.25, 1e-5], ids=["large-update", "update-of-a-few-hundred-ulps"])
@pytest.mark.parametrize("B,K2,N", [(4096, 512, 384), (8192, 256, 256), (3000, 200, 1000), (65536, 128, 256)])
def test_sgd_update_over_several_k_chunks_is_added_once(B, K2, N, lr):
    """A k axis of several accumulation chunks (or k ranges split over the SMs): adding every chunk's partial sum to W
    on its own would round each at the precision of W -- an update of a few hundred ulps of W, spread over 64 chunks,
    came out percents off.  The gradient is finished first (its scale still rides in the product's epilogue) and
    added once: the UPDATE W received is within 4.5e-5 of its largest entry plus half an ulp of W."""
    x = RNG.standard_normal(B * K2).astype(np.float32)
    g = (RNG.standard_normal(B * N) / np.sqrt(B)).astype(np.float32)
    w0 = RNG.standard_normal(K2 * N).astype(np.float32)
    dev = b200()
    ad.set_device(dev)
    ad.eager_dep_opt()
    w = ad.tensor(w0, [K2, N])
    w += -1.0 * (lr * ad.dot(ad.tensor(x, [B, K2]).t(), ad.tensor(g, [B, N])))
    w.forward()
    w.val().keep()
    ad.execute()
    assert "+= product" not in dev.dump_plan(), dev.dump_plan()
    du_ref = -lr * (x.reshape(B, K2).astype(np.float64).T @ g.reshape(B, N).astype(np.float64))
    du_got = np.asarray(w.val().get().data, np.float64).reshape(K2, N) - w0.reshape(K2, N).astype(np.float64)
    half_ulp = np.abs(w0.reshape(K2, N)).astype(np.float64) * 2.0 ** -24 * 1.01
    assert (np.abs(du_got - du_ref) <= 4.5e-5 * np.abs(du_ref).max() + half_ulp).all()


@pytest.mark.parametrize("B,K2,N", [(4096, 512, 384), (16384, 256, 256)])
def test_scaled_product_is_written_directly(B, K2, N):
    """`t = -1 * (lr * dot(x^T, g))` kept as a tensor of its own (what an all-reduce consumes): no scale pass."""
    x = RNG.standard_normal(B * K2).astype(np.float32)
    g = (RNG.standard_normal(B * N) / np.sqrt(B)).astype(np.float32)
    dev = b200()
    ad.set_device(dev)
    ad.eager_dep_opt()
    t = (-1.0 * (0.5 * ad.dot(ad.tensor(x, [B, K2]).t(), ad.tensor(g, [B, N])))).forward()
    t.keep()
    ad.execute()
    assert "= product ; *" in dev.dump_plan(), dev.dump_plan()
    assert dev.stats()["kernel_launches"] == 1
    ref = -0.5 * (x.reshape(B, K2).astype(np.float64).T @ g.reshape(B, N).astype(np.float64))
    got = np.asarray(t.get().data, np.float64).reshape(K2, N)
    assert np.abs(got - ref).max() / np.abs(ref).max() < 4.5e-5


@pytest.mark.parametrize("B,S,D", [(6, 10, 4), (16, 128, 64), (96, 256, 64), (4, 1024, 512)])
def test_batched_product_with_gradients(B, S, D):
    """BatchDot (attention-shaped: scores = Q K^T, out = scores V, and both gradients): many small slices run as one
    launch of the CUDA-core kernel, few large ones on the tensor cores; against the oracle."""
    rng = np.random.default_rng(B * 1000 + S)
    q, k, v = ((rng.standard_normal(B * S * D) / np.sqrt(D)).astype(np.float32) for _ in range(3))

    def prog(dev):
        ad.set_device(dev)
        ad.eager_dep_opt()
        Q, K, V = (ad.tensor(x, [B, S, D]) for x in (q, k, v))
        out = ad.bmm(ad.bmm(Q, K.permute([0, 2, 1])) * (1.0 / np.sqrt(D)), V)
        loss = (out * out).sum(2).sum(1).sum(0)
        loss.forward()
        loss.backward()
        keep = {"out": out.val(), "dq": Q.grad(), "dk": K.grad(), "dv": V.grad()}
        for t in keep.values():
            t.keep()
        ad.execute()
        return {n: t.get() for n, t in keep.items()}
    want = prog(oracle())
    got = prog(b200())
    assert "gemm x%d" % B in b200().dump_plan()
    for name in want:
        assert_rel(name, got[name], want[name], 1e-4)
