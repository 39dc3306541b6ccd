"""The tcgen05 3xTF32 dot product: every operand majorness, ragged edges, long K, against float64."""
import numpy as np
import pytest

from helpers import ad, adb, b200, oracle, assert_rel

pytestmark = pytest.mark.gpu
RNG = np.random.default_rng(23)
_single = None
# The dot products are held to 1e-4 of the largest element.  What the kernels deliver is set by how many k elements the
# tensor core accumulates (with truncation) before the partial sum is added into C with a rounded add: 3e-5 with the
# default chunks of 4096, 8e-6 with ADB_FLAG_SHORT_DOT_CHUNKS (1024), whatever K is.
DOT_TOL = 4.5e-5
SHORT_CHUNK_TOL = 1.5e-5


def _device(kernel):
    """"pair": the default handle (two SMs per 256 x 256 tile whenever M > 128); "single": one SM per 128 x 256 tile."""
    global _single
    if kernel == "pair":
        return b200()
    if _single is None:
        _single = adb.devices.B200(0, flags=adb.devices.FLAG_SINGLE_SM_DOT)
    return _single


def _dot(dev, a, b, ta, tb, M, K, N):
    ad.set_device(dev)
    ad.eager_dep_opt()
    A = ad.tensor(a, [K, M] if ta else [M, K])
    B = ad.tensor(b, [N, K] if tb else [K, N])
    y = ad.dot(A.t() if ta else A, B.t() if tb else B)
    y.forward()
    y.val().keep()
    ad.execute()
    return y.val().get()


@pytest.mark.parametrize("kernel", ["pair", "single"])
@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
@pytest.mark.parametrize("M,K,N", [(128, 64, 256), (256, 32, 512), (200, 100, 300), (384, 1024, 520), (96, 4096, 1000),
                                   (260, 96, 136), (1024, 3200, 392), (640, 2048, 1000)])
def test_tc_dot_matches_float64(M, K, N, ta, tb, kernel):
    a = RNG.standard_normal(M * K).astype(np.float32)
    b = RNG.standard_normal(K * N).astype(np.float32)
    dev = _device(kernel)
    got = _dot(dev, a, b, ta, tb, M, K, N)
    assert dev.stats()["tc_gemm_launches"] == 1, "expected the tensor-core kernel for this shape"
    A = a.reshape(K, M).T if ta else a.reshape(M, K)
    B = b.reshape(N, K).T if tb else b.reshape(K, N)
    ref = A.astype(np.float64) @ B.astype(np.float64)
    g = np.asarray(got.data, np.float64).reshape(M, N)
    err = np.abs(g - ref).max() / np.abs(ref).max()
    # fp32-level: the tensor core truncates when it accumulates, the kernel bounds that by flushing the
    # accumulator every 4096 k-elements; what remains is <= 3e-5 of the largest element for any K
    assert err < DOT_TOL, f"relative error {err:.3e} (3xTF32 should be at fp32 level)"


@pytest.mark.parametrize("kernel", ["pair", "single"])
@pytest.mark.parametrize("M,K,N,ta,tb", [(256, 16384, 256, False, False), (128, 65536, 256, True, False), (512, 65536, 128, True, False)])
def test_tc_dot_error_does_not_grow_with_k(M, K, N, ta, tb, kernel):
    a = RNG.standard_normal(M * K).astype(np.float32)
    b = RNG.standard_normal(K * N).astype(np.float32)
    dev = _device(kernel)
    got = _dot(dev, a, b, ta, tb, M, K, N)
    assert dev.stats()["tc_gemm_launches"] == 1
    A = a.reshape(K, M).T if ta else a.reshape(M, K)
    B = b.reshape(N, K).T if tb else b.reshape(K, N)
    ref = A.astype(np.float64) @ B.astype(np.float64)
    g = np.asarray(got.data, np.float64).reshape(M, N)
    err = np.abs(g - ref).max() / np.abs(ref).max()
    assert err < DOT_TOL, f"relative error {err:.3e} at K={K}"


def test_tc_dot_matches_oracle_and_simt():
    M, K, N = 256, 512, 512
    a = RNG.standard_normal(M * K).astype(np.float32)
    b = RNG.standard_normal(K * N).astype(np.float32)
    want = _dot(oracle(), a, b, False, False, M, K, N)
    got = _dot(b200(), a, b, False, False, M, K, N)
    assert_rel("tc vs oracle", got, want, 1e-4)
    adb = __import__("importlib").import_module("autodiff-ir-rust_b200")
    simt = adb.devices.B200(0, flags=adb.devices.FLAG_SIMT_DOT)
    try:
        ref = _dot(simt, a, b, False, False, M, K, N)
        assert simt.stats()["tc_gemm_launches"] == 0
    finally:
        simt.close()
    assert_rel("tc vs simt", got, ref, 1e-5)


@pytest.mark.parametrize("M,kernel", [(128, "single"), (768, "single"), (768, "pair")])
def test_tc_dot_exact_on_small_integers(M, kernel):
    """Products of small integers are exact in every term of the split: the result must be exact."""
    K, N = 256, 512
    a = RNG.integers(-8, 9, M * K).astype(np.float32)
    b = RNG.integers(-8, 9, K * N).astype(np.float32)
    got = _dot(_device(kernel), a, b, False, False, M, K, N)
    ref = a.reshape(M, K).astype(np.int64) @ b.reshape(K, N).astype(np.int64)
    np.testing.assert_array_equal(np.asarray(got.data).reshape(M, N), ref.astype(np.float32))


@pytest.mark.parametrize("M,K,N,ta,tb", [(512, 8192, 512, False, False), (300, 5000, 200, False, False), (256, 4096, 256, True, True),
                                         (384, 20000, 136, True, False)])
def test_few_tiles_long_k_is_split_across_clusters(M, K, N, ta, tb):
    """Fewer tiles than half the SM pairs and K >= 2048: the paired kernel cuts k into ranges that different
    clusters accumulate into a zeroed C.  Same accuracy bar; the single-SM kernel (no split) must agree."""
    a = RNG.standard_normal(M * K).astype(np.float32)
    b = RNG.standard_normal(K * N).astype(np.float32)
    got = _dot(_device("pair"), a, b, ta, tb, M, K, N)
    ref1 = _dot(_device("single"), a, b, ta, tb, M, K, N)
    A = a.reshape(K, M).T if ta else a.reshape(M, K)
    B = b.reshape(N, K).T if tb else b.reshape(K, N)
    ref = A.astype(np.float64) @ B.astype(np.float64)
    g = np.asarray(got.data, np.float64).reshape(M, N)
    assert np.abs(g - ref).max() / np.abs(ref).max() < DOT_TOL
    assert_rel("pair vs single", got, ref1, DOT_TOL)


@pytest.mark.parametrize("M,K,N,ta", [(128, 16384, 512, False), (64, 8192, 1000, False), (96, 30000, 256, True)])
def test_single_sm_kernel_splits_long_k_too(M, K, N, ta):
    a = RNG.standard_normal(M * K).astype(np.float32)
    b = RNG.standard_normal(K * N).astype(np.float32)
    dev = _device("pair")      # M <= 128 runs the single-SM kernel on any handle
    got = _dot(dev, a, b, ta, False, M, K, N)
    assert dev.stats()["tc_gemm_launches"] == 1
    A = a.reshape(K, M).T if ta else a.reshape(M, K)
    ref = A.astype(np.float64) @ b.reshape(K, N).astype(np.float64)
    g = np.asarray(got.data, np.float64).reshape(M, N)
    assert np.abs(g - ref).max() / np.abs(ref).max() < DOT_TOL


def test_a_dot_kernel_that_gave_up_is_reported_and_the_handle_stays_usable():
    """The host side of the bounded-wait path: the status word the kernels write on a time-out is set from the host
    (no kernel waits for anything), the next execute with a tensor-core product must fail with ADB_ERR_CUDA and name
    the code, and the execute after that must succeed with correct numbers."""
    from helpers import adb
    dev = adb.devices.B200(0)
    try:
        prog = lambda d: adb.configs.c5_dot_loop(d, n=256, max_iters=2)   # noqa: E731
        good = prog(dev)
        assert dev.stats()["tc_gemm_launches"] > 0
        dev.inject_dot_status(3)
        with pytest.raises(adb.devices.AdbError) as e:
            prog(dev)
        assert e.value.status == 3 and "code 3" in str(e.value), str(e.value)
        again = prog(dev)
        for k in good:
            np.testing.assert_array_equal(np.asarray(again[k].data), np.asarray(good[k].data))
    finally:
        dev.close()


@pytest.mark.parametrize("M,K,N", [(512, 1024, 1001), (384, 1001, 512), (1001, 515, 260)])
def test_rows_that_are_not_a_multiple_of_four_are_padded_not_demoted(M, K, N):
    """1001 columns: TMA cannot fetch rows that start on odd 4-byte boundaries, so the operand is copied once into a
    temporary with padded rows and the product still runs on the tensor cores (it used to fall back to the CUDA-core
    kernel)."""
    a = RNG.standard_normal(M * K).astype(np.float32)
    b = RNG.standard_normal(K * N).astype(np.float32)
    dev = _device("pair")
    got = _dot(dev, a, b, False, False, M, K, N)
    assert dev.stats()["tc_gemm_launches"] == 1, dev.dump_plan()
    ref = a.reshape(M, K).astype(np.float64) @ b.reshape(K, N).astype(np.float64)
    g = np.asarray(got.data, np.float64).reshape(M, N)
    assert np.abs(g - ref).max() / np.abs(ref).max() < DOT_TOL


@pytest.mark.parametrize("M,K,N,ta", [(8192, 8192, 1, False), (1, 8192, 8192, False), (4096, 3000, 1, True), (1, 512, 1000, False)])
def test_matrix_vector_products_run_as_row_sums(M, K, N, ta):
    """N = 1 or M = 1: one pass over the matrix through the reduce kernels (row sums of products) instead of a tile
    kernel; against float64."""
    a = RNG.standard_normal(M * K).astype(np.float32)
    b = RNG.standard_normal(K * N).astype(np.float32)
    dev = _device("pair")
    got = _dot(dev, a, b, ta, False, M, K, N)
    plan = dev.dump_plan()
    assert "gemm" not in plan and ("adb_rowsum_" in plan or "adb_colsum_" in plan), plan
    A = a.reshape(K, M).T if ta else a.reshape(M, K)
    ref = A.astype(np.float64) @ b.reshape(K, N).astype(np.float64)
    g = np.asarray(got.data, np.float64).reshape(M, N)
    assert got.dim == [M, N]
    assert np.abs(g - ref).max() / np.abs(ref).max() < 1e-5


def test_deterministic_flag_gives_the_same_bits_on_every_run():
    """512 x 8192 x 512 is cut into k ranges by default (partial sums meet in C in timing order); with
    FLAG_DETERMINISTIC one cluster owns each tile and ten runs give bit-identical results within the accuracy bar."""
    M, K, N = 512, 8192, 512
    a = RNG.standard_normal(M * K).astype(np.float32)
    b = RNG.standard_normal(K * N).astype(np.float32)
    dev = adb.devices.B200(0, flags=adb.devices.FLAG_DETERMINISTIC)
    try:
        runs = [np.asarray(_dot(dev, a, b, False, False, M, K, N).data, np.float32).copy() for _ in range(10)]
    finally:
        dev.close()
    for r in runs[1:]:
        np.testing.assert_array_equal(r, runs[0])
    ref = a.reshape(M, K).astype(np.float64) @ b.reshape(K, N).astype(np.float64)
    assert np.abs(runs[0].reshape(M, N) - ref).max() / np.abs(ref).max() < DOT_TOL


@pytest.mark.parametrize("M,K,N", [(512, 16384, 512), (256, 65536, 384)])
def test_short_accumulation_chunks_buy_accuracy(M, K, N):
    """ADB_FLAG_SHORT_DOT_CHUNKS: the accumulator is added into C every 1024 k elements instead of every 4096; the error
    (truncation inside the tensor core, proportional to the chunk length) drops about fourfold."""
    a = RNG.standard_normal(M * K).astype(np.float32)
    b = RNG.standard_normal(K * N).astype(np.float32)
    ref = a.reshape(M, K).astype(np.float64) @ b.reshape(K, N).astype(np.float64)
    errs = {}
    # (one owner per tile: a k axis split over clusters would cut the long chunks into ranges of 1024 anyway)
    det = adb.devices.FLAG_DETERMINISTIC
    for name, flags in (("long", det), ("short", det | adb.devices.FLAG_SHORT_DOT_CHUNKS)):
        dev = adb.devices.B200(0, flags=flags)
        try:
            g = np.asarray(_dot(dev, a, b, False, False, M, K, N).data, np.float64).reshape(M, N)
        finally:
            dev.close()
        errs[name] = np.abs(g - ref).max() / np.abs(ref).max()
    assert errs["short"] < SHORT_CHUNK_TOL, errs
    assert errs["long"] < DOT_TOL, errs
    assert errs["short"] < 0.6 * errs["long"], errs
