"""The lowering, checked numerically without a GPU: every plan is executed on the CPU by the interpreter in
tests/hostcheck/plan_interp.hpp (same arena layout, same partial-sum layouts as the generated kernels, arena poisoned
with NaN) and the kept tensors are compared with the CPU oracle -- the reference's known-answer programs, the benchmark
programs at sizes that reach every fusion pass, and a few hundred random programs, with and without the passes."""
import importlib
import os
import struct
import subprocess

import numpy as np
import pytest

import fuzz_programs
import ref_programs
from oracle.oracle import OracleDevice

adb = importlib.import_module("autodiff-ir-rust_b200")
ad, nn, cfg = adb.autodiff, adb.nn, adb.configs


class _Both(OracleDevice):
    """Runs the program on the oracle and keeps the self-contained blob for the interpreter."""

    def __init__(self):
        super().__init__()
        self.blobs = []

    def execute(self, proc, dep):
        self.blobs.append(adb.ir.serialize(proc, dep, inline_limit=1 << 40)[0])
        super().execute(proc, dep)


def _read_results(path):
    out = {}
    data = open(path, "rb").read()
    pos = 0
    while pos < len(data):
        (n,) = struct.unpack_from("<I", data, pos); pos += 4
        name = data[pos:pos + n].decode(); pos += n
        (nd,) = struct.unpack_from("<I", data, pos); pos += 4
        dims = struct.unpack_from("<%dQ" % nd, data, pos); pos += 8 * nd
        defined = data[pos]; pos += 1
        if defined:
            cnt = int(np.prod(dims)) if nd else 1
            out[name] = (list(dims), np.frombuffer(data, np.float32, cnt, pos).copy()); pos += 4 * cnt
    return out


def _interpret(binary, tmp_path, blob, flags, tag):
    f = tmp_path / f"{tag}.adir"
    f.write_bytes(blob)
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1", UBSAN_OPTIONS="print_stacktrace=1")
    r = subprocess.run([binary, str(flags | 8), "1", "0", str(f)], capture_output=True, text=True, env=env, timeout=900)
    assert r.returncode == 0, r.stderr[-3000:]
    assert "executed=1" in r.stdout, r.stdout
    return _read_results(str(f) + ".out")


def _compare(got, kept, tol, atol=0.0):
    for name, v in kept.items():
        if v.is_none:
            continue
        assert name in got, f"{name} missing from the interpreted plan"
        dims, data = got[name]
        assert dims == list(v.dim), (name, dims, v.dim)
        want = np.asarray(v.data, np.float64)
        if not np.isfinite(want).all():
            continue
        scale = max(float(np.abs(want).max()), 1e-30) if want.size else 1.0
        diff = float(np.abs(data.astype(np.float64) - want).max()) if want.size else 0.0
        assert diff <= tol * scale + atol, f"{name}: error {diff:.3e} on a tensor of magnitude {scale:.3e}"


@pytest.mark.parametrize("flags", [0, 1, 2, 32], ids=["default", "one-kernel-per-command", "fusions-at-any-size", "one-launch-per-kernel"])
def test_reference_and_benchmark_programs(hostcheck, tmp_path, flags):
    programs = [(n, ref_programs.ALL[n], {}) for n in sorted(ref_programs.ALL)]
    programs += [("c1", cfg.c1_readme_mlp, {}),
                 ("c2", cfg.c2_fused_elementwise, dict(rows=96, cols=136)),
                 ("c3", cfg.c3_reduce_movement, dict(batch=8, n=16)),
                 ("c4", cfg.c4_mlp_train, dict(batch=96, widths=(24, 40, 40, 24, 8), steps=3, lr=1e-2)),
                 ("c5", cfg.c5_dot_loop, dict(n=24, max_iters=4))]
    for name, fn, kw in programs:
        dev = _Both()
        kept = fn(dev, **kw)
        got = _interpret(hostcheck, tmp_path, dev.blobs[-1], flags, name)
        if isinstance(kept, dict):
            by_id = {v.id: v for v in kept.values() if hasattr(v, "id")}
            # (the known-answer programs return values rounded to four decimals, as the reference's tests compare them)
            _compare(got, by_id, 1e-4, atol=6e-5)
        assert got, name


def test_fusions_at_their_real_thresholds(hostcheck, tmp_path):
    """Sizes at which the sum fusion and the row chains switch on by themselves."""
    dev = _Both()
    kept = cfg.c2_fused_elementwise(dev, rows=520, cols=1000)
    _compare(_interpret(hostcheck, tmp_path, dev.blobs[-1], 0, "c2big"), {v.id: v for v in kept.values()}, 1e-4)
    dev = _Both()
    ad.set_device(dev)
    ad.eager_dep_opt()
    x = np.random.default_rng(5).standard_normal(300 * 1024).astype(np.float32)
    y = nn.LayerNorm(1024).f(ad.tensor(x, [300, 1024])).forward()
    y.keep()
    ad.execute()
    _compare(_interpret(hostcheck, tmp_path, dev.blobs[-1], 0, "ln"), {y.id: y.get()}, 1e-4)


@pytest.mark.parametrize("chunk", range(6))
def test_random_programs(hostcheck, tmp_path, chunk):
    """50 random programs per case, each through the default lowering and with every fusion at any size."""
    for seed in range(chunk * 50, chunk * 50 + 50):
        exact = seed % 2 == 0
        dev = _Both()
        with np.errstate(all="ignore"):
            kept = fuzz_programs.build(seed if exact else 1000 + seed, exact=exact)(dev)
        by_id = {v.id: v for v in kept.values()}
        for flags in (0, 2, 128):          # default, every fusion at any size, tiny dot products as dot-product steps
            got = _interpret(hostcheck, tmp_path, dev.blobs[-1], flags, f"fz{seed}_{flags}")
            _compare(got, by_id, 0.0 if exact else 1e-4)


@pytest.mark.parametrize("P,Q", [(7, 5), (33, 131), (40, 64), (3, 1000)])
def test_side_sums_and_row_chains_on_ragged_shapes(hostcheck, tmp_path, P, Q):
    """Element-wise passes with row and column side sums, and max / sum row chains, on shapes that are not multiples
    of the vector width or the tile sizes (fusions forced on at any size)."""
    rng = np.random.default_rng(P * 1000 + Q)
    x = rng.standard_normal(P * Q).astype(np.float32)
    w = rng.standard_normal(Q).astype(np.float32)
    dev = _Both()
    ad.set_device(dev)
    ad.eager_dep_opt()
    t = ad.tensor(x, [P, Q])
    tw = ad.tensor(w, [Q]).view([1, Q]).broadcast(0, P)
    y = ((t * tw + 0.5).sin() * t).forward()
    rows = y.to_node().sum(1).forward() if hasattr(y, "to_node") else None
    cols = (y.to_node() * y.to_node()).sum(0).forward()
    m = t.max(1)
    e = (t - m.unsqueeze(-1).broadcast(-1, Q)).exp()
    sm = (e * e.sum(1).recip().unsqueeze(-1).broadcast(-1, Q)).forward()
    kept = {}
    for v in (y, rows, cols, sm):
        v.keep()
    ad.execute()
    kept = {v.id: v.get() for v in (y, rows, cols, sm)}
    for flags in (0, 2):
        _compare(_interpret(hostcheck, tmp_path, dev.blobs[-1], flags, f"ragged{flags}"), kept, 1e-4)


def test_random_loop_programs(hostcheck, tmp_path):
    """In-place updates, sums and maxima fed back through broadcasts inside IR loops: default lowering, one kernel
    per command, and every fusion at any size."""
    ran = 0
    for seed in range(150):
        dev = _Both()
        try:
            with np.errstate(all="ignore"):
                kept = fuzz_programs.build_loop(seed)(dev)
        except RecursionError:
            continue            # a cyclic update the frontend cannot trace
        ran += 1
        by_id = {v.id: v for v in kept.values()}
        for flags in (0, 1, 2):
            _compare(_interpret(hostcheck, tmp_path, dev.blobs[-1], flags, f"loop{seed}_{flags}"), by_id, 2e-4)
    assert ran >= 30


REFUSAL = "is a view when control flow joins"


def _interpret_or_refused(binary, tmp_path, blob, flags, tag):
    """Interpreted results, or None when the lowering refused the program as path-dependent (a view that one path
    rebinds while another path changes its source)."""
    f = tmp_path / f"{tag}.adir"
    f.write_bytes(blob)
    r = subprocess.run([binary, str(flags | 8), "1", "0", str(f)], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-3000:]
    if "rejected:" in r.stdout:
        assert REFUSAL in r.stdout, r.stdout
        return None
    assert "executed=1" in r.stdout, r.stdout
    return _read_results(str(f) + ".out")


def test_raw_ir_programs_with_reused_ids_and_views_across_blocks(hostcheck, tmp_path):
    """Programs written as IR commands directly: result ids reused, op-assigns on views, views created inside
    branches, branches not taken, loops that run zero times, products written onto their own operands.  Every
    program either interprets to exactly the oracle's result or is refused with the one documented reason."""
    refused = 0
    seeds = range(120)
    for seed in seeds:
        dev = _Both()
        kept = fuzz_programs.build_raw(seed)(dev)
        for flags in (0, 2, 128):
            got = _interpret_or_refused(hostcheck, tmp_path, dev.blobs[-1], flags, f"raw{seed}_{flags}")
            if got is None:
                refused += 1
                break
            _compare(got, kept, 0.0)
    assert refused <= len(seeds) // 4, refused


def _raw(cmds, dep):
    main = adb.ir.IRProcedure("main")
    for c in cmds:
        main.push(c)
    return main, dep


def _block(*cmds):
    b = adb.ir.IRProcedure("blk")
    for c in cmds:
        b.push(c)
    return b


M4 = np.arange(16, dtype=np.float32).reshape(4, 4) - 5.0


@pytest.mark.parametrize("count", [0, 1, 3])
def test_op_assign_on_a_view_inside_a_loop_is_carried_around(hostcheck, tmp_path, count):
    """v5 = Permute(v4); While c {v5 += v5; c += -1}: v5 doubles on every pass (and stays v4^T when the loop never runs)."""
    proc, dep = _raw([("CreateMat", M4, [4, 4], "v4"), ("CreateMat", np.array([count], np.float32), [1], "c"),
                      ("CreateConstant", -1.0, "k", [1]), ("Permute", "v4", [1, 0], "v5"),
                      ("While", "c", _block(("ElwAddEq", "v5", "v5"), ("ElwAddEq", "c", "k")))], ["v5", "v4"])
    dev = _Both()
    dev.execute(proc, dep)
    kept = {d: dev.get_tensor(d) for d in dep}
    assert np.array_equal(kept["v5"].numpy().reshape(4, 4), M4.T * 2.0 ** count)
    for flags in (0, 1, 2):
        _compare(_interpret(hostcheck, tmp_path, dev.blobs[-1], flags, f"loopview{flags}"), kept, 0.0)


@pytest.mark.parametrize("flag", [0.0, 1.0])
def test_views_and_branches(hostcheck, tmp_path, flag):
    """An op-assign on a view inside a branch that may not run, and a branch that turns a tensor into a view."""
    proc, dep = _raw([("CreateMat", M4, [4, 4], "v4"), ("CreateMat", M4 * 2, [4, 4], "v2"),
                      ("CreateMat", np.array([flag], np.float32), [1], "f"),
                      ("View", "v4", [4, 4], "v5"), ("ElwAdd", "v2", "v2", "v6"),
                      ("If", [("f", _block(("ElwMultiplyEq", "v5", "v5"), ("Permute", "v2", [1, 0], "v6")))], None),
                      ("ElwAdd", "v5", "v6", "out")], ["out", "v5", "v6"])
    dev = _Both()
    dev.execute(proc, dep)
    kept = {d: dev.get_tensor(d) for d in dep}
    for flags in (0, 1, 2):
        _compare(_interpret(hostcheck, tmp_path, dev.blobs[-1], flags, f"ifview{flags}"), kept, 0.0)


def test_dot_product_onto_its_own_operand(hostcheck, tmp_path):
    """`DotProduct v w -> v` at top level, in a branch and in a loop: the plan never lets a product land in a buffer
    it reads (hostcheck's plan invariant) and the results match."""
    W = (np.arange(16, dtype=np.float32).reshape(4, 4) % 3) - 1.0
    proc, dep = _raw([("CreateMat", M4, [4, 4], "v"), ("CreateMat", W, [4, 4], "w"),
                      ("CreateMat", np.array([1.0], np.float32), [1], "f"), ("CreateMat", np.array([2.0], np.float32), [1], "c"),
                      ("CreateConstant", -1.0, "k", [1]),
                      ("DotProduct", "v", "w", "v"),
                      ("If", [("f", _block(("DotProduct", "w", "v", "v")))], None),
                      ("While", "c", _block(("DotProduct", "v", "w", "v"), ("ElwAddEq", "c", "k")))], ["v"])
    dev = _Both()
    dev.execute(proc, dep)
    kept = {d: dev.get_tensor(d) for d in dep}
    for flags in (0, 1, 2):
        _compare(_interpret(hostcheck, tmp_path, dev.blobs[-1], flags, f"dotself{flags}"), kept, 0.0)


def test_path_dependent_view_is_refused(hostcheck, tmp_path):
    """`If f {v1 = Permute(v3)}; v3 += v3; read v1`: whether v1 follows v3 depends on f; the lowering says so."""
    proc, dep = _raw([("CreateMat", M4, [4, 4], "v1"), ("CreateMat", M4 * 2, [4, 4], "v3"),
                      ("CreateMat", np.array([1.0], np.float32), [1], "f"),
                      ("If", [("f", _block(("Permute", "v3", [1, 0], "v1")))], None),
                      ("ElwAddEq", "v3", "v3"), ("ElwAdd", "v1", "v3", "out")], ["out"])
    blob = adb.ir.serialize(proc, dep, inline_limit=1 << 40)[0]
    assert _interpret_or_refused(hostcheck, tmp_path, blob, 0, "pathdep") is None


def test_view_of_a_view_that_a_loop_rebinds_is_refused(hostcheck, tmp_path):
    """v2 = Permute(v3); v5 = Permute(v2); While c {v3 = v3 . v3; v2 = v5 + v1; ...}: on the first pass v5 looks through
    v2 at the v3 the loop has just changed, from the second pass on at the tensor v2 has become.  The copy of v2 taken in
    front of the loop cannot follow v3, and v5 -- a view made BEFORE the loop -- reads it: refused (this used to lower,
    with the stale v3 in the first pass)."""
    proc, dep = _raw([("CreateMat", M4, [4, 4], "v1"), ("CreateMat", M4 * 0, [4, 4], "v2"), ("CreateMat", M4 + 1, [4, 4], "v3"),
                      ("CreateConstant", -1.0, "k", [1]), ("Permute", "v3", [1, 0], "v2"), ("Permute", "v2", [1, 0], "v5"),
                      ("CreateMat", np.array([2.0], np.float32), [1], "c"),
                      ("While", "c", _block(("DotProduct", "v3", "v3", "v3"), ("ElwAdd", "v5", "v1", "v2"), ("ElwAddEq", "c", "k")))],
                     ["v1", "v2", "v3", "v5"])
    blob = adb.ir.serialize(proc, dep, inline_limit=1 << 40)[0]
    assert _interpret_or_refused(hostcheck, tmp_path, blob, 0, "viewofview") is None


@pytest.mark.parametrize("M,K,N", [(300, 256, 1), (1, 300, 260)])
def test_matrix_vector_products_through_the_reduce_kernels(hostcheck, tmp_path, M, K, N):
    rng = np.random.default_rng(M + N)
    dev = _Both()
    ad.set_device(dev)
    ad.eager_dep_opt()
    a = ad.tensor(rng.standard_normal(M * K).astype(np.float32), [M, K])
    b = ad.tensor(rng.standard_normal(K * N).astype(np.float32), [K, N])
    y = (ad.dot(a, b) * 2.0).forward()
    y.keep()
    ad.execute()
    for flags in (0, 2):
        _compare(_interpret(hostcheck, tmp_path, dev.blobs[-1], flags, f"mv{flags}"), {y.id: y.get()}, 1e-5)


def test_independent_kernels_share_one_launch(hostcheck, tmp_path):
    """Row sums of a, an element-wise kernel over a and b, and a product-fed sum: kernels that do not depend on one
    another become one launch (hostcheck also verifies, for every plan it sees, that no member of such a launch
    touches what another member writes); the flag that turns grouping off gives the same results."""
    rng = np.random.default_rng(3)
    A, B = rng.standard_normal(96).astype(np.float32), rng.standard_normal(96).astype(np.float32)
    proc, dep = _raw([("CreateMat", A, [2, 48], "a"), ("CreateMat", B, [2, 48], "b"), ("CreateConstant", 3.0, "k", [2, 48]),
                      ("ElwMultiply", "a", "a", "x"), ("ElwAdd", "b", "b", "y"), ("Sum", "x", "s"),
                      ("ElwMultiply", "y", "k", "z"), ("ElwAdd", "x", "y", "w")], ["x", "y", "s", "z", "w"])
    dev = _Both()
    dev.execute(proc, dep)
    kept = {d: dev.get_tensor(d) for d in dep}
    assert "group of 2 kernels in one launch" in adb.devices.lower_check(proc, dep)
    assert "group of" not in adb.devices.lower_check(proc, dep, flags=adb.devices.FLAG_NO_GROUPING)
    for flags in (0, 32):
        _compare(_interpret(hostcheck, tmp_path, dev.blobs[-1], flags, f"group{flags}"), kept, 1e-6)


class _BothRanks(_Both):
    """Oracle whose all-reduce multiplies by the number of ranks: every rank holds the same data."""

    def __init__(self, world):
        OracleDevice.__init__(self, allreduce=lambda arr: np.multiply(arr, np.float32(world), out=arr))
        self.blobs = []


def _interpret_ranks(binary, tmp_path, blob, flags, tag, world):
    f = tmp_path / f"{tag}.adir"
    f.write_bytes(blob)
    r = subprocess.run([binary, str(flags | 8), str(world), "0", str(f)], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-3000:] + r.stdout[-2000:]
    assert "executed=1" in r.stdout, r.stdout
    return _read_results(str(f) + ".out")


@pytest.mark.parametrize("world", [2, 4])
def test_bucketed_all_reduces_on_identical_ranks(hostcheck, tmp_path, world):
    """All-reduces written into the IR by hand, on ranks that all hold the same data (the sum over ranks is then
    `world` times the value): three gradients that nothing reads before the update share one collective over adjacent
    buffers (sizes that are not multiples of the arena's alignment: the padding in between is reduced along with them
    and must not leak); a value that is read right after its all-reduce, a kept value and all-reduces inside a loop
    keep their order.  With and without buckets, against the oracle."""
    rng = np.random.default_rng(7)
    A = rng.integers(-3, 4, 70).astype(np.float32)
    B = rng.integers(-3, 4, 3).astype(np.float32)
    C = rng.integers(-3, 4, 130).astype(np.float32)
    loop = _block(("ElwMultiply", "a", "a", "g1"), ("AllReduce", "g1"), ("ElwAdd", "b", "b", "g2"), ("AllReduce", "g2"),
                  ("ElwMultiply", "c", "h", "g3"), ("AllReduce", "g3"),
                  ("ElwAddEq", "a", "g1"), ("ElwAddEq", "b", "g2"), ("ElwAddEq", "c", "g3"), ("ElwAddEq", "n", "k"))
    proc, dep = _raw([("CreateMat", A, [7, 10], "a"), ("CreateMat", B, [3], "b"), ("CreateMat", C, [2, 65], "c"),
                      ("CreateMat", np.array([2.0], np.float32), [1], "n"), ("CreateConstant", -1.0, "k", [1]),
                      ("CreateConstant", 0.5, "h", [2, 65]),
                      ("ElwMultiply", "a", "a", "t1"), ("AllReduce", "t1"),
                      ("ElwAdd", "b", "b", "t2"), ("AllReduce", "t2"),
                      ("ElwMultiply", "c", "c", "t3"), ("AllReduce", "t3"),
                      ("ElwAdd", "t1", "a", "u"), ("ElwMultiply", "t2", "b", "v"), ("ElwAdd", "t3", "c", "w"),
                      ("ElwAdd", "b", "b", "s1"), ("AllReduce", "s1"), ("ElwMultiply", "s1", "s1", "s2"), ("AllReduce", "s2"),
                      ("While", "n", loop)], ["u", "v", "w", "t2", "s2", "a", "b", "c"])
    dev = _BothRanks(world)
    dev.execute(proc, dep)
    kept = {d: dev.get_tensor(d) for d in dep}
    assert np.array_equal(kept["s2"].numpy(), (2 * B * world) ** 2 * world)
    listing = adb.devices.lower_check(proc, dep, world=world)
    assert " + " in "".join(l for l in listing.splitlines() if " allreduce " in l), listing
    for flags in (0, 64, 1):            # buckets, one collective per command, one kernel per command
        _compare(_interpret_ranks(hostcheck, tmp_path, dev.blobs[-1], flags, f"ar{world}_{flags}", world), kept, 0.0)


def test_raw_ir_programs_with_all_reduces_on_identical_ranks(hostcheck, tmp_path):
    """The raw-IR programs with all-reduces sprinkled over their values (top level, branches, loops), on two ranks that
    hold the same data: bucketed and one collective per command, bit for bit against the oracle."""
    refused = 0
    seeds = range(120)
    for seed in seeds:
        dev = _BothRanks(2)
        kept = fuzz_programs.build_raw(seed, allreduce=True)(dev)
        for flags in (0, 64):
            f = tmp_path / f"rawar{seed}_{flags}.adir"
            f.write_bytes(dev.blobs[-1])
            r = subprocess.run([hostcheck, str(flags | 8), "2", "0", str(f)], capture_output=True, text=True, timeout=900)
            assert r.returncode == 0, (seed, r.stderr[-3000:] + r.stdout[-1500:])
            if "rejected:" in r.stdout:
                assert REFUSAL in r.stdout, r.stdout
                refused += 1
                break
            assert "executed=1" in r.stdout, r.stdout
            _compare(_read_results(str(f) + ".out"), kept, 0.0)
    assert refused <= len(seeds) // 4, refused


def test_values_that_read_each_others_buffers_are_written_out_through_a_temporary(hostcheck, tmp_path):
    """a' = b + 1 and b' = (old a) + 1, both still expressions when an all-reduce forces a' into a's buffer: b' must be
    out of the way first (it reads the old a) and cannot go to b's buffer (a' still reads the old b).  The lowering used to
    recurse without end here; one of the two now waits in a temporary."""
    A = np.arange(4, dtype=np.float32)
    B = np.arange(4, dtype=np.float32) * 10
    proc, dep = _raw([("CreateMat", A, [2, 2], "a"), ("CreateMat", B, [2, 2], "b"), ("CreateConstant", 1.0, "c", [2, 2]),
                      ("Contigious", "a", "s"), ("ElwAdd", "b", "c", "a"), ("ElwAdd", "s", "c", "b"), ("AllReduce", "a")],
                     ["a", "b"])
    dev = _BothRanks(2)
    dev.execute(proc, dep)
    kept = {d: dev.get_tensor(d) for d in dep}
    assert np.array_equal(kept["a"].numpy().reshape(-1), 2 * (B + 1)) and np.array_equal(kept["b"].numpy().reshape(-1), A + 1)
    for flags in (0, 1, 64):
        _compare(_interpret_ranks(hostcheck, tmp_path, dev.blobs[-1], flags, f"swap{flags}", 2), kept, 0.0)


def test_raw_ir_programs_with_sums_rows_and_concats(hostcheck, tmp_path):
    """The raw-IR generator with its richer command mix (row sums broadcast back, single rows repeated, halves cut out
    of a concat -- all as alias chains, inside and outside of branches and loops): default lowering and one kernel per
    command with tiny dot products as dot-product steps, bit for bit or refused for the one documented reason."""
    refused = 0
    seeds = range(100)
    for seed in seeds:
        dev = _Both()
        kept = fuzz_programs.build_raw(seed, rich=True)(dev)
        for flags in (0, 129):
            got = _interpret_or_refused(hostcheck, tmp_path, dev.blobs[-1], flags, f"rich{seed}_{flags}")
            if got is None:
                refused += 1
                break
            _compare(got, kept, 0.0)
    assert refused <= len(seeds) // 3, refused


def test_a_value_computed_twice_survives_a_loop_with_one_kernel_per_command(hostcheck, tmp_path):
    """`v3 = v2 + v2` twice, then a loop: with one kernel per command the second command finds the first one's result
    in memory and v3 stays bound to the expression that forwards to it; the loop moves every buffer version on, and the
    id must follow to the buffer, not fall back to the expression with its outdated operands."""
    proc, dep = _raw([("CreateMat", M4, [4, 4], "v2"), ("ElwAdd", "v2", "v2", "v3"), ("ElwAdd", "v2", "v2", "v3"),
                      ("CreateMat", np.array([1.0], np.float32), [1], "c"), ("CreateConstant", -1.0, "k", [1]),
                      ("While", "c", _block(("ElwAddEq", "c", "k")))], ["v2", "v3"])
    dev = _Both()
    dev.execute(proc, dep)
    kept = {d: dev.get_tensor(d) for d in dep}
    for flags in (0, 1):
        _compare(_interpret(hostcheck, tmp_path, dev.blobs[-1], flags, f"twice{flags}"), kept, 0.0)


def test_tensors_without_elements(hostcheck, tmp_path):
    """A [0, 4] tensor through element-wise work, a sum, a concat with a non-empty tensor: shapes come back as the oracle
    has them, nothing is launched for the empty parts."""
    E = np.zeros(0, np.float32)
    proc, dep = _raw([("CreateMat", E, [0, 4], "a"), ("CreateMat", np.arange(4, dtype=np.float32), [1, 4], "b"),
                      ("ElwAdd", "a", "a", "c"), ("Sum", "a", "s"), ("ElwAdd", "b", "b", "d"),
                      ("Concat", "a", "b", 0, "e"), ("Contigious", "e", "f"),
                      # products and sums over an axis of length 0 (all zeros; -inf for a maximum) and with no rows
                      ("CreateMat", E, [3, 0], "p"), ("CreateMat", E, [0, 4], "q"), ("DotProduct", "p", "q", "pq"),
                      ("CreateMat", np.ones(8, np.float32), [4, 2], "w"), ("DotProduct", "a", "w", "aw"),
                      ("Sum", "p", "ps"), ("Max", "p", "pm")], ["c", "s", "d", "f", "pq", "aw", "ps", "pm"])
    dev = _Both()
    dev.execute(proc, dep)
    kept = {d: dev.get_tensor(d) for d in dep}
    assert kept["c"].dim == [0, 4] and kept["s"].dim == [0] and kept["f"].dim == [1, 4]
    assert kept["pq"].dim == [3, 4] and not kept["pq"].numpy().any() and kept["aw"].dim == [0, 2]
    assert np.isneginf(kept["pm"].numpy()).all() and not kept["ps"].numpy().any()
    for flags in (0, 1, 128):
        got = _interpret(hostcheck, tmp_path, dev.blobs[-1], flags, f"empty{flags}")
        for k, v in kept.items():
            assert got[k][0] == list(v.dim), k
            np.testing.assert_array_equal(got[k][1], v.numpy().reshape(-1), err_msg=k)
