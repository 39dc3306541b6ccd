"""The backend's host code (wire parser, data-parallel rewrite, lowering with its fusion passes, source generation)
built with AddressSanitizer + UndefinedBehaviorSanitizer and run over serialised programs: the reference's
known-answer programs, the benchmark programs at sizes that reach every fusion, random programs, truncated and
corrupted blobs.  Any sanitizer report aborts the helper and fails the test."""
import importlib
import os
import subprocess

import numpy as np
import pytest

import fuzz_programs
import ref_programs

adb = importlib.import_module("autodiff-ir-rust_b200")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "autodiff-ir-rust_b200", "csrc")


class _Capture:
    """Device stand-in that serialises what it is asked to execute into a self-contained blob."""

    def __init__(self):
        self.blobs = []

    def ir_callback(self, irb):
        pass

    def dot_prod_shape(self, a, b):
        return [a[0], b[1]]

    def execute(self, proc, dep):
        blob, _ = adb.ir.serialize(proc, dep, inline_limit=1 << 40)
        self.blobs.append(blob)

    def get_tensor(self, id_):
        return adb.autodiff.ValueData([1], np.zeros(1, np.float32), id_, False)


def _run(binary, files, flags=0, world=1, batch=0):
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1")
    r = subprocess.run([binary, str(flags), str(world), str(batch)] + files, capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-4000:]
    assert "ERROR: AddressSanitizer" not in r.stderr and "runtime error" not in r.stderr, r.stderr[-4000:]
    return dict(kv.split("=") for kv in r.stdout.split())


def _write(tmp_path, blobs):
    files = []
    for i, b in enumerate(blobs):
        p = tmp_path / f"p{i}.adir"
        p.write_bytes(b)
        files.append(str(p))
    return files


def test_reference_and_benchmark_programs_under_sanitizers(hostcheck, tmp_path):
    cap = _Capture()
    for name in sorted(ref_programs.ALL):
        ref_programs.ALL[name](cap)
    cfg = adb.configs
    cfg.c1_readme_mlp(cap)
    cfg.c2_fused_elementwise(cap, rows=512, cols=1024)          # both sums fold into the element-wise pass
    cfg.c3_reduce_movement(cap, batch=8, n=16)
    cfg.c4_mlp_train(cap, batch=2048, widths=(64, 128, 128, 64, 16), steps=2)
    cfg.c5_dot_loop(cap, n=32, max_iters=3)
    adb.autodiff.set_device(cap)                                # row / column maxima (IR extension)
    t = adb.autodiff.tensor(np.arange(300 * 40, dtype=np.float32), [300, 40])
    for axis in (0, 1):
        m = t.max(axis).forward()
        m.keep()
    adb.autodiff.execute()
    files = _write(tmp_path, cap.blobs)
    for flags in (0, 1, 2, 4):
        out = _run(hostcheck, files, flags=flags)
        assert int(out["rejected"]) == 0 and int(out["kernels"]) > 0
    assert int(_run(hostcheck, files, flags=0)["fused_sums"]) >= 2


def test_data_parallel_rewrite_under_sanitizers(hostcheck, tmp_path):
    cap = _Capture()
    adb.configs.c4_mlp_train(cap, batch=256, widths=(64, 128, 128, 64, 16), steps=2)
    out = _run(hostcheck, _write(tmp_path, cap.blobs), world=4, batch=256)
    assert int(out["rejected"]) == 0


def test_random_programs_under_sanitizers(hostcheck, tmp_path):
    cap = _Capture()
    for seed in list(range(30)) + list(range(100, 130)):
        with np.errstate(all="ignore"):
            fuzz_programs.build(seed, exact=seed < 100)(cap)
    files = _write(tmp_path, cap.blobs)
    for flags in (0, 2):
        assert int(_run(hostcheck, files, flags=flags)["rejected"]) == 0


def test_damaged_blobs_are_rejected_not_crashed_on(hostcheck, tmp_path):
    cap = _Capture()
    ref_programs.ALL[sorted(ref_programs.ALL)[0]](cap)
    adb.configs.c4_mlp_train(cap, batch=32, widths=(16, 32, 32, 16, 8), steps=2)
    rng = np.random.default_rng(0)
    damaged = []
    for blob in cap.blobs:
        for cut in (0, 3, 8, 17, len(blob) // 3, len(blob) // 2, len(blob) - 1):
            damaged.append(blob[:cut])
        for _ in range(40):
            b = bytearray(blob)
            for _ in range(int(rng.integers(1, 6))):
                b[int(rng.integers(0, len(b)))] = int(rng.integers(0, 256))
            damaged.append(bytes(b))
    out = _run(hostcheck, _write(tmp_path, damaged))
    assert int(out["rejected"]) > 10     # most are refused; the rest happened to stay valid programs
