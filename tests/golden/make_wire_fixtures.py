"""Writes the byte-level fixtures of the C-ABI wire format: tests/golden/wire/*.adir.

    python tests/golden/make_wire_fixtures.py

`all_variants.adir` is a literal program with every IR command once (nested blocks included); the Rust serialiser
(rust/src/devices/cuda/wire.rs) carries a unit test that builds the same program with the reference's own types and
compares byte for byte.  The other files are the reference's known-answer programs as the frontend mirror traces them
(self-contained: payloads inline), targets for the same comparison once the shim runs inside the reference tree."""
import importlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)
adb = importlib.import_module("autodiff-ir-rust_b200")
P = adb.ir.IRProcedure


def all_variants():
    def blk(name, cmds):
        b = P(name)
        for c in cmds:
            b.push(c)
        return b
    body = blk("b0", [
        ("ElwAddEq", "c", "k"),
        ("If", [("f", blk("b1", [("ElwMultiplyEq", "a", "a")])), ("g", blk("b2", [("EX",)]))], blk("b3", [("Heading", "else")])),
    ])
    f = np.float32
    main = blk("main", [
        ("Heading", "all variants"),
        ("CreateMat", np.array([1, 2, 3, 4, 5, 6], f), [2, 3], "a"),
        ("CreateMat", np.array([2], f), [1], "c"),
        ("CreateMat", np.array([1], f), [1], "f"),
        ("CreateMat", np.array([0], f), [1], "g"),
        ("CreateConstant", -1.0, "k", [1]),
        ("CreateConstant", 0.5, "h", [2, 3]),
        ("ElwMultiply", "a", "h", "m"),
        ("ElwAdd", "a", "m", "n"),
        ("EqualZero", "n", "e0"),
        ("MoreZero", "n", "e1"),
        ("LessZero", "n", "e2"),
        ("Sum", "n", "sm"),
        ("Permute", "a", [1, 0], "at"),
        ("DotProduct", "a", "at", "d"),
        ("View", "a", [3, 2], "v"),
        ("Index", "a", 1, 0, "i"),
        ("Concat", "a", "n", 0, "cc"),
        ("View", "sm", [2, 1], "s1"),
        ("Broadcast", "s1", 1, 3, "bc"),
        ("Contigious", "at", "ct"),
        ("Exp2", "a", "u0"),
        ("Log2", "a", "u1"),
        ("Sin", "a", "u2"),
        ("Recip", "a", "u3"),
        ("Sqrt", "a", "u4"),
        ("While", "c", body),
        ("EX",),
    ])
    return main, ["a", "d", "cc", "bc", "ct", "u4", "c"]


class _Capture:
    def __init__(self):
        self.blobs = []

    def ir_callback(self, irb):
        pass

    def dot_prod_shape(self, a, b):
        return [a[0], b[-1]]

    def execute(self, proc, dep):
        self.blobs.append(adb.ir.serialize(proc, dep, inline_limit=1 << 40)[0])

    def get_tensor(self, id_):
        return adb.autodiff.ValueData([1], np.zeros(1, np.float32), id_, False)


def fixtures():
    out = {}
    proc, dep = all_variants()
    out["all_variants"] = adb.ir.serialize(proc, dep, inline_limit=1 << 40)[0]
    import ref_programs
    for name in sorted(ref_programs.ALL):
        cap = _Capture()
        try:
            ref_programs.ALL[name](cap)
        except Exception:       # programs that read their results back need a real device; the blob exists by then
            pass
        if cap.blobs:
            out["kat_" + name] = cap.blobs[-1]
    return out


if __name__ == "__main__":
    os.makedirs(os.path.join(HERE, "wire"), exist_ok=True)
    for name, blob in fixtures().items():
        with open(os.path.join(HERE, "wire", name + ".adir"), "wb") as f:
            f.write(blob)
        print(name, len(blob), "bytes")
