"""The byte-level fixtures of the wire format (tests/golden/wire/*.adir) are what the Rust serialiser
(rust/src/devices/cuda/wire.rs) is pinned to: they must be exactly what the Python serialiser produces today, and the
backend's own parser and the oracle must accept them."""
import importlib
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_wire_fixtures  # noqa: E402

adb = importlib.import_module("autodiff-ir-rust_b200")
WIRE = os.path.join(HERE, "golden", "wire")


def test_committed_fixtures_are_current():
    fresh = make_wire_fixtures.fixtures()
    on_disk = {f[:-5] for f in os.listdir(WIRE) if f.endswith(".adir")}
    assert on_disk == set(fresh), "run tests/golden/make_wire_fixtures.py"
    for name, blob in fresh.items():
        assert open(os.path.join(WIRE, name + ".adir"), "rb").read() == blob, name


def test_every_variant_appears_in_the_literal_program():
    proc, _ = make_wire_fixtures.all_variants()
    seen = set()

    def walk(p):
        for c in p.main:
            seen.add(c[0])
            if c[0] == "While":
                walk(c[2])
            elif c[0] == "If":
                for _, b in c[1]:
                    walk(b)
                if c[2] is not None:
                    walk(c[2])
    walk(proc)
    reference_variants = {k for k, v in adb.ir.OPC.items() if v <= 26}
    assert seen == reference_variants, reference_variants - seen


@pytest.mark.parametrize("name", sorted(f[:-5] for f in os.listdir(WIRE) if f.endswith(".adir")))
def test_fixture_is_accepted_by_the_oracle(name):
    from oracle.oracle import OracleDevice
    blob = open(os.path.join(WIRE, name + ".adir"), "rb").read()
    dev = OracleDevice()
    dev.execute_blob(blob)
    if name == "all_variants":
        a = dev.get_tensor("a").numpy()
        # the loop runs twice (c = 2, 1); f == 1 squares `a` each time
        np.testing.assert_array_equal(a.reshape(-1), np.array([1, 2, 3, 4, 5, 6], np.float32) ** 4)
        np.testing.assert_array_equal(dev.get_tensor("d").numpy().reshape(2, 2), np.array([[14, 32], [32, 77]], np.float32))


def test_rust_sources_name_every_opcode():
    """The Rust serialiser cannot be compiled here; at least its opcode table must agree with the Python one."""
    import re
    src = open(os.path.join(os.path.dirname(HERE), "rust", "src", "devices", "cuda", "wire.rs")).read()
    for variant, code in adb.ir.OPC.items():
        if code > 26:
            continue
        m = re.search(r"IRCmds::%s\b[^=]*=>\s*\{?(?:[^;]*;){0,3}?\s*self\.u8\((\d+)\)" % variant, src) or \
            re.search(r"IRCmds::%s\b[^=]*=>\s*self\.u8\((\d+)\)" % variant, src)
        assert m and int(m.group(1)) == code, variant
