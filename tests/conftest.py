import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200 box)")


@pytest.fixture(scope="session")
def adb():
    return importlib.import_module("autodiff-ir-rust_b200")


@pytest.fixture()
def oracle_device():
    from oracle.oracle import OracleDevice
    return OracleDevice()


@pytest.fixture(scope="session")
def hostcheck(tmp_path_factory):
    """The backend's host code (parser, data-parallel rewrite, lowering, source generation) plus the CPU plan
    interpreter, built once per session with AddressSanitizer + UndefinedBehaviorSanitizer (tests/hostcheck/)."""
    import subprocess
    csrc = os.path.join(ROOT, "autodiff-ir-rust_b200", "csrc")
    out = tmp_path_factory.mktemp("hostcheck") / "hostcheck"
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined",
           "-I", csrc, os.path.join(ROOT, "tests", "hostcheck", "hostcheck.cpp"), os.path.join(csrc, "adb_lower.cpp"),
           os.path.join(csrc, "adb_codegen.cpp"), os.path.join(csrc, "adb_shard.cpp"), "-o", str(out)]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return str(out)
