"""CPU-side checks of the boundary: the library loads, exports every symbol include/adb200.h
declares, refuses to run without a GPU, and lowers + JIT-compiles (for sm_100a) every program."""
import ctypes
import importlib
import os
import re

import numpy as np
import pytest

import ref_programs

adb = importlib.import_module("autodiff-ir-rust_b200")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ensure_built():
    build = importlib.import_module("autodiff-ir-rust_b200.build")
    build.build()


@pytest.fixture(scope="module", autouse=True)
def built():
    _ensure_built()


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "adb200.h")).read()
    declared = set(re.findall(r"\b(adb_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    lib = ctypes.CDLL(adb.devices.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in adb200.h but not exported"
    assert set(adb.devices.EXPORTS) <= declared


def test_no_silent_cpu_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(adb.devices.AdbError) as e:
        adb.devices.B200(0)
    assert e.value.status == 7  # ADB_ERR_NO_DEVICE


def test_dot_prod_shape_default():
    lib = adb.devices.load_library()
    a = (ctypes.c_uint64 * 2)(5, 3)
    b = (ctypes.c_uint64 * 2)(3, 9)
    out = (ctypes.c_uint64 * 2)()
    lib.adb_dot_prod_shape(a, b, out)
    assert list(out) == [5, 9]


class _LowerOnly:
    """Device stand-in that only lowers + JIT-compiles (host work, no GPU)."""

    def __init__(self, **kw):
        self.kw, self.plan = kw, None

    def ir_callback(self, irb):
        pass

    def execute(self, proc, dep):
        self.plan = adb.devices.lower_check(proc, dep, **self.kw)

    def get_tensor(self, id_):
        return adb.autodiff.ValueData([1], np.zeros(1, np.float32), id_, False)


def _kernel_lines(plan):
    """One line per step of the plan listing; the members of a grouped launch ('  - ...') count as steps."""
    return [l for l in plan.splitlines() if l.startswith("#") or l.lstrip().startswith("- ")]


@pytest.mark.parametrize("name", sorted(ref_programs.ALL))
def test_reference_programs_lower_and_compile(name):
    dev = _LowerOnly()
    ref_programs.ALL[name](dev)
    assert dev.plan.startswith("plan:")


def test_fusion_shapes_of_the_benchmark_programs():
    cfg = adb.configs
    dev = _LowerOnly()
    cfg.c2_fused_elementwise(dev, rows=64, cols=128)
    steps = _kernel_lines(dev.plan)
    # forward chain fused into the row sum; both input gradients from one element-wise kernel
    assert any(" reduce " in l and "ops=2" in l for l in steps)
    assert sum(" elw n=8192" in l for l in steps) == 1
    dev = _LowerOnly()
    cfg.c3_reduce_movement(dev, batch=8, n=16)
    assert "608 IR commands" in dev.plan
    assert len([l for l in dev.plan.splitlines() if l.startswith("#")]) <= 12
    dev = _LowerOnly()
    cfg.c4_mlp_train(dev, batch=32, widths=(16, 32, 32, 16, 8), steps=3)
    assert sum(" gemm " in l for l in dev.plan.splitlines()) == 11   # 4 forward, 4 dW, 3 dX (dX of layer 1 is dead)


def test_sums_ride_along_with_the_element_wise_pass_over_the_same_memory():
    """Config 2 above 2^18 elements: the loss and the bias gradient become side sums of the one kernel that streams
    a and b (plus two tiny second passes); the training loop fuses its loss and every bias gradient; the generated
    kernels compile for sm_100a."""
    cfg = adb.configs
    dev = _LowerOnly(with_source=True)
    cfg.c2_fused_elementwise(dev, rows=512, cols=1024)
    steps = _kernel_lines(dev.plan)
    big = [l for l in steps if " elw n=524288" in l or "rows=512 len=1024" in l or "rows=1024 len=512" in l]
    assert len(big) == 1 and "adb_elwsum_" in big[0], steps
    assert dev.plan.count("    sum v") == 2
    assert "__shfl_xor_sync" in dev.plan and "__shared__ float sm[8][128]" in dev.plan
    small = _LowerOnly()
    cfg.c2_fused_elementwise(small, rows=64, cols=128)
    assert "adb_elwsum_" not in small.plan
    loop = _LowerOnly()
    cfg.c4_mlp_train(loop, batch=2048, widths=(256, 512, 512, 256, 128), steps=2)
    assert loop.plan.count("    sum v") == 5          # loss + four bias gradients
    assert sum(" reduce " in l and "len=2048" in l and "rows=1 " not in l for l in loop.plan.splitlines()) == 0


def test_normalisation_layers_lower_to_one_kernel():
    """mean -> variance -> normalise: consecutive steps over the same rows in which later ones use the per-row results
    of earlier ones become one `adb_rows_*` kernel (it compiles for sm_100a here)."""
    dev = _LowerOnly(with_source=True)
    ad = adb.autodiff
    ad.set_device(dev)
    ad.eager_dep_opt()
    x = np.linspace(-1, 1, 1024 * 512, dtype=np.float32)
    y = adb.nn.LayerNorm(512).f(ad.tensor(x, [1024, 512])).forward()
    y.keep()
    ad.execute()
    steps = _kernel_lines(dev.plan)
    assert sum(" rows [1024,512] phases=2" in l for l in steps) == 1 and not any(" reduce " in l for l in steps), steps
    assert "red0" in dev.plan and "red1" in dev.plan


def test_no_fusion_flag_gives_one_kernel_per_command():
    dev = _LowerOnly(flags=adb.devices.FLAG_NO_FUSION)
    ref_programs.ct(dev)
    fused = _LowerOnly()
    ref_programs.ct(fused)
    count = lambda p: sum(1 for l in _kernel_lines(p) if " elw " in l)
    assert count(dev.plan) > 20 and count(fused.plan) == 1


@pytest.mark.parametrize("blob", [b"", b"ADIR", b"ADIR\x01\x00\x00\x00" + b"\xff" * 40])
def test_malformed_blobs_are_rejected(blob):
    lib = adb.devices.load_library()
    err = ctypes.create_string_buffer(4096)
    need = ctypes.c_size_t()
    rc = lib.adb_lower_check(blob, len(blob), None, 0, None, 0, ctypes.byref(need), err, len(err))
    assert rc == 2 and err.value  # ADB_ERR_INVALID with a message


def test_read_before_definition_is_an_error_not_a_crash():
    ir = adb.ir
    proc = ir.IRProcedure("main")
    proc.push(("ElwAdd", "a", "b", "c"))
    proc.push(("EX",))
    with pytest.raises(adb.devices.AdbError) as e:
        adb.devices.lower_check(proc, {"c"})
    assert "before it is defined" in str(e.value)


def test_products_of_a_few_multiply_adds_become_element_wise_expressions():
    """The README-sized network (2 x 5 inputs, 3 hidden units): its six dot products are sums of at most five products
    per element, so they fuse with the sigmoid, the loss and the update around them -- no dot-product launch is left;
    with one kernel per command they are dot-product steps again."""
    dev = _LowerOnly()
    adb.configs.c1_readme_mlp(dev)
    steps = [l for l in dev.plan.splitlines() if l.startswith("#") and " upload " not in l and " exit" not in l]
    assert not any(" gemm " in l for l in steps), dev.plan
    assert len(steps) <= 4, dev.plan
    unfused = _LowerOnly(flags=adb.devices.FLAG_NO_FUSION)
    adb.configs.c1_readme_mlp(unfused)
    assert sum(" gemm " in l for l in unfused.plan.splitlines()) == 6


_M6 = np.arange(6, dtype=np.float32)
_BAD = {
    "element-wise operands of different size": ([("ElwAdd", "a", "v", "r")], "differ in size"),
    "index beyond the axis": ([("Index", "a", 5, 0, "r")], "Index out of range"),
    "index on an axis that does not exist": ([("Index", "a", 0, 7, "r")], "Index out of range"),
    "view that changes the element count": ([("View", "a", [4, 2], "r")], "changes the element count"),
    "permute of the wrong rank": ([("Permute", "a", [0], "r")], "Permute rank mismatch"),
    "permute that repeats an axis": ([("Permute", "a", [0, 0], "r")], "not a permutation"),
    "concat of different ranks": ([("Concat", "a", "v", 0, "r")], "Concat rank mismatch"),
    "dot product with unequal inner dimensions": ([("DotProduct", "a", "a", "r")], "second dimension must equal"),
    "dot product of a vector": ([("DotProduct", "a", "v", "r")], "must be a 2d array"),
    "sum of a vector": ([("Sum", "v", "r")], "needs dim=2"),
    "broadcast of an axis longer than 1": ([("Broadcast", "a", 0, 4, "r")], "length-1 axis"),
    "loop condition that is not one float": ([("While", "a", [("ElwAddEq", "a", "a")])], "must have dim of [1]"),
    "batched product of matrices": ([("BatchDot", "a", "b", "r")], "3-d operands"),
    "alias written onto its own operand": ([("Permute", "a", [1, 0], "a")], "its own operand"),
}


@pytest.mark.parametrize("case", sorted(_BAD))
def test_malformed_programs_are_refused_with_a_reason(case):
    """What the reference answers with a panic (`expect` / `panic!` in its lowering and its device), the boundary answers
    with ADB_ERR_INVALID and a sentence that names the command: never a crash, never a silent result."""
    ir = adb.ir
    cmds, reason = _BAD[case]
    proc = ir.IRProcedure("main")
    proc.push(("CreateMat", _M6, [2, 3], "a"))
    proc.push(("CreateMat", _M6 * 2, [3, 2], "b"))
    proc.push(("CreateMat", np.arange(4, dtype=np.float32), [4], "v"))
    for c in cmds:
        if c[0] == "While":
            body = ir.IRProcedure("body")
            for bc in c[2]:
                body.push(bc)
            c = ("While", c[1], body)
        proc.push(c)
    with pytest.raises(adb.devices.AdbError) as e:
        adb.devices.lower_check(proc, {"r"} if any(c[-1] == "r" for c in cmds) else {"a"})
    assert e.value.status == 2 and reason in str(e.value), str(e.value)
