"""B200-native execution backend for the autodiff-ir `Device` boundary.

The directory name carries a hyphen, so load the package with
`importlib.import_module("autodiff-ir-rust_b200")` from the repository root.

Layout:
  csrc/        hand-written CUDA (sm_100a) + the C++ lowering/executor behind the C-ABI (include/adb200.h)
  ir.py        HLIR commands and the wire format handed across the C-ABI
  autodiff.py  host-side mirror of the reference frontend (the caller above the boundary)
  nn.py        Linear / Sigmoid / SGD ... composed exactly as upstream composes them
  devices.py   `B200`: the `Device` implementation (execute + get_tensor) over the C-ABI
  configs.py   the five benchmark programs and their seeded synthetic inputs
"""
from . import ir, autodiff, nn, configs  # noqa: F401
from . import devices  # noqa: F401
