"""ctypes wrapper around the CPU oracle (oracle/ir_oracle.c).

TEST INFRASTRUCTURE ONLY.  `OracleDevice` implements the same `execute` / `get_tensor` pair
as the product's device class so the same traced program can be run on both and compared.
Only tests/, the smoke check and the CPU-baseline leg of bench.py may import this module.
"""
from __future__ import annotations

import ctypes
import importlib
import os
import subprocess
import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "_build", "liboracle.so")


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "ir_oracle.c")
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "-B" if force else "-s"])
    return _LIB


_lib = None
_ALLREDUCE_FN = ctypes.CFUNCTYPE(None, ctypes.POINTER(ctypes.c_float), ctypes.c_uint64, ctypes.c_void_p)


def lib():
    global _lib
    if _lib is None:
        L = ctypes.CDLL(build())
        L.oracle_create.restype = ctypes.c_void_p
        L.oracle_destroy.argtypes = [ctypes.c_void_p]
        L.oracle_execute.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
        L.oracle_execute.restype = ctypes.c_int
        L.oracle_last_error.argtypes = [ctypes.c_void_p]
        L.oracle_last_error.restype = ctypes.c_char_p
        L.oracle_get_tensor.argtypes = [ctypes.c_void_p, ctypes.c_char_p,
                                        ctypes.POINTER(ctypes.POINTER(ctypes.c_float)),
                                        ctypes.POINTER(ctypes.POINTER(ctypes.c_uint64)),
                                        ctypes.POINTER(ctypes.c_uint32)]
        L.oracle_get_tensor.restype = ctypes.c_int
        L.oracle_set_f64_acc.argtypes = [ctypes.c_void_p, ctypes.c_int]
        L.oracle_set_allreduce.argtypes = [ctypes.c_void_p, _ALLREDUCE_FN, ctypes.c_void_p]
        L.oracle_cmds_executed.argtypes = [ctypes.c_void_p]
        L.oracle_cmds_executed.restype = ctypes.c_uint64
        L.oracle_set_threads.argtypes = [ctypes.c_int]
        L.oracle_set_threads.restype = ctypes.c_int
        _lib = L
    return _lib


def set_threads(n: int = 0) -> int:
    """Sets the number of OpenMP threads of the oracle's loops (n <= 0: leave it) and returns the count in force.
    An inherited OMP_NUM_THREADS=1 (torch.distributed.run exports it) is overridden this way."""
    return int(lib().oracle_set_threads(int(n)))


def _pkg():
    return importlib.import_module("autodiff-ir-rust_b200")


class OracleDevice:
    """CPU restatement of the reference's `Device` (execute + get_tensor) over raw IR."""

    def __init__(self, f64_acc: bool = False, allreduce=None):
        self._h = lib().oracle_create()
        lib().oracle_set_f64_acc(self._h, 1 if f64_acc else 0)
        self._cb = None
        if allreduce is not None:
            def _cb(ptr, n, _user):
                arr = np.ctypeslib.as_array(ptr, shape=(int(n),))
                allreduce(arr)
            self._cb = _ALLREDUCE_FN(_cb)
            lib().oracle_set_allreduce(self._h, self._cb, None)

    def __del__(self):
        try:
            if self._h:
                lib().oracle_destroy(self._h)
                self._h = None
        except Exception:
            pass

    def ir_callback(self, irb):
        pass

    def dot_prod_shape(self, a, b):
        return [a[0], b[-1]]

    def execute_blob(self, blob: bytes):
        rc = lib().oracle_execute(self._h, blob, len(blob))
        if rc != 0:
            raise RuntimeError(lib().oracle_last_error(self._h).decode())

    def execute(self, proc, dep_list):
        blob, keep = _pkg().ir.serialize(proc, dep_list)
        self.execute_blob(blob)
        del keep

    def get_tensor(self, id_: str):
        VD = _pkg().autodiff.ValueData
        data = ctypes.POINTER(ctypes.c_float)()
        dims = ctypes.POINTER(ctypes.c_uint64)()
        nd = ctypes.c_uint32()
        rc = lib().oracle_get_tensor(self._h, id_.encode(), ctypes.byref(data), ctypes.byref(dims), ctypes.byref(nd))
        if rc != 0:
            return VD.none()
        shape = [int(dims[i]) for i in range(nd.value)]
        n = int(np.prod(shape)) if shape else 1
        arr = np.ctypeslib.as_array(data, shape=(n,)).copy() if n else np.zeros(0, np.float32)
        return VD(shape, arr, id_, False)

    def cmds_executed(self) -> int:
        return int(lib().oracle_cmds_executed(self._h))
