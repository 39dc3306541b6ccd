"""`B200`: the `Device` implementation (src/core/ir.rs:126-143) over the C-ABI in include/adb200.h.

    autodiff.set_device(devices.B200())
    ...build graph, forward(), backward()...
    autodiff.execute()            -> B200.execute(proc, dep_list) -> adb_execute
    t.val().get()                 -> B200.get_tensor(id)          -> adb_get_tensor

There is no CPU fallback: constructing `B200` without a CUDA device, or without the built
library, raises.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

from . import ir as _ir
from .autodiff import ValueData

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libadb200.so")

ADB_OK, ADB_NONE = 0, 1
STATUS = {0: "ADB_OK", 1: "ADB_NONE", 2: "ADB_ERR_INVALID", 3: "ADB_ERR_CUDA", 4: "ADB_ERR_UNSUPPORTED",
          5: "ADB_ERR_OOM", 6: "ADB_ERR_NCCL", 7: "ADB_ERR_NO_DEVICE"}

FLAG_NO_GRAPHS, FLAG_NO_FUSION, FLAG_SIMT_DOT, FLAG_PROFILE, FLAG_COMM_STREAM, FLAG_SINGLE_SM_DOT, FLAG_EXACT_DIV, FLAG_FUSE_SMALL_SUMS = 1, 2, 4, 8, 16, 32, 64, 128
FLAG_NO_GROUPING = 256
FLAG_DETERMINISTIC = 512
FLAG_SERIAL_GRAPHS = 1024
FLAG_NO_BUCKETS = 2048
FLAG_NO_TINY_DOT = 4096
FLAG_SHORT_DOT_CHUNKS = 8192

EXPORTS = ["adb_create", "adb_destroy", "adb_execute", "adb_get_tensor", "adb_get_tensor_device",
           "adb_dot_prod_shape", "adb_last_error", "adb_get_stats", "adb_dump_plan", "adb_lower_check",
           "adb_shard_ir", "adb_nccl_unique_id", "adb_version", "adb_row_sum_noalloc", "adb_inject_dot_status"]

NOALLOC_MAX_PARTIALS = 1 << 20


class AdbConfig(ctypes.Structure):
    _fields_ = [("struct_size", ctypes.c_uint32), ("device_ordinal", ctypes.c_int32), ("rank", ctypes.c_int32),
                ("world_size", ctypes.c_int32), ("nccl_unique_id", ctypes.c_void_p), ("flags", ctypes.c_uint32),
                ("shard_batch", ctypes.c_uint64), ("shard_ids", ctypes.POINTER(ctypes.c_char_p)),
                ("n_shard_ids", ctypes.c_uint32)]


class AdbStats(ctypes.Structure):
    _fields_ = [("device_ms", ctypes.c_double), ("upload_ms", ctypes.c_double), ("readback_ms", ctypes.c_double),
                ("lower_ms", ctypes.c_double), ("h2d_bytes", ctypes.c_uint64), ("d2h_bytes", ctypes.c_uint64),
                ("kernel_launches", ctypes.c_uint64), ("graph_replays", ctypes.c_uint64),
                ("gemm_launches", ctypes.c_uint64), ("jit_compiles", ctypes.c_uint64), ("arena_bytes", ctypes.c_uint64),
                ("while_iterations", ctypes.c_uint64), ("ir_commands", ctypes.c_uint64), ("plan_steps", ctypes.c_uint64),
                ("elw_ms", ctypes.c_double), ("reduce_ms", ctypes.c_double), ("gemm_ms", ctypes.c_double),
                ("collective_ms", ctypes.c_double), ("elw_launches", ctypes.c_uint64), ("reduce_launches", ctypes.c_uint64),
                ("collective_launches", ctypes.c_uint64), ("elw_bytes", ctypes.c_double), ("reduce_bytes", ctypes.c_double),
                ("gemm_flops", ctypes.c_double), ("collective_bytes", ctypes.c_double), ("top_ms", ctypes.c_double),
                ("top_bytes", ctypes.c_double), ("top_launches", ctypes.c_uint64), ("top_name", ctypes.c_char * 64),
                ("tc_gemm_launches", ctypes.c_uint64)]

    def as_dict(self):
        d = {k: getattr(self, k) for k, _ in self._fields_}
        d["top_name"] = d["top_name"].decode(errors="replace")
        return d


class AdbError(RuntimeError):
    def __init__(self, status, msg):
        super().__init__(f"{STATUS.get(status, status)}: {msg}")
        self.status = status


_lib = None


def load_library():
    """dlopen libadb200.so and declare the C-ABI.  Raises if the extension has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: run `python autodiff-ir-rust_b200/build.py` "
                          "(the backend has no fallback without its CUDA library)")
    L = ctypes.CDLL(LIB_PATH)
    u8p = ctypes.POINTER(ctypes.c_uint8)
    L.adb_create.argtypes = [ctypes.POINTER(AdbConfig), ctypes.POINTER(ctypes.c_void_p)]
    L.adb_create.restype = ctypes.c_int
    L.adb_destroy.argtypes = [ctypes.c_void_p]
    L.adb_destroy.restype = None
    L.adb_execute.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    L.adb_execute.restype = ctypes.c_int
    for fn in (L.adb_get_tensor, L.adb_get_tensor_device):
        fn.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.POINTER(ctypes.POINTER(ctypes.c_float)),
                       ctypes.POINTER(ctypes.POINTER(ctypes.c_uint64)), ctypes.POINTER(ctypes.c_uint32)]
        fn.restype = ctypes.c_int
    L.adb_dot_prod_shape.argtypes = [ctypes.POINTER(ctypes.c_uint64)] * 3
    L.adb_dot_prod_shape.restype = None
    L.adb_last_error.argtypes = [ctypes.c_void_p]
    L.adb_last_error.restype = ctypes.c_char_p
    L.adb_get_stats.argtypes = [ctypes.c_void_p, ctypes.POINTER(AdbStats)]
    L.adb_get_stats.restype = ctypes.c_int
    L.adb_dump_plan.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    L.adb_dump_plan.restype = ctypes.c_size_t
    L.adb_lower_check.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(AdbConfig), ctypes.c_int,
                                  ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_size_t),
                                  ctypes.c_char_p, ctypes.c_size_t]
    L.adb_lower_check.restype = ctypes.c_int
    L.adb_shard_ir.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(AdbConfig),
                               u8p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_size_t), ctypes.c_char_p, ctypes.c_size_t]
    L.adb_shard_ir.restype = ctypes.c_int
    L.adb_nccl_unique_id.argtypes = [ctypes.c_void_p]
    L.adb_nccl_unique_id.restype = ctypes.c_int
    L.adb_version.restype = ctypes.c_char_p
    L.adb_row_sum_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_void_p,
                                      ctypes.c_char_p, ctypes.c_size_t]
    L.adb_row_sum_noalloc.restype = ctypes.c_int
    L.adb_inject_dot_status.argtypes = [ctypes.c_void_p, ctypes.c_int]
    L.adb_inject_dot_status.restype = ctypes.c_int
    _lib = L
    return L


def _id_array(ids):
    if not ids:
        return None, 0
    arr = (ctypes.c_char_p * len(ids))(*[i.encode() for i in ids])
    return arr, len(ids)


def lower_check(proc, dep_list, *, with_source=False, flags=0, rank=0, world=1, shard_batch=0, shard_ids=None) -> str:
    """Host-only: lower a traced program and JIT-compile every generated kernel for sm_100a
    (no GPU needed).  Returns the plan listing; raises AdbError with the reason on failure."""
    L = load_library()
    blob, keep = _ir.serialize(proc, dep_list)
    ids, n_ids = _id_array(shard_ids)
    cfg = AdbConfig(ctypes.sizeof(AdbConfig), 0, rank, world, None, flags, shard_batch, ids, n_ids)
    err = ctypes.create_string_buffer(1 << 16)
    need = ctypes.c_size_t(0)
    cap = 1 << 20
    while True:
        buf = ctypes.create_string_buffer(cap)
        rc = L.adb_lower_check(blob, len(blob), ctypes.byref(cfg), 1 if with_source else 0, buf, cap,
                               ctypes.byref(need), err, len(err))
        if rc != ADB_OK:
            raise AdbError(rc, err.value.decode(errors="replace"))
        if need.value <= cap:
            del keep
            return buf.value.decode(errors="replace")
        cap = need.value + 16


def shard_ir(blob: bytes, rank: int, world: int, shard_batch: int, shard_ids=None) -> bytes:
    """Host-only: the data-parallel rewrite applied when world_size > 1, as a blob -> blob function."""
    L = load_library()
    err = ctypes.create_string_buffer(1 << 14)
    need = ctypes.c_size_t(0)
    ids, n_ids = _id_array(shard_ids)
    cfg = AdbConfig(ctypes.sizeof(AdbConfig), 0, rank, world, None, 0, shard_batch, ids, n_ids)
    rc = L.adb_shard_ir(blob, len(blob), ctypes.byref(cfg), None, 0, ctypes.byref(need), err, len(err))
    if rc != ADB_OK:
        raise AdbError(rc, err.value.decode(errors="replace"))
    out = (ctypes.c_uint8 * need.value)()
    rc = L.adb_shard_ir(blob, len(blob), ctypes.byref(cfg), out, need.value, ctypes.byref(need), err, len(err))
    if rc != ADB_OK:
        raise AdbError(rc, err.value.decode(errors="replace"))
    return bytes(out)


class B200:
    """One handle per GPU (one process per GPU).  `execute` and `get_tensor` are the two methods of the
    reference's `Device` trait; `ir_callback` is a no-op and `dot_prod_shape` the trait's default."""

    def __init__(self, device_ordinal: int = 0, *, rank: int = 0, world_size: int = 1, nccl_unique_id: bytes | None = None,
                 flags: int = 0, shard_batch: int = 0, shard_ids=None):
        L = load_library()
        self._L = L
        uid = None
        if nccl_unique_id is not None:
            assert len(nccl_unique_id) == 128
            self._uid = ctypes.create_string_buffer(nccl_unique_id, 128)
            uid = ctypes.cast(self._uid, ctypes.c_void_p)
        ids, n_ids = _id_array(shard_ids)   # the ids of the CreateMat tensors that hold the batch (optional)
        cfg = AdbConfig(ctypes.sizeof(AdbConfig), device_ordinal, rank, world_size, uid, flags, shard_batch, ids, n_ids)
        h = ctypes.c_void_p()
        rc = L.adb_create(ctypes.byref(cfg), ctypes.byref(h))
        if rc != ADB_OK:
            raise AdbError(rc, "adb_create failed (a B200 and the CUDA driver are required; there is no CPU path)")
        self._h = h
        self.rank, self.world_size = rank, world_size
        self._keep = None

    def close(self):
        if getattr(self, "_h", None):
            self._L.adb_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- Device trait ---------------------------------------------------------------------------
    def ir_callback(self, irb):
        """`Device::ir_callback` (src/core/ir.rs:135): this backend wants the IR as traced."""

    def dot_prod_shape(self, a, b):
        """`Device::dot_prod_shape` default (src/core/ir.rs:140-142)."""
        aa = (ctypes.c_uint64 * 2)(*a)
        bb = (ctypes.c_uint64 * 2)(*b)
        out = (ctypes.c_uint64 * 2)()
        self._L.adb_dot_prod_shape(aa, bb, out)
        return [int(out[0]), int(out[1])]

    def execute(self, proc, dep_list):
        """`Device::execute` (src/core/ir.rs:128)."""
        blob, keep = _ir.serialize(proc, dep_list)
        self.execute_blob(blob)
        del keep

    def execute_blob(self, blob: bytes):
        rc = self._L.adb_execute(self._h, blob, len(blob))
        if rc != ADB_OK:
            raise AdbError(rc, self._L.adb_last_error(self._h).decode(errors="replace"))

    def get_tensor(self, id_: str) -> ValueData:
        """`Device::get_tensor` (src/core/ir.rs:131): a host copy, or ValueData.none() if not kept."""
        data = ctypes.POINTER(ctypes.c_float)()
        dims = ctypes.POINTER(ctypes.c_uint64)()
        nd = ctypes.c_uint32()
        rc = self._L.adb_get_tensor(self._h, id_.encode(), ctypes.byref(data), ctypes.byref(dims), ctypes.byref(nd))
        if rc == ADB_NONE:
            return ValueData.none()
        if rc != ADB_OK:
            raise AdbError(rc, self._L.adb_last_error(self._h).decode(errors="replace"))
        shape = [int(dims[i]) for i in range(nd.value)]
        n = int(np.prod(shape)) if shape else 1
        arr = np.ctypeslib.as_array(data, shape=(n,)).copy() if n else np.zeros(0, np.float32)
        return ValueData(shape, arr, id_, False)

    # -- extras ---------------------------------------------------------------------------------
    def get_tensor_device(self, id_: str):
        """(device address, shape) of a kept tensor, left in HBM."""
        data = ctypes.POINTER(ctypes.c_float)()
        dims = ctypes.POINTER(ctypes.c_uint64)()
        nd = ctypes.c_uint32()
        rc = self._L.adb_get_tensor_device(self._h, id_.encode(), ctypes.byref(data), ctypes.byref(dims), ctypes.byref(nd))
        if rc != ADB_OK:
            return None
        return ctypes.cast(data, ctypes.c_void_p).value, [int(dims[i]) for i in range(nd.value)]

    def save_tensors(self, path: str, ids) -> list:
        """Checkpoint helper: writes the kept tensors named in `ids` (Tensor / Value objects or id strings) of the last
        execute to one `.npz` file, keyed by id, and returns the ids written.  The reference has no checkpointing;
        weights are only reachable through `keep()` + `get()` (src/core/value.rs:97-99), which is what this wraps."""
        out = {}
        for t in ids:
            id_ = t if isinstance(t, str) else (t.val().id if hasattr(t, "val") and not hasattr(t, "get") else t.id)
            v = self.get_tensor(id_)
            if v.is_none:
                raise KeyError(f"'{id_}' was not kept by the last execute")
            out[id_] = np.asarray(v.data, np.float32).reshape(v.dim)
        np.savez(path, **out)
        return list(out)

    def stats(self) -> dict:
        s = AdbStats()
        self._L.adb_get_stats(self._h, ctypes.byref(s))
        return s.as_dict()

    def inject_dot_status(self, code: int) -> None:
        """Diagnostic: makes the next execute that runs a tensor-core dot product fail as if a bounded wait inside the
        kernel had run out (`adb_inject_dot_status`)."""
        rc = self._L.adb_inject_dot_status(self._h, int(code))
        if rc != ADB_OK:
            raise AdbError(rc, "adb_inject_dot_status failed")

    def dump_plan(self) -> str:
        n = self._L.adb_dump_plan(self._h, None, 0)
        buf = ctypes.create_string_buffer(int(n) + 16)
        self._L.adb_dump_plan(self._h, buf, len(buf))
        return buf.value.decode(errors="replace")


def row_sum_noalloc(d_in: int, d_out: int, rows: int, length: int, stream: int = 0) -> None:
    """out[r] = sum(in[r, :]) on device pointers, through the entry point that allocates nothing.

    For callers that cannot allocate device memory where they call from: the scratch of the two-pass
    sum is a fixed array inside the library (see include/adb200.h for the limit and the sharing rules).
    Raises AdbError when `rows` exceeds NOALLOC_MAX_PARTIALS."""
    err = ctypes.create_string_buffer(256)
    rc = load_library().adb_row_sum_noalloc(d_in, d_out, rows, length, stream, err, len(err))
    if rc != ADB_OK:
        raise AdbError(rc, err.value.decode(errors="replace"))


def nccl_unique_id() -> bytes:
    buf = ctypes.create_string_buffer(128)
    rc = load_library().adb_nccl_unique_id(buf)
    if rc != ADB_OK:
        raise AdbError(rc, "ncclGetUniqueId failed")
    return buf.raw
