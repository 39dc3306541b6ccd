"""HLIR commands and the flat wire format handed across the C-ABI.

The command set is the reference's `enum IRCmds` (src/core/ir.rs:8-105) and
`struct IRProcedure` (src/core/ir.rs:109-112).  A command is a plain tuple whose
first element is the variant name; nested blocks are `IRProcedure` objects.

Wire format (little-endian, version 1) — the exact layout is also documented in
`include/adb200.h`:

    u32 magic 'ADIR'   u32 version   u32 flags   u32 n_ids
    n_ids  x { u16 len, bytes }                      id string table
    u32 n_dep, n_dep x u32                           ids that must be readable afterwards
    procedure := u32 n_cmds, n_cmds x cmd
    cmd       := u8 opcode, operands (see OPC below)
    payload section: raw f32 data referenced by CreateMat(kind=inline)

ids are referenced by their index in the string table.
"""
from __future__ import annotations

import struct
import numpy as np

MAGIC = 0x52494441  # 'ADIR'
VERSION = 1

OPC = {
    "CreateMat": 1, "CreateConstant": 2,
    "ElwMultiply": 3, "ElwAdd": 4, "ElwMultiplyEq": 5, "ElwAddEq": 6,
    "EqualZero": 7, "MoreZero": 8, "LessZero": 9,
    "Sum": 10, "DotProduct": 11,
    "View": 12, "Index": 13, "Concat": 14, "Permute": 15, "Broadcast": 16, "Contigious": 17,
    "Exp2": 18, "Log2": 19, "Sin": 20, "Recip": 21, "Sqrt": 22,
    "While": 23, "If": 24, "EX": 25, "Heading": 26,
    # extension (no counterpart in the reference): in-place sum of `id` over all data-parallel ranks
    "AllReduce": 27,
    # extension: row maximum of a 2-d tensor, same shape contract as Sum (the reference's kernel layer names
    # `ReduceOp::Max`, src/kernel/kernel_decl.rs:77, but no IR command reaches it)
    "Max": 28,
    # extension: batched matrix product [B, M, K] x [B, K, N] -> [B, M, N] (the reference lists it as missing,
    # TODO.md:22; its attention runs one 2-d DotProduct per head, src/nn/transformer.rs:10-18)
    "BatchDot": 29,
}

PAYLOAD_INLINE = 0   # u64 = byte offset of the data inside the blob
PAYLOAD_HOST = 1     # u64 = host address of n f32 (borrowed for the duration of execute)
PAYLOAD_DEVICE = 2   # u64 = device address of n f32 already resident in HBM

INLINE_LIMIT = 1 << 16  # bytes; larger CreateMat payloads are passed by pointer (zero copy)


class IRProcedure:
    """`struct IRProcedure { main: Vec<IRCmds>, id: String }` (src/core/ir.rs:109-112)."""

    def __init__(self, id: str):
        self.main: list = []
        self.id = id

    def push(self, cmd):
        self.main.append(cmd)

    def __len__(self):
        return len(self.main)

    def __iter__(self):
        return iter(self.main)

    def count(self) -> int:
        """Total number of commands including nested blocks."""
        n = 0
        for c in self.main:
            n += 1
            if c[0] == "While":
                n += c[2].count()
            elif c[0] == "If":
                for _, blk in c[1]:
                    n += blk.count()
                if c[2] is not None:
                    n += c[2].count()
        return n


class DevicePayload:
    """A CreateMat payload that is already resident in HBM (`ptr` = device address of `n` f32)."""

    def __init__(self, ptr: int, n: int, owner=None):
        self.ptr, self.n, self.owner = int(ptr), int(n), owner

    def __len__(self):
        return self.n


def format_ir(proc: IRProcedure, indent: int = 0) -> str:
    """Readable listing of a procedure (same role as the reference's `ir_print`, src/ir/debug.rs:85-185)."""
    pad = "    " * indent
    out = []
    for c in proc.main:
        k = c[0]
        if k == "CreateMat":
            out.append(f"{pad}{c[3]} = mat(dim={list(c[2])})")
        elif k == "CreateConstant":
            out.append(f"{pad}{c[2]} = {c[1]!r} (dim={list(c[3])})")
        elif k == "While":
            out.append(f"{pad}while ({c[1]} != 0) {{")
            out.append(format_ir(c[2], indent + 1))
            out.append(f"{pad}}}")
        elif k == "If":
            for i, (cond, blk) in enumerate(c[1]):
                out.append(f"{pad}{'if' if i == 0 else 'else if'} ({cond} == 1) {{")
                out.append(format_ir(blk, indent + 1))
                out.append(f"{pad}}}")
            if c[2] is not None:
                out.append(f"{pad}else {{")
                out.append(format_ir(c[2], indent + 1))
                out.append(f"{pad}}}")
        else:
            out.append(f"{pad}{k} {', '.join(str(x) for x in c[1:])}")
    return "\n".join(out)


class _Writer:
    def __init__(self):
        self.ids: dict[str, int] = {}
        self.body = bytearray()
        self.inline: list[tuple[int, np.ndarray]] = []  # (patch position in body, data)
        self.keepalive: list = []
        self.inline_limit = INLINE_LIMIT

    def idx(self, s: str) -> int:
        i = self.ids.get(s)
        if i is None:
            i = len(self.ids)
            self.ids[s] = i
        return i

    def u8(self, v):
        self.body += struct.pack("<B", v)

    def u16(self, v):
        self.body += struct.pack("<H", v)

    def u32(self, v):
        self.body += struct.pack("<I", v)

    def u64(self, v):
        self.body += struct.pack("<Q", v)

    def f32(self, v):
        self.body += struct.pack("<f", float(v))

    def dims(self, d):
        self.u8(len(d))
        for x in d:
            self.u64(int(x))

    def proc(self, p: IRProcedure):
        self.u32(len(p.main))
        for c in p.main:
            self.cmd(c)

    def cmd(self, c):
        k = c[0]
        self.u8(OPC[k])
        if k == "CreateMat":
            _, contents, dim, id_ = c
            self.u32(self.idx(id_))
            self.dims(dim)
            if isinstance(contents, DevicePayload):
                self.u8(PAYLOAD_DEVICE)
                self.u64(contents.ptr)
                self.u64(contents.n)
                self.keepalive.append(contents)
                return
            arr = np.ascontiguousarray(contents, dtype=np.float32).reshape(-1)
            if arr.nbytes <= self.inline_limit:
                self.u8(PAYLOAD_INLINE)
                self.inline.append((len(self.body), arr))
                self.u64(0)
            else:
                self.u8(PAYLOAD_HOST)
                self.u64(arr.ctypes.data)
                self.keepalive.append(arr)
            self.u64(arr.size)
        elif k == "CreateConstant":
            _, contents, id_, dim = c
            self.u32(self.idx(id_))
            self.f32(contents)
            self.dims(dim)
        elif k in ("ElwMultiply", "ElwAdd", "DotProduct", "BatchDot"):
            self.u32(self.idx(c[1])); self.u32(self.idx(c[2])); self.u32(self.idx(c[3]))
        elif k in ("ElwMultiplyEq", "ElwAddEq"):
            self.u32(self.idx(c[1])); self.u32(self.idx(c[2]))
        elif k in ("EqualZero", "MoreZero", "LessZero", "Sum", "Max", "Contigious",
                   "Exp2", "Log2", "Sin", "Recip", "Sqrt"):
            self.u32(self.idx(c[1])); self.u32(self.idx(c[2]))
        elif k == "View":
            _, a, target_dim, res = c
            self.u32(self.idx(a)); self.u32(self.idx(res)); self.dims(target_dim)
        elif k == "Index":
            _, a, index, dim, res = c
            self.u32(self.idx(a)); self.u32(self.idx(res)); self.u64(index); self.u32(dim)
        elif k == "Concat":
            _, a, b, dim, res = c
            self.u32(self.idx(a)); self.u32(self.idx(b)); self.u32(self.idx(res)); self.u32(dim)
        elif k == "Permute":
            _, a, p, res = c
            self.u32(self.idx(a)); self.u32(self.idx(res)); self.u8(len(p))
            for x in p:
                self.u32(x)
        elif k == "Broadcast":
            _, a, dim, r, res = c
            self.u32(self.idx(a)); self.u32(self.idx(res)); self.u32(dim); self.u64(r)
        elif k == "While":
            _, cond, block = c
            self.u32(self.idx(cond)); self.proc(block)
        elif k == "If":
            _, conditions, else_proc = c
            self.u32(len(conditions))
            for cond, blk in conditions:
                self.u32(self.idx(cond)); self.proc(blk)
            self.u8(0 if else_proc is None else 1)
            if else_proc is not None:
                self.proc(else_proc)
        elif k == "EX":
            pass
        elif k == "Heading":
            b = c[1].encode("utf-8")[:65535]
            self.u16(len(b)); self.body += b
        elif k == "AllReduce":
            self.u32(self.idx(c[1]))
        else:
            raise ValueError(f"unknown IR command {k}")


def serialize(proc: IRProcedure, dep_list, inline_limit: int | None = None) -> tuple[bytes, list]:
    """Flatten (procedure, dep list) into the wire blob.

    Returns (blob, keepalive): `keepalive` holds the arrays whose addresses the
    blob references (PAYLOAD_HOST / PAYLOAD_DEVICE); the caller keeps it alive
    until `adb_execute` has returned.  `inline_limit` (bytes) overrides the size up to which
    host payloads are copied into the blob instead of being passed by address; a very large value
    gives a self-contained blob that can be written to a file.
    """
    w = _Writer()
    if inline_limit is not None:
        w.inline_limit = inline_limit
    w.proc(proc)
    dep = sorted(dep_list)
    dep_idx = [w.idx(d) for d in dep]
    head = bytearray()
    head += struct.pack("<IIII", MAGIC, VERSION, 0, len(w.ids))
    for s in w.ids:  # insertion order == index order
        b = s.encode("utf-8")
        head += struct.pack("<H", len(b)) + b
    head += struct.pack("<I", len(dep_idx))
    for i in dep_idx:
        head += struct.pack("<I", i)
    body_off = len(head)
    blob = head + w.body
    # payload section, 16-byte aligned
    for pos, arr in w.inline:
        while len(blob) % 16:
            blob += b"\0"
        struct.pack_into("<Q", blob, body_off + pos, len(blob))
        blob += arr.tobytes()
    return bytes(blob), w.keepalive
