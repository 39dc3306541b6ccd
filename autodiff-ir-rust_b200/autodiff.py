"""Host-side mirror of the reference's lazy-autodiff frontend, used as the caller above the C-ABI.

This is the piece that sits *above* the `Device` boundary: user code builds a graph of
`Tensor` nodes, `.forward()` / `.backward()` append IR commands to a global builder, and
`execute()` hands the finished procedure to the installed device.  It follows the
reference's decompositions command by command so that the IR a program emits here is
the IR the reference frontend would hand to `Device::execute`:

  * global builder / id allocator            src/ir/base.rs:5-61, src/core/ir.rs:145-232
  * Tensor handle and node protocol          src/core/node.rs:6-107
  * leaf / value / constant nodes            src/core/tensor.rs, value.rs, constant.rs
  * + and * (with op-assign forms) and sugar src/graph/ops/ops.rs:7-340
  * unary functions and their derivatives    src/graph/ops/func.rs:5-139
  * sum / mean / var                         src/graph/ops/sum.rs
  * dot                                      src/graph/ops/dot_product.rs
  * comparisons and .all()                   src/graph/ops/equality.rs
  * broadcast/view/permute/index/concat/...  src/graph/data/*.rs
  * ir_if / ir_if_else / ir_while / ir_for   src/core/control.rs
  * dependency ("keep") list                 src/core/dependency.rs

Known upstream behaviours that are reproduced on purpose (they shape the IR):
`Tensor -= f32` adds (ops.rs:288-292); Index backward pads with `i_dim[0]`
(index.rs:37-53); a node whose operand was replaced by an op-assign is re-forwarded
into the *same* result id (ops.rs:33-49), which is how loop-carried ids arise.
"""
from __future__ import annotations

import copy
import math
import numpy as np

from .ir import IRProcedure, format_ir

f32 = np.float32

LN_2 = f32(np.log(f32(2.0)))                 # 2.0f32.ln()
INV_LN_2 = f32(1.0) / LN_2                   # 1.0 / 2.0f32.ln()
LOG2_E = f32(np.log2(f32(math.e)))           # E.log2()
FRAC_PI_2 = f32(math.pi / 2)                 # std::f32::consts::FRAC_PI_2


# --------------------------------------------------------------------------------------
# global builder state (IRB, DEVICE, DEP_TRACKER, HARSH_DEP_LIST)
# --------------------------------------------------------------------------------------
class _IRBase:
    def __init__(self):
        self.id = 0
        self.proc_id = 0
        self.proc = IRProcedure("main")
        self.temp_proc: list[IRProcedure] = []

    @staticmethod
    def unique_id_idx(idx: int) -> str:
        # base-26 ids a..z, ba.. (src/ir/base.rs:17-31)
        alphabet = "abcdefghijklmnopqrstuvwxyz"
        base = 26
        out = []
        while idx >= base:
            out.append(alphabet[idx % base])
            idx //= base
            idx -= 1
        out.append(alphabet[idx])
        return "".join(reversed(out))

    def unique_id(self) -> str:
        r = self.unique_id_idx(self.id)
        self.id += 1
        return r

    def unique_id_proc(self) -> str:
        r = self.unique_id_idx(self.proc_id)
        self.proc_id += 1
        return r

    def add_cmd(self, cmd):
        (self.temp_proc[-1] if self.temp_proc else self.proc).push(cmd)


class _State:
    irb: _IRBase | None = None
    device = None
    dep: set | None = None
    harsh = False


def _irb() -> _IRBase:
    if _State.irb is None:
        raise RuntimeError("Can't unpack IRBuilder: call set_device first")
    return _State.irb


def ir_b_add(cmd):
    _irb().add_cmd(cmd)


def ir_b_id() -> str:
    return _irb().unique_id()


def add_to_dep(id_: str):
    if _State.dep is None:
        raise RuntimeError("Can't unpack dep tracker")
    _State.dep.add(id_)


def ret_dep_list() -> set:
    return set(_State.dep)


def is_harsh() -> bool:
    return _State.harsh


# --------------------------------------------------------------------------------------
# Value: (dim, id) handle of something the device will compute
# --------------------------------------------------------------------------------------
class Value:
    __slots__ = ("dim", "id")

    def __init__(self, dim, id_):
        self.dim = list(dim)
        self.id = id_

    @staticmethod
    def new(data, dim) -> "Value":
        id_ = ir_b_id()
        ir_b_add(("CreateMat", data, list(dim), id_))
        return Value(dim, id_)

    @staticmethod
    def fill(val, dim) -> "Value":
        n = int(np.prod(dim)) if len(dim) else 1
        return Value.new(np.full(n, val, dtype=f32), dim)

    @staticmethod
    def ones(dim):
        return Value.fill(1.0, dim)

    @staticmethod
    def zeros(dim):
        return Value.fill(0.0, dim)

    @staticmethod
    def empty():
        return Value([], "")

    def to_node(self) -> "Tensor":
        return Tensor(ValueNode(self))

    def to_node_with_grad(self) -> "Tensor":
        return Tensor(TensorNode(self, None))

    def get(self):
        """`Value::get` (src/core/value.rs:83-90): ask the device for the tensor behind this id."""
        if _State.device is None:
            raise RuntimeError("Can't unpack device")
        return _State.device.get_tensor(self.id)

    def keep(self):
        add_to_dep(self.id)

    def clone(self):
        return Value(self.dim, self.id)

    def __repr__(self):
        return f"Value(id={self.id!r}, dim={self.dim})"


class ValueData:
    """`struct ValueData` (src/core/value_data.rs:6-11)."""

    def __init__(self, dim, data, id_, is_none=False):
        self.dim = list(dim)
        self.data = data
        self.id = id_
        self.is_none = is_none

    @staticmethod
    def none():
        return ValueData([], np.zeros(0, dtype=f32), "", True)

    def round(self, num_digits: int) -> "ValueData":
        mult = f32(10.0) ** num_digits
        d = np.asarray(self.data, dtype=f32)
        r = (d * f32(mult))
        # Rust f32::round rounds half away from zero
        r = np.where(r >= 0, np.floor(r + f32(0.5)), np.ceil(r - f32(0.5))).astype(f32) / f32(mult)
        return ValueData(self.dim, r.astype(f32), self.id, self.is_none)

    def numpy(self) -> np.ndarray:
        return np.asarray(self.data, dtype=f32).reshape(self.dim)


# --------------------------------------------------------------------------------------
# Tensor handle + node protocol
# --------------------------------------------------------------------------------------
class Node:
    def forward(self) -> Value: raise NotImplementedError
    def backward(self, grad: Value): raise NotImplementedError
    def dim(self) -> list: raise NotImplementedError
    def val(self): raise NotImplementedError
    def grad(self) -> Value: raise RuntimeError("Calling .grad() on a non-tensor node")
    def reset_grad(self): raise RuntimeError("Calling .reset_grad() on a non-tensor node")
    def is_const(self) -> bool: return False
    def deep_copy(self) -> "Node": return copy.copy(self)


class Tensor:
    """Shared, replaceable handle on a node (`Rc<RefCell<Box<dyn NodeTrait>>>`, src/core/node.rs:39-44)."""

    __array_priority__ = 1000
    __array_ufunc__ = None  # numpy scalars defer to Tensor.__radd__/__rmul__/...

    def __init__(self, n: Node):
        self.n = n

    # Rc clone == same handle object
    def clone(self) -> "Tensor":
        return self

    def replace(self, node: Node):
        self.n = node

    def forward(self) -> Value:
        return self.n.forward()

    def backward(self):
        self.n.backward(Value.ones(self.dim()))

    def dim(self) -> list:
        return self.n.dim()

    def val(self):
        return self.n.val()

    def grad(self) -> Value:
        return self.n.grad()

    def reset_grad(self):
        self.n.reset_grad()

    def detach(self) -> "Tensor":
        self.forward()
        return self.val().to_node()

    def detach_grad(self) -> "Tensor":
        self.forward()
        return self.val().to_node_with_grad()

    def is_const(self) -> bool:
        return self.n.is_const()

    def deep_copy(self) -> "Tensor":
        return Tensor(self.n.deep_copy())

    # ------------------------------------------------------------------ + and *
    def __add__(self, other):
        return _binary(AddNode, self, other, False)

    def __radd__(self, other):
        return _binary(AddNode, other, self, False)

    def __mul__(self, other):
        return _binary(MultiplyNode, self, other, False)

    def __rmul__(self, other):
        return _binary(MultiplyNode, other, self, False)

    def __iadd__(self, rhs):
        _op_assign(AddNode, self, rhs)
        return self

    def __imul__(self, rhs):
        _op_assign(MultiplyNode, self, rhs)
        return self

    # ------------------------------------------------------------------ sugar (ops.rs:250-341)
    def __neg__(self):
        return f32(-1.0) * self

    def __sub__(self, other):
        if isinstance(other, Tensor):
            return self + f32(-1.0) * other
        return self + f32(f32(-1.0) * f32(other))

    def __rsub__(self, other):  # f32 - Tensor
        return f32(other) + f32(-1.0) * self

    def __isub__(self, rhs):
        if isinstance(rhs, Tensor):
            self += f32(-1.0) * rhs
        elif isinstance(rhs, Value):
            self += f32(-1.0) * rhs.to_node()
        else:
            # upstream: `impl SubAssign<f32>` adds rhs unchanged (src/graph/ops/ops.rs:288-292)
            self += f32(rhs)
        return self

    def __truediv__(self, other):
        if isinstance(other, Tensor):
            return self * other.recip()
        return self * f32(f32(1.0) / f32(other))

    def __rtruediv__(self, other):  # f32 / Tensor
        return f32(other) * self.recip()

    def __itruediv__(self, rhs):
        if isinstance(rhs, Tensor):
            self *= rhs.recip()
        elif isinstance(rhs, Value):
            self *= rhs.to_node().recip()
        else:
            self *= f32(f32(1.0) / f32(rhs))
        return self

    # ------------------------------------------------------------------ unary functions (func.rs)
    def exp2(self): return Tensor(FuncNode("Exp2", self))
    def log2(self): return Tensor(FuncNode("Log2", self))
    def recip(self): return Tensor(FuncNode("Recip", self))
    def sqrt(self): return Tensor(FuncNode("Sqrt", self))
    def sin(self): return Tensor(FuncNode("Sin", self))

    def cos(self):
        return (FRAC_PI_2 - self).sin()

    def exp(self):
        return (self * INV_LN_2).exp2()

    def ln(self):
        return self.log2() * LN_2

    def pow2(self):
        return self * self

    def abs(self):
        """|x| composed from existing primitives (upstream lists abs as missing, TODO.md:47): the device's Sqrt is
        sqrt(fabs(.)) (src/devices/opencl/kernels/unary.rs:11), so sqrt(x*x) is exact up to the rounding of x*x;
        the gradient x / |x| comes out of the pow2 / sqrt backward rules."""
        return self.pow2().sqrt()

    def pow3(self):
        return self.pow2() * self

    def pow(self, p: "Tensor"):
        return (p * self.log2()).exp2()

    def powf(self, p: float):
        if p == 2.0:
            return self.pow2()
        if p == 3.0:
            return self.pow3()
        return (f32(p) * self.log2()).exp2()

    # ------------------------------------------------------------------ reductions (sum.rs)
    def sum(self, dim: int) -> "Tensor":
        p_dim = len(self.dim())
        dim = p_dim + dim if dim < 0 else dim
        permute_to = list(range(p_dim))
        permute_to[-1] = dim
        permute_to[dim] = p_dim - 1
        node = self.permute(permute_to)
        new_dim = node.dim()
        node = node.view([-1, new_dim[-1]])
        node = Tensor(SumNode(node))
        new_dim = new_dim[:-1]
        node = node.view(list(new_dim))
        permute_to = permute_to[:dim] + permute_to[dim + 1:]
        return node.permute(permute_to)

    def max(self, dim: int) -> "Tensor":
        """Maximum along one axis: the same permute / view / reduce / view / permute sandwich as `sum`."""
        p_dim = len(self.dim())
        dim = p_dim + dim if dim < 0 else dim
        permute_to = list(range(p_dim))
        permute_to[-1] = dim
        permute_to[dim] = p_dim - 1
        node = self.permute(permute_to)
        new_dim = node.dim()
        node = node.view([-1, new_dim[-1]])
        node = Tensor(MaxNode(node))
        new_dim = new_dim[:-1]
        node = node.view(list(new_dim))
        permute_to = permute_to[:dim] + permute_to[dim + 1:]
        return node.permute(permute_to)

    def mean(self, dim: int) -> "Tensor":
        p_dim = self.dim()
        d = len(p_dim) + dim if dim < 0 else dim
        return self.sum(d) / f32(p_dim[d])

    def var(self, dim: int, correction: int) -> "Tensor":
        a = (self - self.mean(dim).unsqueeze(dim)).pow2()
        p_dim = self.dim()
        d = len(p_dim) + dim if dim < 0 else dim
        return a.sum(dim) / f32(p_dim[d] - correction)

    # ------------------------------------------------------------------ data movement
    def permute(self, p) -> "Tensor":
        p = list(p)
        if all(i == v for i, v in enumerate(p)):
            return self
        return Tensor(PermuteNode(self, p))

    def t(self) -> "Tensor":
        assert len(self.dim()) == 2, "Transpose only supprots 2D matrix"
        return Tensor(PermuteNode(self, [1, 0]))

    def view(self, target_dim) -> "Tensor":
        target_dim = list(target_dim) if len(target_dim) else [1]
        source_dim = self.dim()
        target = handle_minus_dim(source_dim, target_dim)
        if target != source_dim:
            return Tensor(ViewNode(self, target))
        return self

    def flatten(self):
        return self.view([int(np.prod(self.dim()))])

    def unsqueeze(self, dim: int):
        p = len(self.dim())
        dim = p + dim + 1 if dim < 0 else dim
        nd = list(self.dim())
        nd.insert(dim, 1)
        return self.view(nd)

    def squeeze(self, dim: int):
        if len(self.dim()) <= 1:
            return self
        nd = list(self.dim())
        assert nd[dim] == 1, "Squeeze dim must be one"
        del nd[dim]
        return self.view(nd)

    def i(self, i: int, dim: int) -> "Tensor":
        p_dim = self.dim()
        dim = len(p_dim) + dim if dim < 0 else dim
        assert dim < len(p_dim), "invalid dimension!"
        assert i < p_dim[dim], "invalid index!"
        return Tensor(IndexNode(self, i, dim))

    def r(self, rng, dim: int) -> "Tensor":
        return concat([self.i(i, dim).unsqueeze(dim) for i in rng], dim)

    def repeat(self, f, length: int, dim: int) -> "Tensor":
        return concat([f(self, i).unsqueeze(dim) for i in range(length)], dim)

    def broadcast(self, dim: int, r: int) -> "Tensor":
        target = list(self.dim())
        dim = len(target) + dim if dim < 0 else dim
        target[dim] = r
        return _make_broadcast_node(self, target)

    def contigious(self) -> "Tensor":
        return Tensor(ContigiousNode(self))

    # ------------------------------------------------------------------ comparisons (equality.rs)
    def equal(self, b: "Tensor"): return Tensor(CompareNode("EqualZero", self - b))
    def more_than(self, b: "Tensor"): return Tensor(CompareNode("MoreZero", self - b))
    def less_than(self, b: "Tensor"): return Tensor(CompareNode("LessZero", self - b))

    def all(self) -> "Tensor":
        x = self
        total = int(np.prod(self.dim()))
        for _ in self.dim():
            x = x.sum(0)
        return x.equal(constant(float(total), [1]))

    # ------------------------------------------------------------------ activations (src/nn/activations)
    def sigmoid(self):
        return f32(1.0) / (f32(1.0) + (-self).exp())

    def relu(self):
        return self * self.more_than(constant(0.0, self.dim()))

    def softmax(self, dim: int):
        return self.exp() / self.exp().sum(dim)


def _as_tensor_pair(a, b):
    """Wrap a scalar operand as a ConstantNode with the other operand's dims (ops.rs:147-176)."""
    if not isinstance(a, Tensor):
        a = constant(a, b.dim())
    elif not isinstance(b, Tensor):
        if isinstance(b, Value):
            b = b.to_node()
        else:
            b = constant(b, a.dim())
    return a, b


def _binary(cls, a, b, is_op_equal):
    a, b = _as_tensor_pair(a, b)
    a, b = try_broadcast(a, b)
    return Tensor(cls(a, b, is_op_equal))


def _op_assign(cls, self_t: Tensor, rhs):
    s_clone = self_t.deep_copy()
    if isinstance(rhs, Value):
        rhs = rhs.to_node()
    elif not isinstance(rhs, Tensor):
        rhs = constant(rhs, self_t.dim())
    a, b = try_broadcast(s_clone, rhs)
    self_t.replace(cls(a, b, True))


# --------------------------------------------------------------------------------------
# leaf nodes
# --------------------------------------------------------------------------------------
class TensorNode(Node):
    def __init__(self, v: Value, gd):
        self.v = v
        self.gd = gd

    def forward(self): return self.v.clone()

    def backward(self, grad: Value):
        if self.gd is not None:
            g = self.gd.to_node()
            g += grad.to_node()
            g.forward()
        else:
            self.gd = grad.clone()
            if not is_harsh():
                self.gd.keep()

    def dim(self): return list(self.v.dim)
    def val(self): return self.v.clone()

    def grad(self):
        if self.gd is None:
            raise RuntimeError("Must run backwards before calling grad()")
        return self.gd.clone()

    def reset_grad(self): self.gd = None


class ValueNode(Node):
    def __init__(self, v: Value): self.v = v
    def forward(self): return self.v.clone()
    def backward(self, grad): pass
    def dim(self): return list(self.v.dim)
    def val(self): return self.v.clone()


class ConstantNode(Node):
    def __init__(self, content, dim):
        self.content = f32(content)
        self._dim = list(dim)
        self._val = None

    def forward(self):
        if self._val is None:
            id_ = ir_b_id()
            ir_b_add(("CreateConstant", float(self.content), id_, list(self._dim)))
            self._val = Value(self._dim, id_)
        return self._val.clone()

    def backward(self, grad): pass
    def dim(self): return list(self._dim)
    def val(self): return None if self._val is None else self._val.clone()
    def is_const(self): return True


# --------------------------------------------------------------------------------------
# + and *  (create_op!, src/graph/ops/ops.rs:7-219)
# --------------------------------------------------------------------------------------
class _BinaryNode(Node):
    IR = IR_EQ = None

    def __init__(self, left: Tensor, right: Tensor, is_op_equal: bool):
        self.left, self.right = left, right
        self._val = None
        self.is_op_equal = is_op_equal

    def forward(self):
        v = self.val()
        if v is not None:
            return v
        left = self.left.forward()
        right = self.right.forward()
        if self.is_op_equal:
            ir_b_add((self.IR_EQ, left.id, right.id))
            res = Value(left.dim, left.id)
        else:
            id_ = self._val.id if self._val is not None else ir_b_id()
            ir_b_add((self.IR, left.id, right.id, id_))
            res = Value(left.dim, id_)
        self._val = res.clone()
        return res

    def dim(self):
        return self.right.dim() if self.left.is_const() else self.left.dim()

    def val(self):
        if self.left.val() is None or self.right.val() is None:
            return None
        return None if self._val is None else self._val.clone()

    def grad(self):
        if self.is_op_equal:
            return self.left.grad()
        raise RuntimeError("Calling .grad() on a non-tensor node")

    def reset_grad(self):
        if self.is_op_equal:
            self.left.reset_grad()
        else:
            raise RuntimeError("Calling .reset_grad() on a non-tensor node")


class AddNode(_BinaryNode):
    IR, IR_EQ = "ElwAdd", "ElwAddEq"

    def backward(self, grad):
        assert self.left.val() is not None and self.right.val() is not None, "forward first"
        self.left.n.backward(grad.clone())
        self.right.n.backward(grad.clone())


class MultiplyNode(_BinaryNode):
    IR, IR_EQ = "ElwMultiply", "ElwMultiplyEq"

    def backward(self, grad):
        l = self.left.val()
        r = self.right.val()
        assert l is not None and r is not None, "forward first"
        self.left.n.backward((r.to_node() * grad.to_node()).forward())
        self.right.n.backward((l.to_node() * grad.to_node()).forward())


# --------------------------------------------------------------------------------------
# unary functions (create_func!, src/graph/ops/func.rs:5-70)
# --------------------------------------------------------------------------------------
class _UnaryBase(Node):
    def __init__(self, parent: Tensor):
        self.parent = parent
        self._val = None

    def dim(self): return self.parent.dim()

    def val(self):
        if self.parent.val() is None:
            return None
        return None if self._val is None else self._val.clone()

    def _emit(self, p: Value) -> Value:
        raise NotImplementedError

    def forward(self):
        v = self.val()
        if v is not None:
            return v
        res = self._emit(self.parent.forward())
        self._val = res.clone()
        return res

    def _res_id(self):
        return self._val.id if self._val is not None else ir_b_id()


class FuncNode(_UnaryBase):
    def __init__(self, ir: str, parent: Tensor):
        super().__init__(parent)
        self.ir = ir

    def _emit(self, a):
        id_ = self._res_id()
        ir_b_add((self.ir, a.id, id_))
        return Value(a.dim, id_)

    def backward(self, grad):
        v = self.parent.val()
        assert v is not None, "parent val invalid at unary func"
        g, x = grad.to_node(), v.to_node()
        if self.ir == "Exp2":
            out = g * LN_2 * x.exp2()
        elif self.ir == "Log2":
            out = g * x.recip() * LOG2_E
        elif self.ir == "Recip":
            out = g * (f32(-1.0) / x.pow2())
        elif self.ir == "Sqrt":
            out = g * (f32(1.0) / (f32(2.0) * x.sqrt()))
        elif self.ir == "Sin":
            out = g * x.cos()
        else:
            raise AssertionError(self.ir)
        self.parent.n.backward(out.forward())


class CompareNode(_UnaryBase):
    def __init__(self, ir: str, parent: Tensor):
        super().__init__(parent)
        self.ir = ir

    def _emit(self, a):
        id_ = self._res_id()
        ir_b_add((self.ir, a.id, id_))
        return Value(a.dim, id_)

    def backward(self, grad): pass

    def grad(self): return Value.zeros(self.dim())


class SumNode(_UnaryBase):
    def forward(self):
        v = self.val()
        if v is not None:
            return v
        val = self.parent.forward()
        assert len(self.parent.dim()) == 2, "Reduce (sum) node needs dim=2"
        id_ = self._res_id()
        ir_b_add(("Sum", val.id, id_))
        res = Value(val.dim[:-1], id_)
        self._val = res.clone()
        return res

    def dim(self): return self.parent.dim()[:-1]

    def backward(self, grad):
        n = self.parent.dim()[-1]
        self.parent.n.backward(grad.to_node().unsqueeze(-1).broadcast(-1, n).forward())


class MaxNode(_UnaryBase):
    """Row maximum of a 2-d tensor (IR extension `Max`).  Backward sends the gradient to every position that holds
    the maximum of its row (ties share it undivided, like the comparison-based masks upstream uses for relu)."""

    def forward(self):
        v = self.val()
        if v is not None:
            return v
        val = self.parent.forward()
        assert len(self.parent.dim()) == 2, "Reduce (max) node needs dim=2"
        id_ = self._res_id()
        ir_b_add(("Max", val.id, id_))
        res = Value(val.dim[:-1], id_)
        self._val = res.clone()
        return res

    def dim(self): return self.parent.dim()[:-1]

    def backward(self, grad):
        n = self.parent.dim()[-1]
        top = Tensor(self).unsqueeze(-1).broadcast(-1, n)
        mask = self.parent.equal(top)
        self.parent.n.backward((grad.to_node().unsqueeze(-1).broadcast(-1, n) * mask).forward())


class DotProductNode(Node):
    def __init__(self, left, right):
        self.left, self.right = left, right
        self._val = None

    def forward(self):
        v = self.val()
        if v is not None:
            return v
        left, right = self.left.forward(), self.right.forward()
        assert len(left.dim) == 2, "A must be a 2d array"
        assert len(right.dim) == 2, "B must be a 2d array"
        assert left.dim[1] == right.dim[0], "A's second dimension must equal B's first dimension"
        id_ = self._val.id if self._val is not None else ir_b_id()
        ir_b_add(("DotProduct", left.id, right.id, id_))
        res = Value([left.dim[0], right.dim[-1]], id_)
        self._val = res.clone()
        return res

    def dim(self): return [self.left.dim()[0], self.right.dim()[-1]]

    def val(self):
        if self.left.val() is None or self.right.val() is None:
            return None
        return None if self._val is None else self._val.clone()

    def backward(self, grad):
        g = grad.to_node()
        self.left.n.backward(dot(g, self.right.t()).forward())
        self.right.n.backward(dot(self.left.t(), g).forward())


def dot(a: Tensor, b: Tensor) -> Tensor:
    return Tensor(DotProductNode(a, b))


class BatchDotNode(Node):
    """Batched matrix product [B, M, K] x [B, K, N] -> [B, M, N] (IR extension `BatchDot`).  Upstream lists batched
    matmul as missing (TODO.md:22) and runs attention as one 2-d `dot` per head (src/nn/transformer.rs:10-18); the
    gradients follow DotProductNode slice by slice: dA = g . B^T, dB = A^T . g with the last two axes swapped."""

    def __init__(self, left, right):
        self.left, self.right = left, right
        self._val = None

    def forward(self):
        v = self.val()
        if v is not None:
            return v
        left, right = self.left.forward(), self.right.forward()
        assert len(left.dim) == 3 and len(right.dim) == 3, "bmm needs 3d operands"
        assert left.dim[0] == right.dim[0], "bmm operands differ in their batch size"
        assert left.dim[2] == right.dim[1], "A's last dimension must equal B's second dimension"
        id_ = self._val.id if self._val is not None else ir_b_id()
        ir_b_add(("BatchDot", left.id, right.id, id_))
        res = Value([left.dim[0], left.dim[1], right.dim[2]], id_)
        self._val = res.clone()
        return res

    def dim(self): return [self.left.dim()[0], self.left.dim()[1], self.right.dim()[2]]

    def val(self):
        if self.left.val() is None or self.right.val() is None:
            return None
        return None if self._val is None else self._val.clone()

    def backward(self, grad):
        g = grad.to_node()
        self.left.n.backward(bmm(g, self.right.permute([0, 2, 1])).forward())
        self.right.n.backward(bmm(self.left.permute([0, 2, 1]), g).forward())


def bmm(a: Tensor, b: Tensor) -> Tensor:
    return Tensor(BatchDotNode(a, b))


# --------------------------------------------------------------------------------------
# data-movement nodes (src/graph/data)
# --------------------------------------------------------------------------------------
def handle_minus_dim(source_dim, input_dim):
    input_dim = [int(x) for x in input_dim]
    if -1 in input_dim:
        idx = input_dim.index(-1)
        total = int(np.prod(source_dim))
        inp = -int(np.prod(input_dim))
        assert total % inp == 0, "Can't fill in -1"
        ret = list(input_dim)
        ret[idx] = total // inp
        return ret
    return list(input_dim)


def _c_view(p: Value, target_dim, id_=None) -> Value:
    assert int(np.prod(target_dim)) == int(np.prod(p.dim)), "Target dim must be same size as input dim"
    id_ = id_ or ir_b_id()
    ir_b_add(("View", p.id, list(target_dim), id_))
    return Value(target_dim, id_)


def _c_permute(a: Value, permute, id_=None) -> Value:
    assert len(permute) == len(a.dim), "Permute dimension mismatch"
    for i in permute:
        if i >= len(a.dim):
            raise IndexError("Permute index out of bounds")
    if all(i == v for i, v in enumerate(permute)):
        return a.clone()
    id_ = id_ or ir_b_id()
    ir_b_add(("Permute", a.id, list(permute), id_))
    return Value([a.dim[permute[i]] for i in range(len(a.dim))], id_)


class ViewNode(_UnaryBase):
    def __init__(self, parent, target_dim):
        super().__init__(parent)
        self.target_dim = list(target_dim)

    def forward(self):
        # Divergence from upstream: there the cached field is returned unconditionally
        # (src/graph/data/view.rs:19-27), so a reshape inside a loop condition is never
        # re-forwarded and the condition goes stale.  Here a view re-forwards like every other
        # node (same result id), which is what `.all()` inside `ir_while` needs.
        v = self.val()
        if v is not None:
            return v
        p = self.parent.forward()
        res = _c_view(p, self.target_dim, self._val.id if self._val is not None else None)
        self._val = res.clone()
        return res

    def dim(self): return list(self.target_dim)

    def backward(self, grad):
        self.parent.n.backward(_c_view(grad, self.parent.dim(), None))


class PermuteNode(_UnaryBase):
    def __init__(self, parent, permute):
        super().__init__(parent)
        self.permute = list(permute)

    def _emit(self, p):
        return _c_permute(p, self.permute, self._val.id if self._val is not None else None)

    def dim(self):
        c = self.parent.dim()
        return [c[self.permute[i]] for i in range(len(c))]

    def backward(self, grad):
        inv = [0] * len(self.permute)
        for i, p in enumerate(self.permute):
            inv[p] = i
        self.parent.n.backward(_c_permute(grad, inv, None))


class BroadcastNode(_UnaryBase):
    def __init__(self, parent, repeat, dim):
        super().__init__(parent)
        self.repeat, self._bdim = repeat, dim

    def _emit(self, p):
        id_ = self._res_id()
        ir_b_add(("Broadcast", p.id, self._bdim, self.repeat, id_))
        d = list(p.dim)
        d[self._bdim] = self.repeat
        return Value(d, id_)

    def dim(self):
        d = self.parent.dim()
        d[self._bdim] = self.repeat
        return d

    def backward(self, grad):
        self.parent.n.backward(grad.to_node().sum(self._bdim).forward())


class IndexNode(_UnaryBase):
    def __init__(self, parent, idx, dim):
        super().__init__(parent)
        self.idx, self._idim = idx, dim

    def _emit(self, a):
        id_ = self._res_id()
        ir_b_add(("Index", a.id, self.idx, self._idim, id_))
        d = list(a.dim)
        del d[self._idim]
        return Value(d, id_)

    def dim(self):
        d = self.parent.dim()
        del d[self._idim]
        return d

    def backward(self, grad):
        i_dim = self.parent.dim()
        z1 = list(i_dim); z1[self._idim] = self.idx
        # upstream uses i_dim[0] here regardless of self.dim (src/graph/data/index.rs:43-44)
        z2 = list(i_dim); z2[self._idim] = i_dim[0] - self.idx - 1
        first_zero = Value.zeros(z1).to_node()
        second_zero = Value.zeros(z2).to_node()
        g = grad.to_node()
        self.parent.n.backward(concat([first_zero, g.unsqueeze(0), second_zero], self._idim).forward())


class ConcatNode(Node):
    def __init__(self, nodes, dim):
        self.nodes, self._cdim = list(nodes), dim
        self._val = None

    def forward(self):
        v = self.val()
        if v is not None:
            return v
        values = [n.forward() for n in self.nodes]
        res = _c_concat(values, self._cdim, self._val.id if self._val is not None else None)
        self._val = res.clone()
        return res

    def dim(self):
        d = self.nodes[0].dim()
        for n in self.nodes[1:]:
            d[self._cdim] += n.dim()[self._cdim]
        return d

    def backward(self, grad):
        c = 0
        for n in self.nodes:
            d = n.dim()[self._cdim]
            g = grad.to_node().r(range(c, c + d), self._cdim).forward()
            n.n.backward(g)
            c += d

    def val(self):
        for n in self.nodes:
            if n.val() is None:
                return None
        return None if self._val is None else self._val.clone()


def _c_concat(values, dim, id_=None) -> Value:
    first = list(values[0].dim)
    for v in values[1:]:
        assert len(first) == len(v.dim), "Dimensions are not equal at concat"
        a, b = list(first), list(v.dim)
        del a[dim]; del b[dim]
        assert a == b, "Dim misaligned at concat"
    prev = values[0].id
    total = list(values[0].dim)
    last_id = id_ or ir_b_id()
    for i in range(1, len(values)):
        new_id = last_id if i == len(values) - 1 else ir_b_id()
        ir_b_add(("Concat", prev, values[i].id, dim, new_id))
        prev = new_id
        total[dim] += values[i].dim[dim]
    return Value(total, prev)


def concat(nodes, dim: int) -> Tensor:
    n_dim = len(nodes[0].dim())
    dim = n_dim + dim if dim < 0 else dim
    return Tensor(ConcatNode(nodes, dim))


class ContigiousNode(_UnaryBase):
    def _emit(self, a):
        id_ = self._res_id()
        ir_b_add(("Contigious", a.id, id_))
        return Value(a.dim, id_)

    def backward(self, grad):
        self.parent.n.backward(grad)


# --------------------------------------------------------------------------------------
# implicit broadcasting (src/graph/data/broadcast.rs:44-190)
# --------------------------------------------------------------------------------------
def _is_broadcastable(da, db) -> bool:
    la, lb = len(da), len(db)
    if la == 0 or lb == 0:
        return False
    for i in range(max(la, lb)):
        if i >= la or i >= lb:
            return True
        a, b = da[la - i - 1], db[lb - i - 1]
        if a != b and a != 1 and b != 1:
            return False
    return True


def _make_broadcast_node(n: Tensor, target_dim) -> Tensor:
    n_dim = list(n.dim())
    assert len(target_dim) >= len(n_dim), "Wrong broadcasted node"
    n_dim = [1] * (len(target_dim) - len(n_dim)) + n_dim
    ret = n.view(n_dim)
    for i in range(len(target_dim)):
        if target_dim[i] != n_dim[i]:
            assert n_dim[i] == 1, "Can't broadcast to target dim"
            ret = Tensor(BroadcastNode(ret, target_dim[i], i))
    return ret


def try_broadcast(a: Tensor, b: Tensor):
    if len(a.dim()) == 0 and len(b.dim()) > 0:
        a = a.unsqueeze(0)
    if len(b.dim()) == 0 and len(a.dim()) > 0:
        b = b.unsqueeze(0)
    if a.dim() == b.dim():
        return a, b
    if a.is_const() or b.is_const():
        return a, b
    if _is_broadcastable(a.dim(), b.dim()):
        la, lb = len(a.dim()), len(b.dim())
        is_a = (sum(a.dim()) < sum(b.dim())) if la == lb else (la < lb)
        if is_a:
            return _make_broadcast_node(a, b.dim()), b
        return a, _make_broadcast_node(b, a.dim())
    raise ValueError(f"Cannot broadcast {a.dim()} to {b.dim()}")


# --------------------------------------------------------------------------------------
# public constructors and session control (src/core/autodiff.rs)
# --------------------------------------------------------------------------------------
def tensor(data, dim, local_rows=None) -> Tensor:
    """`autodiff::tensor` (src/core/autodiff.rs:24-41).  `local_rows`: for data-parallel runs the caller may
    hand over only its own rows of a tensor whose `dim` is the global shape (the device splits axis 0)."""
    dim = list(dim)
    if isinstance(data, (list, tuple)):
        data = np.asarray(data, dtype=f32)
    n = len(data)
    full = int(np.prod(dim)) if dim else 1
    if local_rows is not None:
        full = full // dim[0] * local_rows
    if n != full:
        raise ValueError("# of values doesn't match dim size when calling from_vec")
    v = Value.new(data, dim)
    if not is_harsh():
        add_to_dep(v.id)
    return Tensor(TensorNode(v, None))


def scalar(val: float) -> Tensor:
    return tensor(np.asarray([val], dtype=f32), [1])


def constant(val: float, dim) -> Tensor:
    return Tensor(ConstantNode(val, dim))


def fill(val, dim) -> Tensor:
    return tensor(np.full(int(np.prod(dim)), val, dtype=f32), dim)


def ones(dim): return fill(1.0, dim)
def zeros(dim): return fill(0.0, dim)


def empty() -> Tensor:
    return Tensor(TensorNode(Value.empty(), None))


def randn(dim, rng=None) -> Tensor:
    """Standard-normal tensor.  The reference draws from an unseeded thread RNG
    (src/core/autodiff.rs:75-80); here a numpy Generator may be passed for reproducibility."""
    rng = rng or np.random.default_rng()
    return tensor(rng.standard_normal(int(np.prod(dim)), dtype=f32), dim)


def set_device(device):
    """`autodiff::set_device` (src/core/autodiff.rs:82-97): fresh builder, device and dep list.
    Unlike upstream, the eager-dep flag is also reset so sessions do not leak into each other."""
    _State.irb = _IRBase()
    _State.device = device
    _State.dep = set()
    _State.harsh = False


def add_heading(cmt: str):
    ir_b_add(("Heading", cmt))


def eager_dep_opt():
    _State.harsh = True


def current_ir() -> IRProcedure:
    return _irb().proc


def execute():
    """`autodiff::execute` (src/core/autodiff.rs:108-114).  The reference's host-side IR clean-up
    passes run before the boundary and do not change results; the device does its own
    dead-code elimination from the dep list, so the procedure is handed over as traced."""
    ir_b_add(("EX",))
    dev = _State.device
    dev.ir_callback(_irb())
    dev.execute(_irb().proc, ret_dep_list())


def print_and_exec():
    ir_b_add(("EX",))
    dev = _State.device
    dev.ir_callback(_irb())
    print(format_ir(_irb().proc))
    dev.execute(_irb().proc, ret_dep_list())


# --------------------------------------------------------------------------------------
# control flow (src/core/control.rs)
# --------------------------------------------------------------------------------------
def _create_temp_proc():
    b = _irb()
    b.temp_proc.append(IRProcedure(b.unique_id_proc()))


def _return_temp_proc() -> IRProcedure:
    return _irb().temp_proc.pop()


def ir_if(expr, func):
    v = expr().forward()
    add_to_dep(v.id)
    if v.dim != [1]:
        raise ValueError("If expression must have dim of [1]")
    _create_temp_proc()
    func()
    blk = _return_temp_proc()
    ir_b_add(("If", [(v.id, blk)], None))


def ir_if_else(expr, func, func_else):
    v = expr().forward()
    add_to_dep(v.id)
    if v.dim != [1]:
        raise ValueError("Expr must return a boolean")
    _create_temp_proc()
    func()
    blk = _return_temp_proc()
    _create_temp_proc()
    func_else()
    blk_else = _return_temp_proc()
    ir_b_add(("If", [(v.id, blk)], blk_else))


def ir_while(var: Tensor, func):
    v = var.forward()
    add_to_dep(v.id)
    if v.dim != [1]:
        raise ValueError("Expr must return a boolean.")
    _create_temp_proc()
    func()
    r = var.forward()
    blk = _return_temp_proc()
    ir_b_add(("While", r.id, blk))


def ir_for(rng: range, func):
    x = scalar(float(rng.start))
    x_end = constant(float(rng.stop), [1])
    result = x.less_than(x_end)

    def body():
        nonlocal x
        func(x)
        x += f32(1.0)

    ir_while(result, body)
