"""The five benchmark programs and their seeded synthetic inputs.

Each `cN_*` function traces one program with the frontend mirror (so the device receives the IR the
reference frontend would emit for it), executes it on the installed device and returns the kept
tensors.  Sizes are parameters: the defaults are the full benchmark sizes, tests pass small ones.

Inputs are synthetic: element i of tensor t of a config is a pure function of (seed, t, i), produced
by a counter-based generator (Philox via numpy, then Box-Muller for normals), so any rank can
generate any row range of a tensor without generating the rest.
"""
from __future__ import annotations

import math

import numpy as np

from . import autodiff as ad
from . import nn
from .autodiff import f32


# --------------------------------------------------------------------------------------------------
# counter-based synthetic data
# --------------------------------------------------------------------------------------------------
def _raw_u32(seed: int, stream: int, start: int, count: int) -> np.ndarray:
    """`count` uint32 words starting at word `start` of stream (seed, stream)."""
    if count == 0:
        return np.zeros(0, np.uint32)
    bg = np.random.Philox(key=[seed & 0xFFFFFFFFFFFFFFFF, stream & 0xFFFFFFFFFFFFFFFF])
    # one Philox block = 4 x 64-bit outputs = 8 uint32 words
    first_block = start // 8
    bg.advance(first_block)
    skip = start - first_block * 8
    n64 = (skip + count + 1) // 2 + 1
    raw = bg.random_raw(n64).view(np.uint32)
    return raw[skip:skip + count]


def uniform(seed: int, stream: int, n: int, lo: float, hi: float, start: int = 0) -> np.ndarray:
    """U(lo, hi) as float32; element i depends only on (seed, stream, start + i)."""
    u = _raw_u32(seed, stream, start, n)
    x = (u >> np.uint32(8)).astype(np.float32) * f32(1.0 / (1 << 24))
    return (f32(lo) + x * f32(hi - lo)).astype(np.float32)


def normal(seed: int, stream: int, n: int, std: float = 1.0, start: int = 0) -> np.ndarray:
    """N(0, std^2) as float32 (Box-Muller on two words per element)."""
    u = _raw_u32(seed, stream, 2 * start, 2 * n).reshape(-1, 2)
    u1 = ((u[:, 0] >> np.uint32(8)).astype(np.float64) + 1.0) * (1.0 / (1 << 24))  # (0, 1]
    u2 = (u[:, 1] >> np.uint32(8)).astype(np.float64) * (1.0 / (1 << 24))
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * math.pi * u2)
    return (z * std).astype(np.float32)


# A second generator for tensors too large to draw on the host in reasonable time (the full-size benchmark batch):
# integer hashing only, so the same few lines run on numpy arrays and on torch tensors (CPU or CUDA) and give the
# same bits everywhere; any rank can produce any row range of a tensor.  Element i of (seed, stream) takes three
# 64-bit words  mix64(base + GOLDEN * (3 i + j + 1)),  j = 0..2  (mix64 = the splitmix64 finaliser); their twelve 16-bit
# fields are summed (Irwin-Hall), which is exact in integers:  z = (sum - 12 * 32767.5) / 65536  has mean 0, variance
# 1 - 2^-32 and the bell shape of a sum of twelve uniforms (support +-6).  It stands in for N(0, 1).
GOLDEN = 0x9E3779B97F4A7C15
_M1, _M2 = 0xBF58476D1CE4E5B9, 0x94D049BB133111EB


def _mix64(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> np.uint64(30))) * np.uint64(_M1)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(_M2)
    return z ^ (z >> np.uint64(31))


def hash_base(seed: int, stream: int) -> int:
    """Start of the counter space of (seed, stream) as a Python int in [0, 2^64)."""
    with np.errstate(over="ignore"):
        a = _mix64(np.array([(seed * GOLDEN + 0x1234567) % (1 << 64)], np.uint64))
        b = _mix64(np.array([(int(a[0]) ^ ((stream + 1) * _M2)) % (1 << 64)], np.uint64))
    return int(b[0])


def hash_normal(seed: int, stream: int, n: int, std: float = 1.0, start: int = 0) -> np.ndarray:
    """~N(0, std^2) as float32 (Irwin-Hall of twelve 16-bit uniforms); element i depends only on
    (seed, stream, start + i).  Bit-identical to `bench.py`'s torch version of the same arithmetic."""
    base = np.uint64(hash_base(seed, stream))
    out = np.empty(n, np.float32)
    step = 1 << 22
    with np.errstate(over="ignore"):
        for lo in range(0, n, step):
            cnt = min(step, n - lo)
            i = np.arange(start + lo, start + lo + cnt, dtype=np.uint64) * np.uint64(3)
            total = np.zeros(cnt, np.int64)
            for j in range(3):
                w = _mix64(base + np.uint64(GOLDEN) * (i + np.uint64(j + 1)))
                for f in range(4):
                    total += ((w >> np.uint64(16 * f)) & np.uint64(0xFFFF)).astype(np.int64)
            out[lo:lo + cnt] = ((total - 393210).astype(np.float32) * f32(1.0 / 65536.0)) * f32(std)
    return out


def _kept(names_values):
    return {k: v.get() for k, v in names_values.items()}


# --------------------------------------------------------------------------------------------------
# C1: README MLP, one SGD step
# --------------------------------------------------------------------------------------------------
def c1_inputs(seed: int = 0):
    k1, k2 = 1.0 / math.sqrt(5.0), 1.0 / math.sqrt(3.0)
    return {
        "x": np.asarray([1, 2, 3, 4, 5, 6, 7, 8, 3.2, 6.3], np.float32),
        "w1": uniform(seed, 0, 15, -k1, k1),
        "w2": uniform(seed, 1, 6, -k2, k2),
        "b2": uniform(seed, 2, 2, -k2, k2),
    }


def c1_readme_mlp(dev, inputs=None, lr: float = 0.1):
    """x[2,5] -> Linear(5,3, no bias) -> sigmoid -> Linear(3,2, bias); loss = sum of outputs;
    forward, backward and one SGD step (the README example of the reference, README.md:5-45)."""
    inp = inputs or c1_inputs()
    ad.set_device(dev)
    w1 = ad.tensor(inp["w1"], [5, 3])
    w2 = ad.tensor(inp["w2"], [3, 2])
    b2 = ad.tensor(inp["b2"], [2])
    x = ad.tensor(inp["x"], [2, 5])
    net = nn.Sequential()
    net.insert(nn.LinearWithWeights(w1, None))
    net.insert(nn.Sigmoid())
    net.insert(nn.LinearWithWeights(w2, b2))
    opt = nn.SGD(net.params(), lr)
    y = net.f(x)
    y.forward()
    y.backward()
    grads = {"w1_grad": w1.grad(), "w2_grad": w2.grad(), "b2_grad": b2.grad(), "x_grad": x.grad()}
    opt.step()
    y.val().keep()
    ad.execute()
    out = {"y": y.val(), "w1": w1.val(), "w2": w2.val(), "b2": b2.val()}
    out.update(grads)
    return _kept(out)


# --------------------------------------------------------------------------------------------------
# C2: fused element-wise chain with broadcast, forward + backward
# --------------------------------------------------------------------------------------------------
def c2_inputs(rows: int = 8192, cols: int = 8192, seed: int = 1):
    return {
        "a": normal(seed, 0, rows * cols),
        "b": normal(seed, 1, rows * cols),
        "bias": uniform(seed, 2, cols, -1.0, 1.0),
    }


def c2_fused_elementwise(dev, rows: int = 8192, cols: int = 8192, inputs=None, execute=True):
    """y = sigmoid(a*b + bias + 3).powf(2) * exp(-a) + sin(b) - cos(a) / (1 + b*b);
    loss = y.sum(1).sum(0); gradients w.r.t. a, b and bias."""
    inp = inputs or c2_inputs(rows, cols)
    ad.set_device(dev)
    ad.eager_dep_opt()
    a = ad.tensor(inp["a"], [rows, cols])
    b = ad.tensor(inp["b"], [rows, cols])
    bias = ad.tensor(inp["bias"], [cols])
    y = (a * b + bias + 3.0).sigmoid().powf(2.0) * (-a).exp() + b.sin() - a.cos() / (1.0 + b * b)
    loss = y.sum(1).sum(0)
    loss.forward()
    loss.backward()
    keep = {"loss": loss.val(), "a_grad": a.grad(), "b_grad": b.grad(), "bias_grad": bias.grad()}
    for v in keep.values():
        v.keep()
    if not execute:
        return keep
    ad.execute()
    return _kept(keep)


# --------------------------------------------------------------------------------------------------
# C3: reductions and data movement
# --------------------------------------------------------------------------------------------------
def c3_inputs(batch: int = 64, n: int = 1024, seed: int = 2):
    return {"x": uniform(seed, 0, batch * n * n, -1.0, 1.0)}


def c3_reduce_movement(dev, batch: int = 64, n: int = 1024, inputs=None, execute=True):
    """z = x.permute(0,2,1); s = z.sum(1); c = concat(s, 2s) along 0; rows batch/2 .. 3*batch/2;
    mask = (c > 0); per-row all; reshape to [batch*n]; backward from the slice to x.grad."""
    inp = inputs or c3_inputs(batch, n)
    ad.set_device(dev)
    ad.eager_dep_opt()
    x = ad.tensor(inp["x"], [batch, n, n])
    z = x.permute([0, 2, 1])
    s = z.sum(1)
    c = ad.concat([s, s * 2.0], 0)
    r = c.r(range(batch // 2, batch // 2 + batch), 0)
    mask = r.more_than(ad.constant(0.0, r.dim()))
    row_all = mask.sum(1).equal(ad.constant(float(n), [batch]))
    flat = mask.view([batch * n]).contigious()
    sc = s.contigious()
    rc = r.contigious()
    for t in (sc, rc, flat, row_all):
        t.forward()
    r.backward()
    keep = {"s": sc.val(), "slice": rc.val(), "mask": flat.val(), "row_all": row_all.val(), "x_grad": x.grad()}
    for v in keep.values():
        v.keep()
    if not execute:
        return keep
    ad.execute()
    return _kept(keep)


# --------------------------------------------------------------------------------------------------
# C4: MLP training (the data-parallel workload)
# --------------------------------------------------------------------------------------------------
C4_WIDTHS = (4096, 8192, 8192, 4096, 1000)


def c4_inputs(batch: int = 65536, widths=C4_WIDTHS, seed: int = 3, row_range=None):
    """X ~ N(0,1) [batch, widths[0]], T ~ N(0,1) [batch, widths[-1]], weights / biases U(+-1/sqrt(fan_in)).
    `row_range=(lo, hi)` generates only those rows of X and T (what one data-parallel rank needs)."""
    lo, hi = row_range or (0, batch)
    out = {
        "x": normal(seed, 0, (hi - lo) * widths[0], start=lo * widths[0]),
        "t": normal(seed, 1, (hi - lo) * widths[-1], start=lo * widths[-1]),
    }
    for i in range(len(widths) - 1):
        k = 1.0 / math.sqrt(widths[i])
        out[f"w{i}"] = uniform(seed, 10 + 2 * i, widths[i] * widths[i + 1], -k, k)
        out[f"b{i}"] = uniform(seed, 11 + 2 * i, widths[i + 1], -k, k)
    return out


def c4_mlp_train(dev, batch: int = 65536, widths=C4_WIDTHS, steps: int = 100, lr: float = 1e-3, inputs=None,
                 local_batch=None, execute=True):
    """Linear -> sigmoid (x3) -> Linear, MSE loss, SGD, `steps` iterations inside one IR for-loop.
    `batch` is the global batch; when the device shards the batch, pass `local_batch` rows of X / T per
    rank (dims in the IR stay global, the device rewrites them)."""
    inp = inputs or c4_inputs(batch, widths)
    ad.set_device(dev)
    ad.eager_dep_opt()
    n_layers = len(widths) - 1
    ws = [ad.tensor(inp[f"w{i}"], [widths[i], widths[i + 1]]) for i in range(n_layers)]
    bs = [ad.tensor(inp[f"b{i}"], [widths[i + 1]]) for i in range(n_layers)]
    x = ad.tensor(inp["x"], [batch, widths[0]])
    t = ad.tensor(inp["t"], [batch, widths[-1]])
    net = nn.Sequential()
    for i in range(n_layers):
        net.insert(nn.LinearWithWeights(ws[i], bs[i]))
        if i < n_layers - 1:
            net.insert(nn.Sigmoid())
    opt = nn.SGD(net.params(), lr)
    box = {}

    def body(_):
        y = net.f(x)
        d = y - t
        loss = d.pow2().sum(1).sum(0) * f32(1.0 / (batch * widths[-1]))
        opt.zero_grad()
        loss.forward()
        loss.backward()
        opt.step()
        box["loss"] = loss

    ad.ir_for(range(0, steps), body)
    keep = {"loss": box["loss"].val()}
    for i in range(n_layers):
        keep[f"w{i}"] = ws[i].val()
        keep[f"b{i}"] = bs[i].val()
    for v in keep.values():
        v.keep()
    if not execute:
        return keep
    ad.execute()
    return _kept(keep)


# --------------------------------------------------------------------------------------------------
# C5: dense dot products inside a while loop
# --------------------------------------------------------------------------------------------------
def c5_inputs(n: int = 8192, seed: int = 4):
    std = 1.0 / math.sqrt(n)
    return {"a": normal(seed, 0, n * n, std), "b": normal(seed, 1, n * n, std)}


def c5_dot_loop(dev, n: int = 8192, max_iters: int = 50, tol: float = 1e-3, step: float = 0.01, inputs=None,
                execute=True):
    """X <- X - step * (A.X - B) from X = 0 while not all(|A.X - B| < tol) and fewer than max_iters
    iterations; the forward product and both gradient products run every iteration."""
    inp = inputs or c5_inputs(n)
    ad.set_device(dev)
    a = ad.tensor(inp["a"], [n, n])
    b = ad.tensor(inp["b"], [n, n])
    x = ad.tensor(np.zeros(n * n, np.float32), [n, n])
    it = ad.scalar(0.0)
    resid = ad.dot(a, x) - b
    small = resid.pow2().sqrt().less_than(ad.constant(tol, [n, n])).all()
    cond = it.less_than(ad.constant(float(max_iters), [1])) * (1.0 - small)

    def body():
        nonlocal x, it
        resid.backward()
        # the op-assigns are emitted when the loop condition is re-forwarded (it depends on both), which
        # is what makes the residual product re-run on the updated X (src/core/control.rs:87-91)
        x += f32(-step) * resid.val().to_node()
        it += 1.0

    ad.ir_while(cond, body)
    keep = {"x": x.val(), "iters": it.val(), "a_grad": a.grad(), "x_grad": x.grad()}
    for v in keep.values():
        v.keep()
    if not execute:
        return keep
    ad.execute()
    return _kept(keep)
