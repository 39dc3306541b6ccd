"""Seeded random programs over the frontend mirror, for differential testing of the lowering.

`build(seed, exact)` returns a function `prog(dev) -> {name: ValueData}`.  With `exact=True` only
operations whose results are exactly representable are used (small integers, + * compare, views,
index, concat, permute, sums), so device and oracle must agree bit for bit; otherwise transcendental
functions, reciprocals and dot products are mixed in and a relative tolerance applies."""
from __future__ import annotations

import importlib

import numpy as np

adb = importlib.import_module("autodiff-ir-rust_b200")
ad = adb.autodiff

DIMS = [1, 2, 3, 4, 5, 8]


def build(seed: int, exact: bool, n_ops: int = 14):
    def prog(dev):
        rng = np.random.default_rng(seed)
        ad.set_device(dev)
        ad.eager_dep_opt()

        def leaf(shape):
            n = int(np.prod(shape))
            data = rng.integers(-3, 4, n).astype(np.float32) if exact else rng.standard_normal(n).astype(np.float32)
            return ad.tensor(data, list(shape))

        pool = []
        for _ in range(3):
            rank = int(rng.integers(1, 4))
            pool.append(leaf([int(rng.choice(DIMS)) for _ in range(rank)]))
        leaves = list(pool)

        def pick():
            return pool[int(rng.integers(0, len(pool)))]

        for _ in range(n_ops):
            kind = int(rng.integers(0, 12))
            t = pick()
            d = t.dim()
            try:
                if kind == 0:      # binary with a fresh same-shape leaf or broadcastable row
                    other = leaf(d) if rng.random() < 0.5 else leaf(d[-1:])
                    r = t + other if rng.random() < 0.5 else t * other
                elif kind == 1:    # scalar ops
                    c = float(rng.integers(-2, 3)) if exact else float(rng.standard_normal())
                    r = t * c + (1.0 if exact else 0.5)
                elif kind == 2:    # comparison against a leaf
                    other = leaf(d)
                    r = [t.equal, t.more_than, t.less_than][int(rng.integers(0, 3))](other)
                elif kind == 3:    # sum over an axis
                    if len(d) < 1 or int(np.prod(d)) > 4096:
                        continue
                    r = t.sum(int(rng.integers(0, len(d))))
                elif kind == 4:    # permute
                    if len(d) < 2:
                        continue
                    r = t.permute([int(x) for x in rng.permutation(len(d))])
                elif kind == 5:    # reshape
                    n = int(np.prod(d))
                    opts = [[n], [1, n], [n, 1]] + [[a, n // a] for a in (2, 3, 4) if n % a == 0]
                    r = t.view(opts[int(rng.integers(0, len(opts)))])
                elif kind == 6:    # index
                    if len(d) < 2:
                        continue
                    ax = int(rng.integers(0, len(d)))
                    r = t.i(int(rng.integers(0, d[ax])), ax)
                elif kind == 7:    # concat with a transformed copy of itself
                    ax = int(rng.integers(0, len(d)))
                    r = ad.concat([t, t * 2.0, t], ax) if rng.random() < 0.5 else ad.concat([t, leaf(d)], ax)
                elif kind == 8:    # range slice
                    ax = int(rng.integers(0, len(d)))
                    if d[ax] < 2:
                        continue
                    lo = int(rng.integers(0, d[ax] - 1))
                    hi = int(rng.integers(lo + 1, d[ax] + 1))
                    r = t.r(range(lo, hi), ax)
                elif kind == 9:    # dot with a fresh matrix
                    if len(d) != 2:
                        continue
                    w = leaf([d[1], int(rng.choice(DIMS))])
                    r = ad.dot(t, w) if rng.random() < 0.6 else ad.dot(t.t().t(), w)
                elif kind == 10:   # in-place update of a leaf
                    if exact:
                        t2 = leaves[int(rng.integers(0, len(leaves)))]
                        t2 += 1.0
                        t2.forward()
                        continue
                    r = (t * t + 1.0).recip()
                else:              # transcendental chain (bounded)
                    if exact:
                        r = t * t
                    else:
                        r = [lambda x: x.sin(), lambda x: (x.sin() * 2.0).exp2(), lambda x: (x * x + 1.0).log2(),
                             lambda x: (x * x + 0.5).sqrt(), lambda x: x.sigmoid()][int(rng.integers(0, 5))](t)
            except (AssertionError, ValueError):
                continue
            if int(np.prod(r.dim())) <= 1 << 14:
                pool.append(r)
        outs = {}
        chosen = list(range(len(pool)))[-5:]
        for k in chosen:
            v = pool[k].forward()
            v.keep()
            outs[f"t{k}"] = v
        # gradients through the last value back to the leaves
        last = pool[-1]
        try:
            last.backward()
        except (AssertionError, ValueError, IndexError):
            # upstream's Index backward only works along axis 0 (src/graph/data/index.rs:37-53); whatever was
            # emitted before the frontend gave up is still a valid program
            pass
        for i, lf in enumerate(leaves):
            try:
                g = lf.grad()
            except RuntimeError:
                continue
            g.keep()
            outs[f"g{i}"] = g
        ad.execute()
        return {k: v.get() for k, v in outs.items()}
    return prog


def build_loop(seed: int):
    """A random loop program: two matrices, a row vector and two accumulators updated in place by a random sequence of
    statements (scaled adds, sin chains, row / column sums and maxima fed back through broadcasts) for a few
    iterations of an IR for-loop.  Some seeds describe cyclic updates the frontend cannot trace (RecursionError);
    callers skip those."""
    rng = np.random.default_rng(seed)
    P, Q, iters = int(rng.integers(1, 12)), int(rng.integers(1, 20)), int(rng.integers(1, 4))
    xa = rng.standard_normal(P * Q).astype(np.float32)
    xb = rng.standard_normal(P * Q).astype(np.float32)
    xw = rng.standard_normal(Q).astype(np.float32)
    plan = [int(k) for k in rng.integers(0, 8, size=int(rng.integers(2, 7)))]

    def prog(dev):
        ad.set_device(dev)
        st = {"a": ad.tensor(xa, [P, Q]), "b": ad.tensor(xb, [P, Q]), "w": ad.tensor(xw, [Q]),
              "c": ad.tensor(np.zeros(Q, np.float32), [Q]), "r": ad.tensor(np.zeros(P, np.float32), [P])}

        def body(i):
            for k in plan:
                a, b, w, c, r = st["a"], st["b"], st["w"], st["c"], st["r"]
                wb = w.view([1, Q]).broadcast(0, P)
                if k == 0:
                    a += b * 0.5
                    a.forward()
                elif k == 1:
                    b += (a * wb).sin() * 0.1
                    b.forward()
                elif k == 2:
                    c += a.sum(0)
                    c.forward()
                elif k == 3:
                    r += (a * b).sum(1)
                    r.forward()
                elif k == 4:
                    w += a.sum(0) * 0.01
                    w.forward()
                elif k == 5:
                    a += r.unsqueeze(-1).broadcast(-1, Q) * 0.01
                    a.forward()
                elif k == 6:
                    b += c.view([1, Q]).broadcast(0, P) * 0.01
                    b.forward()
                else:
                    m = a.max(1)
                    a += (a - m.unsqueeze(-1).broadcast(-1, Q)) * 0.1
                    a.forward()
        ad.ir_for(range(0, iters), body)
        ad.execute()
        return {k: v.val().get() for k, v in st.items()}
    return prog


def build_raw(seed: int, allreduce: bool = False, rich: bool = False):
    """A random program written directly as IR commands (no frontend in between): ids are reused as results, op-assigns
    hit ids that are views / permutes of other tensors, views are created inside branches, branches are not taken and
    loops run zero times.  Square [n, n] tensors of small integers and a few additions / multiplications per path, so
    every value is exact in fp32 and device and oracle must agree bit for bit.

    With `rich`, row sums broadcast back to [n, n], single rows repeated over the tensor and halves cut out of a concat
    join the mix (reductions, Index / Broadcast / Concat / View chains as alias ids).

    With `allreduce`, about a third of the values are all-reduced right after they are assigned (the caller runs the
    program on ranks that hold identical data, so the sum over ranks is a multiplication by their number).

    Returns `prog(dev) -> {id: ValueData}`.  Only ids that are certainly defined are read: an id first assigned inside
    a block is local to that block."""
    IRP = adb.ir.IRProcedure

    def prog(dev):
        rng = np.random.default_rng(seed)
        n = int(rng.integers(2, 5))
        counter = [0]

        def fresh(prefix="v"):
            counter[0] += 1
            return f"{prefix}{counter[0]}"

        main = IRP("main")
        mats = []
        for _ in range(3):
            id_ = fresh()
            main.push(("CreateMat", rng.integers(-1, 3, n * n).astype(np.float32), [n, n], id_))
            mats.append(id_)
        one = fresh("k")
        main.push(("CreateConstant", -1.0, one, [1]))
        budget = {"mul": 3}   # multiplications per program: keeps values small enough to stay exact
        # ids that an id may be a view of, transitively (never shrinks: a view command whose result is one of its own
        # sources would make the alias chain cyclic, which no device can evaluate)
        anc: dict = {}

        def may_alias(res, a):
            return res == a or res in anc.get(a, ())

        def note_alias(res, a):
            new = set(anc.get(a, ())) | {a}
            anc.setdefault(res, set()).update(new)
            for x, s in anc.items():
                if res in s:
                    s.update(new)

        def emit(block, pool, depth):
            """Appends random commands to `block`; `pool` = ids (shape [n, n]) that are defined at this point."""
            pool = list(pool)
            for _ in range(int(rng.integers(2, 7))):
                kind = int(rng.integers(0, 13 if rich else 10))
                a = pool[int(rng.integers(0, len(pool)))]
                b = pool[int(rng.integers(0, len(pool)))]
                # results go to a fresh id or overwrite an existing one
                res = fresh() if rng.random() < 0.5 else pool[int(rng.integers(0, len(pool)))]
                if kind == 0:
                    block.push(("ElwAdd", a, b, res))
                elif kind == 1:
                    if budget["mul"] <= 0:
                        continue
                    budget["mul"] -= 1
                    block.push(("ElwMultiply", a, b, res))
                elif kind == 2:
                    block.push(("ElwAddEq", a, b))
                    res = a
                elif kind == 3:
                    if budget["mul"] <= 0:
                        continue
                    budget["mul"] -= 1
                    block.push(("ElwMultiplyEq", a, b))
                    res = a
                elif kind == 4:
                    if may_alias(res, a):
                        continue
                    note_alias(res, a)
                    block.push(("Permute", a, [1, 0], res))
                elif kind == 5:
                    if may_alias(res, a):
                        continue
                    note_alias(res, a)
                    block.push(("View", a, [n, n], res))
                elif kind == 6:
                    block.push(("Contigious", a, res))
                elif kind == 7:
                    if budget["mul"] <= 0:
                        continue
                    budget["mul"] -= 1
                    block.push(("DotProduct", a, b, res))
                elif kind == 10:
                    # row sums, repeated along the rows again: [n, n] -> [n] -> [n, 1] -> [n, n]
                    if budget["mul"] <= 0 or may_alias(res, a):
                        continue
                    budget["mul"] -= 1
                    s_, v_ = fresh("s"), fresh("w")
                    block.push(("Sum", a, s_))
                    block.push(("View", s_, [n, 1], v_))
                    block.push(("Broadcast", v_, 1, n, res))
                    note_alias(v_, s_)
                    note_alias(res, v_)
                elif kind == 11:
                    # one row of a, repeated over all rows
                    if may_alias(res, a):
                        continue
                    i_, v_ = fresh("i"), fresh("w")
                    block.push(("Index", a, int(rng.integers(0, n)), 0, i_))
                    block.push(("View", i_, [1, n], v_))
                    block.push(("Broadcast", v_, 0, n, res))
                    note_alias(i_, a)
                    note_alias(v_, i_)
                    note_alias(res, v_)
                elif kind == 12:
                    # a on top of b, then one of the two halves again
                    if may_alias(res, a) or may_alias(res, b):
                        continue
                    c_, v_, i_ = fresh("c"), fresh("w"), fresh("i")
                    block.push(("Concat", a, b, 0, c_))
                    block.push(("View", c_, [2, n * n], v_))
                    block.push(("Index", v_, int(rng.integers(0, 2)), 0, i_))
                    block.push(("View", i_, [n, n], res))
                    note_alias(c_, a)
                    note_alias(c_, b)
                    note_alias(v_, c_)
                    note_alias(i_, v_)
                    note_alias(res, i_)
                elif kind == 8 and depth < 2:
                    # If on a flag that is 0 or 1 (optionally with an else block)
                    flag = fresh("f")
                    block.push(("CreateMat", np.array([float(rng.integers(0, 2))], np.float32), [1], flag))
                    then = IRP(fresh("blk"))
                    emit(then, pool, depth + 1)
                    other = None
                    if rng.random() < 0.4:
                        other = IRP(fresh("blk"))
                        emit(other, pool, depth + 1)
                    block.push(("If", [(flag, then)], other))
                    continue
                elif kind == 9 and depth < 2:
                    # While on a counter that starts at 0 .. 2 and is decremented at the end of the body
                    cnt = fresh("c")
                    block.push(("CreateMat", np.array([float(rng.integers(0, 3))], np.float32), [1], cnt))
                    body = IRP(fresh("blk"))
                    saved = budget["mul"]
                    budget["mul"] = min(budget["mul"], 1)
                    emit(body, pool, depth + 1)
                    budget["mul"] = max(0, saved - 1)
                    body.push(("ElwAddEq", cnt, one))
                    block.push(("While", cnt, body))
                    continue
                else:
                    continue
                if allreduce and kind in (0, 1, 2, 3, 6, 7) and rng.random() < 0.35:
                    block.push(("AllReduce", res))
                if res not in pool:
                    pool.append(res)
            return pool

        pool = emit(main, mats, 0)
        dep = list(dict.fromkeys(pool[-6:] + mats))
        dev.execute(main, dep)
        return {d: dev.get_tensor(d) for d in dep}
    return prog
