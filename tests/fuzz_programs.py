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
