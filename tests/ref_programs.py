"""The reference's own integration tests, restated against the frontend mirror.

Each function traces one program (same tensors, same operations, same order as the cited
Rust test), executes it on whatever device is installed, and returns
{name: ValueData} for the tensors the Rust test asserts on.  Expected values live in
tests/golden/reference_kat.json (transcribed from the cited lines).
"""
from __future__ import annotations

import importlib

adb = importlib.import_module("autodiff-ir-rust_b200")
ad = adb.autodiff
nn = adb.nn


def ct(dev):
    """src/tests/ct.rs:9-59"""
    ad.set_device(dev)
    x = ad.tensor([1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0, 8.0], [2, 4])
    y = ad.tensor([7.0, 2.0, 6.0, 4.0, 9.0, 2.0, 6.0, 4.0], [2, 4])
    t = (2.0 * x + 3.0).cos()
    t2 = ((t * y) + 3.0 * (t + x)).sqrt()
    res = t2 / t
    res.forward()
    res.backward()
    res.val().keep()
    ad.execute()
    return {"res": res.val().get().round(4), "x_grad": x.grad().get().round(4), "y_grad": y.grad().get().round(4)}


def if_ctrl(dev):
    """src/tests/ctrl.rs:8-34"""
    ad.set_device(dev)
    x = ad.scalar(1.0)
    y = ad.scalar(3.0)

    def body():
        nonlocal y
        y += 4.0
        y.forward()
    ad.ir_if(lambda: x, body)
    y += 3.0
    y.forward()
    x_two = ad.scalar(0.0)
    ad.ir_if(lambda: x_two, body)
    ad.execute()
    return {"y": y.val().get()}


def if_else_ctrl(dev):
    """src/tests/ctrl.rs:36-71"""
    ad.set_device(dev)
    x = ad.scalar(1.0)
    y = ad.scalar(3.0)
    y_two = ad.scalar(3.0)

    def a():
        nonlocal y
        y += 4.0
        y.forward()

    def b():
        nonlocal y_two
        y_two += 5.0
        y_two.forward()

    def c():
        nonlocal y
        y += 9.0
        y.forward()

    def d():
        nonlocal y_two
        y_two += 10.0
        y_two.forward()

    ad.ir_if_else(lambda: x.clone(), a, b)
    ad.ir_if_else(lambda: x - 1.0, c, d)
    ad.execute()
    return {"y": y.val().get(), "y_two": y_two.val().get()}


def for_ctrl(dev):
    """src/tests/ctrl.rs:73-89"""
    ad.set_device(dev)
    y = ad.scalar(10.0)

    def body(i):
        nonlocal y
        y += i.clone()
        y.forward()
    ad.ir_for(range(-3, 5), body)
    ad.execute()
    return {"y": y.val().get()}


def evrty_ctrl(dev):
    """src/tests/ctrl.rs:92-127"""
    ad.set_device(dev)
    y = ad.scalar(3.0)
    y_two = ad.scalar(3.0)

    def body(i):
        def neg():
            nonlocal y
            y *= i.clone()
            y.forward()

        def nonneg():
            def pos():
                nonlocal y_two
                y_two *= i.clone()
                y_two.forward()
            ad.ir_if(lambda: i.more_than(ad.scalar(0.0)), pos)
        ad.ir_if_else(lambda: i.less_than(ad.scalar(0.0)), neg, nonneg)
    ad.ir_for(range(-3, 5), body)
    ad.execute()
    return {"y": y.val().get(), "y_two": y_two.val().get()}


def eq(dev):
    """src/tests/eq.rs:7-68"""
    ad.set_device(dev)
    x = ad.tensor([0.0, 1.0, 3.0, 2.0, 1.0, 3.0], [6])
    res = 3.0 * (x.clone() * (x.equal(ad.constant(3.0, x.dim())))).pow2()
    y = res.sum(0)
    ad.add_heading("Forward")
    y.forward()
    ad.add_heading("Backward")
    y.backward()
    all_no = ad.tensor([0.0, 1.0, 1.0], [3]).all()
    ad.add_heading("All No Forward")
    all_no.forward()
    all_yes = ad.tensor([1.0, 1.0, 1.0], [3]).all()
    ad.add_heading("All Yes Forward")
    all_yes.forward()
    res.val().keep()
    all_no.val().keep()
    all_yes.val().keep()
    ad.execute()
    return {"res": res.val().get(), "x_grad": x.grad().get(),
            "all_no": all_no.val().get(), "all_yes": all_yes.val().get()}


def everything(dev):
    """src/tests/evryt.rs:8-68 (ignored upstream: concat is unimplemented in the OpenCL device)"""
    ad.set_device(dev)
    x = ad.tensor([1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0, 8.0], [2, 4])
    y = ad.tensor([7.0, 2.0, 6.0, 4.0, 9.0, 2.0, 6.0, 4.0], [2, 4])
    z = ad.tensor([7.0, 2.0], [2, 1])
    v = ad.tensor([1.0, 2.0, 4.0], [3, 1])
    t1 = ad.dot(x.clone(), y.t())
    t2 = t1.sum(0).repeat(lambda n, _: n.clone(), 3, 0)
    t3 = ad.dot(t2, z.clone())
    result = ad.concat([t3, 3.0 * v.pow2()], 1)
    result.forward()
    result.r(range(0, 2), 0).backward()
    result.val().keep()
    ad.execute()
    return {"result": result.val().get(), "x_grad": x.grad().get(), "y_grad": y.grad().get(),
            "z_grad": z.grad().get(), "v_grad": v.grad().get()}


def grd(dev):
    """src/tests/grd.rs:11-41"""
    ad.set_device(dev)
    a = ad.tensor([3.0, 2.0, 1.0, 3.0], [2, 2])
    b = ad.tensor([2.0, 5.0, 2.0, 1.0], [2, 2])
    l = a.clone() * b.clone()
    l.forward()
    l.backward()
    a += a.grad()
    l = a.clone() * b.clone()
    l.forward()
    l.backward()
    ad.execute()
    return {"a": a.val().get(), "a_grad": a.grad().get()}


def nn_train(dev, iters=10):
    """src/tests/nn.rs:8-101"""
    ad.set_device(dev)
    ad.eager_dep_opt()
    l1_w = ad.tensor([0.03, 0.02, 0.01, 0.04, 0.05, 0.063, 0.01, 0.10, 0.07,
                      0.02, 0.01, 0.08, 0.05, 0.03, 0.06], [5, 3])
    l1_b = ad.tensor([0.03, 0.01, 0.032], [3])
    l2_w = ad.tensor([0.022, 0.016, 0.007, 0.093, 0.013, 0.09], [3, 2])
    net = nn.Sequential()
    net.insert(nn.LinearWithWeights(l1_w.clone(), l1_b.clone()))
    net.insert(nn.Sigmoid())
    net.insert(nn.LinearWithWeights(l2_w.clone(), None))
    opt = nn.SGD(net.params(), 0.1)
    x = ad.tensor([0.01, 0.02, 0.037, 0.04, 0.05, 0.063, 0.07, 0.08, 0.09, 0.013], [2, 5])
    box = {}

    def body(_):
        y = net.f(x.clone())
        opt.zero_grad()
        ad.add_heading("Forward")
        y.forward()
        ad.add_heading("Backward")
        y.backward()
        ad.add_heading("Stepping")
        opt.step()
        box["res"] = y
    ad.ir_for(range(0, iters), body)
    res = box["res"]
    res.val().keep()
    l1_w.val().keep()
    l1_b.val().keep()
    l2_w.val().keep()
    ad.execute()
    return {"res": res.val().get().round(4), "l1_w": l1_w.val().get().round(4),
            "l1_b": l1_b.val().get().round(4), "l2_w": l2_w.val().get().round(4)}


def rmsnorm(dev):
    """src/tests/norm.rs:8-29"""
    ad.set_device(dev)
    x = ad.tensor([1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0, 8.0], [2, 4])
    res = nn.RMS(4).f(x)
    res.forward()
    res.val().keep()
    ad.execute()
    return {"res": res.val().get().round(4)}


def layernorm(dev):
    """src/tests/norm.rs:31-53"""
    ad.set_device(dev)
    x = ad.tensor([1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0, 9.0], [2, 4])
    res = nn.LayerNorm(4).f(x)
    res.forward()
    res.val().keep()
    ad.execute()
    return {"res": res.val().get().round(4)}


def view(dev):
    """src/tests/view.rs:5-16 (ignored upstream, no assertion there: a kept alias id has no buffer)"""
    ad.set_device(dev)
    a = ad.tensor([2.0, 1.0, 3.0, 4.0], [2, 2])
    res = a.view([1, 1, 2, -1])
    res.forward()
    res.val().keep()
    ad.execute()
    return {"res": res.val().get()}


ALL = {
    "ct": ct, "if_ctrl": if_ctrl, "if_else_ctrl": if_else_ctrl, "for_ctrl": for_ctrl,
    "evrty_ctrl": evrty_ctrl, "eq": eq, "everything": everything, "grd": grd,
    "nn": nn_train, "rmsnorm": rmsnorm, "layernorm": layernorm, "view": view,
}
