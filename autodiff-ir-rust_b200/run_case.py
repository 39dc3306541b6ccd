"""Runs one benchmark program a few times on cuda:0 (inputs resident in HBM) and prints its timing.

    python autodiff-ir-rust_b200/run_case.py c2 --size 8192 --reps 3
    python autodiff-ir-rust_b200/run_case.py c3 --batch 64 --n 1024
    python autodiff-ir-rust_b200/run_case.py dot --m 4096 --n 4096 --k 4096 [--ta] [--tb]
    python autodiff-ir-rust_b200/run_case.py c5 --size 4096 --iters 3
    python autodiff-ir-rust_b200/run_case.py ln --batch 65536 --n 1024        (layer normalisation of [batch, n])

Small, single-purpose entry point for profilers (ncu -k regex:adb_ ...) and for quick timing of one
kernel family; bench.py remains the benchmark.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["c2", "c3", "c5", "dot", "ln"])
    ap.add_argument("--size", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--n", type=int, default=1024)
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--ta", action="store_true")
    ap.add_argument("--tb", action="store_true")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--no-profile-flag", action="store_true")
    ap.add_argument("--flags", type=int, default=0, help="extra ADB_FLAG_* bits for the handle (e.g. 32 = single-SM dot kernel)")
    args = ap.parse_args()

    import torch
    adb = importlib.import_module("autodiff-ir-rust_b200")
    ad, cfg, DP = adb.autodiff, adb.configs, adb.ir.DevicePayload
    torch.cuda.set_device(0)
    dev = adb.devices.B200(0, flags=args.flags | (0 if args.no_profile_flag else adb.devices.FLAG_PROFILE))
    g = torch.Generator(device="cuda").manual_seed(1)

    def resident(n, scale=1.0):
        t = torch.randn(n, device="cuda", generator=g) * scale
        return t, DP(t.data_ptr(), t.numel(), t)

    keep = []
    for rep in range(args.reps):
        if args.case == "c2":
            n = args.size
            a, pa = resident(n * n)
            b, pb = resident(n * n)
            bias, pbias = resident(n)
            keep += [a, b, bias]
            cfg.c2_fused_elementwise(dev, rows=n, cols=n, inputs={"a": pa, "b": pb, "bias": pbias}, execute=False)
        elif args.case == "c3":
            x = torch.rand(args.batch * args.n * args.n, device="cuda", generator=g) * 2 - 1
            keep.append(x)
            cfg.c3_reduce_movement(dev, batch=args.batch, n=args.n, inputs={"x": DP(x.data_ptr(), x.numel(), x)}, execute=False)
        elif args.case == "ln":
            x = torch.randn(args.batch * args.n, device="cuda", generator=g) * 3 + 1
            keep.append(x)
            ad.set_device(dev)
            ad.eager_dep_opt()
            y = adb.nn.LayerNorm(args.n).f(ad.tensor(DP(x.data_ptr(), x.numel(), x), [args.batch, args.n])).forward()
            y.keep()            # (read back with the result; the timing below is the device time of the kernels)
        elif args.case == "c5":
            n = args.size
            a, pa = resident(n * n, n ** -0.5)
            b, pb = resident(n * n, n ** -0.5)
            keep += [a, b]
            cfg.c5_dot_loop(dev, n=n, max_iters=args.iters, inputs={"a": pa, "b": pb}, execute=False)
        else:
            M, N, K = args.m, args.n, args.k
            a, pa = resident(M * K)
            b, pb = resident(K * N)
            keep += [a, b]
            ad.set_device(dev)
            ad.eager_dep_opt()
            A = ad.tensor(pa, [K, M] if args.ta else [M, K])
            B = ad.tensor(pb, [N, K] if args.tb else [K, N])
            y = ad.dot(A.t() if args.ta else A, B.t() if args.tb else B).contigious()
            y.forward()
            y.val().keep()
        ad.execute()
        st = dev.stats()
        out = {k: st[k] for k in ("device_ms", "kernel_launches", "gemm_launches", "tc_gemm_launches", "elw_ms", "reduce_ms",
                                  "gemm_ms", "elw_bytes", "reduce_bytes", "gemm_flops", "top_name", "top_ms", "top_bytes", "arena_bytes")}
        if st["gemm_ms"] > 0:
            out["gemm_tflops"] = st["gemm_flops"] / st["gemm_ms"] / 1e9
        if st["top_ms"] > 0:
            out["top_GBps"] = st["top_bytes"] / st["top_ms"] / 1e6
        print(json.dumps(out))
    if os.environ.get("ADB_DUMP_PLAN"):
        print(dev.dump_plan())
    dev.close()


if __name__ == "__main__":
    main()
