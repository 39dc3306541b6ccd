"""Benchmark of the B200 backend on the reference's headline workloads.

    python bench.py --gpus N --steps K --warmup W            # this backend
    python bench.py --impl reference --gpus N --steps K ...  # CPU restatement of the reference path

One "step" is one training step of the data-parallel MLP (BASELINE config 4: batch 65536,
4096-8192-8192-4096-1000, sigmoid, MSE, SGD), executed as one iteration of an IR for-loop.
  value  steps/s over all GPUs with inputs resident in HBM; CUDA events inside the library around
         the compute region of one `adb_execute` of a K-iteration loop, max over ranks
  e2e    the same metric through the C-ABI with pinned HOST inputs: the batch (X, T) is created
         inside the loop body, so every step uploads it again (the reference re-uploads a CreateMat
         each time it executes, src/devices/opencl/kernels/alloc.rs:5-12); wall clock around adb_execute
At N=1 the line also carries the fused element-wise workload (BASELINE config 2) and the CPU baseline.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "mlp_train_steps_per_s"
UNIT = "steps/s"
BATCH = 65536


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d["bf16_tflops_sustained"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "200"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = [s for s, p in zip(sm, power) if p > 250] or sm
        return {"sm_mhz": float(np.median(busy)) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------
def mlp_flops_per_step(batch, widths):
    fwd = sum(2 * batch * widths[i] * widths[i + 1] for i in range(len(widths) - 1))
    dw = fwd
    dx = sum(2 * batch * widths[i] * widths[i + 1] for i in range(1, len(widths) - 1))
    return fwd + dw + dx


def trace_c4(adb, dev, inputs, batch, widths, steps, upload_in_loop, local_rows=None):
    """Traces config 4.  With `upload_in_loop` the batch tensors are created inside the loop body."""
    ad, nn, f32 = adb.autodiff, adb.nn, adb.autodiff.f32
    ad.set_device(dev)
    ad.eager_dep_opt()
    L = len(widths) - 1
    ws = [ad.tensor(inputs[f"w{i}"], [widths[i], widths[i + 1]]) for i in range(L)]
    bs = [ad.tensor(inputs[f"b{i}"], [widths[i + 1]]) for i in range(L)]
    if not upload_in_loop:
        x = ad.tensor(inputs["x"], [batch, widths[0]], local_rows)
        t = ad.tensor(inputs["t"], [batch, widths[-1]], local_rows)
    net = nn.Sequential()
    for i in range(L):
        net.insert(nn.LinearWithWeights(ws[i], bs[i]))
        if i < L - 1:
            net.insert(nn.Sigmoid())
    opt = nn.SGD(net.params(), 1e-3)
    box = {}

    def body(_):
        xx = ad.tensor(inputs["x"], [batch, widths[0]], local_rows) if upload_in_loop else x
        tt = ad.tensor(inputs["t"], [batch, widths[-1]], local_rows) if upload_in_loop else t
        y = net.f(xx)
        d = y - tt
        loss = d.pow2().sum(1).sum(0) * f32(1.0 / (batch * widths[-1]))
        opt.zero_grad()
        loss.forward()
        loss.backward()
        opt.step()
        box["loss"] = loss
    ad.ir_for(range(0, steps), body)
    box["loss"].val().keep()
    return box["loss"].val()


def run_ours(args):
    import torch
    import torch.distributed as dist
    adb = importlib.import_module("autodiff-ir-rust_b200")
    cfg = adb.configs
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(local)
    uid = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        box = [adb.devices.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        uid = box[0]
    pk = peaks()
    widths = cfg.C4_WIDTHS
    batch = args.batch
    lb = batch // world
    flags = adb.devices.FLAG_PROFILE if args.dev_flags is None else args.dev_flags
    dev = adb.devices.B200(local, rank=rank, world_size=world, nccl_unique_id=uid, flags=flags, shard_batch=batch if world > 1 else 0)

    # synthetic data: weights from the documented counter-based generator, the batch from torch's
    # seeded generators (device-side for the resident run, pinned host memory for the end-to-end run)
    small = cfg.c4_inputs(batch=0, widths=widths)
    g = torch.Generator(device="cuda").manual_seed(3 + 1000 * rank)
    x_dev = torch.randn(lb * widths[0], device="cuda", generator=g)
    t_dev = torch.randn(lb * widths[-1], device="cuda", generator=g)
    w_dev = {k: torch.from_numpy(v).cuda() for k, v in small.items() if k[0] in "wb"}
    DP = adb.ir.DevicePayload
    resident = {k: DP(v.data_ptr(), v.numel(), v) for k, v in w_dev.items()}
    resident["x"] = DP(x_dev.data_ptr(), x_dev.numel(), x_dev)
    resident["t"] = DP(t_dev.data_ptr(), t_dev.numel(), t_dev)
    x_host = torch.empty(lb * widths[0], pin_memory=True).copy_(x_dev)
    t_host = torch.empty(lb * widths[-1], pin_memory=True).copy_(t_dev)
    # end-to-end run: every payload is a host buffer (weights once per execute, the batch every step), all pinned
    pinned = {k: torch.empty(v.size, pin_memory=True).copy_(torch.from_numpy(v)) for k, v in small.items() if k[0] in "wb"}
    host = {k: v.numpy() for k, v in pinned.items()}
    host["x"], host["t"] = x_host.numpy(), t_host.numpy()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def once(inputs, steps, upload_in_loop):
        loss = trace_c4(adb, dev, inputs, batch, widths, steps, upload_in_loop, lb if world > 1 else None)
        barrier()
        t0 = time.perf_counter()
        adb.autodiff.execute()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        barrier()
        return wall, dev.stats(), float(loss.get().data[0])

    K, W = args.steps, max(args.warmup, 3)
    # warm-up: at least W steps of the very program that is timed (same plan, same kernels)
    for _ in range((W + K - 1) // K):
        once(resident, K, False)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    wall, st, loss = once(resident, K, False)
    clocks = sampler.stop() if rank == 0 else None
    dev_ms = max_over_ranks(st["device_ms"])
    value = K / (dev_ms / 1e3)
    flops = mlp_flops_per_step(batch, widths)

    # end to end: pinned host batch uploaded every step inside the loop
    for _ in range((W + K - 1) // K):
        once(host, K, True)
    wall_e, st_e, loss_e = once(host, K, True)
    e2e_s = max_over_ranks(wall_e)
    e2e = {"value": K / e2e_s, "unit": UNIT, "h2d_bytes_per_step": int((x_host.numel() + t_host.numel()) * 4),
           "d2h_bytes_per_step": int(st_e["d2h_bytes"] // K), "ms_per_step": e2e_s * 1e3 / K,
           "upload_ms_per_step": st_e["upload_ms"] / K}

    gemm_tflops = st["gemm_flops"] / max(st["gemm_ms"], 1e-9) / 1e9
    peak_3xtf32 = pk["bf16_tflops_sustained"] / 6.0
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": dev_ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic (seeded: Philox weights, torch-generated N(0,1) batch and targets)",
        "config": {"workload": "C4 data-parallel MLP training: batch %d f32 [%d,%d] -> %s, sigmoid, MSE, SGD lr 1e-3, "
                               "one IR for-loop iteration per step" % (batch, batch, widths[0], "-".join(map(str, widths[1:]))),
                   "global_batch": batch, "parallelism": f"dp{world}", "l2": "working set (GBs per kernel) far exceeds the 126 MB L2",
                   "loss_after_timed_run": loss},
        "e2e": e2e, "gpu_launches": int(st["kernel_launches"]), "clocks": clocks,
        "effective_fp32_tflops_per_gpu": flops * value / world / 1e12,
        "roofline": {"bound": "tensor", "achieved": gemm_tflops, "peak": peak_3xtf32, "unit": "TFLOP/s",
                     "frac": gemm_tflops / peak_3xtf32, "traffic": None,
                     "peak_note": "3xTF32 peak taken as %s bf16 sustained / 2 (tf32) / 3 (passes) of %s" % (pk["bf16_tflops_sustained"], pk["source"]),
                     "kernel": "dot product (all GEMM launches of the timed region)", "launches": int(st["gemm_launches"]),
                     "avg_ms": st["gemm_ms"] / max(1, st["gemm_launches"])},
        "breakdown_ms_per_step": {"gemm": st["gemm_ms"] / K, "elementwise": st["elw_ms"] / K, "reduce": st["reduce_ms"] / K,
                                  "allreduce": st["collective_ms"] / K},
        # the HBM-bound kernels of the same timed region: fused bias + sigmoid chains, sigmoid backward, SGD updates
        "elementwise_in_step": {"bound": "hbm", "achieved": st["elw_bytes"] / max(st["elw_ms"], 1e-9) / 1e6, "peak": pk["hbm_gbs"],
                                "unit": "GB/s", "frac": st["elw_bytes"] / max(st["elw_ms"], 1e-9) / 1e6 / pk["hbm_gbs"],
                                "launches": int(st["elw_launches"]), "peak_note": "copy bandwidth of " + pk["source"]},
    }
    if world == 1 and rank == 0 and not args.skip_extras:
        line["fused_elw"] = bench_c2(adb, dev, pk, args)
        line["other_configs"] = bench_small_configs(adb, pk)
        line["cpu_baseline"] = cpu_baseline_c4(adb, widths, batch, args)
    if rank == 0:
        print(json.dumps(line))
    dev.close()
    if world > 1:
        dist.destroy_process_group()


def bench_c2(adb, dev, pk, args):
    """BASELINE config 2 at full size (8192x8192), resident inputs; returns the element-wise roofline."""
    import torch
    cfg = adb.configs
    rows = cols = args.c2_size
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randn(rows * cols, device="cuda", generator=g)
    b = torch.randn(rows * cols, device="cuda", generator=g)
    bias = torch.rand(cols, device="cuda", generator=g) * 2 - 1
    DP = adb.ir.DevicePayload
    inp = {"a": DP(a.data_ptr(), a.numel(), a), "b": DP(b.data_ptr(), b.numel(), b), "bias": DP(bias.data_ptr(), bias.numel(), bias)}
    # whole-program time on a handle without per-kernel events (cached plan -> one CUDA-graph replay);
    # per-kernel figures from the profiling handle
    plain = adb.devices.B200(0)
    best = None
    for it in range(7):
        cfg.c2_fused_elementwise(plain, rows=rows, cols=cols, inputs=inp, execute=False)
        adb.autodiff.execute()
        st = plain.stats()
        if it >= 3 and (best is None or st["device_ms"] < best["device_ms"]):
            best = st
    plain.close()
    prof = None
    for it in range(3):
        cfg.c2_fused_elementwise(dev, rows=rows, cols=cols, inputs=inp, execute=False)
        adb.autodiff.execute()
        st = dev.stats()
        if prof is None or st["top_ms"] < prof["top_ms"]:
            prof = st
    for k in ("top_ms", "top_bytes", "top_name", "top_launches"):
        best[k] = prof[k]
    n = rows * cols
    algorithmic = 4.0 * n * 4  # read a, b once; write a.grad, b.grad once
    achieved = algorithmic / (best["device_ms"] / 1e3) / 1e9
    top = best["top_bytes"] / max(best["top_ms"], 1e-9) / 1e6
    return {"workload": "C2 fused element-wise + broadcast, forward + backward, f32 [%d,%d]" % (rows, cols),
            "ms": best["device_ms"], "algorithmic_bytes": algorithmic, "algorithmic_GBps": achieved,
            "frac_of_hbm_peak": achieved / pk["hbm_gbs"], "kernels": int(best["kernel_launches"]),
            "roofline": {"bound": "hbm", "kernel": best["top_name"], "achieved": top, "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": top / pk["hbm_gbs"],
                         # dram__bytes_read + dram__bytes_write of this kernel at this size, from the ncu capture summarised in
                         # profiles/c2_fused_elementwise_8192.md (one launch)
                         "traffic": 1034001664 if rows == 8192 else None, "launches": int(best["top_launches"]),
                         "peak_note": "copy bandwidth of " + pk["source"]}}


def bench_small_configs(adb, pk):
    """BASELINE configs 1, 3 and 5 on one GPU with resident inputs: whole-program device time of a cached plan
    (best of a few executes on a handle without per-kernel events)."""
    import torch
    cfg, DP = adb.configs, adb.ir.DevicePayload
    g = torch.Generator(device="cuda").manual_seed(2)
    dev = adb.devices.B200(0)
    out = {}

    def best_of(n, build):
        best = None
        for it in range(n):
            build()
            t0 = time.perf_counter()
            adb.autodiff.execute()
            wall = time.perf_counter() - t0
            st = dev.stats()
            st["wall_ms"] = wall * 1e3
            if it >= 2 and (best is None or st["device_ms"] < best["device_ms"]):
                best = st
        return best

    # config 1: the README-sized MLP step (trace, execute, read back: the whole user-level call); nothing but latency
    best = None
    for it in range(12):
        t0 = time.perf_counter()
        cfg.c1_readme_mlp(dev)
        wall = time.perf_counter() - t0
        st = dev.stats()
        if it >= 2 and (best is None or wall < best[0]):
            best = (wall, st)
    wall, st = best

    # the same step through the C-ABI alone: the serialised program is handed to adb_execute again and again
    # (cached plan, one CUDA-graph replay, read-back of the kept tensors included)
    class Capture:
        def ir_callback(self, irb): pass
        def dot_prod_shape(self, a, b): return [a[0], b[1]]
        def execute(self, proc, dep): self.blob, self.keep = adb.ir.serialize(proc, dep)
        def get_tensor(self, id_): return adb.autodiff.ValueData([1], np.zeros(1, np.float32), id_, False)
    cap = Capture()
    cfg.c1_readme_mlp(cap)
    abi = []
    for it in range(200):
        t0 = time.perf_counter()
        dev.execute_blob(cap.blob)
        abi.append(time.perf_counter() - t0)
    abi_s = float(np.median(abi[20:]))
    out["c1_readme_mlp"] = {"device_us": st["device_ms"] * 1e3, "abi_call_us": abi_s * 1e6, "steps_per_s": 1.0 / abi_s,
                            "python_call_us": wall * 1e6, "kernels": int(st["kernel_launches"]),
                            "graph_replays": int(st["graph_replays"]),
                            "note": "abi_call_us = one adb_execute of the serialised step (cached plan, graph replay, read-back of "
                                    "8 tensors), median of 180; python_call_us adds tracing and serialising in the Python mirror"}
    # config 3: reductions and data movement, f32 [64,1024,1024]
    batch, n = 64, 1024
    x = torch.rand(batch * n * n, device="cuda", generator=g) * 2 - 1
    st = best_of(6, lambda: cfg.c3_reduce_movement(dev, batch=batch, n=n, inputs={"x": DP(x.data_ptr(), x.numel(), x)}, execute=False))
    alg = 2.0 * batch * n * n * 4  # read x once, write x.grad once
    out["c3_reduce_movement"] = {"ms": st["device_ms"], "algorithmic_bytes": alg, "algorithmic_GBps": alg / st["device_ms"] / 1e6,
                                 "frac_of_hbm_peak": alg / st["device_ms"] / 1e6 / pk["hbm_gbs"], "kernels": int(st["kernel_launches"])}
    del x
    # config 5: 8192^2 fixed-point loop, three dot products per iteration, 50 iterations
    n, iters = 8192, 50
    a = torch.randn(n * n, device="cuda", generator=g) * n ** -0.5
    b = torch.randn(n * n, device="cuda", generator=g) * n ** -0.5
    st = best_of(3, lambda: cfg.c5_dot_loop(dev, n=n, max_iters=iters, inputs={"a": DP(a.data_ptr(), a.numel(), a),
                                                                               "b": DP(b.data_ptr(), b.numel(), b)}, execute=False))
    flops = 2.0 * n ** 3 * st["gemm_launches"]
    out["c5_dot_loop"] = {"ms": st["device_ms"], "iterations": int(st["while_iterations"]), "dot_products": int(st["gemm_launches"]),
                          "effective_fp32_tflops": flops / st["device_ms"] / 1e9,
                          "frac_of_3xtf32_peak": flops / st["device_ms"] / 1e9 / (pk["bf16_tflops_sustained"] / 6.0)}
    dev.close()
    return out


def cpu_baseline_c4(adb, widths, batch, args, sample_batch=None):
    """The CPU restatement of the reference path (oracle) on the host cores: one training step at a
    reduced batch, extrapolated linearly to the full batch (the work is linear in the batch)."""
    from oracle.oracle import OracleDevice
    cfg = adb.configs
    sb = sample_batch or args.cpu_sample_batch
    inp = cfg.c4_inputs(batch=sb, widths=widths)
    t0 = time.perf_counter()
    cfg.c4_mlp_train(OracleDevice(), batch=sb, widths=widths, steps=1, inputs=inp)
    dt = time.perf_counter() - t0
    cores = os.cpu_count() or 1
    return {"value": (1.0 / dt) * (sb / batch), "unit": UNIT, "cores": cores, "kind": "port",
            "sample": "1 training step at batch %d of %d (%.1f s), extrapolated linearly in the batch" % (sb, batch, dt)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    adb = importlib.import_module("autodiff-ir-rust_b200")
    widths = adb.configs.C4_WIDTHS
    vals = []
    for _ in range(max(1, min(args.steps, 2))):
        vals.append(cpu_baseline_c4(adb, widths, args.batch, args))
    best = max(vals, key=lambda v: v["value"])
    line = {"impl": "reference", "metric": METRIC, "value": best["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "ms_per_step": 1e3 / best["value"],
            "config": {"workload": "C4 data-parallel MLP training (CPU restatement of the reference path, host cores)",
                       "global_batch": args.batch},
            "cpu_baseline": best,
            "e2e": {"value": best["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--c2-size", type=int, default=8192)
    ap.add_argument("--cpu-sample-batch", type=int, default=512)
    ap.add_argument("--skip-extras", action="store_true")
    ap.add_argument("--dev-flags", type=int, default=None, help="ADB_FLAG_* bits of the handle (default: per-kernel profiling events)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
