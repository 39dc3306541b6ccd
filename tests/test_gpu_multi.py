"""Data-parallel MLP training on 2 GPUs (one process per GPU, NCCL all-reduce of the gradients) against
the same program on one GPU.  Skipped when fewer than two GPUs are visible."""
import importlib
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KW = dict(batch=256, widths=(64, 128, 128, 64, 16), steps=4, lr=1e-2)


def _batch_ids(adb, kw):
    """ids of x and t in the program `c4_mlp_train` traces (weights first, then biases, then x and t)"""
    class Probe:
        def ir_callback(self, irb): pass
        def dot_prod_shape(self, a, b): return [a[0], b[1]]
        def execute(self, proc, dep): self.mats = [c[3] for c in proc.main if c[0] == "CreateMat"]
        def get_tensor(self, id_): return adb.autodiff.ValueData([1], np.zeros(1, np.float32), id_, False)
    probe = Probe()
    adb.configs.c4_mlp_train(probe, inputs=adb.configs.c4_inputs(batch=kw["batch"], widths=kw["widths"]), **kw)
    n_layers = len(kw["widths"]) - 1
    return probe.mats[2 * n_layers: 2 * n_layers + 2]


def _worker(rank, world, port, out_dir, flags, kw=None, name_batch=False):
    kw = kw or KW
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    adb = importlib.import_module("autodiff-ir-rust_b200")
    box = [adb.devices.nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    dev = adb.devices.B200(rank, rank=rank, world_size=world, nccl_unique_id=box[0], shard_batch=kw["batch"], flags=flags,
                           shard_ids=_batch_ids(adb, kw) if name_batch else None)
    inputs = adb.configs.c4_inputs(batch=kw["batch"], widths=kw["widths"])     # full tensors: the device takes its rows
    out = adb.configs.c4_mlp_train(dev, inputs=inputs, **kw)
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), **{k: v.numpy() for k, v in out.items()})
    dev.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("flags", [0, 16], ids=["compute-stream", "comm-stream"])
def test_two_gpus_match_one_gpu(tmp_path, flags):
    """flags 16 = ADB_FLAG_COMM_STREAM: collectives on their own stream, ordered against the compute stream by events."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    adb = importlib.import_module("autodiff-ir-rust_b200")
    port = 29600 + (os.getpid() % 2000) + flags
    mp.spawn(_worker, args=(2, port, str(tmp_path), flags), nprocs=2, join=True)
    dev = adb.devices.B200(0)
    want = adb.configs.c4_mlp_train(dev, inputs=adb.configs.c4_inputs(batch=KW["batch"], widths=KW["widths"]), **KW)
    dev.close()
    for r in range(2):
        got = np.load(tmp_path / f"rank{r}.npz")
        for k, v in want.items():
            ref = v.numpy()
            err = np.abs(got[k] - ref).max() / max(np.abs(ref).max(), 1e-30)
            assert err < 1e-4, (r, k, err)


def test_two_gpus_match_one_gpu_at_the_benchmark_widths(tmp_path):
    """The benchmark network (4096-8192-8192-4096-1000) at batch 16384: tensor-core dot products on CTA pairs, sums
    fused into the element-wise passes, NCCL all-reduce of 553 MB of gradients per step; two steps, 2 GPUs against 1."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    adb = importlib.import_module("autodiff-ir-rust_b200")
    kw = dict(batch=16384, widths=adb.configs.C4_WIDTHS, steps=2, lr=1e-3)   # (a batch equal to a layer width would be ambiguous)
    port = 29700 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path), 0, kw), nprocs=2, join=True)
    dev = adb.devices.B200(0)
    want = adb.configs.c4_mlp_train(dev, inputs=adb.configs.c4_inputs(batch=kw["batch"], widths=kw["widths"]), **kw)
    assert dev.stats()["tc_gemm_launches"] == 22
    dev.close()
    for r in range(2):
        got = np.load(tmp_path / f"rank{r}.npz")
        for k, v in want.items():
            ref = v.numpy()
            err = np.abs(got[k] - ref).max() / max(np.abs(ref).max(), 1e-30)
            assert err < 1e-4, (r, k, err)


def test_batch_equal_to_a_layer_width_with_named_batch_tensors(tmp_path):
    """batch 128 with 128-wide layers: shapes alone cannot tell the weights from the batch tensors; with x and t named
    (adb_config.shard_ids) two GPUs reproduce the single-GPU run."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    adb = importlib.import_module("autodiff-ir-rust_b200")
    kw = dict(batch=128, widths=(64, 128, 128, 64, 16), steps=3, lr=1e-2)
    port = 29800 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path), 0, kw, True), nprocs=2, join=True)
    dev = adb.devices.B200(0)
    want = adb.configs.c4_mlp_train(dev, inputs=adb.configs.c4_inputs(batch=kw["batch"], widths=kw["widths"]), **kw)
    dev.close()
    for r in range(2):
        got = np.load(tmp_path / f"rank{r}.npz")
        for k, v in want.items():
            ref = v.numpy()
            err = np.abs(got[k] - ref).max() / max(np.abs(ref).max(), 1e-30)
            assert err < 1e-4, (r, k, err)


def _raw_worker(rank, world, port, out_dir, seeds):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    adb = importlib.import_module("autodiff-ir-rust_b200")
    import fuzz_programs
    box = [adb.devices.nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    dev = adb.devices.B200(rank, rank=rank, world_size=world, nccl_unique_id=box[0], shard_batch=0)
    out = {}
    for seed in seeds:
        # every rank must issue the same collectives: a program this rank would refuse is refused on all of them
        try:
            got = fuzz_programs.build_raw(seed, allreduce=True)(dev)
        except adb.devices.AdbError as e:
            assert "is a view when control flow joins" in str(e), str(e)
            continue
        for k, v in got.items():
            out[f"{seed}:{k}"] = v.numpy()
    np.savez(os.path.join(out_dir, f"raw{rank}.npz"), **out)
    dev.close()
    dist.destroy_process_group()


def test_hand_written_all_reduces_on_two_identical_ranks(tmp_path):
    """Raw-IR programs with all-reduces sprinkled over their values, run on two GPUs that hold the same data (nothing
    is sharded): the sum over ranks is twice the value, which the oracle reproduces with an all-reduce hook.  Exact
    integer arithmetic: bit for bit, with the collectives bucketed as the default lowering does."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import fuzz_programs
    from oracle.oracle import OracleDevice
    seeds = list(range(40))
    port = 29900 + (os.getpid() % 2000)
    mp.spawn(_raw_worker, args=(2, port, str(tmp_path), seeds), nprocs=2, join=True)
    got = [np.load(tmp_path / f"raw{r}.npz") for r in range(2)]
    checked = 0
    for seed in seeds:
        ora = OracleDevice(allreduce=lambda arr: np.multiply(arr, np.float32(2), out=arr))
        want = fuzz_programs.build_raw(seed, allreduce=True)(ora)
        for k, v in want.items():
            key = f"{seed}:{k}"
            if key not in got[0].files:
                continue            # refused on the device
            for r in range(2):
                np.testing.assert_array_equal(got[r][key].reshape(-1), v.numpy().reshape(-1), err_msg=f"{key} rank {r}")
            checked += 1
    assert checked >= 60, checked
