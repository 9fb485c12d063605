"""Two ranks on two GPUs (one process per GPU, NCCL): every benchmark configuration, at a reduced size, cut the way
the configuration names, computed shard by shard through the entry points, all-gathered with sharding/gather.py and
compared with the same problem computed on one GPU.  Needs two visible GPUs; skipped where there is one."""
import os
import socket
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

pytestmark = pytest.mark.gpu

SMALL = {"c2": dict(batch=2, q_heads=16, kv_heads=4, seq=384, head_dim=128),
         "c3": dict(n_seqs=7, lo=30, hi=700),
         "c4": dict(batch=8, lo=100, hi=3000),
         "c5": dict(batch=4, lo=200, hi=5000)}


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    for p in (os.path.join(ROOT, "triton-kernels_b200"), ROOT):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from benchmarks import workloads as W
    from kernels import _native
    from sharding import all_gather_outputs, all_gather_ragged

    for name, cfg in SMALL.items():
        shard, full, assemble = W.STRONG[name](dev, 5, rank, world, **cfg)
        out = shard.run()
        parts = (all_gather_ragged if name == "c3" else all_gather_outputs)(out)
        got = assemble(parts)
        whole = full.run()
        torch.cuda.synchronize()
        assert got.shape == whole.shape, name
        if name in ("c2", "c3"):
            # a prefill unit is computed tile by tile in the same order wherever it runs: bit-identical
            assert torch.equal(got, whole), name
        else:
            # split-KV chunking follows the batch a rank holds, so partial sums are grouped differently
            torch.testing.assert_close(got.float(), whole.float(), atol=2e-2, rtol=2e-2)
    torch.cuda.synchronize()
    _native.check_device_errors()
    dist.barrier()
    dist.destroy_process_group()
    open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")


def test_sharded_outputs_gathered_over_nccl_equal_single_gpu(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
