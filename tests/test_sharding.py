"""Multi-rank host logic on CPU (gloo, world_size 2): the shard planners partition the benchmark
configurations without overlap, and the optional output gather reassembles per-rank shards in rank order.
The oracle plays the kernel here (the tests are about partitioning, not arithmetic)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


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
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import sdpa_ref
    from sharding import all_gather_outputs, all_gather_ragged, balance_sequences, batch_head_units, contiguous_shard

    # --- dense prefill sharded by (batch, kv head) units: every rank computes its q-head groups ---
    g = torch.Generator().manual_seed(0)
    B, QH, KVH, S, D = 2, 8, 4, 24, 16
    q = torch.randn((B, QH, S, D), generator=g)
    k = torch.randn((B, KVH, S, D), generator=g)
    v = torch.randn((B, KVH, S, D), generator=g)
    grp = QH // KVH
    units = batch_head_units(B, KVH, world, rank)
    outs = []
    for (b, h) in units:
        qs = q[b, h * grp:(h + 1) * grp].transpose(0, 1)
        outs.append(sdpa_ref.prefill_reference([qs], [k[b, h:h + 1].transpose(0, 1)], [v[b, h:h + 1].transpose(0, 1)],
                                               grp, 1, True)[0].transpose(0, 1))
    shard = torch.stack(outs)                       # (units, grp, S, D)
    gathered = torch.cat(all_gather_outputs(shard))  # rank order == unit order
    full = sdpa_ref.prefill_reference([q[b].transpose(0, 1) for b in range(B)], [k[b].transpose(0, 1) for b in range(B)],
                                      [v[b].transpose(0, 1) for b in range(B)], QH, KVH, True)
    want = torch.stack([f.transpose(0, 1) for f in full]).reshape(B * KVH, grp, S, D)
    assert torch.allclose(gathered, want, atol=1e-6)

    # --- ragged prefill: sequences balanced by causal cost; gather of unequal shards ---
    lens = [5, 40, 17, 33, 8, 29]
    seqs_q = [torch.randn((n, QH, D), generator=g) for n in lens]
    seqs_k = [torch.randn((n, KVH, D), generator=g) for n in lens]
    seqs_v = [torch.randn((n, KVH, D), generator=g) for n in lens]
    bins = balance_sequences(lens, world)
    mine = bins[rank]
    my_out = torch.cat(sdpa_ref.prefill_reference([seqs_q[i] for i in mine], [seqs_k[i] for i in mine],
                                                  [seqs_v[i] for i in mine], QH, KVH, True)) if mine else torch.zeros((0, QH, D))
    parts = all_gather_ragged(my_out)
    ref = sdpa_ref.prefill_reference(seqs_q, seqs_k, seqs_v, QH, KVH, True)
    for r in range(world):
        want_r = torch.cat([ref[i] for i in bins[r]]) if bins[r] else torch.zeros((0, QH, D))
        assert torch.allclose(parts[r], want_r, atol=1e-6)

    # --- decode sharded by batch ---
    b0, b1 = contiguous_shard(len(lens), world, rank)
    qd = [torch.randn((QH, D), generator=g) for _ in lens]
    refs = sdpa_ref.decode_reference(qd, seqs_k, seqs_v, QH, KVH)
    mine_out = torch.stack(refs[b0:b1])
    allo = torch.cat(all_gather_outputs(mine_out)) if len(lens) % world == 0 else None
    if allo is not None:
        assert torch.allclose(allo, torch.stack(refs), atol=1e-6)
    dist.barrier()
    dist.destroy_process_group()
    open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")


@pytest.mark.parametrize("world", [2])
def test_sharded_attention_two_ranks(tmp_path, world):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_failed_rank_is_detected_on_the_host(tmp_path):
    """A rank that raises before the gather must surface as an error in the parent, not a hang."""
    def run():
        mp.spawn(_failing_worker, args=(2, _free_port()), nprocs=2, join=True)

    with pytest.raises(Exception):
        run()


def _failing_worker(rank, world, port):
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=10))
    if rank == 1:
        raise RuntimeError("injected host-side failure before the collective")
    t = torch.zeros(4)
    dist.all_reduce(t)   # rank 0 must not hang forever: the group times out or the peer's exit is noticed


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("name", ["c2", "c3", "c4", "c5"])
def test_strong_shards_reassemble_to_the_whole_problem(name, world):
    """The strong-scaling cut of every benchmark configuration (benchmarks/workloads.STRONG), at a small size on
    CPU with the oracle playing the kernel: the shards' outputs, put back together by `assemble`, are the whole
    problem's output, and the shards' algorithmic work adds up to the whole."""
    from benchmarks import workloads as W
    from oracle import sdpa_ref

    cpu = torch.device("cpu")
    cfg = {"c2": dict(batch=2, q_heads=16, kv_heads=8, seq=24, head_dim=16, dtype=torch.float32),
           "c3": dict(n_seqs=9, lo=3, hi=40, q_heads=8, kv_heads=2, head_dim=16, dtype=torch.float32),
           "c4": dict(batch=16, lo=5, hi=70, q_heads=8, kv_heads=2, head_dim=16, dtype=torch.float32),
           "c5": dict(batch=4, drafts=3, lo=5, hi=50, q_heads=16, kv_heads=8, head_dim=16, dtype=torch.float32)}[name]

    def oracle_run(wl):
        t, m = wl.tensors, wl.meta
        if name == "c2":
            b, qh = t["q"].shape[0], t["q"].shape[1]
            kvh = t["k"].shape[1]
            outs = sdpa_ref.prefill_reference([t["q"][i].transpose(0, 1) for i in range(b)],
                                              [t["k"][i].transpose(0, 1) for i in range(b)],
                                              [t["v"][i].transpose(0, 1) for i in range(b)], qh, kvh, True)
            return torch.stack([o.transpose(0, 1) for o in outs]) if outs else t["q"][:0]
        if name == "c3":
            ip = t["indptr"].tolist()
            seq = lambda x: [x[ip[i]:ip[i + 1]] for i in range(len(ip) - 1)]
            outs = sdpa_ref.prefill_reference(seq(t["q"]), seq(t["k"]), seq(t["v"]), t["q"].shape[1], t["k"].shape[1], True)
            return torch.cat(outs) if outs else t["q"][:0]
        lens = t["lens"].tolist()
        ks = [W.gather_paged(t["k_cache"], t["k_table"][i], lens[i], m["page_size"]) for i in range(len(lens))]
        vs = [W.gather_paged(t["v_cache"], t["v_table"][i], lens[i], m["page_size"]) for i in range(len(lens))]
        qh, kvh = t["q"].shape[1], t["k_cache"].shape[1]
        if name == "c4":
            outs = sdpa_ref.decode_reference([t["q"][i] for i in range(len(lens))], ks, vs, qh, kvh)
        else:
            outs = sdpa_ref.spec_decode_reference([t["q"][i] for i in range(len(lens))], ks, vs, qh, kvh, True)
        return torch.stack(outs) if outs else t["q"][:0]

    parts, flops, kvb = [], 0.0, 0.0
    for rank in range(world):
        shard, full, assemble = W.STRONG[name](cpu, 3, rank, world, **cfg)
        parts.append(oracle_run(shard))
        flops += shard.flops
        kvb += shard.kv_bytes
    got = assemble(parts)
    want = oracle_run(full)
    assert got.shape == want.shape
    torch.testing.assert_close(got.float(), want.float(), atol=1e-6, rtol=1e-6)
    assert abs(flops - full.flops) <= 1e-9 * full.flops
    if name in ("c4", "c5"):
        assert abs(kvb - full.kv_bytes) <= 1e-9 * full.kv_bytes
