#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c3|c4|c5]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Prints ONE JSON line on rank 0.  The headline workload is the dense causal GQA bf16 prefill
(batch 2, 32/8 heads, seq 2048, head_dim 128); the ragged prefill, paged decode and paged
speculative decode configurations are measured in the same run and reported under "workloads".

A step is one call of the entry point on one batch of seeded synthetic inputs.
  value : algorithmic FLOPs (prefill) or KV bytes (decode) of all ranks / device time of the slowest
          rank, inputs resident in HBM, CUDA events on the launch stream, L2 flushed between steps.
  e2e   : the same quantity through the Python entry point with the per-step inputs in pinned host
          memory: H2D copies, the call, and the D2H copy of the output are all inside the timed region
          (upload, kernels and download on three streams, two sets of device input buffers).  Every step
          is timed by its own event pair; the figure is the median step, with min / max, the PCIe link and
          the achieved copy rates beside it.
Multi-GPU runs: the headline `value` is weak scaling (every rank runs the full single-GPU configuration
on its own seeded inputs, global batch = N x the configuration's batch, no data-path collective).  At
N > 1 every workload also carries a "strong" entry: ONE problem cut the way the configuration names
(dense prefill by batch x KV-head units, ragged prefill by balanced token cost, paged decode by batch,
speculative decode by KV head), timed as max over ranks, and - once, outside the timed region - the
shards are all-gathered over NCCL and compared with the same problem computed on rank 0's GPU.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "triton-kernels_b200")
for _p in (PKG, ROOT):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
NOMINAL = {"hbm_gbs": 8000.0, "bf16_tflops": 2250.0}
L2_FLUSH_BYTES = 512 << 20

# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum), one ncu capture per kernel and workload.
NCU_TRAFFIC_BYTES = {"c2": 54.2e6, "c3": 778.6e6, "c4": 1137.2e6, "c5": 1805.4e6}
# kernels of this library launched per call of the entry point (prefill: the persistent kernel;
# decode: planner + split kernel with fused merge)
LAUNCHES_PER_STEP = {"c2": 1, "c3": 1, "c4": 2, "c5": 2}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {k: float(d[k]) for k in FALLBACK_PEAKS if k in d} | {"source": "measured"}
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_indices):
        self.gpus = set(int(i) for i in gpu_indices)
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                if int(parts[0]) not in self.gpus:
                    continue
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.unlink(self.file.name)
        except OSError:
            pass
        busy = [x for x in sm if x > 0]
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def build_workload(name, device, rank, world, seed):
    from benchmarks import workloads as W

    shard = (rank, world)
    if name == "c2":
        return W.c2_dense_prefill(device, seed, shard=shard)
    if name == "c3":
        return W.c3_ragged_prefill(device, seed, shard=shard, weak=True)
    if name == "c4":
        return W.c4_paged_decode(device, seed, shard=shard, weak=True)
    if name == "c5":
        return W.c5_paged_spec_decode(device, seed, shard=shard, weak=True)
    raise ValueError(name)


def dist_max(x: float, world: int, device) -> float:
    if world == 1:
        return x
    import torch.distributed as dist

    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def dist_sum(x: float, world: int, device) -> float:
    if world == 1:
        return x
    import torch.distributed as dist

    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def barrier(world):
    if world > 1:
        import torch.distributed as dist

        dist.barrier()


def time_resident(wl, steps, warmup, flush, world):
    """Device time of `steps` calls, L2 flushed (and the launch queue primed) before each one."""
    for _ in range(warmup):
        wl.run()
    torch.cuda.synchronize()
    barrier(world)
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        flush.zero_()                      # evicts L2; also keeps the GPU busy while the host prepares the launch
        torch.cuda._sleep(2_000_000)   # ~1 ms: the host finishes preparing the launch meanwhile
        starts[i].record()
        wl.run()
        stops[i].record()
    torch.cuda.synchronize()
    barrier(world)
    torch.cuda.synchronize()
    return [s.elapsed_time(e) for s, e in zip(starts, stops)]  # ms


def time_end_to_end(wl, steps, warmup, world):
    """Every step copies its inputs from pinned host memory, calls the public entry point and copies the output back
    to pinned host memory, all inside the timed region.  The three stages run on three streams with two sets of
    device input buffers, the way a serving loop would: step i's upload overlaps step i-1's kernels and download
    (PCIe is full duplex), ordered by events; nothing is skipped or cached."""
    dev = next(iter(wl.tensors.values())).device
    host = {n: wl.tensors[n].cpu().pin_memory() for n in wl.host_inputs}
    dev_sets = [{n: wl.tensors[n] for n in wl.host_inputs}, {n: torch.empty_like(wl.tensors[n]) for n in wl.host_inputs}]
    out0 = wl.run()
    out_host = torch.empty(out0.shape, dtype=out0.dtype).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host.values())
    d2h = out_host.numel() * out_host.element_size()
    s_comp = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    comp_done = [None, None]     # last compute event that read each input set
    out_done = None              # the previous download (out_host is reused)

    def step(i):
        nonlocal out_done
        cur = dev_sets[i & 1]
        with torch.cuda.stream(s_in):
            if comp_done[i & 1] is not None:
                s_in.wait_event(comp_done[i & 1])          # the kernels that read this set two steps ago are done
            for n, t in host.items():
                cur[n].copy_(t, non_blocking=True)
            uploaded = torch.cuda.Event()
            uploaded.record(s_in)
        s_comp.wait_event(uploaded)
        for n in wl.host_inputs:
            wl.tensors[n] = cur[n]
        out = wl.run()
        ev = torch.cuda.Event()
        ev.record(s_comp)
        comp_done[i & 1] = ev
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev)
            if out_done is not None:
                s_out.wait_event(out_done)
            out.record_stream(s_out)
            out_host.copy_(out, non_blocking=True)
            out_done = torch.cuda.Event()
            out_done.record(s_out)

    for i in range(max(2, warmup)):
        step(i)
    torch.cuda.synchronize()
    barrier(world)
    torch.cuda.synchronize()
    # one event per step, recorded behind the step's download: the interval between two of them is what one more
    # step costs the pipeline (upload, kernels and download of neighbouring steps overlap)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    s_out.wait_stream(s_comp)
    marks[0].record(s_out)
    s_in.wait_event(marks[0])
    s_comp.wait_event(marks[0])
    for i in range(steps):
        step(i)
        marks[i + 1].record(s_out)
    torch.cuda.synchronize()
    barrier(world)
    for n in wl.host_inputs:
        wl.tensors[n] = dev_sets[0][n]
    intervals = [marks[i].elapsed_time(marks[i + 1]) for i in range(steps)]
    return intervals, h2d, d2h


def pin_rank_to_cores(local_rank, world):
    """With several ranks on one host, give each its own equal slice of the cores this process may use, so that the
    ranks' launch and copy-submission threads do not migrate onto each other.  Returns the slice (or None)."""
    if world <= 1 or not hasattr(os, "sched_getaffinity"):
        return None
    try:
        cores = sorted(os.sched_getaffinity(0))
        per = len(cores) // world
        if per < 1:
            return None
        mine = cores[local_rank * per:(local_rank + 1) * per]
        os.sched_setaffinity(0, mine)
        return [mine[0], mine[-1]]
    except OSError:
        return None


def pcie_link(index):
    """Current PCIe link of the GPU (read-only query), e.g. {"gen": 5, "width": 16}."""
    try:
        out = subprocess.run(["nvidia-smi", "--query-gpu=pcie.link.gen.current,pcie.link.width.current",
                              "--format=csv,noheader,nounits", "-i", str(index)], capture_output=True, text=True,
                             timeout=20).stdout.strip().splitlines()[0]
        gen, width = [int(x.strip()) for x in out.split(",")]
        # usable payload rate per direction, GB/s: 128b/130b encoding from gen 3 on, ~1 GB/s per lane at gen 3
        rate = {1: 0.25, 2: 0.5, 3: 0.985, 4: 1.969, 5: 3.938, 6: 7.56}.get(gen, 0.0) * width
        return {"gen": gen, "width": width, "nominal_gbs_per_direction": round(rate, 1)}
    except Exception:  # noqa: BLE001 - the query is informational
        return None


def summarize_e2e(intervals, h2d, d2h, work_all, scale, unit, world, device, link):
    """Median / min / max of the per-step intervals (max over ranks of each), achieved copy rates, and what bounds it."""
    med = dist_max(statistics.median(intervals), world, device)
    lo = dist_max(min(intervals), world, device)
    hi = dist_max(max(intervals), world, device)
    mean = dist_max(sum(intervals) / len(intervals), world, device)
    res = {"value": work_all * scale / (med * 1e-3), "unit": unit, "ms_per_step": med, "ms_min": lo, "ms_max": hi,
           "ms_mean": mean, "steps": len(intervals), "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "h2d_gbs": h2d / (med * 1e-3) * 1e-9, "d2h_gbs": d2h / (med * 1e-3) * 1e-9, "pcie": link}
    return res


def measure(name, device, rank, world, steps, warmup, seed, peaks, flush, e2e_steps, link):
    wl = build_workload(name, device, rank, world, seed)
    times = time_resident(wl, steps, warmup, flush, world)
    ms = sum(times) / len(times)
    ms_max = dist_max(ms, world, device)
    work = wl.flops if wl.kind == "prefill" else wl.kv_bytes
    work_all = dist_sum(work, world, device)
    if wl.kind == "prefill":
        unit, scale, bound, peak_key = "TFLOP/s", 1e-12, "tensor", "bf16_tflops"
    else:
        unit, scale, bound, peak_key = "GB/s", 1e-9, "hbm", "hbm_gbs"
    intervals, h2d, d2h = time_end_to_end(wl, e2e_steps, 5, world)
    e2e = summarize_e2e(intervals, h2d, d2h, work_all, scale, unit, world, device, link)
    # what the end-to-end step cannot beat: the larger copy direction over the link, or the kernel itself
    if link and link.get("nominal_gbs_per_direction"):
        copy_ms = max(h2d, d2h) / (link["nominal_gbs_per_direction"] * 1e9) * 1e3
        e2e["bound"] = {"copy_ms_at_link_rate": copy_ms, "kernel_ms": ms,
                        "limiter": "pcie copies" if copy_ms > ms else "kernel"}
    value = work_all * scale / (ms_max * 1e-3)
    achieved = work * scale / (ms * 1e-3)          # this rank's kernel
    peak = peaks[peak_key]
    res = {
        "workload": wl.name, "value": value, "unit": unit, "ms_per_step": ms_max,
        "ms_min": min(times), "ms_median": statistics.median(times),
        "e2e": e2e,
        "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                     "frac_of_nominal": achieved / NOMINAL[peak_key], "peak_source": peaks["source"],
                     "traffic": NCU_TRAFFIC_BYTES[name]},
        "gpu_launches": LAUNCHES_PER_STEP[name] * steps,
        "algorithmic_work_per_step": work, "meta": {k: v for k, v in wl.meta.items() if k != "lengths"},
    }
    del wl
    torch.cuda.empty_cache()
    if world > 1:
        res["strong"] = measure_strong(name, device, rank, world, steps, warmup, seed, peaks, flush, scale, unit, peak_key)
    return res


def measure_strong(name, device, rank, world, steps, warmup, seed, peaks, flush, scale, unit, peak_key):
    """ONE problem cut across the ranks the way the configuration names; max over ranks; plus, outside the timed
    region, the all-gather of the shards over NCCL compared with the whole problem computed on rank 0's GPU."""
    import torch.distributed as dist

    from benchmarks import workloads as W
    from sharding import all_gather_outputs, all_gather_ragged

    shard, full, assemble = W.STRONG[name](device, seed, rank, world)
    work_full = full.flops if full.kind == "prefill" else full.kv_bytes
    work_mine = shard.flops if shard.kind == "prefill" else shard.kv_bytes
    # --- the check: gather the shards and compare with the whole problem on one GPU
    out = shard.run()
    torch.cuda.synchronize()
    gather = all_gather_ragged if name == "c3" else all_gather_outputs
    parts = gather(out)                     # warm-up of the collective
    torch.cuda.synchronize()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    parts = gather(out)
    e1.record()
    torch.cuda.synchronize()
    gather_us = dist_max(e0.elapsed_time(e1) * 1e3, world, device)
    check = None
    if rank == 0:
        whole = full.run()
        got = assemble(parts)
        torch.cuda.synchronize()
        diff = (got.float() - whole.float()).abs().max().item() if whole.numel() else 0.0
        # bit equality where shard and whole take the same path (prefill without the KV split); otherwise partial
        # sums are grouped differently and the two agree to rounding: the reference's own bar for this dtype at N = 1
        # (bf16: atol 2.4e-2, rtol 2e-2; tests/test_attention.py:20-30 of the reference) is reported beside it
        close = bool(torch.allclose(got.float(), whole.float(), atol=2.4e-2, rtol=2e-2)) if whole.numel() else True
        check = {"sharded_equals_single": bool(torch.equal(got, whole)), "max_abs_diff": diff,
                 "within_reference_tolerance": close,
                 "gather_us": gather_us, "gathered_bytes": got.numel() * got.element_size()}
        del whole, got
    del parts, out
    # only the shard stays resident for the timing (rank 0 held the whole problem for the check)
    shard_names = set(id(t) for t in shard.tensors.values())
    for k in list(full.tensors):
        if id(full.tensors[k]) not in shard_names:
            full.tensors[k] = None
    del full
    torch.cuda.empty_cache()
    times = time_resident(shard, steps, warmup, flush, world)
    ms = sum(times) / len(times)
    ms_max = dist_max(ms, world, device)
    ms_min_rank = -dist_max(-ms, world, device)
    res = {"value": work_full * scale / (ms_max * 1e-3), "unit": unit, "ms_per_step": ms_max,
           "ms_fastest_rank": ms_min_rank, "frac_per_gpu": work_full * scale / (ms_max * 1e-3) / world / peaks[peak_key],
           "work_share_of_slowest": dist_max(work_mine, world, device) / work_full,
           "parallelism": {"c2": "batch x KV-head units, contiguous", "c3": "sequences by balanced causal cost (LPT)",
                           "c4": "batch, contiguous", "c5": "KV heads, contiguous"}[name]}
    if check is not None:
        res["check"] = check
    del shard
    torch.cuda.empty_cache()
    return res


# ---------------------------------------------------------------------------
# CPU arm: the reference's own PyTorch path (fp32 scaled_dot_product_attention per sequence, the
# oracle its tests compare against), on the host cores of this box.
# ---------------------------------------------------------------------------
def cpu_reference(name, steps, warmup, seed):
    from benchmarks import workloads as W
    from oracle import sdpa_ref

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cpu = torch.device("cpu")
    g = torch.Generator().manual_seed(seed)
    if name == "c2":
        qh, kvh, seq, d, b = 32, 8, 2048, 128, 2
        qs = [torch.randn((seq, qh, d), generator=g).bfloat16() for _ in range(b)]
        ks = [torch.randn((seq, kvh, d), generator=g).bfloat16() for _ in range(b)]
        vs = [torch.randn((seq, kvh, d), generator=g).bfloat16() for _ in range(b)]
        fn = lambda: sdpa_ref.prefill_reference(qs, ks, vs, qh, kvh, True)
        work, unit, scale = 4.0 * d * qh * b * seq * (seq + 1) / 2, "TFLOP/s", 1e-12
        sample = "full configuration: 2 sequences x 32 q heads x 2048 x 2048 causal, fp32 SDPA per sequence"
    elif name == "c3":
        qh, kvh, d = 32, 8, 128
        lens = W.c3_lengths(seed)[:4]
        qs = [torch.randn((n, qh, d), generator=g).bfloat16() for n in lens]
        ks = [torch.randn((n, kvh, d), generator=g).bfloat16() for n in lens]
        vs = [torch.randn((n, kvh, d), generator=g).bfloat16() for n in lens]
        fn = lambda: sdpa_ref.prefill_reference(qs, ks, vs, qh, kvh, True)
        work, unit, scale = sum(4.0 * d * qh * n * (n + 1) / 2 for n in lens), "TFLOP/s", 1e-12
        sample = f"first 4 of the 16 sequences (lengths {lens})"
    elif name == "c4":
        qh, kvh, d = 32, 8, 128
        lens = W._lengths(seed, 64, 512, 8192)[:16]
        qs = [torch.randn((qh, d), generator=g).bfloat16() for _ in lens]
        ks = [torch.randn((n, kvh, d), generator=g).bfloat16() for n in lens]
        vs = [torch.randn((n, kvh, d), generator=g).bfloat16() for n in lens]
        fn = lambda: sdpa_ref.decode_reference(qs, ks, vs, qh, kvh)
        work, unit, scale = float(sum(lens)) * kvh * d * 2 * 2, "GB/s", 1e-9
        sample = "first 16 of the 64 sequences, K/V already gathered from their pages"
    else:
        qh, kvh, d, m = 64, 8, 128, 5
        lens = [c + m for c in W._lengths(seed, 32, 1024, 32768)[:4]]
        qs = [torch.randn((qh, m, d), generator=g).bfloat16() for _ in lens]
        ks = [torch.randn((n, kvh, d), generator=g).bfloat16() for n in lens]
        vs = [torch.randn((n, kvh, d), generator=g).bfloat16() for n in lens]
        fn = lambda: sdpa_ref.spec_decode_reference(qs, ks, vs, qh, kvh, True)
        work, unit, scale = float(sum(lens)) * kvh * d * 2 * 2, "GB/s", 1e-9
        sample = "first 4 of the 32 sequences, K/V already gathered from their pages"
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter()
        fn()
        ts.append(time.perf_counter() - t0)
    sec = sum(ts) / len(ts)
    return {"value": work * scale / sec, "unit": unit, "cores": cores, "kind": "port", "sample": sample,
            "ms_per_step": sec * 1e3}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c2", "c3", "c4", "c5"])
    ap.add_argument("--only", action="store_true", help="measure only --workload, not the other configurations")
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    metric = {"c2": "prefill_attn_tflops", "c3": "prefill_attn_tflops", "c4": "paged_decode_kv_gbs",
              "c5": "paged_decode_kv_gbs"}[args.workload]
    wl_names = {"c2": "c2_dense_causal_prefill", "c3": "c3_ragged_causal_prefill", "c4": "c4_paged_decode",
                "c5": "c5_paged_spec_decode"}

    if args.impl == "reference":
        if rank != 0:
            return
        base = cpu_reference(args.workload, max(1, args.steps), max(1, min(args.warmup, 2)), args.seed)
        line = {
            "impl": "reference", "metric": metric, "value": base["value"], "unit": base["unit"], "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": wl_names[args.workload], "sample": base["sample"]},
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": base["value"], "unit": base["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        }
        print(json.dumps(line), flush=True)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (sm_100a); there is no CPU fallback")
    affinity = pin_rank_to_cores(local_rank, world)
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
    from kernels import _native

    peaks = load_peaks()
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    sampler = ClockSampler(range(world)) if rank == 0 else None
    if sampler:
        sampler.start()
    order = [args.workload] + ([] if args.only else [n for n in ("c2", "c3", "c4", "c5") if n != args.workload])
    link = pcie_link(local_rank)
    results = {}
    for i, name in enumerate(order):
        steps = args.steps if i == 0 else max(5, min(args.steps, 10))
        results[name] = measure(name, device, rank, world, steps, args.warmup, args.seed, peaks, flush,
                                e2e_steps=30 if name != "c3" else 20, link=link)
    clocks = sampler.stop() if sampler else None
    torch.cuda.synchronize()
    _native.check_device_errors()

    if rank == 0:
        main_res = results[args.workload]
        line = {
            "metric": metric, "value": main_res["value"], "unit": main_res["unit"], "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": main_res["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": main_res["workload"], "l2": "flushed between timed steps (512 MiB memset)",
                       "timing": "CUDA events per step on the launch stream, mean over steps, max over ranks; "
                                 "e2e: median of per-step event intervals",
                       "parallelism": f"independent replicas x{world} (batch-sharded, no collective)",
                       **main_res["meta"]},
            "e2e": main_res["e2e"],
            "gpu_launches": main_res["gpu_launches"],
            "roofline": main_res["roofline"],
            "clocks": clocks,
            "cpu_affinity_rank0": affinity,
            "workloads": {n: {k: r[k] for k in ("workload", "value", "unit", "ms_per_step", "ms_min", "e2e", "roofline",
                                                "strong") if k in r}
                          for n, r in results.items()},
        }
        if world == 1:
            cb = cpu_reference(args.workload, 3, 1, args.seed)
            line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


if __name__ == "__main__":
    main()
