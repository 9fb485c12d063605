"""Secondary sweeps over the reference's own benchmark grids (benchmarks/attention.py:11-55,
benchmarks/decode.py:11-43, benchmarks/speculative_decode.py:11-50 of the reference):

  prefill : BATCH 16, HEAD_DIM 128, PAGE 16, Q in {128, 512}, KV in {128, 512, 2048}, self + cross,
            mha 8/8, gqa 8/2, mqa 8/1, fp16 / bf16, dense / ragged / paged, causal for self attention
  decode  : BATCH 16, HEAD_DIM 64, N in {16 ... 8192}, same topologies and layouts
  spec    : as decode with M in {2, 4, 6, 8, 10} draft tokens, causal and not
  softmax : the shapes of benchmarks/benchmark_softmx.py:68-84 plus tensors far larger than L2; GB/s counts one read
            and one write of the tensor (the reference's bytes_softmax, :21-22)

Timing: CUDA events, median of `iters` calls after warm-up, L2 flushed between calls (the reference uses
triton.testing.do_bench, which flushes L2 the same way).  Prints one line per cell: milliseconds and the derived
TFLOP/s (prefill, visible score pairs only) or KV GB/s (decode).

    PYTHONPATH=triton-kernels_b200 python -m benchmarks.sweeps [prefill|decode|spec|softmax] [--quick]
    PYTHONPATH=triton-kernels_b200 python -m benchmarks.sweeps softmax --rows 8192 --cols 8192 --dtype float32
"""
from __future__ import annotations

import argparse
import statistics

import torch

from kernels import decode_attention, flash_attention_v2, log_softmax, softmax, speculative_decode_attention

DEVICE = "cuda"
BATCH = 16
PAGE = 16
TOPOLOGIES = {"mha": (8, 8), "gqa": (8, 2), "mqa": (8, 1)}


def _time(fn, iters=20, warmup=5):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEVICE)
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        torch.cuda._sleep(1_000_000)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return statistics.median(ts)


def _paged(k, v, n):
    """k, v: (B*n, H, D) packed equal-length sequences -> caches with a random page permutation."""
    blocks = (n + PAGE - 1) // PAGE
    g = torch.Generator().manual_seed(0)
    perm = torch.randperm(BATCH * blocks, generator=g).to(torch.int32).reshape(BATCH, blocks).to(DEVICE)
    kc = torch.zeros((BATCH * blocks * PAGE,) + tuple(k.shape[1:]), dtype=k.dtype, device=DEVICE)
    vc = torch.zeros_like(kc)
    rows = (perm.to(torch.int64)[:, :, None] * PAGE + torch.arange(PAGE, device=DEVICE)[None, None, :]).reshape(BATCH, -1)[:, :n]
    kc[rows.reshape(-1)] = k
    vc[rows.reshape(-1)] = v
    lens = torch.full((BATCH,), n, dtype=torch.int32, device=DEVICE)
    return kc, vc, perm, lens


def sweep_prefill(quick):
    D = 128
    print(f"{'layout':7s}{'attn':6s}{'topo':5s}{'dtype':6s}{'causal':7s}{'Q':>5s}{'KV':>6s}{'ms':>9s}{'TFLOP/s':>10s}")
    for layout in ("dense", "ragged", "paged"):
        for attn in ("self", "cross"):
            for topo, (qh, kvh) in TOPOLOGIES.items():
                for dtype in (torch.float16, torch.bfloat16):
                    for causal in (False, True):
                        if causal and attn == "cross":
                            continue
                        for lq in (128, 512):
                            for lkv in ((lq,) if attn == "self" else (128, 512, 2048)):
                                if quick and (dtype == torch.float16 or topo == "mha"):
                                    continue
                                q = torch.randn((BATCH, qh, lq, D), device=DEVICE, dtype=dtype)
                                k = torch.randn((BATCH, kvh, lkv, D), device=DEVICE, dtype=dtype)
                                v = torch.randn_like(k)
                                if layout == "dense":
                                    fn = lambda: flash_attention_v2(q, k, v, is_causal=causal)
                                elif layout == "ragged":
                                    qr = q.transpose(1, 2).reshape(BATCH * lq, qh, D).contiguous()
                                    kr = k.transpose(1, 2).reshape(BATCH * lkv, kvh, D).contiguous()
                                    vr = v.transpose(1, 2).reshape(BATCH * lkv, kvh, D).contiguous()
                                    qi = torch.arange(0, (BATCH + 1) * lq, lq, device=DEVICE, dtype=torch.int32)
                                    ki = torch.arange(0, (BATCH + 1) * lkv, lkv, device=DEVICE, dtype=torch.int32)
                                    fn = lambda: flash_attention_v2(qr, kr, vr, is_causal=causal, q_indptr=qi, kv_indptr=ki)
                                else:
                                    kr = k.transpose(1, 2).reshape(BATCH * lkv, kvh, D).contiguous()
                                    vr = v.transpose(1, 2).reshape(BATCH * lkv, kvh, D).contiguous()
                                    kc, vc, tab, lens = _paged(kr, vr, lkv)
                                    fn = lambda: flash_attention_v2(q, kc, vc, is_causal=causal, kv_indptr=lens,
                                                                    k_block_table=tab, v_block_table=tab, kv_page_size=PAGE)
                                ms = _time(fn)
                                pairs = lq * (lq + 1) / 2 if causal else lq * lkv
                                tf = 4.0 * D * BATCH * qh * pairs / ms / 1e9
                                print(f"{layout:7s}{attn:6s}{topo:5s}{str(dtype)[6:10]:6s}{str(causal):7s}{lq:5d}{lkv:6d}{ms:9.4f}{tf:10.1f}")


def sweep_decode(quick, spec):
    D = 64
    ns = (16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192)
    ms_list = (2, 4, 6, 8, 10) if spec else (1,)
    print(f"{'layout':7s}{'topo':5s}{'dtype':6s}{'M':>3s}{'causal':>7s}{'N':>6s}{'ms':>9s}{'KV GB/s':>10s}")
    for layout in ("dense", "ragged", "paged"):
        for topo, (qh, kvh) in TOPOLOGIES.items():
            for dtype in (torch.float16, torch.bfloat16, torch.float32):
                for m in ms_list:
                    for causal in ((True, False) if spec else (False,)):
                        for n in ns:
                            if quick and (dtype != torch.bfloat16 or topo == "mha" or n not in (128, 2048, 8192) or m not in (1, 4)):
                                continue
                            k = torch.randn((BATCH * n, kvh, D), device=DEVICE, dtype=dtype)
                            v = torch.randn_like(k)
                            q = torch.randn((BATCH, qh, m, D) if spec else (BATCH, qh, D), device=DEVICE, dtype=dtype)
                            kw = dict(causal=causal) if spec else {}
                            f = speculative_decode_attention if spec else decode_attention
                            if layout == "dense":
                                kd = k.reshape(BATCH, n, kvh, D).transpose(1, 2).contiguous()
                                vd = v.reshape(BATCH, n, kvh, D).transpose(1, 2).contiguous()
                                fn = lambda: f(q, kd, vd, **kw)
                            elif layout == "ragged":
                                ip = torch.arange(0, (BATCH + 1) * n, n, device=DEVICE, dtype=torch.int32)
                                fn = lambda: f(q, k, v, kv_indptr=ip, **kw)
                            else:
                                kc, vc, tab, lens = _paged(k, v, n)
                                fn = lambda: f(q, kc, vc, kv_indptr=lens, k_block_table=tab, v_block_table=tab,
                                               kv_page_size=PAGE, **kw)
                            t = _time(fn)
                            gbs = BATCH * n * kvh * D * 2 * k.element_size() / t / 1e6
                            print(f"{layout:7s}{topo:5s}{str(dtype)[6:10]:6s}{m:3d}{str(causal):>7s}{n:6d}{t:9.4f}{gbs:10.1f}")


SOFTMAX_SHAPES = [(1024,), (4096,), (64, 128), (128, 512), (512, 1024), (2048, 2048), (4096, 4096), (1, 32768),
                  (2, 32768), (8, 32768), (16, 32768), (1, 65536), (2, 65536), (8, 65536), (1, 131072),
                  # HBM-bound sizes (the grid above fits in L2)
                  (8192, 8192), (16384, 16384), (65536, 2048), (1024, 131072), (64, 1048576)]


def sweep_softmax(quick, only=None, dtypes=None):
    print("softmax: op dtype rows cols ms GB/s")
    shapes = [only] if only else (SOFTMAX_SHAPES[::3] if quick else SOFTMAX_SHAPES)
    for dtype in dtypes or (torch.float16, torch.bfloat16, torch.float32):
        for shape in shapes:
            x = torch.randn(shape, device=DEVICE, dtype=dtype)
            out = torch.empty_like(x)
            for name, f in (("softmax", softmax), ("log_softmax", log_softmax)):
                t = _time(lambda: f(x, out=out))
                gbs = 2 * x.numel() * x.element_size() / t / 1e6
                rows = x.numel() // x.shape[-1]
                print(f"{name:12s}{str(dtype)[6:]:9s}{rows:8d}{x.shape[-1]:9d}{t:10.4f}{gbs:10.1f}")
            del x, out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("which", nargs="?", default="all", choices=["all", "prefill", "decode", "spec", "softmax"])
    ap.add_argument("--quick", action="store_true", help="a thin slice of each grid")
    ap.add_argument("--rows", type=int, default=0, help="softmax: one shape only")
    ap.add_argument("--cols", type=int, default=0)
    ap.add_argument("--dtype", default="", choices=["", "float16", "bfloat16", "float32"])
    a = ap.parse_args()
    if a.which in ("all", "prefill"):
        sweep_prefill(a.quick)
    if a.which in ("all", "decode"):
        sweep_decode(a.quick, spec=False)
    if a.which in ("all", "spec"):
        sweep_decode(a.quick, spec=True)
    if a.which in ("all", "softmax"):
        only = (a.rows, a.cols) if a.rows > 0 and a.cols > 0 else None
        sweep_softmax(a.quick, only, [getattr(torch, a.dtype)] if a.dtype else None)


if __name__ == "__main__":
    main()
