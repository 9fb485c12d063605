"""GPU parity on the corner cells of the reference's own benchmark grids (benchmarks/attention.py:11-55:
BATCH 16, HEAD_DIM 128, Q in {128, 512}, KV in {128, 512, 2048}, self + cross, mha / gqa / mqa;
benchmarks/decode.py:28-43 and benchmarks/speculative_decode.py:29-50: BATCH 16, HEAD_DIM 64, N in {16 .. 8192},
M in {2 .. 10}).  The reference's tests stay at B = 4, D = 64 and sequences of at most 256 keys; these cells reach
cross attention with 16 KV tiles per query tile, launches with fewer work items than SMs, and one-page sequences."""
import pytest
import torch

from helpers import TOPOLOGIES, assert_close_both, make_rngs
from oracle import sdpa_ref
from test_attention import run_prefill
from test_decode import run_decode
from test_speculative_decode import run_spec

pytestmark = pytest.mark.gpu
DEVICE = "cuda"
BATCH = 16


def _seqs(gen, n, heads, d, dtype, count=BATCH):
    return [torch.randn((n, heads, d), generator=gen).to(dtype).to(DEVICE) for _ in range(count)]


@pytest.mark.parametrize("layout", ["dense", "ragged", "paged"])
@pytest.mark.parametrize("topology", list(TOPOLOGIES))
@pytest.mark.parametrize("cell", [("cross", 128, 2048, False), ("cross", 512, 128, False), ("self", 512, 512, True),
                                  ("self", 128, 128, True), ("cross", 128, 128, False)],
                         ids=["cross-q128-kv2048", "cross-q512-kv128", "self-q512-causal", "self-q128-causal", "cross-q128-kv128"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
def test_prefill_bench_grid_cell(layout, topology, cell, dtype):
    attn, lq, lkv, causal = cell
    qh, kvh = TOPOLOGIES[topology]
    _, gen = make_rngs("grid-prefill", layout, topology, cell, dtype)
    qs, ks, vs = _seqs(gen, lq, qh, 128, dtype), _seqs(gen, lkv, kvh, 128, dtype), _seqs(gen, lkv, kvh, 128, dtype)
    refs = sdpa_ref.prefill_reference(qs, ks, vs, qh, kvh, causal)
    outs = run_prefill(layout, qs, ks, vs, causal, permute=9, pad=-1)
    for b in (0, 7, 15):
        assert_close_both(outs[b], refs[b], dtype, lkv, f"{attn} q{lq} kv{lkv} seq {b}")


@pytest.mark.parametrize("layout", ["dense", "ragged", "paged"])
@pytest.mark.parametrize("topology", list(TOPOLOGIES))
@pytest.mark.parametrize("n", [16, 1024, 8192])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32], ids=["bf16", "fp32"])
def test_decode_bench_grid_cell(layout, topology, n, dtype):
    qh, kvh = TOPOLOGIES[topology]
    _, gen = make_rngs("grid-decode", layout, topology, n, dtype)
    qs = [torch.randn((qh, 64), generator=gen).to(dtype).to(DEVICE) for _ in range(BATCH)]
    ks, vs = _seqs(gen, n, kvh, 64, dtype), _seqs(gen, n, kvh, 64, dtype)
    refs = sdpa_ref.decode_reference(qs, ks, vs, qh, kvh)
    out = run_decode(layout, qs, ks, vs, [n] * BATCH, permute=3, pad=-1)
    for b in (0, 9, 15):
        assert_close_both(out[b], refs[b], dtype, n, f"decode n{n} seq {b}")


@pytest.mark.parametrize("layout", ["dense", "ragged", "paged"])
@pytest.mark.parametrize("topology", list(TOPOLOGIES))
@pytest.mark.parametrize("m", [2, 10])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("n", [16, 2048])
def test_spec_decode_bench_grid_cell(layout, topology, m, causal, n):
    dtype = torch.bfloat16
    qh, kvh = TOPOLOGIES[topology]
    _, gen = make_rngs("grid-spec", layout, topology, m, causal, n)
    qs = [torch.randn((qh, m, 64), generator=gen).to(dtype).to(DEVICE) for _ in range(BATCH)]
    total = n + m if causal else n           # causal: the m draft K/V rows are the tail of the sequence
    ks, vs = _seqs(gen, total, kvh, 64, dtype), _seqs(gen, total, kvh, 64, dtype)
    refs = sdpa_ref.spec_decode_reference(qs, ks, vs, qh, kvh, causal)
    out = run_spec(layout, qs, ks, vs, causal, permute=5, pad=-1)
    for b in (0, 4, 15):
        assert_close_both(out[b], refs[b], dtype, total, f"spec m{m} n{n} seq {b}")
