"""Seeded random sweep over the three entry points: layouts x head topologies x head dims x dtypes x
lengths that no hand-written grid enumerates (ragged length mixes, long-KV / few-query launches that take
the split-KV path, wide GQA groups, every page size), each checked against the fp32 SDPA oracle with the
reference's tolerance (tests/test_attention.py:20-30,246-251) and the stricter un-scaled bar."""
import random

import pytest
import torch

import test_attention as TA
import test_decode as TD
import test_speculative_decode as TS
from helpers import PREFILL_F32_STRICT, assert_close_both, spec_strict
from oracle import sdpa_ref

pytestmark = pytest.mark.gpu
DEVICE = "cuda"
HEADS = [(8, 8), (8, 2), (8, 1), (32, 8), (12, 4), (4, 1), (16, 2), (2, 2), (64, 8), (24, 3)]
DTYPES = [torch.float16, torch.bfloat16, torch.float32]
CASES_PER_CHUNK = 40


def _randn(shape, gen, dtype):
    return torch.randn(shape, generator=gen).to(dtype).to(DEVICE)


def _prefill_case(rng, gen, it):
    QH, KVH = rng.choice(HEADS)
    D, dtype = rng.choice([64, 128]), rng.choice(DTYPES)
    layout = rng.choice(["dense", "ragged", "paged"])
    B = rng.choice([1, 1, 2, 3, 5])
    causal = rng.random() < 0.5
    long_kv = rng.random() < 0.4
    max_q = rng.choice([128, 256, 500]) if long_kv else rng.choice([8, 130, 300, 700])
    max_kv = rng.choice([1100, 2100, 4200]) if long_kv else rng.choice([40, 300, 900])
    fixed_q, fixed_kv = rng.randint(1, max_q), rng.randint(1, max_kv)
    q_lens, kv_lens = [], []
    for _ in range(B):
        l_q = fixed_q if layout == "dense" else rng.randint(1, max_q)
        l_kv = l_q if causal else (fixed_kv if layout == "dense" else rng.randint(1, max_kv))
        if long_kv and causal:
            l_q = l_kv = fixed_kv if layout == "dense" else rng.randint(1, max_kv)
        q_lens.append(l_q)
        kv_lens.append(l_kv)
    what = f"prefill {layout} {QH}/{KVH} D{D} {dtype} causal={causal} q{q_lens} kv{kv_lens}"
    qs = [_randn((n, QH, D), gen, dtype) for n in q_lens]
    ks = [_randn((n, KVH, D), gen, dtype) for n in kv_lens]
    vs = [_randn((n, KVH, D), gen, dtype) for n in kv_lens]
    refs = sdpa_ref.prefill_reference(qs, ks, vs, QH, KVH, causal)
    outs = TA.run_prefill(layout, qs, ks, vs, causal, permute=it, poison=float("nan"), pad=-1,
                          page_size=rng.choice([16, 16, 8, 32, 64, 128]),
                          index_dtype=rng.choice([torch.int32, torch.int64]))
    for b in range(B):
        assert torch.isfinite(outs[b].float()).all(), what
        assert_close_both(outs[b], refs[b], dtype, max(kv_lens), f"{what} seq {b}",
                          strict=PREFILL_F32_STRICT if dtype == torch.float32 else None)


def _decode_case(rng, gen, it, spec):
    QH, KVH = rng.choice(HEADS)
    D, dtype = rng.choice([64, 128]), rng.choice(DTYPES)
    layout = rng.choice(["dense", "ragged", "paged"])
    B = rng.choice([1, 2, 4, 9, 33])
    max_kv = rng.choice([20, 300, 2000, 6000])
    fixed_kv = rng.randint(1, max_kv)
    M = rng.randint(1, 16) if spec else None
    causal = spec and rng.random() < 0.6
    kv_lens = [fixed_kv if layout == "dense" else rng.randint(1, max_kv) for _ in range(B)]
    drafts = M if causal else 0           # in causal mode the draft rows are the last M rows of each KV
    what = f"{'spec' if spec else 'decode'} {layout} {QH}/{KVH} D{D} {dtype} M={M} causal={causal} kv{kv_lens}"
    qs = [_randn((QH, D) if M is None else (QH, M, D), gen, dtype) for _ in range(B)]
    ks = [_randn((n + drafts, KVH, D), gen, dtype) for n in kv_lens]
    vs = [_randn((n + drafts, KVH, D), gen, dtype) for n in kv_lens]
    index_dtype = rng.choice([torch.int32, torch.int64])
    if spec:
        refs = sdpa_ref.spec_decode_reference(qs, ks, vs, QH, KVH, causal)
        out = TS.run_spec(layout, qs, ks, vs, causal, permute=it, poison=float("nan"), pad=-1, index_dtype=index_dtype)
    else:
        refs = sdpa_ref.decode_reference(qs, ks, vs, QH, KVH)
        out = TD.run_decode(layout, qs, ks, vs, kv_lens, permute=it, poison=float("nan"), pad=-1,
                            index_dtype=index_dtype)
    assert torch.isfinite(out.float()).all(), what
    for b in range(B):
        assert_close_both(out[b], refs[b], dtype, max(kv_lens) + drafts, f"{what} seq {b}",
                          strict=spec_strict(dtype, QH, KVH, M) if spec else None)


@pytest.mark.parametrize("chunk", range(6))
def test_random_configurations(chunk):
    for i in range(CASES_PER_CHUNK):
        it = chunk * CASES_PER_CHUNK + i
        rng, gen = random.Random(7919 * it + 13), torch.Generator().manual_seed(7919 * it + 13)
        kind = rng.choice(["prefill", "prefill", "decode", "spec"])
        if kind == "prefill":
            _prefill_case(rng, gen, it)
        else:
            _decode_case(rng, gen, it, spec=kind == "spec")
