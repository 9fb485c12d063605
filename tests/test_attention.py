"""GPU parity tests for flash_attention_v2 / flash_attention_v1.  Mirrors the reference's
tests/test_attention.py:137-251 (layout x self/cross x topology x causal x dtype, B=4, D=64,
causal+cross skipped) with seeded inputs, then adds D=128, multi-tile sequences, hostile paged
caches, both index widths and known answers."""
import pytest
import torch

from helpers import (DTYPE_IDS, DTYPES, PREFILL_F32_STRICT, TOPOLOGIES, assert_close_both, make_rngs,
                     prefill_sequences)
from oracle import sdpa_ref

pytestmark = pytest.mark.gpu
DEVICE = "cuda"
PAGE_SIZE = 16

HALF_DTYPES = [torch.float16, torch.bfloat16]


def run_prefill(layout, qs, ks, vs, causal, *, index_dtype=torch.int32, permute=None, poison=None, pad=0,
                page_size=PAGE_SIZE, fn=None):
    if fn is None:
        from kernels.attention import flash_attention_v2 as fn
    B = len(qs)
    q_lens = [int(x.shape[0]) for x in qs]
    if layout == "dense":
        q, k, v = sdpa_ref.pack_dense_prefill(qs, ks, vs)
        out = fn(q, k, v, is_causal=causal)
        return [out[b, :, : q_lens[b], :].transpose(0, 1) for b in range(B)]
    if layout == "ragged":
        q, q_indptr = sdpa_ref.pack_ragged(qs, index_dtype)
        k, kv_indptr = sdpa_ref.pack_ragged(ks, index_dtype)
        v, _ = sdpa_ref.pack_ragged(vs, index_dtype)
        out = fn(q, k, v, is_causal=causal, q_indptr=q_indptr, kv_indptr=kv_indptr)
        ip = q_indptr.tolist()
        return [out[ip[b]: ip[b + 1]] for b in range(B)]
    QH, D = qs[0].shape[1], qs[0].shape[2]
    q = torch.zeros((B, QH, max(q_lens), D), device=DEVICE, dtype=qs[0].dtype)
    for b in range(B):
        q[b, :, : q_lens[b]] = qs[b].transpose(0, 1)
    kc, kt, lens = sdpa_ref.pack_paged(ks, page_size, permute_seed=permute, extra_pages=3 if permute is not None else 0,
                                       pad_value=pad, poison=poison)
    vc, vt, _ = sdpa_ref.pack_paged(vs, page_size, permute_seed=None if permute is None else permute + 1,
                                    extra_pages=3 if permute is not None else 0, pad_value=pad, poison=poison)
    out = fn(q, kc, vc, is_causal=causal, kv_indptr=lens.to(index_dtype), k_block_table=kt, v_block_table=vt,
             kv_page_size=page_size)
    return [out[b, :, : q_lens[b], :].transpose(0, 1) for b in range(B)]


@pytest.mark.parametrize("layout", ["dense", "paged", "ragged"])
@pytest.mark.parametrize("attn_type", ["self", "cross"])
@pytest.mark.parametrize("topology", list(TOPOLOGIES))
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("dtype", DTYPES, ids=DTYPE_IDS)
def test_attention_reference_grid(layout, attn_type, topology, causal, dtype):
    if causal and attn_type == "cross":
        pytest.skip("Causal masking on cross attention is undefined in the reference (tests/test_attention.py:145-146).")
    QH, KVH = TOPOLOGIES[topology]
    rng, gen = make_rngs("prefill", layout, attn_type, topology, causal, dtype)
    qs, ks, vs, q_lens, kv_lens = prefill_sequences(rng, gen, 4, QH, KVH, 64, attn_type, dtype, layout, DEVICE)
    refs = sdpa_ref.prefill_reference(qs, ks, vs, QH, KVH, causal)
    outs = run_prefill(layout, qs, ks, vs, causal)
    for b in range(4):
        assert_close_both(outs[b], refs[b], dtype, max(kv_lens), f"seq {b} lq {q_lens[b]} lkv {kv_lens[b]}",
                          strict=PREFILL_F32_STRICT if dtype == torch.float32 else None)


@pytest.mark.parametrize("layout", ["dense", "paged", "ragged"])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("dtype", DTYPES, ids=DTYPE_IDS)
@pytest.mark.parametrize("D", [64, 128])
def test_attention_multi_tile(layout, causal, dtype, D):
    """Sequences spanning several 128-row tiles (and an odd number of them), GQA 8/2."""
    QH, KVH = 8, 2
    rng, gen = make_rngs("prefill-multi", layout, causal, dtype, D)
    lens = [300, 300, 300] if layout == "dense" else [513, 129, 700]
    qs = [torch.randn((n, QH, D), generator=gen).to(dtype).to(DEVICE) for n in lens]
    ks = [torch.randn((n, KVH, D), generator=gen).to(dtype).to(DEVICE) for n in lens]
    vs = [torch.randn((n, KVH, D), generator=gen).to(dtype).to(DEVICE) for n in lens]
    refs = sdpa_ref.prefill_reference(qs, ks, vs, QH, KVH, causal)
    outs = run_prefill(layout, qs, ks, vs, causal, permute=4, poison=float("nan"), pad=-1, index_dtype=torch.int64)
    for b in range(3):
        assert torch.isfinite(outs[b].float()).all()
        assert_close_both(outs[b], refs[b], dtype, max(lens), f"seq {b}",
                          strict=PREFILL_F32_STRICT if dtype == torch.float32 else None)


@pytest.mark.parametrize("dtype", HALF_DTYPES, ids=["fp16", "bf16"])
def test_attention_cross_long_kv(dtype):
    """Few query rows against a long KV (cross attention), non-causal."""
    QH, KVH, D = 8, 2, 128
    gen = torch.Generator().manual_seed(77)
    qs = [torch.randn((n, QH, D), generator=gen).to(dtype).to(DEVICE) for n in (5, 140)]
    ks = [torch.randn((n, KVH, D), generator=gen).to(dtype).to(DEVICE) for n in (1500, 999)]
    vs = [torch.randn((n, KVH, D), generator=gen).to(dtype).to(DEVICE) for n in (1500, 999)]
    refs = sdpa_ref.prefill_reference(qs, ks, vs, QH, KVH, False)
    for layout in ("ragged", "paged"):
        outs = run_prefill(layout, qs, ks, vs, False, permute=8, poison=float("nan"), pad=-1)
        for b in range(2):
            assert_close_both(outs[b], refs[b], dtype, 1500, f"{layout} seq {b}")


def test_attention_known_answers():
    from kernels.attention import flash_attention_v2

    gen = torch.Generator().manual_seed(2)
    q = torch.randn((1, 8, 200, 64), generator=gen).to(torch.bfloat16).to(DEVICE)
    k = torch.randn((1, 2, 200, 64), generator=gen).to(torch.bfloat16).to(DEVICE)
    v = torch.randn((1, 2, 200, 64), generator=gen).to(torch.bfloat16).to(DEVICE)
    out = flash_attention_v2(q, k, v, is_causal=True)
    # causal row 0 sees only key 0
    assert torch.equal(out[0, :, 0, :], v[0, :, 0, :].repeat_interleave(4, dim=0))
    # uniform V -> every output row equals that V row
    row = torch.randn((1, 2, 1, 64), generator=gen).to(torch.bfloat16).to(DEVICE)
    out2 = flash_attention_v2(q, k, row.expand(1, 2, 200, 64).contiguous(), is_causal=False)
    torch.testing.assert_close(out2.float(), row.repeat_interleave(4, dim=1).expand(1, 8, 200, 64).float(), atol=8e-3, rtol=8e-3)


def test_flash_attention_v1_alias():
    from kernels import flash_attention_v1, flash_attention_v2

    gen = torch.Generator().manual_seed(4)
    q = torch.randn((2, 8, 70, 64), generator=gen).to(torch.float16).to(DEVICE)
    k = torch.randn((2, 2, 70, 64), generator=gen).to(torch.float16).to(DEVICE)
    v = torch.randn((2, 2, 70, 64), generator=gen).to(torch.float16).to(DEVICE)
    assert torch.equal(flash_attention_v1(q, k, v, is_causal=True), flash_attention_v2(q, k, v, is_causal=True))


def test_attention_page_sizes():
    for page in (8, 32, 48, 128, 256):
        QH, KVH = 8, 2
        rng, gen = make_rngs("prefill-page", page)
        qs, ks, vs, q_lens, kv_lens = prefill_sequences(rng, gen, 3, QH, KVH, 64, "self", torch.float16, "paged", DEVICE,
                                                        max_q=300)
        refs = sdpa_ref.prefill_reference(qs, ks, vs, QH, KVH, True)
        outs = run_prefill("paged", qs, ks, vs, True, permute=6, poison=float("nan"), pad=-1, page_size=page)
        for b in range(3):
            assert_close_both(outs[b], refs[b], torch.float16, max(kv_lens), f"page {page} seq {b}")


def test_attention_validation_errors():
    from kernels.attention import flash_attention_v2

    q = torch.zeros((2, 8, 16, 64), device=DEVICE, dtype=torch.float16)
    k = torch.zeros((2, 2, 16, 64), device=DEVICE, dtype=torch.float16)
    with pytest.raises(AssertionError):
        flash_attention_v2(q, k, k.float())
    with pytest.raises(AssertionError):
        flash_attention_v2(q, k[:, :1].expand(2, 3, 16, 64).contiguous(), k[:, :1].expand(2, 3, 16, 64).contiguous())
    with pytest.raises(AssertionError):
        flash_attention_v2(q[0], k, k)
    with pytest.raises(AssertionError):
        flash_attention_v2(q.cpu(), k.cpu(), k.cpu())
