"""GPU parity tests for decode_attention.  The parametrisation mirrors the reference's
tests/test_decode.py:133-244 (3 layouts x 3 head topologies x 3 dtypes, B=4, D=64) with seeded
inputs, then adds what the reference never exercises: permuted and distinct K/V block tables,
-1 table padding, NaN-poisoned page tails, int32/int64 index tensors, D=128, long split sequences."""
import pytest
import torch

from helpers import DTYPE_IDS, DTYPES, TOPOLOGIES, assert_close_both, decode_sequences, make_rngs
from oracle import sdpa_ref

pytestmark = pytest.mark.gpu
DEVICE = "cuda"
PAGE_SIZE = 16


def run_decode(layout, qs, ks, vs, kv_lens, *, index_dtype=torch.int32, permute=None, poison=None, pad=0,
               page_size=PAGE_SIZE):
    from kernels.decode import decode_attention

    B = len(qs)
    q = torch.stack(qs)
    if layout == "dense":
        KVH, D = ks[0].shape[1], ks[0].shape[2]
        n = max(kv_lens)
        k = torch.zeros((B, KVH, n, D), device=DEVICE, dtype=q.dtype)
        v = torch.zeros_like(k)
        for b in range(B):
            k[b, :, : kv_lens[b]] = ks[b].transpose(0, 1)
            v[b, :, : kv_lens[b]] = vs[b].transpose(0, 1)
        return decode_attention(q, k, v)
    if layout == "ragged":
        k, indptr = sdpa_ref.pack_ragged(ks, index_dtype)
        v, _ = sdpa_ref.pack_ragged(vs, index_dtype)
        return decode_attention(q, k, v, kv_indptr=indptr)
    kc, kt, lens = sdpa_ref.pack_paged(ks, page_size, permute_seed=permute, extra_pages=3 if permute is not None else 0,
                                       pad_value=pad, poison=poison)
    vc, vt, _ = sdpa_ref.pack_paged(vs, page_size, permute_seed=None if permute is None else permute + 1,
                                    extra_pages=3 if permute is not None else 0, pad_value=pad, poison=poison)
    return decode_attention(q, kc, vc, kv_indptr=lens.to(index_dtype), k_block_table=kt, v_block_table=vt,
                            kv_page_size=page_size)


@pytest.mark.parametrize("layout", ["dense", "ragged", "paged"])
@pytest.mark.parametrize("topology", list(TOPOLOGIES))
@pytest.mark.parametrize("dtype", DTYPES, ids=DTYPE_IDS)
def test_decode_reference_grid(layout, topology, dtype):
    QH, KVH = TOPOLOGIES[topology]
    rng, gen = make_rngs("decode", layout, topology, dtype)
    qs, ks, vs, kv_lens = decode_sequences(rng, gen, 4, QH, KVH, 64, dtype, layout, DEVICE)
    refs = sdpa_ref.decode_reference(qs, ks, vs, QH, KVH)
    out = run_decode(layout, qs, ks, vs, kv_lens)
    for b in range(4):
        assert_close_both(out[b], refs[b], dtype, max(kv_lens), f"seq {b} len {kv_lens[b]}")


@pytest.mark.parametrize("dtype", DTYPES, ids=DTYPE_IDS)
@pytest.mark.parametrize("index_dtype", [torch.int32, torch.int64], ids=["i32", "i64"])
def test_decode_paged_hostile_cache(dtype, index_dtype):
    """Random page permutation, K table != V table, -1 padding, NaN in every unused slot."""
    QH, KVH = 8, 2
    rng, gen = make_rngs("decode-hostile", dtype, index_dtype)
    qs, ks, vs, kv_lens = decode_sequences(rng, gen, 5, QH, KVH, 64, dtype, "paged", DEVICE)
    refs = sdpa_ref.decode_reference(qs, ks, vs, QH, KVH)
    out = run_decode("paged", qs, ks, vs, kv_lens, index_dtype=index_dtype, permute=11, poison=float("nan"), pad=-1)
    assert torch.isfinite(out.float()).all()
    for b in range(5):
        assert_close_both(out[b], refs[b], dtype, max(kv_lens), f"seq {b}")


@pytest.mark.parametrize("index_dtype", [torch.int32, torch.int64], ids=["i32", "i64"])
def test_decode_ragged_index_width(index_dtype):
    rng, gen = make_rngs("decode-ragged-width", index_dtype)
    qs, ks, vs, kv_lens = decode_sequences(rng, gen, 6, 8, 2, 64, torch.bfloat16, "ragged", DEVICE)
    refs = sdpa_ref.decode_reference(qs, ks, vs, 8, 2)
    out = run_decode("ragged", qs, ks, vs, kv_lens, index_dtype=index_dtype)
    for b in range(6):
        assert_close_both(out[b], refs[b], torch.bfloat16, max(kv_lens))


@pytest.mark.parametrize("dtype", DTYPES, ids=DTYPE_IDS)
@pytest.mark.parametrize("layout", ["dense", "ragged", "paged"])
def test_decode_head_dim_128_long(dtype, layout):
    """D=128, GQA 32/8, lengths long enough that sequences split into several KV chunks (merge path)."""
    QH, KVH, B = 32, 8, 3
    rng, gen = make_rngs("decode-128", dtype, layout)
    lens = [3000, 3000, 3000] if layout == "dense" else [4097, 130, 2511]
    qs = [torch.randn((QH, 128), generator=gen).to(dtype).to(DEVICE) for _ in range(B)]
    ks = [torch.randn((n, KVH, 128), generator=gen).to(dtype).to(DEVICE) for n in lens]
    vs = [torch.randn((n, KVH, 128), generator=gen).to(dtype).to(DEVICE) for n in lens]
    refs = sdpa_ref.decode_reference(qs, ks, vs, QH, KVH)
    out = run_decode(layout, qs, ks, vs, lens, permute=5, poison=float("nan"), pad=-1)
    for b in range(B):
        assert_close_both(out[b], refs[b], dtype, max(lens), f"seq {b}")


def test_decode_known_answers():
    from kernels.decode import decode_attention

    gen = torch.Generator().manual_seed(1)
    q = torch.randn((2, 8, 64), generator=gen).to(torch.bfloat16).to(DEVICE)
    # single key -> v0
    k = torch.randn((2, 2, 1, 64), generator=gen).to(torch.bfloat16).to(DEVICE)
    v = torch.randn((2, 2, 1, 64), generator=gen).to(torch.bfloat16).to(DEVICE)
    out = decode_attention(q, k, v)
    assert torch.equal(out, v[:, :, 0, :].repeat_interleave(4, dim=1))
    # uniform V rows -> that row (up to rounding of the normalisation)
    k2 = torch.randn((2, 2, 300, 64), generator=gen).to(torch.bfloat16).to(DEVICE)
    row = torch.randn((2, 2, 1, 64), generator=gen).to(torch.bfloat16).to(DEVICE)
    out2 = decode_attention(q, k2, row.expand(2, 2, 300, 64).contiguous())
    torch.testing.assert_close(out2.float(), row[:, :, 0, :].repeat_interleave(4, dim=1).float(), atol=8e-3, rtol=8e-3)


def test_decode_page_sizes():
    """Page sizes other than 16, including a non-power-of-two one."""
    for page in (1, 8, 24, 64, 256):
        rng, gen = make_rngs("decode-page", page)
        qs, ks, vs, kv_lens = decode_sequences(rng, gen, 3, 8, 2, 64, torch.float16, "paged", DEVICE, max_kv=300)
        refs = sdpa_ref.decode_reference(qs, ks, vs, 8, 2)
        out = run_decode("paged", qs, ks, vs, kv_lens, permute=2, poison=float("nan"), pad=-1, page_size=page)
        for b in range(3):
            assert_close_both(out[b], refs[b], torch.float16, max(kv_lens), f"page {page} seq {b}")


def test_decode_out_of_range_page_is_reported_not_dereferenced():
    """A block-table entry outside the cache must not be read; the error word reports it."""
    from kernels import _native
    from kernels.decode import decode_attention

    gen = torch.Generator().manual_seed(3)
    q = torch.randn((1, 8, 64), generator=gen).to(torch.bfloat16).to(DEVICE)
    cache = torch.randn((4 * 16, 2, 64), generator=gen).to(torch.bfloat16).to(DEVICE)
    table = torch.tensor([[0, 1000000, 2]], dtype=torch.int32, device=DEVICE)
    lens = torch.tensor([40], dtype=torch.int32, device=DEVICE)
    out = decode_attention(q, cache, cache, kv_indptr=lens, k_block_table=table, v_block_table=table, kv_page_size=16)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    with pytest.raises(RuntimeError, match="device error"):
        _native.check_device_errors()
    _native.check_device_errors()  # cleared


def test_decode_validation_errors():
    from kernels.decode import decode_attention

    q = torch.zeros((2, 8, 64), device=DEVICE, dtype=torch.float16)
    k = torch.zeros((2, 2, 10, 64), device=DEVICE, dtype=torch.float16)
    with pytest.raises(AssertionError):
        decode_attention(q, k.float(), k)
    with pytest.raises(AssertionError):
        decode_attention(q.cpu(), k.cpu(), k.cpu())
    with pytest.raises(AssertionError):
        decode_attention(q, k, k, k_block_table=torch.zeros((2, 1), dtype=torch.int32, device=DEVICE))
