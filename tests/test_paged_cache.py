"""Paged KV-cache append kernel: bit-exact against the reference fixture's scatter loop restated in
oracle/sdpa_ref.pack_paged (tests/test_attention.py:101-134 of the reference)."""
import pytest
import torch

from oracle import sdpa_ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(dtype, heads, dim, lens, page, seed, index_dtype=torch.int32):
    from kernels import append_paged_kv

    g = torch.Generator().manual_seed(seed)
    seqs = [torch.randn((n, heads, dim), generator=g).to(dtype) for n in lens]
    want, table, _ = sdpa_ref.pack_paged(seqs, page, permute_seed=seed, extra_pages=2, pad_value=-1)
    cache = torch.zeros_like(want).to(DEV)
    src, indptr = sdpa_ref.pack_ragged([s.to(DEV) for s in seqs], index_dtype)
    out = append_paged_kv(cache, table.to(DEV), src, indptr, page)
    assert out.data_ptr() == cache.data_ptr()
    assert torch.equal(cache.cpu().view(torch.uint8), want.view(torch.uint8))
    return seqs, table, cache


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("page", [1, 16, 24, 128])
def test_append_from_scratch_is_bit_exact(dtype, page):
    _case(dtype, 2, 64, [1, 16, 17, 40, 255], page, seed=page)
    _case(dtype, 8, 128, [300, 5], page, seed=page + 1, index_dtype=torch.int64)


def test_append_at_the_tail_like_a_decode_step():
    from kernels import append_paged_kv

    page = 16
    seqs, table, cache = _case(torch.bfloat16, 2, 64, [30, 16, 1], page, seed=9)
    # room for 5 more tokens per sequence: extend the tables with fresh pages
    lens = [30, 16, 1]
    g = torch.Generator().manual_seed(10)
    new = [torch.randn((5, 2, 64), generator=g).to(torch.bfloat16) for _ in lens]
    full = [torch.cat([a, b]) for a, b in zip(seqs, new)]
    want, table2, _ = sdpa_ref.pack_paged(full, page, permute_seed=None, pad_value=-1)
    cache2 = torch.zeros_like(want).to(DEV)
    src_old, ip_old = sdpa_ref.pack_ragged([s.to(DEV) for s in seqs])
    append_paged_kv(cache2, table2.to(DEV), src_old, ip_old, page)
    src_new, ip_new = sdpa_ref.pack_ragged([s.to(DEV) for s in new])
    append_paged_kv(cache2, table2.to(DEV), src_new, ip_new, page, dst_pos=torch.tensor(lens, dtype=torch.int32, device=DEV))
    assert torch.equal(cache2.cpu().view(torch.uint8), want.view(torch.uint8))


def test_out_of_range_table_entry_is_reported_and_skipped():
    from kernels import _native, append_paged_kv

    cache = torch.zeros((4 * 16, 2, 64), dtype=torch.float16, device=DEV)
    table = torch.tensor([[1, 99]], dtype=torch.int32, device=DEV)
    src = torch.ones((20, 2, 64), dtype=torch.float16, device=DEV)
    ip = torch.tensor([0, 20], dtype=torch.int32, device=DEV)
    append_paged_kv(cache, table, src, ip, 16)
    torch.cuda.synchronize()
    assert cache[16:32].eq(1).all() and cache[:16].eq(0).all() and cache[32:].eq(0).all()
    with pytest.raises(RuntimeError, match="device error"):
        _native.check_device_errors()


def test_append_then_decode_roundtrip():
    """Cache built by the append kernel feeds paged decode; result equals the oracle on the source rows."""
    from kernels import append_paged_kv, decode_attention

    g = torch.Generator().manual_seed(3)
    lens = [700, 33, 129]
    ks = [torch.randn((n, 2, 64), generator=g).to(torch.bfloat16).to(DEV) for n in lens]
    vs = [torch.randn((n, 2, 64), generator=g).to(torch.bfloat16).to(DEV) for n in lens]
    qs = [torch.randn((8, 64), generator=g).to(torch.bfloat16).to(DEV) for _ in lens]
    blocks = [(n + 15) // 16 for n in lens]
    perm = torch.randperm(sum(blocks), generator=g).to(torch.int32)
    table = torch.full((3, max(blocks)), -1, dtype=torch.int32)
    cur = 0
    for i, nb in enumerate(blocks):
        table[i, :nb] = perm[cur:cur + nb]
        cur += nb
    table = table.to(DEV)
    kc = torch.full((sum(blocks) * 16, 2, 64), float("nan"), dtype=torch.bfloat16, device=DEV)
    vc = kc.clone()
    ksrc, ip = sdpa_ref.pack_ragged(ks)
    vsrc, _ = sdpa_ref.pack_ragged(vs)
    append_paged_kv(kc, table, ksrc, ip, 16)
    append_paged_kv(vc, table, vsrc, ip, 16)
    out = decode_attention(torch.stack(qs), kc, vc, kv_indptr=torch.tensor(lens, dtype=torch.int32, device=DEV),
                           k_block_table=table, v_block_table=table, kv_page_size=16)
    refs = sdpa_ref.decode_reference(qs, ks, vs, 8, 2)
    for i in range(3):
        torch.testing.assert_close(out[i].float().cpu(), refs[i].cpu(), atol=2e-2, rtol=2e-2)
