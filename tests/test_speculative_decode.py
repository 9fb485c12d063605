"""GPU parity tests for speculative_decode_attention.  Mirrors the reference's
tests/test_speculative_decode.py:169-332 (causal x M x layout x topology x dtype, B=4, D=64) with
seeded inputs; in causal mode the M draft K/V rows are appended to each sequence and the length
passed to the kernel includes them (:202-224, :242-251, :280-289)."""
import pytest
import torch

from helpers import DTYPE_IDS, DTYPES, TOPOLOGIES, assert_close_both, decode_sequences, make_rngs, spec_strict
from oracle import sdpa_ref

pytestmark = pytest.mark.gpu
DEVICE = "cuda"
PAGE_SIZE = 16
M_VALUES = [2, 3, 4, 6, 8, 10, 12, 16]


def run_spec(layout, qs, ks, vs, causal, *, index_dtype=torch.int32, permute=None, poison=None, pad=0,
             page_size=PAGE_SIZE):
    from kernels.speculative_decode import speculative_decode_attention

    B = len(qs)
    q = torch.stack(qs)
    lens = [int(k.shape[0]) for k in ks]
    if layout == "dense":
        KVH, D = ks[0].shape[1], ks[0].shape[2]
        n = max(lens)
        k = torch.zeros((B, KVH, n, D), device=DEVICE, dtype=q.dtype)
        v = torch.zeros_like(k)
        for b in range(B):
            k[b, :, : lens[b]] = ks[b].transpose(0, 1)
            v[b, :, : lens[b]] = vs[b].transpose(0, 1)
        return speculative_decode_attention(q, k, v, causal=causal)
    if layout == "ragged":
        k, indptr = sdpa_ref.pack_ragged(ks, index_dtype)
        v, _ = sdpa_ref.pack_ragged(vs, index_dtype)
        return speculative_decode_attention(q, k, v, kv_indptr=indptr, causal=causal)
    kc, kt, lens_t = sdpa_ref.pack_paged(ks, page_size, permute_seed=permute, extra_pages=2 if permute is not None else 0,
                                         pad_value=pad, poison=poison)
    vc, vt, _ = sdpa_ref.pack_paged(vs, page_size, permute_seed=None if permute is None else permute + 1,
                                    extra_pages=2 if permute is not None else 0, pad_value=pad, poison=poison)
    return speculative_decode_attention(q, kc, vc, kv_indptr=lens_t.to(index_dtype), k_block_table=kt, v_block_table=vt,
                                        kv_page_size=page_size, causal=causal)


def with_drafts(rng, gen, B, QH, KVH, M, D, dtype, layout, causal):
    qs, ks, vs, kv_lens = decode_sequences(rng, gen, B, QH, KVH, D, dtype, layout, DEVICE, M=M)
    if causal:
        ks = [torch.cat([k, torch.randn((M, KVH, D), generator=gen).to(dtype).to(DEVICE)]) for k in ks]
        vs = [torch.cat([v, torch.randn((M, KVH, D), generator=gen).to(dtype).to(DEVICE)]) for v in vs]
    return qs, ks, vs


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("M", M_VALUES)
@pytest.mark.parametrize("layout", ["dense", "ragged", "paged"])
@pytest.mark.parametrize("topology", list(TOPOLOGIES))
@pytest.mark.parametrize("dtype", DTYPES, ids=DTYPE_IDS)
def test_speculative_decode_reference_grid(M, layout, topology, dtype, causal):
    QH, KVH = TOPOLOGIES[topology]
    rng, gen = make_rngs("spec", M, layout, topology, dtype, causal)
    qs, ks, vs = with_drafts(rng, gen, 4, QH, KVH, M, 64, dtype, layout, causal)
    refs = sdpa_ref.spec_decode_reference(qs, ks, vs, QH, KVH, causal)
    out = run_spec(layout, qs, ks, vs, causal)
    n = max(int(k.shape[0]) for k in ks)
    for b in range(4):
        assert_close_both(out[b], refs[b], dtype, n, f"seq {b}", strict=spec_strict(dtype, QH, KVH, M))


@pytest.mark.parametrize("dtype", DTYPES, ids=DTYPE_IDS)
@pytest.mark.parametrize("M", [1, 5, 16])
def test_spec_paged_hostile_cache_d128(dtype, M):
    """The benchmark's shape family: 64/8 heads, D=128, random tables, poisoned tails, long contexts."""
    QH, KVH, B = 64, 8, 2
    rng, gen = make_rngs("spec-hostile", dtype, M)
    lens = [2500 + M, 77 + M]
    qs = [torch.randn((QH, M, 128), generator=gen).to(dtype).to(DEVICE) for _ in range(B)]
    ks = [torch.randn((n, KVH, 128), generator=gen).to(dtype).to(DEVICE) for n in lens]
    vs = [torch.randn((n, KVH, 128), generator=gen).to(dtype).to(DEVICE) for n in lens]
    refs = sdpa_ref.spec_decode_reference(qs, ks, vs, QH, KVH, True)
    out = run_spec("paged", qs, ks, vs, True, permute=9, poison=float("nan"), pad=-1, index_dtype=torch.int64)
    assert torch.isfinite(out.float()).all()
    for b in range(B):
        assert_close_both(out[b], refs[b], dtype, max(lens), f"seq {b}", strict=spec_strict(dtype, QH, KVH, M))


def test_spec_draft_only_context():
    """Sequences that consist of the drafts alone (context length 0): row i sees keys 0..i."""
    M, QH, KVH = 4, 8, 2
    gen = torch.Generator().manual_seed(12)
    qs = [torch.randn((QH, M, 64), generator=gen).to(torch.float16).to(DEVICE) for _ in range(2)]
    ks = [torch.randn((M, KVH, 64), generator=gen).to(torch.float16).to(DEVICE) for _ in range(2)]
    vs = [torch.randn((M, KVH, 64), generator=gen).to(torch.float16).to(DEVICE) for _ in range(2)]
    refs = sdpa_ref.spec_decode_reference(qs, ks, vs, QH, KVH, True)
    for layout in ("dense", "ragged", "paged"):
        out = run_spec(layout, qs, ks, vs, True)
        for b in range(2):
            assert_close_both(out[b], refs[b], torch.float16, M, layout)
        # row 0 of every head sees exactly key 0
        assert torch.equal(out[0][:, 0, :], vs[0][0].repeat_interleave(QH // KVH, dim=0))


def test_spec_m_too_large_rejected():
    from kernels.speculative_decode import speculative_decode_attention

    q = torch.zeros((1, 8, 17, 64), device=DEVICE, dtype=torch.float16)
    k = torch.zeros((1, 2, 32, 64), device=DEVICE, dtype=torch.float16)
    with pytest.raises(AssertionError):
        speculative_decode_attention(q, k, k)


@pytest.mark.parametrize("qh,kvh,m", [(32, 1, 5), (24, 1, 16), (64, 2, 6)], ids=["mqa32x5=160rows", "mqa24x16=384rows", "gqa32x6=192rows"])
@pytest.mark.parametrize("layout", ["ragged", "paged"])
def test_spec_more_than_128_rows_per_kv_head(qh, kvh, m, layout):
    """Any head ratio with M <= 16 is legal in the reference (kernels/speculative_decode.py:262-299); group x M beyond
    the 128 rows one CTA holds is served by several launches over the same K/V."""
    dtype = torch.bfloat16
    rng, gen = make_rngs("spec-wide", qh, kvh, m, layout)
    lens = [700, 90, 2300]
    qs = [torch.randn((qh, m, 128), generator=gen).to(dtype).to(DEVICE) for _ in lens]
    ks = [torch.randn((n + m, kvh, 128), generator=gen).to(dtype).to(DEVICE) for n in lens]
    vs = [torch.randn((n + m, kvh, 128), generator=gen).to(dtype).to(DEVICE) for n in lens]
    refs = sdpa_ref.spec_decode_reference(qs, ks, vs, qh, kvh, True)
    out = run_spec(layout, qs, ks, vs, True, permute=7, pad=-1, poison=float("nan"))
    for b in range(len(lens)):
        assert_close_both(out[b], refs[b], dtype, lens[b] + m, f"seq {b}")


@pytest.mark.parametrize("qh,kvh,m", [(64, 8, 5), (64, 8, 16), (16, 8, 3)], ids=["40rows", "128rows", "6rows-warp-kernel"])
@pytest.mark.parametrize("layout", ["ragged", "paged"])
def test_spec_several_units_per_cta(qh, kvh, m, layout):
    """More sequences than one wave of CTAs holds and uneven lengths: the planner stays with several waves, so a CTA
    of the persistent tcgen05 kernel works through several (item, kv head) units, some of them chunks of a split
    sequence whose merge is claimed in a teardown, others whole short sequences written directly (2, 4 and 1 softmax
    warps; the 6-row case runs the one-CTA-per-unit warp-level kernel over the same plan)."""
    from kernels import _native
    from utils.launch_config import decode_items, decode_plan

    dtype = torch.bfloat16
    rng, gen = make_rngs("spec-units", qh, kvh, m, layout)
    lens = [rng.choice([60, 300, 1500, 4000, 9000]) + rng.randint(0, 63) for _ in range(60)]
    info = _native.device_info(torch.cuda.current_device())
    plan = decode_plan(info.sm_count, len(lens), qh, kvh, m)
    items = decode_items(plan, [n + m for n in lens])
    assert sum(items) * kvh > 2 * info.sm_count and max(items) > 1      # several rounds, split sequences
    qs = [torch.randn((qh, m, 64), generator=gen).to(dtype).to(DEVICE) for _ in lens]
    ks = [torch.randn((n + m, kvh, 64), generator=gen).to(dtype).to(DEVICE) for n in lens]
    vs = [torch.randn((n + m, kvh, 64), generator=gen).to(dtype).to(DEVICE) for n in lens]
    refs = sdpa_ref.spec_decode_reference(qs, ks, vs, qh, kvh, True)
    out = run_spec(layout, qs, ks, vs, True, permute=11, pad=-1, poison=float("nan"))
    assert torch.isfinite(out.float()).all()
    for b in range(len(lens)):
        assert_close_both(out[b], refs[b], dtype, lens[b] + m, f"seq {b} len {lens[b]}")
    # the same call again on the same workspace: tickets and the ready count were left clean
    out2 = run_spec(layout, qs, ks, vs, True, permute=11, pad=-1, poison=float("nan"))
    assert torch.equal(out, out2)


@pytest.mark.parametrize("page", [1, 8, 24, 64, 256])
@pytest.mark.parametrize("qh,kvh,m", [(64, 8, 5), (8, 2, 3)], ids=["tcgen05-40rows", "warp-kernel-12rows"])
def test_spec_page_sizes(page, qh, kvh, m):
    """Page sizes other than 16 under both tensor-core kernels: one key per page (more boxes per tile than lanes, no
    table read-ahead), a non-power-of-two size, pages larger than a tile; sequences long enough for several tiles and
    a split."""
    dtype = torch.bfloat16
    rng, gen = make_rngs("spec-page", page, qh, kvh, m)
    lens = [rng.randint(1, 700) for _ in range(5)] + [2300]
    qs = [torch.randn((qh, m, 64), generator=gen).to(dtype).to(DEVICE) for _ in lens]
    ks = [torch.randn((n + m, kvh, 64), generator=gen).to(dtype).to(DEVICE) for n in lens]
    vs = [torch.randn((n + m, kvh, 64), generator=gen).to(dtype).to(DEVICE) for n in lens]
    refs = sdpa_ref.spec_decode_reference(qs, ks, vs, qh, kvh, True)
    out = run_spec("paged", qs, ks, vs, True, permute=13, pad=-1, poison=float("nan"), page_size=page)
    assert torch.isfinite(out.float()).all()
    for b in range(len(lens)):
        assert_close_both(out[b], refs[b], dtype, lens[b] + m, f"page {page} seq {b}")
