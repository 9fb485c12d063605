"""The five benchmark configurations at full size on the GPU.

Parity against the CPU oracle on a sample of the units (the oracle needs seconds per sequence at these sizes)
plus size-independent properties on the whole output: finiteness, row-convexity (every output row lies inside
the per-column min/max of the V rows it may attend to), invariance under a permutation of the physical pages,
and agreement between split and unsplit evaluation of the same sequence."""
import pytest
import torch

from benchmarks import workloads as W
from helpers import assert_close_both
from oracle import sdpa_ref

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")


def test_c1_cpu_reference_shape_on_gpu():
    """The CPU-runnable config (fp32, 8/2 heads, seq 512, D 64, causal) through the GPU entry point."""
    from kernels.attention import flash_attention_v2

    q, k, v = W.c1_cpu_case(0)
    ref = sdpa_ref.prefill_reference([q], [k], [v], 8, 2, True)[0]
    out = flash_attention_v2(q.transpose(0, 1).unsqueeze(0).contiguous().to(DEV), k.transpose(0, 1).unsqueeze(0).contiguous().to(DEV),
                             v.transpose(0, 1).unsqueeze(0).contiguous().to(DEV), is_causal=True)
    assert_close_both(out[0].transpose(0, 1), ref, torch.float32, 512, "c1", strict=4e-3)


def test_c2_dense_causal_prefill_full_size():
    wl = W.c2_dense_prefill(DEV, 0)
    out = wl.run()
    q, k, v = wl.tensors["q"], wl.tensors["k"], wl.tensors["v"]
    assert torch.isfinite(out.float()).all()
    for b in range(2):
        ref = sdpa_ref.prefill_reference([q[b].transpose(0, 1).cpu()], [k[b].transpose(0, 1).cpu()], [v[b].transpose(0, 1).cpu()],
                                         32, 8, True)[0]
        assert_close_both(out[b].transpose(0, 1), ref, torch.bfloat16, 2048, f"c2 batch {b}")
    # causal row 0 of every head is exactly v[0] of its kv head
    assert torch.equal(out[:, :, 0, :], v[:, :, 0, :].repeat_interleave(4, dim=1))


def test_c3_ragged_causal_prefill_full_size():
    wl = W.c3_ragged_prefill(DEV, 0)
    out = wl.run()
    lens = wl.meta["lengths"]
    assert sum(lens) == 39332 and out.shape == (39332, 32, 128)
    assert torch.isfinite(out.float()).all()
    q, k, v = wl.tensors["q"], wl.tensors["k"], wl.tensors["v"]
    ip = [0]
    for n in lens:
        ip.append(ip[-1] + n)
    # oracle on the shortest and on one long sequence (heads 0-7 of the long one to bound CPU time)
    order = sorted(range(len(lens)), key=lambda i: lens[i])
    for i in (order[0], order[-1]):
        a, e = ip[i], ip[i + 1]
        ref = sdpa_ref.prefill_reference([q[a:e, :8].cpu()], [k[a:e, :2].cpu()], [v[a:e, :2].cpu()], 8, 2, True)[0]
        assert_close_both(out[a:e, :8], ref, torch.bfloat16, lens[i], f"c3 seq {i} len {lens[i]}")
    # first row of every sequence sees only its own first key
    for i in range(len(lens)):
        assert torch.equal(out[ip[i]], v[ip[i]].repeat_interleave(4, dim=0))
    # int64 index tensors give the same bits
    wl64 = W.c3_ragged_prefill(DEV, 0, index_dtype=torch.int64)
    assert torch.equal(wl64.run(), out)


def test_c4_paged_decode_full_size():
    wl = W.c4_paged_decode(DEV, 0)
    out = wl.run()
    t, lens = wl.tensors, wl.meta["lengths"]
    assert wl.meta["tokens"] == 275479 and wl.meta["pages"] == 17244
    assert torch.isfinite(out.float()).all()
    ks = [W.gather_paged(t["k_cache"], t["k_table"][i], lens[i], 16) for i in range(64)]
    vs = [W.gather_paged(t["v_cache"], t["v_table"][i], lens[i], 16) for i in range(64)]
    refs = sdpa_ref.decode_reference([t["q"][i].cpu() for i in range(64)], [x.cpu() for x in ks], [x.cpu() for x in vs], 32, 8)
    for i in range(64):
        assert_close_both(out[i], refs[i], torch.bfloat16, lens[i], f"c4 seq {i}")
    # convexity: each output lies within the column-wise range of the V rows of its sequence and head
    for i in (0, 17, 63):
        lo = vs[i].float().amin(dim=0).repeat_interleave(4, dim=0) - 1e-2
        hi = vs[i].float().amax(dim=0).repeat_interleave(4, dim=0) + 1e-2
        assert ((out[i].float() >= lo) & (out[i].float() <= hi)).all()
    # the same logical sequences through the ragged layout give the same result up to rounding of the split merge
    from kernels.decode import decode_attention

    kr, ip = sdpa_ref.pack_ragged(ks)
    vr, _ = sdpa_ref.pack_ragged(vs)
    out_r = decode_attention(t["q"], kr, vr, kv_indptr=ip)
    torch.testing.assert_close(out_r.float(), out.float(), atol=4e-3, rtol=2e-2)


def test_c5_paged_speculative_decode_full_size():
    wl = W.c5_paged_spec_decode(DEV, 0)
    out = wl.run()
    t, lens = wl.tensors, wl.meta["lengths"]
    assert wl.meta["tokens"] == 429958
    assert torch.isfinite(out.float()).all()
    sample = [0, 7, 31]
    ks = {i: W.gather_paged(t["k_cache"], t["k_table"][i], lens[i], 16) for i in sample}
    vs = {i: W.gather_paged(t["v_cache"], t["v_table"][i], lens[i], 16) for i in sample}
    refs = sdpa_ref.spec_decode_reference([t["q"][i].cpu() for i in sample], [ks[i].cpu() for i in sample],
                                          [vs[i].cpu() for i in sample], 64, 8, True)
    for n, i in enumerate(sample):
        assert_close_both(out[i], refs[n], torch.bfloat16, lens[i], f"c5 seq {i}")
    # one KV head per rank (the 8-GPU sharding) reproduces the corresponding q heads bit for bit
    from kernels.speculative_decode import speculative_decode_attention

    h = 3
    out_h = speculative_decode_attention(t["q"][:, h * 8:(h + 1) * 8].contiguous(), t["k_cache"][:, h:h + 1].contiguous(),
                                         t["v_cache"][:, h:h + 1].contiguous(), causal=True, kv_indptr=t["lens"],
                                         k_block_table=t["k_table"], v_block_table=t["v_table"], kv_page_size=16)
    torch.testing.assert_close(out_h.float(), out[:, h * 8:(h + 1) * 8].float(), atol=4e-3, rtol=2e-2)
