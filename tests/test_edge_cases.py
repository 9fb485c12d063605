"""Edge cases the reference never exercises: empty sequences, very many short sequences (device-side planner and
work search beyond one warp / one thread block of sequences), lengths around tile and chunk boundaries."""
import pytest
import torch

from helpers import assert_close_both
from oracle import sdpa_ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(gen, shape, dtype=torch.bfloat16):
    return torch.randn(shape, generator=gen).to(dtype).to(DEV)


def test_decode_many_short_sequences_and_empty_ones():
    from kernels.decode import decode_attention

    gen = torch.Generator().manual_seed(21)
    B, QH, KVH, D = 1500, 8, 2, 64
    lens = torch.randint(0, 41, (B,), generator=gen).tolist()
    lens[0] = 0
    lens[-1] = 0
    qs = [_rand(gen, (QH, D)) for _ in range(B)]
    ks = [_rand(gen, (n, KVH, D)) for n in lens]
    vs = [_rand(gen, (n, KVH, D)) for n in lens]
    k, ip = sdpa_ref.pack_ragged(ks)
    v, _ = sdpa_ref.pack_ragged(vs)
    out = decode_attention(torch.stack(qs), k, v, kv_indptr=ip)
    assert torch.isfinite(out.float()).all()
    live = [i for i in range(B) if lens[i] > 0]
    refs = sdpa_ref.decode_reference([qs[i] for i in live], [ks[i] for i in live], [vs[i] for i in live], QH, KVH)
    got = out[live].float().cpu()
    torch.testing.assert_close(got, torch.stack(refs).cpu(), atol=2e-2, rtol=2e-2)
    assert (out[[0, B - 1]] == 0).all()      # empty sequences: defined as zeros here (0/0 in the reference)


def test_prefill_many_short_sequences_and_empty_ones():
    from kernels.attention import flash_attention_v2

    gen = torch.Generator().manual_seed(22)
    B, QH, KVH, D = 300, 8, 2, 64
    lens = torch.randint(0, 50, (B,), generator=gen).tolist()
    lens[3] = 0
    lens[150] = 300
    qs = [_rand(gen, (n, QH, D)) for n in lens]
    ks = [_rand(gen, (n, KVH, D)) for n in lens]
    vs = [_rand(gen, (n, KVH, D)) for n in lens]
    q, ip = sdpa_ref.pack_ragged(qs, torch.int64)
    k, _ = sdpa_ref.pack_ragged(ks, torch.int64)
    v, _ = sdpa_ref.pack_ragged(vs, torch.int64)
    out = flash_attention_v2(q, k, v, is_causal=True, q_indptr=ip, kv_indptr=ip)
    assert torch.isfinite(out.float()).all()
    live = [i for i in range(B) if lens[i] > 0]
    refs = sdpa_ref.prefill_reference([qs[i] for i in live], [ks[i] for i in live], [vs[i] for i in live], QH, KVH, True)
    torch.testing.assert_close(out.float().cpu(), torch.cat(refs).cpu(), atol=2e-2, rtol=2e-2)


def test_prefill_queries_without_keys_give_zeros():
    from kernels.attention import flash_attention_v2

    gen = torch.Generator().manual_seed(23)
    q = _rand(gen, (40, 8, 64))
    k = _rand(gen, (17, 2, 64))
    v = _rand(gen, (17, 2, 64))
    qi = torch.tensor([0, 25, 40], dtype=torch.int32, device=DEV)
    ki = torch.tensor([0, 0, 17], dtype=torch.int32, device=DEV)   # first sequence has no keys
    out = flash_attention_v2(q, k, v, q_indptr=qi, kv_indptr=ki)
    assert (out[:25] == 0).all()
    ref = sdpa_ref.prefill_reference([q[25:]], [k], [v], 8, 2, False)[0]
    assert_close_both(out[25:], ref, torch.bfloat16, 17)


@pytest.mark.parametrize("n", [63, 64, 65, 127, 128, 129, 191, 192, 193, 255, 256, 257])
def test_lengths_around_tile_boundaries(n):
    from kernels.attention import flash_attention_v2
    from kernels.decode import decode_attention
    from kernels.speculative_decode import speculative_decode_attention

    gen = torch.Generator().manual_seed(100 + n)
    QH, KVH, D = 8, 2, 128
    q = _rand(gen, (1, QH, n, D))
    k = _rand(gen, (1, KVH, n, D))
    v = _rand(gen, (1, KVH, n, D))
    ref = sdpa_ref.prefill_reference([q[0].transpose(0, 1)], [k[0].transpose(0, 1)], [v[0].transpose(0, 1)], QH, KVH, True)[0]
    assert_close_both(flash_attention_v2(q, k, v, is_causal=True)[0].transpose(0, 1), ref, torch.bfloat16, n, "prefill")
    qd = _rand(gen, (1, QH, D))
    refd = sdpa_ref.decode_reference([qd[0]], [k[0].transpose(0, 1)], [v[0].transpose(0, 1)], QH, KVH)[0]
    assert_close_both(decode_attention(qd, k, v)[0], refd, torch.bfloat16, n, "decode")
    qs = _rand(gen, (1, QH, 7, D))   # 28 rows per KV head: tcgen05 decode path
    refs = sdpa_ref.spec_decode_reference([qs[0]], [k[0].transpose(0, 1)], [v[0].transpose(0, 1)], QH, KVH, True)[0]
    assert_close_both(speculative_decode_attention(qs, k, v, causal=True)[0], refs, torch.bfloat16, n, "spec")


def test_decode_chunk_boundaries_long_sequence():
    """One long sequence splits into many chunks; lengths one below / at / above a multiple of the chunk size."""
    from kernels.decode import decode_attention

    gen = torch.Generator().manual_seed(31)
    QH, KVH, D = 32, 8, 128
    for n in (8191, 8192, 8193):
        q = _rand(gen, (1, QH, D))
        k = _rand(gen, (1, KVH, n, D))
        v = _rand(gen, (1, KVH, n, D))
        ref = sdpa_ref.decode_reference([q[0]], [k[0].transpose(0, 1)], [v[0].transpose(0, 1)], QH, KVH)[0]
        assert_close_both(decode_attention(q, k, v)[0], ref, torch.bfloat16, n, f"n={n}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("layout", ["dense", "ragged"])
def test_prefill_output_aligned_to_16_bytes_only(monkeypatch, dtype, layout):
    """The C ABI asks for 16-byte alignment; the kernel's 32-byte stores are an option it may only take when the
    output pointer allows.  The entry point's output allocation is replaced by one that starts 16 bytes past a
    32-byte boundary."""
    import kernels.attention as attn
    from kernels.attention import flash_attention_v2

    keep = []

    def offset_empty_like(t):
        raw = torch.empty(t.numel() * t.element_size() + 64, dtype=torch.uint8, device=t.device)
        keep.append(raw)
        start = (-raw.data_ptr()) % 32 + 16
        out = raw[start:start + t.numel() * t.element_size()].view(t.dtype).view(t.shape)
        assert out.data_ptr() % 32 == 16
        return out

    monkeypatch.setattr(attn.torch, "empty_like", offset_empty_like)
    gen = torch.Generator().manual_seed(77)
    QH, KVH, D, n = 8, 2, 128, 300
    if layout == "dense":
        q = _rand(gen, (1, QH, n, D), dtype)
        k = _rand(gen, (1, KVH, n, D), dtype)
        v = _rand(gen, (1, KVH, n, D), dtype)
        out = flash_attention_v2(q, k, v, is_causal=True)
        got = out[0].transpose(0, 1)
        qs, ks, vs = q[0].transpose(0, 1), k[0].transpose(0, 1), v[0].transpose(0, 1)
    else:
        q = _rand(gen, (n, QH, D), dtype)
        k = _rand(gen, (n, KVH, D), dtype)
        v = _rand(gen, (n, KVH, D), dtype)
        ip = torch.tensor([0, n], dtype=torch.int32, device=DEV)
        out = flash_attention_v2(q, k, v, is_causal=True, q_indptr=ip, kv_indptr=ip)
        got, qs, ks, vs = out, q, k, v
    assert out.data_ptr() % 32 == 16
    ref = sdpa_ref.prefill_reference([qs], [ks], [vs], QH, KVH, True)[0]
    from helpers import PREFILL_F32_STRICT
    assert_close_both(got, ref, dtype, n, layout, strict=PREFILL_F32_STRICT if dtype == torch.float32 else None)


def test_two_streams_run_concurrently():
    """Calls on different streams use different workspaces (one per stream) and may overlap on the GPU: the
    persistent prefill kernel's work counters and the decode planner's tables must not be shared between them."""
    from kernels.attention import flash_attention_v2
    from kernels.decode import decode_attention

    gen = torch.Generator().manual_seed(91)
    QH, KVH, D = 8, 2, 128
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    work = []
    for i, st in enumerate(streams):
        n = 700 + 300 * i
        q = _rand(gen, (2, QH, n, D))
        k = _rand(gen, (2, KVH, n, D))
        v = _rand(gen, (2, KVH, n, D))
        qd = _rand(gen, (2, QH, D))
        work.append((st, n, q, k, v, qd))
    torch.cuda.synchronize()
    outs = []
    for rep in range(3):
        outs = []
        for st, n, q, k, v, qd in work:
            with torch.cuda.stream(st):
                outs.append((flash_attention_v2(q, k, v, is_causal=True), decode_attention(qd, k, v)))
    torch.cuda.synchronize()
    for (st, n, q, k, v, qd), (po, do) in zip(work, outs):
        for b in range(2):
            ref = sdpa_ref.prefill_reference([q[b].transpose(0, 1)], [k[b].transpose(0, 1)], [v[b].transpose(0, 1)], QH, KVH, True)[0]
            assert_close_both(po[b].transpose(0, 1), ref, torch.bfloat16, n, "prefill")
            refd = sdpa_ref.decode_reference([qd[b]], [k[b].transpose(0, 1)], [v[b].transpose(0, 1)], QH, KVH)[0]
            assert_close_both(do[b], refd, torch.bfloat16, n, "decode")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [False, True])
def test_prefill_outlier_keys_move_the_exponent_reference(dtype, causal):
    """Keys whose score towers over everything seen so far, planted in the first and in the second 64 keys of a
    128-key tile and in later tiles: the running exponent reference has to jump (by far more than the 2^8 the
    kernel tolerates before it rescales), including between the two halves of one tile, where the first half's P
    is already in tensor memory when the jump comes."""
    from kernels import flash_attention_v2

    gen = torch.Generator().manual_seed(77)
    s, d, qh, kvh = 400, 128, 4, 2
    q = torch.randn((1, qh, s, d), generator=gen)
    k = torch.randn((1, kvh, s, d), generator=gen)
    v = torch.randn((1, kvh, s, d), generator=gen)
    # key t is made parallel to query row r of the first q head of its group, scaled so that the score is ~ +25..+40
    # (log2 domain: 36..58 above a typical score); rows before and after see it or not depending on the mask
    for t, r, gain in [(5, 390, 2.2), (70, 200, 2.6), (100, 300, 3.0), (127, 127, 2.4), (130, 350, 2.8), (200, 399, 3.3),
                       (330, 340, 2.9)]:
        for h in range(kvh):
            k[0, h, t] = q[0, h * (qh // kvh), r] * gain / q[0, h * (qh // kvh), r].norm() * (d ** 0.5)
    q, k, v = q.to(dtype).to(DEV), k.to(dtype).to(DEV), v.to(dtype).to(DEV)
    out = flash_attention_v2(q, k, v, is_causal=causal)
    ref = sdpa_ref.prefill_reference([q[0].transpose(0, 1)], [k[0].transpose(0, 1)], [v[0].transpose(0, 1)], qh, kvh, causal)[0]
    assert torch.isfinite(out.float()).all()
    assert_close_both(out[0].transpose(0, 1), ref, dtype, s, "outlier keys")


@pytest.mark.gpu
@pytest.mark.parametrize("layout", ["dense", "paged"])
@pytest.mark.parametrize("shape", [(1, 8, 2, 128, 2048, False, 128), (1, 8, 8, 128, 4096, False, 64), (2, 4, 1, 200, 1000, False, 128),
                                   (1, 2, 1, 2048, 2048, True, 128), (1, 4, 2, 1100, 1100, True, 64), (3, 2, 2, 128, 1280, False, 128)],
                         ids=["b1-q128-kv2048", "b1-mha-kv4096-d64", "b2-q200-kv1000", "b1-causal-2048", "b1-causal-1100-d64", "b3-kv1280"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32], ids=["bf16", "fp32"])
def test_prefill_few_work_items_split_kv(layout, shape, dtype):
    """Launches with far fewer (query tile, head pair, sequence) items than SMs: the library cuts every sequence's KV
    range into parts that run as work items of their own and merges them by their log-sum-exps (the reference splits KV
    when B x QH < SMs, kernels/attention.py:836-841).  Paged sequences are shorter than the table allows, so some parts
    see no key at all."""
    import ctypes as C

    from kernels import _native
    from test_attention import run_prefill

    b, qh, kvh, lq, lkv, causal, d = shape
    gen = torch.Generator().manual_seed(lq * 7 + lkv + qh)
    qs = [torch.randn((lq, qh, d), generator=gen).to(dtype).to(DEV) for _ in range(b)]
    if layout == "paged" and not causal:
        kv_lens = [max(1, lkv - 300 * i - 77) for i in range(b)]      # shorter than the widest table row
    else:
        kv_lens = [lkv] * b
    ks = [torch.randn((n, kvh, d), generator=gen).to(dtype).to(DEV) for n in kv_lens]
    vs = [torch.randn((n, kvh, d), generator=gen).to(dtype).to(DEV) for n in kv_lens]
    refs = sdpa_ref.prefill_reference(qs, ks, vs, qh, kvh, causal)
    outs = run_prefill(layout, qs, ks, vs, causal, permute=11, pad=-1, poison=float("nan"))
    for i in range(b):
        assert_close_both(outs[i], refs[i], dtype, kv_lens[i], f"seq {i}", strict=4e-3 if dtype == torch.float32 else None)
    # the split really is in play for these shapes: the library asks for room for the parts
    a = _native.PrefillArgs()
    a.dtype, a.layout = _native.DTYPE_CODE[dtype], _native.DENSE
    a.batch, a.q_heads, a.kv_heads, a.max_q, a.max_kv, a.head_dim = b, qh, kvh, lq, lkv, d
    a.device = torch.cuda.current_device()
    assert _native.lib().b200attn_prefill_workspace_bytes(C.byref(a)) > b * qh * lq * d * 2
