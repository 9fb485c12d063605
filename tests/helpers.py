"""Seeded per-sequence generators shared by the GPU parity tests.

They produce what the reference's tests produce with unseeded ``random`` / ``torch.randn``
(tests/test_attention.py:52-77, tests/test_decode.py:49-66, tests/test_speculative_decode.py:52-74)."""
import random

import torch

TOPOLOGIES = {"mha": (8, 8), "gqa": (8, 2), "mqa": (8, 1)}
DTYPES = [torch.float16, torch.bfloat16, torch.float32]
DTYPE_IDS = ["fp16", "bf16", "fp32"]


def seed_for(*parts) -> int:
    return abs(hash(tuple(str(p) for p in parts))) % (2**31)


def stable_seed(*parts) -> int:
    # hash() of str is salted per process; use a simple deterministic mix instead
    s = 0
    for p in parts:
        for ch in str(p):
            s = (s * 131 + ord(ch)) % (2**31 - 1)
    return s


def prefill_sequences(rng, gen, B, QH, KVH, D, attn_type, dtype, layout, device, max_q=128, max_kv=256):
    qs, ks, vs, q_lens, kv_lens = [], [], [], [], []
    fixed_q = rng.randint(16, max_q)
    fixed_kv = fixed_q if attn_type == "self" else rng.randint(16, max_kv)
    for _ in range(B):
        l_q = fixed_q if layout == "dense" else rng.randint(1, max_q)
        if attn_type == "self":
            l_kv = l_q
        else:
            l_kv = fixed_kv if layout == "dense" else rng.randint(1, max_kv)
        q_lens.append(l_q)
        kv_lens.append(l_kv)
        qs.append(torch.randn((l_q, QH, D), generator=gen).to(dtype).to(device))
        ks.append(torch.randn((l_kv, KVH, D), generator=gen).to(dtype).to(device))
        vs.append(torch.randn((l_kv, KVH, D), generator=gen).to(dtype).to(device))
    return qs, ks, vs, q_lens, kv_lens


def decode_sequences(rng, gen, B, QH, KVH, D, dtype, layout, device, M=None, max_kv=256):
    """M is None for decode (q is (QH, D)) or the draft count (q is (QH, M, D))."""
    qs, ks, vs, kv_lens = [], [], [], []
    fixed_kv = rng.randint(16, max_kv)
    for _ in range(B):
        l_kv = fixed_kv if layout == "dense" else rng.randint(1, max_kv)
        kv_lens.append(l_kv)
        qshape = (QH, D) if M is None else (QH, M, D)
        qs.append(torch.randn(qshape, generator=gen).to(dtype).to(device))
        ks.append(torch.randn((l_kv, KVH, D), generator=gen).to(dtype).to(device))
        vs.append(torch.randn((l_kv, KVH, D), generator=gen).to(dtype).to(device))
    return qs, ks, vs, kv_lens


def make_rngs(*parts):
    s = stable_seed(*parts)
    return random.Random(s), torch.Generator().manual_seed(s)


# fp32 prefill multiplies in fp16 on the tensor cores, exactly as the reference kernel does (it casts
# q, k, v and p to fp16 whatever the input dtype: kernels/attention.py:547,572,594,607,614), so its
# un-scaled bar is the 16-bit class one; fp32 decode uses fp32 FMAs and keeps the 1e-3 bar.
PREFILL_F32_STRICT = 4e-3


def spec_strict(dtype, qh, kvh, m):
    """Un-scaled bar of a speculative-decode call: fp32 inputs with several q rows per head (or more than 16 per KV
    head) are multiplied in fp16 with fp32 accumulation - the ten mantissa bits of the TF32 `tl.dot` the reference
    runs on its fp32 operands (kernels/speculative_decode.py:153,175) - so their bar is the 16-bit class one; every
    other case keeps the bar of its dtype."""
    return PREFILL_F32_STRICT if dtype == torch.float32 and (m > 1 or (qh // kvh) * m > 16) else None


def assert_close_both(out, ref, dtype, n_kv, what="", strict=None):
    """The reference tolerance (atol = base*sqrt(N)+eps, rtol) and the stricter un-scaled max-abs bar
    (bf16 2e-2, fp16 1e-2, fp32 1e-3 unless `strict` overrides it)."""
    from oracle.sdpa_ref import attn_tolerances, strict_max_abs

    out = out.float().cpu()
    ref = ref.float().cpu()
    torch.testing.assert_close(out, ref, **attn_tolerances(dtype, n_kv), msg=lambda m: f"{what}: {m}")
    err = (out - ref).abs().max().item() if out.numel() else 0.0
    bar = strict if strict is not None else strict_max_abs(dtype)
    assert err <= bar, f"{what}: max-abs {err:.3e} exceeds strict bar {bar:.1e}"
