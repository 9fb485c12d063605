"""Generates tests/golden/attention_golden.pt: small seeded inputs with the outputs of the oracle
(fp32 torch scaled_dot_product_attention, the reference tests' own oracle).  The reference ships
no golden vectors, so these pin the oracle against drift (torch upgrades, edits to oracle/).

    python tests/golden/make_golden.py
"""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import sdpa_ref  # noqa: E402


def main():
    gen = torch.Generator().manual_seed(20240)
    r = lambda *s: torch.randn(s, generator=gen)
    cases = []
    for qh, kvh, lq, lk, causal in [(8, 2, 21, 21, True), (8, 8, 5, 33, False), (8, 1, 16, 16, True)]:
        q, k, v = r(lq, qh, 64), r(lk, kvh, 64), r(lk, kvh, 64)
        out = sdpa_ref.prefill_reference([q], [k], [v], qh, kvh, causal)[0]
        cases.append(dict(kind="prefill", qh=qh, kvh=kvh, causal=causal, q=q, k=k, v=v, out=out))
    for qh, kvh, lk in [(8, 2, 47), (8, 8, 1)]:
        q, k, v = r(qh, 64), r(lk, kvh, 64), r(lk, kvh, 64)
        out = sdpa_ref.decode_reference([q], [k], [v], qh, kvh)[0]
        cases.append(dict(kind="decode", qh=qh, kvh=kvh, causal=False, q=q, k=k, v=v, out=out))
    for qh, kvh, m, lk, causal in [(8, 2, 5, 30, True), (8, 1, 16, 16, True), (8, 8, 3, 19, False)]:
        q, k, v = r(qh, m, 64), r(lk, kvh, 64), r(lk, kvh, 64)
        out = sdpa_ref.spec_decode_reference([q], [k], [v], qh, kvh, causal)[0]
        cases.append(dict(kind="spec", qh=qh, kvh=kvh, causal=causal, q=q, k=k, v=v, out=out))
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "attention_golden.pt")
    torch.save(dict(torch_version=str(torch.__version__), cases=cases), path)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
