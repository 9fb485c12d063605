"""Generates tests/golden/attention_golden.pt FROM THE REFERENCE'S OWN TEST-ORACLE FUNCTIONS.

The reference ships no stored vectors; what it has are the pure-torch oracle functions its tests
compare the kernels with.  This script imports those functions from the reference checkout (they run
on CPU once the module-level ``from kernels... import`` resolves, which this build's ``kernels``
package satisfies without a GPU) and records their outputs on small seeded inputs:

  tests/test_attention.py          get_reference_outputs :79-98, allocate_paged_cache :101-134,
                                   attn_tolerances :27-30
  tests/test_decode.py             get_reference_outputs :69-90, allocate_paged_cache :93-130
  tests/test_speculative_decode.py get_reference_outputs :76-126 (appends the draft K/V itself when
                                   causal), allocate_paged_cache :129-166

``tests/test_oracle.py::test_golden_vectors`` then checks ``oracle/sdpa_ref.py`` (the restatement
that travels to the GPU box, where the reference checkout does not exist) against these values.

    python tests/golden/make_golden.py [path-to-reference-checkout]
"""
import importlib.util
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
PKG = os.path.join(ROOT, "triton-kernels_b200")


def load_reference_tests(ref_root):
    """Import the three reference test modules as they stand, with this build's package first on
    the path so that their top-level kernel imports resolve.  DEVICE is pointed at the CPU for the
    fixture builders that allocate on it."""
    if PKG not in sys.path:
        sys.path.insert(0, PKG)
    mods = {}
    for name in ("test_attention", "test_decode", "test_speculative_decode"):
        path = os.path.join(ref_root, "tests", name + ".py")
        spec = importlib.util.spec_from_file_location("reference_" + name, path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.DEVICE = "cpu"
        mods[name] = mod
    return mods


def main():
    # the checkout: first argument, else $B200ATTN_REFERENCE_CHECKOUT, else a directory `reference` beside this repository
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get(
        "B200ATTN_REFERENCE_CHECKOUT", os.path.join(os.path.dirname(ROOT), "reference"))
    ref = load_reference_tests(ref_root)
    t_att, t_dec, t_spec = ref["test_attention"], ref["test_decode"], ref["test_speculative_decode"]

    gen = torch.Generator().manual_seed(20240)
    r = lambda *s: torch.randn(s, generator=gen)
    cases = []
    # prefill: (L, H, D) per sequence, as the reference's generate_sequences builds them
    for qh, kvh, lq, lk, causal, dt in [(8, 2, 21, 21, True, torch.float32), (8, 8, 5, 33, False, torch.float32),
                                        (8, 1, 16, 16, True, torch.float32), (8, 2, 40, 40, True, torch.bfloat16),
                                        (8, 2, 7, 130, False, torch.float16), (32, 8, 9, 9, True, torch.float32)]:
        d = 128 if qh == 32 else 64
        q, k, v = r(lq, qh, d).to(dt), r(lk, kvh, d).to(dt), r(lk, kvh, d).to(dt)
        out = t_att.get_reference_outputs([q], [k], [v], qh, kvh, causal)[0]
        cases.append(dict(kind="prefill", qh=qh, kvh=kvh, causal=causal, q=q, k=k, v=v, out=out))
    # decode: q (H, D)
    for qh, kvh, lk, dt in [(8, 2, 47, torch.float32), (8, 8, 1, torch.float32), (8, 1, 200, torch.bfloat16)]:
        q, k, v = r(qh, 64).to(dt), r(lk, kvh, 64).to(dt), r(lk, kvh, 64).to(dt)
        out = t_dec.get_reference_outputs([q], [k], [v], qh, kvh)[0]
        cases.append(dict(kind="decode", qh=qh, kvh=kvh, causal=False, q=q, k=k, v=v, out=out))
    # speculative decode: q (H, M, D); the reference oracle takes the context K/V and the draft K/V
    # separately and appends the drafts only when causal (tests/test_speculative_decode.py:84-94)
    for qh, kvh, m, lk, causal, dt in [(8, 2, 5, 25, True, torch.float32), (8, 1, 16, 1, True, torch.float32),
                                       (8, 8, 3, 19, False, torch.float32), (8, 2, 2, 77, True, torch.float16),
                                       (8, 2, 10, 33, False, torch.bfloat16)]:
        q, k, v = r(qh, m, 64).to(dt), r(lk, kvh, 64).to(dt), r(lk, kvh, 64).to(dt)
        dk, dv = r(m, kvh, 64).to(dt), r(m, kvh, 64).to(dt)
        out = t_spec.get_reference_outputs([q], [k], [v], [dk], [dv], qh, kvh, causal)[0]
        cases.append(dict(kind="spec", qh=qh, kvh=kvh, causal=causal, q=q, k=k, v=v, dk=dk, dv=dv, out=out))

    # fixture builders: the reference's paged scatter (pages handed out in order, zero cache, zero table)
    paged = []
    for mod, lens in [(t_att, [1, 16, 17, 40]), (t_dec, [33, 5]), (t_spec, [64, 3, 18])]:
        seqs = [r(n, 2, 64) for n in lens]
        cache, table = mod.allocate_paged_cache(seqs, lens, 2, 64, 16)
        paged.append(dict(seqs=seqs, lens=lens, cache=cache, table=table))

    # tolerance rule (identical in the three modules: tests/test_attention.py:27-30, tests/test_decode.py:27-30,
    # tests/test_speculative_decode.py:27-30)
    tol = []
    for dt in (torch.float16, torch.bfloat16, torch.float32):
        for n in (0, 1, 16, 300, 2048):
            vals = [t_att.attn_tolerances(dt, n), t_dec.decode_tolerances(dt, n), t_spec.decode_tolerances(dt, n)]
            assert all(x == vals[0] for x in vals)
            tol.append(dict(dtype=dt, n=n, **vals[0]))

    path = os.path.join(HERE, "attention_golden.pt")
    torch.save(dict(torch_version=str(torch.__version__), source="reference tests' get_reference_outputs",
                    cases=cases, paged=paged, tolerances=tol), path)
    print("wrote", path, os.path.getsize(path), "bytes,", len(cases), "cases")


if __name__ == "__main__":
    main()
