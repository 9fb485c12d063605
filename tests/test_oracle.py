"""CPU tests of the oracle itself: SDPA restatement vs the fp64 numpy formula, analytic
known-answer cases, and the committed golden vectors."""
import os

import numpy as np
import pytest
import torch

from oracle import sdpa_ref, softmax_ref

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "attention_golden.pt")


def _rand(gen, *shape):
    return torch.randn(shape, generator=gen)


@pytest.mark.parametrize("qh,kvh", [(8, 8), (8, 2), (8, 1)])
@pytest.mark.parametrize("causal", [False, True])
def test_prefill_oracle_matches_fp64(qh, kvh, causal):
    gen = torch.Generator().manual_seed(qh * 10 + kvh + causal)
    lq = 37
    lk = 37 if causal else 53
    q, k, v = _rand(gen, lq, qh, 64), _rand(gen, lk, kvh, 64), _rand(gen, lk, kvh, 64)
    ref = sdpa_ref.prefill_reference([q], [k], [v], qh, kvh, causal)[0]
    mask = softmax_ref.causal_top_left(lq, lk) if causal else None
    f64 = softmax_ref.attention_f64(q.transpose(0, 1).numpy(), k.transpose(0, 1).numpy(), v.transpose(0, 1).numpy(), mask=mask)
    np.testing.assert_allclose(ref.transpose(0, 1).numpy(), f64, atol=2e-6, rtol=1e-5)


@pytest.mark.parametrize("qh,kvh", [(8, 8), (8, 2), (8, 1)])
def test_decode_oracle_matches_fp64(qh, kvh):
    gen = torch.Generator().manual_seed(3 + kvh)
    q, k, v = _rand(gen, qh, 64), _rand(gen, 91, kvh, 64), _rand(gen, 91, kvh, 64)
    ref = sdpa_ref.decode_reference([q], [k], [v], qh, kvh)[0]
    f64 = softmax_ref.attention_f64(q[:, None, :].numpy(), k.transpose(0, 1).numpy(), v.transpose(0, 1).numpy())
    np.testing.assert_allclose(ref.numpy(), f64[:, 0, :], atol=2e-6, rtol=1e-5)


@pytest.mark.parametrize("m", [1, 2, 5, 16])
@pytest.mark.parametrize("causal", [False, True])
def test_spec_oracle_matches_fp64(m, causal):
    gen = torch.Generator().manual_seed(100 + m)
    qh, kvh, lk = 8, 2, 40 + m
    q, k, v = _rand(gen, qh, m, 64), _rand(gen, lk, kvh, 64), _rand(gen, lk, kvh, 64)
    ref = sdpa_ref.spec_decode_reference([q], [k], [v], qh, kvh, causal)[0]
    mask = softmax_ref.draft_tail_mask(m, lk) if causal else None
    f64 = softmax_ref.attention_f64(q.numpy(), k.transpose(0, 1).numpy(), v.transpose(0, 1).numpy(), mask=mask)
    np.testing.assert_allclose(ref.numpy(), f64, atol=2e-6, rtol=1e-5)


def test_draft_mask_rule_matches_reference_rule():
    # tests/test_speculative_decode.py:113-114 vs kernels/speculative_decode.py:155-160
    for m, n in [(1, 1), (3, 3), (4, 20), (16, 16), (16, 300)]:
        a = sdpa_ref.draft_mask(m, n).numpy()
        b = softmax_ref.draft_tail_mask(m, n)
        assert (a == b).all()


def test_known_answers():
    gen = torch.Generator().manual_seed(7)
    # single key: output is v0 whatever q is
    q, k, v = _rand(gen, 4, 8, 64), _rand(gen, 1, 2, 64), _rand(gen, 1, 2, 64)
    out = sdpa_ref.prefill_reference([q], [k], [v], 8, 2, False)[0]
    torch.testing.assert_close(out, v.repeat_interleave(4, dim=1).expand(4, 8, 64))
    # uniform V rows: output equals that row
    k2 = _rand(gen, 19, 2, 64)
    v2 = _rand(gen, 1, 2, 64).expand(19, 2, 64).contiguous()
    out2 = sdpa_ref.decode_reference([q[0]], [k2], [v2], 8, 2)[0]
    torch.testing.assert_close(out2, v2[0].repeat_interleave(4, dim=0), atol=1e-6, rtol=1e-6)
    # causal row 0 sees only key 0
    q3, k3, v3 = _rand(gen, 9, 8, 64), _rand(gen, 9, 8, 64), _rand(gen, 9, 8, 64)
    out3 = sdpa_ref.prefill_reference([q3], [k3], [v3], 8, 8, True)[0]
    torch.testing.assert_close(out3[0], v3[0])
    # zero q: uniform softmax -> mean of V
    out4 = sdpa_ref.decode_reference([torch.zeros(8, 64)], [k3], [v3], 8, 8)[0]
    torch.testing.assert_close(out4, v3.mean(dim=0), atol=1e-6, rtol=1e-6)


def test_lse_merge_equals_unsplit():
    rng = np.random.default_rng(0)
    q = rng.standard_normal((3, 5, 64))
    k = rng.standard_normal((3, 200, 64))
    v = rng.standard_normal((3, 200, 64))
    full = softmax_ref.attention_f64(q, k, v)
    for h in range(3):
        ms, ls, accs = [], [], []
        for a, b in [(0, 64), (64, 64), (64, 200)]:  # one empty split
            s = (q[h] @ k[h, a:b].T) / 8.0
            if b > a:
                m = s.max(axis=1)
                p = np.exp(s - m[:, None])
                ms.append(m); ls.append(p.sum(axis=1)); accs.append(p @ v[h, a:b])
            else:
                ms.append(np.full(5, -np.inf)); ls.append(np.zeros(5)); accs.append(np.zeros((5, 64)))
        merged = softmax_ref.lse_merge_f64(ms, ls, accs)
        np.testing.assert_allclose(merged, full[h], atol=1e-12, rtol=1e-10)


def test_packers_roundtrip():
    gen = torch.Generator().manual_seed(5)
    seqs = [_rand(gen, n, 2, 64) for n in (1, 16, 17, 40)]
    cache, table, lens = sdpa_ref.pack_paged(seqs, 16, permute_seed=3, extra_pages=2, pad_value=-1, poison=float("nan"))
    assert lens.tolist() == [1, 16, 17, 40]
    for i, s in enumerate(seqs):
        nb = (s.shape[0] + 15) // 16
        rows = torch.cat([cache[int(p) * 16: int(p) * 16 + 16] for p in table[i, :nb]])[: s.shape[0]]
        assert torch.equal(rows, s)
        assert (table[i, nb:] == -1).all()
    packed, indptr = sdpa_ref.pack_ragged(seqs, torch.int64)
    assert indptr.tolist() == [0, 1, 17, 34, 74] and packed.shape[0] == 74


def test_golden_vectors():
    """The committed fixtures hold outputs of the REFERENCE's own oracle functions (its tests'
    get_reference_outputs, imported from the reference checkout by tests/golden/make_golden.py);
    the restatement in oracle/sdpa_ref.py must reproduce them."""
    blob = torch.load(GOLDEN)
    assert blob["source"] == "reference tests' get_reference_outputs"
    kinds = [c["kind"] for c in blob["cases"]]
    assert kinds.count("prefill") >= 3 and kinds.count("decode") >= 2 and kinds.count("spec") >= 3
    for case in blob["cases"]:
        kind = case["kind"]
        if kind == "prefill":
            out = sdpa_ref.prefill_reference([case["q"]], [case["k"]], [case["v"]], case["qh"], case["kvh"], case["causal"])[0]
        elif kind == "decode":
            out = sdpa_ref.decode_reference([case["q"]], [case["k"]], [case["v"]], case["qh"], case["kvh"])[0]
        else:
            k, v = case["k"], case["v"]
            if case["causal"]:
                # the reference oracle appends the draft K/V itself (tests/test_speculative_decode.py:84-94);
                # the restatement takes what the kernel sees: K/V with the drafts already at the tail
                k, v = torch.cat([k, case["dk"]]), torch.cat([v, case["dv"]])
            out = sdpa_ref.spec_decode_reference([case["q"]], [k], [v], case["qh"], case["kvh"], case["causal"])[0]
        assert out.dtype == case["out"].dtype == torch.float32 and out.shape == case["out"].shape
        torch.testing.assert_close(out, case["out"], atol=1e-5, rtol=1e-5)


def test_golden_paged_fixture_and_tolerances():
    """pack_paged with its defaults is the reference fixture's scatter (tests/test_attention.py:101-134,
    tests/test_decode.py:93-130, tests/test_speculative_decode.py:129-166) bit for bit, and
    attn_tolerances is the reference's rule (tests/test_attention.py:27-30)."""
    blob = torch.load(GOLDEN)
    assert len(blob["paged"]) == 3
    for fx in blob["paged"]:
        cache, table, lens = sdpa_ref.pack_paged(fx["seqs"], 16)
        assert lens.tolist() == fx["lens"]
        assert torch.equal(cache, fx["cache"]) and torch.equal(table, fx["table"])
    assert len(blob["tolerances"]) == 15
    for t in blob["tolerances"]:
        got = sdpa_ref.attn_tolerances(t["dtype"], t["n"])
        assert got == dict(atol=t["atol"], rtol=t["rtol"])


def test_c1_cpu_config_runs():
    from benchmarks.workloads import c1_cpu_case

    q, k, v = c1_cpu_case(0)
    out = sdpa_ref.prefill_reference([q], [k], [v], 8, 2, True)[0]
    f64 = softmax_ref.attention_f64(q.transpose(0, 1).numpy(), k.transpose(0, 1).numpy(), v.transpose(0, 1).numpy(),
                                    mask=softmax_ref.causal_top_left(512, 512))
    np.testing.assert_allclose(out.transpose(0, 1).numpy(), f64, atol=5e-6, rtol=1e-5)


@pytest.mark.parametrize("shape", [(7,), (5, 33), (3, 4, 129)])
@pytest.mark.parametrize("log", [False, True])
def test_row_softmax_oracle_matches_torch_and_split(shape, log):
    """The row-softmax restatement against the reference tests' own oracle (torch's softmax / log_softmax) and
    against the split-and-merge form the long-row kernels use."""
    import numpy as np
    from oracle import softmax_ref

    x = torch.randn(shape, generator=torch.Generator().manual_seed(len(shape)), dtype=torch.float64) * 5
    want = (torch.log_softmax if log else torch.softmax)(x, dim=-1).numpy()
    got = softmax_ref.row_softmax_f64(x.numpy(), log=log)
    np.testing.assert_allclose(got, want, rtol=1e-12, atol=1e-14)
    split = softmax_ref.row_softmax_split_f64(x.numpy(), 3, log=log)
    np.testing.assert_allclose(split, want, rtol=1e-12, atol=1e-13)
    # known answers: a constant row is uniform, a dominant entry takes everything
    u = softmax_ref.row_softmax_f64(np.full((4,), 2.5))
    np.testing.assert_allclose(u, np.full((4,), 0.25))
    d = softmax_ref.row_softmax_f64(np.array([0.0, 800.0, -3.0]))
    np.testing.assert_allclose(d, np.array([0.0, 1.0, 0.0]), atol=1e-300)
