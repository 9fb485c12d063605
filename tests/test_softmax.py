"""Row softmax / log-softmax parity (GPU, through the C ABI).

Oracle: torch's softmax / log_softmax on the same input (the reference tests' oracle, tests/test_softmax.py:47,95),
evaluated in float64 on the CPU and rounded to the tensor's dtype, plus the numpy restatement in oracle/softmax_ref.py.
Tolerances are the reference's: ``torch.testing.assert_close`` defaults for the dtype."""
import numpy as np
import pytest
import torch

from oracle import softmax_ref

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float16, torch.bfloat16, torch.float32]

# the reference grid (tests/test_softmax.py:18-40: its small, medium, large and higher-dimensional shapes) ...
REFERENCE_SHAPES = [(1024,), (512,), (32, 1024), (4096,), (64, 2048), (128, 4096), (16, 1025), (8, 3072), (1, 32768),
                    (2, 32768), (4, 20000), (8, 32768), (1, 65536), (1, 131072), (8, 16, 1024), (4, 8, 32, 1024)]
# ... and shapes it never visits: single elements, odd widths (scalar path), rows around the shared-memory and the
# cluster limits (51 200 fp32 / 102 400 16-bit elements per CTA, eight times that per cluster), many short rows
EXTRA_SHAPES = [(1,), (3, 1), (5, 7), (33, 127), (2, 51200), (2, 51204), (3, 102400), (2, 102408), (2, 300001),
                (1, 409600), (1, 500000), (1, 1000003), (4096, 64), (70000, 8)]


def _expected(x: torch.Tensor, log: bool) -> torch.Tensor:
    ref = (torch.log_softmax if log else torch.softmax)(x.detach().cpu().double(), dim=-1)
    return ref.to(x.dtype)


def _check(out: torch.Tensor, x: torch.Tensor, log: bool):
    exp = _expected(x, log)
    assert out.shape == x.shape and out.dtype == x.dtype
    torch.testing.assert_close(out.cpu(), exp)


def _fn(log):
    from kernels import log_softmax, softmax
    return log_softmax if log else softmax


@pytest.mark.parametrize("log", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", REFERENCE_SHAPES + EXTRA_SHAPES)
def test_matches_oracle(shape, dtype, log):
    g = torch.Generator().manual_seed(hash((shape, str(dtype))) & 0xffff)
    x = torch.randn(shape, generator=g).to(dtype).to(DEV)
    _check(_fn(log)(x), x, log)


@pytest.mark.parametrize("log", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(32, 1024), (16, 1025), (4, 20000), (2, 300001), (1, 1000003)])
def test_out_and_in_place(shape, dtype, log):
    g = torch.Generator().manual_seed(7)
    x = torch.randn(shape, generator=g).to(dtype).to(DEV)
    keep = x.clone()
    out = torch.empty_like(x)
    returned = _fn(log)(x, out=out)
    assert returned.data_ptr() == out.data_ptr()
    assert torch.equal(x, keep)                       # the input is untouched
    _check(out, keep, log)
    returned = _fn(log)(x, out=x)                     # in place
    assert returned.data_ptr() == x.data_ptr()
    _check(x, keep, log)


# long rows: the pipelined kernel (one CTA up to 108 KiB, clusters of 2, 4, 8 up to 864 KiB; slice edges that do not
# divide the row; more rows than resident CTAs, so every stage of the ring is reused), the register cluster kernel
# beyond it (up to 1 MiB) and the lengths right at and right after each limit
@pytest.mark.parametrize("log", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(3, 16388), (700, 20000), (3000, 4100), (3, 27648), (3, 27652), (300, 55296),
                                   (2, 55304), (5, 65544), (2, 131080), (3, 200000), (2, 221184), (2, 221188),
                                   (2, 262144), (2, 442368), (2, 442376), (2, 524288)])
def test_long_rows(shape, dtype, log):
    g = torch.Generator().manual_seed(shape[1] & 0xffff)
    x = (torch.randn(shape, generator=g) * 3).to(dtype).to(DEV)
    _check(_fn(log)(x), x, log)


@pytest.mark.parametrize("dtype", DTYPES)
def test_cluster_slices_of_minus_inf(dtype):
    """Whole slices of a clustered row are -inf: those CTAs contribute (max, sum) = (-inf, 0) and write zeros."""
    from kernels import log_softmax, softmax

    g = torch.Generator().manual_seed(5)
    x = torch.randn((4, 131072), generator=g).to(dtype)
    x[0, 40000:] = -float("inf")
    x[1, :100000] = -float("inf")
    x[2, 20000:110000] = -float("inf")
    x[3, :] = -float("inf")
    x = x.to(DEV)
    s = softmax(x)
    exp = _expected(x, False)
    torch.testing.assert_close(s.cpu()[:3], exp[:3])
    assert torch.isnan(s[3]).all()
    assert float(s[0, 40000:].abs().max()) == 0.0 and float(s[1, :100000].abs().max()) == 0.0
    ls = log_softmax(x).cpu()
    lexp = _expected(x, True)
    assert torch.equal(torch.isinf(ls[:3]), torch.isinf(lexp[:3]))
    fin = torch.isfinite(lexp)
    torch.testing.assert_close(ls[fin], lexp[fin])


@pytest.mark.parametrize("log", [False, True])
def test_against_numpy_restatement_fp32(log):
    g = torch.Generator().manual_seed(11)
    x = (torch.randn((6, 3000), generator=g) * 4).to(DEV)
    got = _fn(log)(x).cpu().double().numpy()
    want = softmax_ref.row_softmax_f64(x.cpu().numpy(), log=log)
    np.testing.assert_allclose(got, want, rtol=2e-6, atol=2e-6 if log else 1e-9)


@pytest.mark.parametrize("dtype", DTYPES)
def test_extreme_values(dtype):
    from kernels import log_softmax, softmax

    big = 3e4 if dtype == torch.float16 else 1e30
    x = torch.tensor([[big, big, -big, 0.0], [-big, -big, -big, -big], [0.0, -float("inf"), 1.0, -float("inf")],
                      [5.0, 5.0, 5.0, 5.0]], dtype=dtype, device=DEV)
    s = softmax(x)
    _check(s, x, False)
    assert torch.isfinite(s).all()
    torch.testing.assert_close(s.float().sum(-1).cpu(), torch.ones(4), atol=1e-2, rtol=0)
    ls = log_softmax(x)
    exp = _expected(x, True)
    assert torch.equal(torch.isinf(ls).cpu(), torch.isinf(exp))      # -inf exactly where the oracle has it
    fin = torch.isfinite(exp)
    torch.testing.assert_close(ls.cpu()[fin], exp[fin])
    # a row of -inf only: NaN, like torch
    n = softmax(torch.full((1, 8), -float("inf"), dtype=dtype, device=DEV))
    assert torch.isnan(n).all()


@pytest.mark.parametrize("log", [False, True])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(4, 4096), (3, 16384), (2, 40000), (2, 131072), (2, 524288)])
def test_large_magnitudes_on_the_vector_paths(shape, dtype, log):
    """Values of huge magnitude with ties at the maximum, on every 16-byte path: the difference x - max has to be taken
    before anything is scaled, or the exponent's rounding error (proportional to |max|) ruins the result."""
    big = 3e4 if dtype == torch.float16 else 1e30
    g = torch.Generator().manual_seed(shape[1])
    levels = torch.tensor([0.0, 0.5 * big, big, -big])
    x = levels[torch.randint(0, 4, shape, generator=g)].to(dtype).to(DEV)
    got = _fn(log)(x)
    exp = _expected(x, log)
    assert torch.equal(torch.isinf(got).cpu(), torch.isinf(exp)) and not torch.isnan(got).any()
    fin = torch.isfinite(exp)
    torch.testing.assert_close(got.cpu()[fin], exp[fin])


def test_seeded_sweep_around_the_kernel_limits():
    """Seeded random cases at and next to every row length where the launcher changes kernel, cluster size or stage
    count, some with a tail of -inf, against the float64 oracle."""
    import random

    rnd = random.Random(1)
    edges = [4096, 8192, 16384, 16388, 24576, 27648, 27652, 32768, 55296, 55300, 65536, 110592, 110600, 131072, 221184,
             221188, 262144, 262148, 442368, 442376, 524288, 524296]
    for _ in range(80):
        dtype = rnd.choice(DTYPES)
        cols = max(1, rnd.choice(edges) + rnd.choice([0, 0, -8, 8, -4, 4, -1, 1, rnd.randint(-3000, 3000)]))
        rows = max(1, min(rnd.choice([1, 2, 3, 7, 37, 150]), 2_000_000 // cols))
        log = rnd.random() < 0.5
        g = torch.Generator().manual_seed(cols)
        x = (torch.randn((rows, cols), generator=g) * rnd.choice([0.5, 3.0, 20.0])).to(dtype)
        if rnd.random() < 0.3:
            x[:, rnd.randint(0, cols - 1):] = -float("inf")
        x = x.to(DEV)
        got = _fn(log)(x).cpu()
        exp = _expected(x, log)
        assert torch.equal(torch.isinf(got), torch.isinf(exp)) and not torch.isnan(got).any(), (dtype, rows, cols, log)
        fin = torch.isfinite(exp)
        torch.testing.assert_close(got[fin], exp[fin], msg=lambda m: f"{dtype} {rows}x{cols} log={log}: {m}")


def test_rows_sum_to_one_at_scale():
    """Size-independent property on a tensor far beyond what the CPU oracle is run on: rows sum to 1, entries are
    in [0, 1], exp(log_softmax) equals softmax, softmax is invariant under a per-row shift."""
    from kernels import log_softmax, softmax

    g = torch.Generator(device=DEV).manual_seed(3)
    x = torch.randn((8192, 16384), generator=g, device=DEV, dtype=torch.float32)
    s = softmax(x)
    assert float(s.min()) >= 0.0 and float(s.max()) <= 1.0
    torch.testing.assert_close(s.sum(-1), torch.ones(8192, device=DEV), atol=1e-5, rtol=0)
    torch.testing.assert_close(log_softmax(x).exp(), s, atol=1e-7, rtol=1e-5)
    shift = torch.randn((8192, 1), generator=g, device=DEV) * 10
    torch.testing.assert_close(softmax(x + shift), s, atol=1e-6, rtol=1e-4)


def test_argument_errors():
    from kernels import softmax

    with pytest.raises(AssertionError):
        softmax(torch.randn(4, 8))                                    # not on the GPU
    with pytest.raises(AssertionError):
        softmax(torch.randn(8, 4, device=DEV).t())                    # not contiguous
    with pytest.raises(AssertionError):
        softmax(torch.empty(0, 4, device=DEV))                        # empty
    with pytest.raises(AssertionError):
        softmax(torch.randn(4, 8, device=DEV).double())               # unsupported dtype
    with pytest.raises(AssertionError):
        softmax(torch.randn(4, 8, device=DEV), out=torch.empty(4, 9, device=DEV))
