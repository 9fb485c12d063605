"""fp64 numpy restatement of scaled-dot-product attention.  TEST INFRASTRUCTURE ONLY.

The reference's oracle is ``torch.nn.functional.scaled_dot_product_attention``
(call sites tests/test_attention.py:94, tests/test_decode.py:82-86,
tests/test_speculative_decode.py:116-122).  torch is a third-party dependency
whose source is not part of the reference tree, so this file restates the
published formula

    O = softmax(Q K^T / sqrt(D) + mask) V

explicitly, one sequence at a time, in float64, with the GQA head map
``kv_head = q_head * KVH // QH`` (kernels/attention.py:463) and the two mask
conventions of the path:

  * prefill causal: top-left aligned, key j visible to query i iff j <= i
    (kernels/attention.py:566-569);
  * speculative decode causal: the M draft keys are the last M keys; draft row
    i sees key j iff not (j >= L-M and j-(L-M) > i)
    (kernels/speculative_decode.py:155-160).

Parity status: pinned against torch SDPA and analytic known-answer cases in
``tests/test_oracle.py``; the reference holds no golden vectors of its own.
"""
from __future__ import annotations

import numpy as np


def attention_f64(q, k, v, *, mask=None) -> np.ndarray:
    """q (QH, Lq, D), k/v (KVH, Lk, D) array-likes -> (QH, Lq, D) float64.
    ``mask`` is an optional boolean (Lq, Lk) array, True = visible."""
    q = np.asarray(q, dtype=np.float64)
    k = np.asarray(k, dtype=np.float64)
    v = np.asarray(v, dtype=np.float64)
    qh, lq, d = q.shape
    kvh = k.shape[0]
    out = np.zeros((qh, lq, d), dtype=np.float64)
    scale = 1.0 / np.sqrt(d)
    for h in range(qh):
        g = h * kvh // qh
        s = (q[h] @ k[g].T) * scale
        if mask is not None:
            s = np.where(mask, s, -np.inf)
        s = s - s.max(axis=1, keepdims=True)
        p = np.exp(s)
        p /= p.sum(axis=1, keepdims=True)
        out[h] = p @ v[g]
    return out


def causal_top_left(lq: int, lk: int) -> np.ndarray:
    i = np.arange(lq)[:, None]
    j = np.arange(lk)[None, :]
    return j <= i


def draft_tail_mask(m: int, lk: int) -> np.ndarray:
    i = np.arange(m)[:, None]
    j = np.arange(lk)[None, :]
    start = lk - m
    return ~((j >= start) & ((j - start) > i))


def lse_merge_f64(ms, ls, accs) -> np.ndarray:
    """Merge split-KV partials (m_s, l_s, acc_s): g = max m_s,
    O = sum exp(m_s-g) acc_s / sum exp(m_s-g) l_s
    (kernels/decode.py:186-197, kernels/attention.py:710-724).
    ms, ls: (S, R); accs: (S, R, D).  Empty splits carry m=-inf, l=0."""
    ms = np.asarray(ms, dtype=np.float64)
    ls = np.asarray(ls, dtype=np.float64)
    accs = np.asarray(accs, dtype=np.float64)
    g = ms.max(axis=0)
    with np.errstate(invalid="ignore"):
        a = np.where(np.isneginf(ms), 0.0, np.exp(ms - g[None, :]))
    num = (a[:, :, None] * accs).sum(axis=0)
    den = (a * ls).sum(axis=0)
    return num / den[:, None]


def row_softmax_f64(x, *, log: bool = False) -> np.ndarray:
    """Softmax (or log-softmax) over the last axis in float64: the formula behind the reference's test oracle
    ``torch.nn.functional.softmax`` / ``log_softmax`` (tests/test_softmax.py:47,95), written out as
    ``exp(x - max) / sum(exp(x - max))`` and ``x - max - log(sum(exp(x - max)))`` (kernels/softmax.py:26-31,247-250)."""
    x = np.asarray(x, dtype=np.float64)
    m = np.max(x, axis=-1, keepdims=True)
    with np.errstate(invalid="ignore", divide="ignore"):
        e = np.exp(x - m)
        s = np.sum(e, axis=-1, keepdims=True)
        return (x - m - np.log(s)) if log else e / s


def row_softmax_split_f64(x, parts: int, *, log: bool = False) -> np.ndarray:
    """The same result through per-slice (max, sum) pairs merged as the reference merges its programs
    (kernels/softmax.py:114-127): what the cluster kernel computes, slice by slice."""
    x = np.asarray(x, dtype=np.float64)
    pieces = np.array_split(x, parts, axis=-1)
    ms = [np.max(p, axis=-1, keepdims=True) for p in pieces]
    ls = [np.sum(np.exp(p - m), axis=-1, keepdims=True) for p, m in zip(pieces, ms)]
    g = np.max(np.concatenate(ms, axis=-1), axis=-1, keepdims=True)
    total = sum(l * np.exp(m - g) for l, m in zip(ls, ms))
    return (x - g - np.log(total)) if log else np.exp(x - g) / total
