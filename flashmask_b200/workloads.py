"""Seeded synthetic inputs: FlashMask column-bound masks and the benchmark shapes.

A FlashMask mask is an int32 array ``[B, Hm, Sk, ncols]`` of row bounds per key
column.  Column meaning (flashmask/frontend/torch/__init__.py:53-55 and
flashmask/cute/mask.py:575-606 of the reference):

* ``ncols == 1``                 ``[LTS]``            rows ``i >= LTS`` masked
* causal, ``ncols == 2``         ``[LTS, LTE]``       rows ``LTS <= i < LTE`` masked
* non-causal, ``ncols == 2``     ``[LTS, UTE]``       rows ``i >= LTS`` or ``i < UTE`` masked
* ``ncols == 4``                 ``[LTS, LTE, UTS, UTE]``

``causal=True`` additionally masks ``j > i + Sk - Sq`` (bottom-right aligned).

The public benchmark masks of the reference are document layouts read from a
text file; here seeded synthetic layouts with the same shapes and value
distributions stand in for them.  Everything is numpy so that tests, the
benchmark and the CPU checker build identical inputs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np

__all__ = [
    "lognormal_doc_lengths", "causal_document", "bidirectional_document",
    "sliding_window", "share_question", "random_eviction", "causal_only",
    "full_visible", "prefix_lm_document", "four_column_bands", "empty_mask",
    "uniform_doc_lengths", "count_visible", "block_density", "Workload",
    "make_workload", "WORKLOADS", "window_bounds",
]


# --------------------------------------------------------------------------
# document layouts
# --------------------------------------------------------------------------
def lognormal_doc_lengths(rng: np.random.Generator, total: int, mu: float, sigma: float,
                          lo: int, hi: int) -> np.ndarray:
    """Document lengths ~ round(exp(N(mu, sigma))) clipped to [lo, hi], drawn
    until they cover ``total``; the last one is truncated to pack exactly."""
    lens = []
    left = total
    while left > 0:
        n = int(round(math.exp(rng.normal(mu, sigma))))
        n = max(lo, min(hi, n))
        n = min(n, left)
        lens.append(n)
        left -= n
    return np.asarray(lens, dtype=np.int64)


def uniform_doc_lengths(rng: np.random.Generator, total: int, ndocs: int) -> np.ndarray:
    """``ndocs`` documents whose cut points are drawn uniformly without
    replacement from [1, total-1]."""
    cuts = np.sort(rng.choice(np.arange(1, total), size=ndocs - 1, replace=False))
    edges = np.concatenate([[0], cuts, [total]])
    return np.diff(edges).astype(np.int64)


def _stack(cols, B: int, Sq: int) -> np.ndarray:
    arr = np.stack([np.asarray(c, dtype=np.int64) for c in cols], axis=-1)  # [Sk, n]
    arr = np.clip(arr, None, Sq).astype(np.int32)
    return np.ascontiguousarray(np.broadcast_to(arr[None, None], (B, 1) + arr.shape))


def _doc_ends_starts(lens: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    ends = np.cumsum(lens)
    starts = ends - lens
    return np.repeat(ends, lens), np.repeat(starts, lens)


# --------------------------------------------------------------------------
# mask generators: each returns (startend_row_indices | None, causal)
# --------------------------------------------------------------------------
def causal_only(B, Sq, Sk):
    return None, True


def full_visible(B, Sq, Sk):
    return None, False


def empty_mask(B, Sq, Sk):
    """Every element masked (LTS = 0 everywhere): exercises empty rows."""
    return _stack([np.zeros(Sk)], B, Sq), True


def causal_document(B, Sq, Sk, doc_lens):
    """Causal attention inside packed documents: LTS[j] = end(doc(j))."""
    ends, _ = _doc_ends_starts(np.asarray(doc_lens))
    assert ends.shape[0] == Sk
    return _stack([ends], B, Sq), True


def bidirectional_document(B, Sq, Sk, doc_lens):
    """Block-diagonal attention: [LTS = end(doc), UTE = start(doc)], non-causal."""
    ends, starts = _doc_ends_starts(np.asarray(doc_lens))
    assert ends.shape[0] == Sk
    return _stack([ends, starts], B, Sq), False


def causal_document_noncausal_form(B, Sq, Sk, doc_lens):
    """The causal document mask written as a non-causal 2-column mask
    [LTS = end(doc(j)), UTE = j]: the form the context-parallel entry points
    accept (they take only 2/4-column non-causal masks)."""
    ends, _ = _doc_ends_starts(np.asarray(doc_lens))
    return _stack([ends, np.arange(Sk)], B, Sq), False


def window_bounds(Sk: int, window: int) -> np.ndarray:
    """LTS bound of a causal sliding window of ``window`` keys:
    key j is seen by rows j .. j+window-1."""
    return np.minimum(np.arange(Sk, dtype=np.int64) + window, np.iinfo(np.int32).max)


def sliding_window(B, Sq, Sk, window):
    return _stack([window_bounds(Sk, window)], B, Sq), True


def share_question(B, Sq, Sk, prefix, answer, n_answers):
    """Groups of one shared prefix followed by answers; every answer sees the
    prefix and itself only.  Causal 2-column [LTS, LTE]: prefix columns are
    masked from the end of their group on, answer columns from the end of that
    answer on; LTE = Sq (masked to the bottom)."""
    lts = np.empty(Sk, dtype=np.int64)
    pos = 0
    while pos < Sk:
        g_start = pos
        p = min(prefix, Sk - pos)
        pos += p
        ans = []
        for _ in range(n_answers):
            if pos >= Sk:
                break
            a = min(answer, Sk - pos)
            ans.append((pos, pos + a))
            pos += a
        g_end = pos
        lts[g_start:g_start + p] = g_end
        for s, e in ans:
            lts[s:e] = e
    lte = np.full(Sk, Sq, dtype=np.int64)
    return _stack([lts, lte], B, Sq), True


def random_eviction(B, Sq, Sk, rng: np.random.Generator):
    """Causal 2-column: LTS[j] ~ U{j+1..S}, LTE[j] ~ U{LTS[j]..S} (key j is
    evicted for rows LTS..LTE-1)."""
    j = np.arange(Sk, dtype=np.int64)
    lo = np.minimum(j + 1, Sq)
    lts = lo + np.floor(rng.random(Sk) * (Sq - lo + 1)).astype(np.int64)
    lte = lts + np.floor(rng.random(Sk) * (Sq - lts + 1)).astype(np.int64)
    return _stack([lts, lte], B, Sq), True


def prefix_lm_document(B, Sq, Sk, docs):
    """Per document (prefix, length): bidirectional over the prefix, causal after."""
    lens = np.asarray([d for _, d in docs])
    ends, _ = _doc_ends_starts(lens)
    ute = np.empty(Sk, dtype=np.int64)
    cur = 0
    for p, d in docs:
        ute[cur:cur + p] = cur
        ute[cur + p:cur + d] = np.arange(cur + p, cur + d)
        cur += d
    return _stack([ends, ute], B, Sq), False


def four_column_bands(B, Sq, Sk, rng: np.random.Generator):
    """Random 4-column mask [LTS, LTE, UTS, UTE] with a masked band below and a
    masked band above the diagonal of every column."""
    j = np.arange(Sk, dtype=np.int64) * Sq // max(Sk, 1)
    lts = np.minimum(j + 1 + rng.integers(0, max(Sq // 4, 1), Sk), Sq)
    lte = np.minimum(lts + rng.integers(0, max(Sq // 2, 1), Sk), Sq)
    ute = np.maximum(j - rng.integers(0, max(Sq // 4, 1), Sk), 0)
    uts = np.maximum(ute - rng.integers(0, max(Sq // 2, 1), Sk), 0)
    return _stack([lts, lte, uts, ute], B, Sq), False


# --------------------------------------------------------------------------
# work measures
# --------------------------------------------------------------------------
def _masked_rows_per_column(idx: np.ndarray, Sq: int, Sk: int, causal: bool) -> np.ndarray:
    """Number of masked query rows per key column, exact, from the bounds."""
    ncols = idx.shape[-1]
    a = idx.astype(np.int64)
    lts = np.clip(a[..., 0], 0, Sq)
    if ncols == 1:
        lo1, hi1 = lts, np.full_like(lts, Sq)
    elif (causal and ncols == 2) or ncols == 4:
        lo1, hi1 = lts, np.clip(a[..., 1], 0, Sq)
    else:
        lo1, hi1 = lts, np.full_like(lts, Sq)
    hi1 = np.maximum(hi1, lo1)
    j = np.arange(Sk, dtype=np.int64)
    if causal:
        lo2 = np.zeros_like(lts)
        hi2 = np.broadcast_to(np.clip(j - (Sk - Sq), 0, Sq), lts.shape)
    elif ncols == 2:
        lo2, hi2 = np.zeros_like(lts), np.clip(a[..., 1], 0, Sq)
    elif ncols == 4:
        lo2, hi2 = np.clip(a[..., 2], 0, Sq), np.clip(a[..., 3], 0, Sq)
    else:
        lo2, hi2 = np.zeros_like(lts), np.zeros_like(lts)
    hi2 = np.maximum(hi2, lo2)
    len1 = hi1 - lo1
    len2 = hi2 - lo2
    inter = np.maximum(0, np.minimum(hi1, hi2) - np.maximum(lo1, lo2))
    return len1 + len2 - inter


def count_visible(idx: Optional[np.ndarray], B: int, Sq: int, Sk: int, causal: bool) -> np.ndarray:
    """Exact number of unmasked (query, key) pairs per (batch, mask head)."""
    if idx is None:
        if causal:
            j = np.arange(Sk, dtype=np.int64)
            vis = Sq - np.clip(j - (Sk - Sq), 0, Sq)
            return np.full((B, 1), int(vis.sum()), dtype=np.int64)
        return np.full((B, 1), Sq * Sk, dtype=np.int64)
    masked = _masked_rows_per_column(idx, Sq, Sk, causal)
    return (Sq - masked).sum(axis=-1).astype(np.int64)


def block_density(idx: Optional[np.ndarray], B: int, Sq: int, Sk: int, causal: bool,
                  block: int = 128) -> float:
    """Fraction of block x block tiles with at least one unmasked element — the
    FLOP accounting of the reference benchmark
    (tests/torch/benchmark_flashmask.py:272-398)."""
    tq, tk = -(-Sq // block), -(-Sk // block)
    if idx is None:
        if not causal:
            return 1.0
        i_hi = np.minimum((np.arange(tq) + 1) * block, Sq) - 1
        n_lo = np.arange(tk) * block
        return float((n_lo[None, :] <= i_hi[:, None] + (Sk - Sq)).mean())
    total = 0
    alive = 0
    for b in range(idx.shape[0]):
        for h in range(idx.shape[1]):
            bias = dense_visible(idx[b:b + 1, h:h + 1], Sq, causal)[0, 0]
            pad = np.zeros((tq * block, tk * block), dtype=bool)
            pad[:Sq, :Sk] = bias
            blk = pad.reshape(tq, block, tk, block).any(axis=(1, 3))
            alive += int(blk.sum())
            total += tq * tk
    return alive / total


def dense_visible(idx: np.ndarray, Sq: int, causal: bool) -> np.ndarray:
    """Boolean [B, Hm, Sq, Sk] visibility expanded from the bounds (small sizes)."""
    Bm, Hm, Sk, ncols = idx.shape
    i = np.arange(Sq, dtype=np.int64)[None, None, :, None]
    j = np.arange(Sk, dtype=np.int64)[None, None, None, :]
    a = idx.astype(np.int64)
    c = [a[..., t][:, :, None, :] for t in range(ncols)]
    if ncols == 1:
        masked = i >= c[0]
    elif ncols == 2 and causal:
        masked = (i >= c[0]) & (i < c[1])
    elif ncols == 2:
        masked = (i >= c[0]) | (i < c[1])
    else:
        masked = ((i >= c[0]) & (i < c[1])) | ((i >= c[2]) & (i < c[3]))
    if causal:
        masked = masked | (j > i + (Sk - Sq))
    return ~masked


# --------------------------------------------------------------------------
# named benchmark / parity workloads
# --------------------------------------------------------------------------
@dataclass
class Workload:
    name: str
    B: int
    Sq: int
    Sk: int
    Hq: int
    Hkv: int
    d: int
    dv: int
    idx: Optional[np.ndarray]
    causal: bool
    sink: bool = False
    deterministic: bool = False
    seed: int = 0

    def n_visible(self) -> int:
        """Unmasked (batch, q-head, query, key) pairs."""
        per = count_visible(self.idx, self.B, self.Sq, self.Sk, self.causal)
        hm = per.shape[1]
        return int(per.sum()) * (self.Hq // hm)

    def flops(self) -> Tuple[int, int]:
        """(forward, backward) FLOPs counting unmasked pairs only:
        fwd 2*N*(d+dv), bwd 2*N*(3d+2dv)."""
        n = self.n_visible()
        return 2 * n * (self.d + self.dv), 2 * n * (3 * self.d + 2 * self.dv)

    def sparsity(self) -> float:
        return 1.0 - self.n_visible() / (self.B * self.Hq * self.Sq * self.Sk)


def _docs_per_batch(rng, B, S, mu, sigma, lo, hi):
    return [lognormal_doc_lengths(rng, S, mu, sigma, lo, hi) for _ in range(B)]


def _cat_batches(masks):
    return np.ascontiguousarray(np.concatenate(masks, axis=0))


def make_workload(name: str, S: Optional[int] = None) -> Workload:
    """Build one of the named configurations.  ``S`` overrides the sequence
    length (parity tests run reduced sizes of the same distributions)."""
    if name == "cpu_causal_doc_1k":            # the CPU-runnable case
        S = S or 1024
        rng = np.random.default_rng(0)
        idx, causal = causal_document(1, S, S, uniform_doc_lengths(rng, S, 4))
        return Workload(name, 1, S, S, 2, 2, 64, 64, idx, causal, seed=0)
    if name in ("causal_doc_8k_gqa", "causal_doc_8k_gqa_d64"):   # the headline single-GPU case; the same mask at d = 64
        S = S or 8192
        rng = np.random.default_rng(1)
        docs = _docs_per_batch(rng, 2, S, math.log(1024), 1.0, 64, 8192)
        idx = _cat_batches([causal_document(1, S, S, d)[0] for d in docs])
        hd = 64 if name.endswith("_d64") else 128
        return Workload(name, 2, S, S, 32, 8, hd, hd, idx, True, seed=1)
    if name.startswith("sweep32k_"):
        S = S or 32768
        kind = name[len("sweep32k_"):]
        rng = np.random.default_rng(2)
        scale = S / 32768
        if kind == "sliding_window":
            idx, causal = sliding_window(1, S, S, max(1, int(1024 * scale)))
        elif kind == "causal_doc":
            idx, causal = causal_document(
                1, S, S, lognormal_doc_lengths(rng, S, math.log(1024), 1.0, 64, 8192))
        elif kind == "share_question":
            idx, causal = share_question(1, S, S, max(1, int(4096 * scale)),
                                         max(1, int(2048 * scale)), 4)
        elif kind == "bidir_doc":
            idx, causal = bidirectional_document(
                1, S, S, lognormal_doc_lengths(rng, S, math.log(1024), 1.0, 64, 8192))
        elif kind == "random_eviction":
            idx, causal = random_eviction(1, S, S, rng)
        else:
            raise KeyError(name)
        return Workload(name, 1, S, S, 16, 16, 128, 128, idx, causal, seed=2)
    if name.startswith("bigd16k_"):
        S = S or 16384
        kind = name[len("bigd16k_"):]
        shapes = {"192_128": (32, 8, 192, 128), "576_512": (16, 1, 576, 512),
                  "256_256": (16, 16, 256, 256)}
        hq, hkv, d, dv = shapes[kind]
        return Workload(name, 1, S, S, hq, hkv, d, dv, None, True, sink=True,
                        deterministic=True, seed=3)
    if name in ("dense8k_full_gqa", "dense8k_causal_gqa"):     # no mask tensor: the dense points of the headline shape
        S = S or 8192
        return Workload(name, 2, S, S, 32, 8, 128, 128, None, name == "dense8k_causal_gqa", seed=5)
    if name == "cp_causal_doc_128k":
        S = S or 131072
        rng = np.random.default_rng(4)
        scale = S / 131072
        docs = lognormal_doc_lengths(rng, S, math.log(4096 * scale), 1.5,
                                     max(1, int(512 * scale)), max(1, int(32768 * scale)))
        idx, causal = causal_document_noncausal_form(1, S, S, docs)
        return Workload(name, 1, S, S, 32, 8, 128, 128, idx, causal, seed=4)
    raise KeyError(name)


WORKLOADS = [
    "cpu_causal_doc_1k", "causal_doc_8k_gqa", "causal_doc_8k_gqa_d64",
    "sweep32k_sliding_window", "sweep32k_causal_doc", "sweep32k_share_question",
    "sweep32k_bidir_doc", "sweep32k_random_eviction",
    "bigd16k_192_128", "bigd16k_576_512", "bigd16k_256_256",
    "dense8k_full_gqa", "dense8k_causal_gqa",
    "cp_causal_doc_128k",
]
