"""Mask preprocessing and tile classification on the CPU (checker only).

Integer restatement, in numpy, of
  * _compute_nblock_seqlen     flashmask/cute/flashmask_utils.py:96-103
  * scan_max_min_kernel        flashmask/cute/flashmask_utils.py:139-169
    (max reduced from 0, min from INT_MAX, pad entries 0 — :239-240)
  * reduce_block_count_kernel  flashmask/cute/flashmask_utils.py:396-424
  * the skip / partial / unmasked predicates of
    compute_flashmask_block_lists, flashmask/cute/flashmask_utils.py:596-670
    (same predicates as the in-kernel generate_block,
    flashmask/cute/flash_fwd_sm100.py:2297-2427).
No stored vector of the reference covers these bit patterns: parity unpinned;
this restatement is the pin.
"""
from __future__ import annotations

import numpy as np

TILE_SKIP, TILE_PARTIAL, TILE_FULL = 0, 1, 2
INT_MAX = np.iinfo(np.int32).max

# slots of the eight reductions
LTS_MAX, LTS_MIN, LTE_MAX, LTE_MIN, UTS_MAX, UTS_MIN, UTE_MAX, UTE_MIN = range(8)


def nblk_pad(Sk: int, tile_n: int) -> int:
    return ((Sk + tile_n - 1) // tile_n + 3) & 0xFFFFFFFC


def column_slots(ncols: int, causal: bool):
    """Which bound each mask column carries: list of (max_slot, min_slot)."""
    if ncols == 1:
        return [(LTS_MAX, LTS_MIN)]
    if ncols == 2 and causal:
        return [(LTS_MAX, LTS_MIN), (LTE_MAX, LTE_MIN)]
    if ncols == 2:
        return [(LTS_MAX, LTS_MIN), (UTE_MAX, UTE_MIN)]
    if ncols == 4:
        return [(LTS_MAX, LTS_MIN), (LTE_MAX, LTE_MIN), (UTS_MAX, UTS_MIN), (UTE_MAX, UTE_MIN)]
    raise ValueError(ncols)


def scan_max_min(idx: np.ndarray, tile_n: int, causal: bool) -> np.ndarray:
    """[8, B*Hm, nblk_pad] int32; slots of absent bounds and pads are 0."""
    B, Hm, Sk, ncols = idx.shape
    nb = (Sk + tile_n - 1) // tile_n
    pad = nblk_pad(Sk, tile_n)
    out = np.zeros((8, B * Hm, pad), dtype=np.int32)
    flat = idx.reshape(B * Hm, Sk, ncols).astype(np.int64)
    for c, (smax, smin) in enumerate(column_slots(ncols, causal)):
        for n in range(nb):
            seg = flat[:, n * tile_n:min((n + 1) * tile_n, Sk), c]
            out[smax, :, n] = np.maximum(seg.max(axis=1), 0)
            out[smin, :, n] = np.minimum(seg.min(axis=1), INT_MAX)
    return out


def _predicates(mm, ncols, causal, ms, me):
    """fully-masked and partial predicates for row range [ms, me) against the
    per-tile reductions mm[slot] (broadcastable arrays)."""
    if ncols == 4:
        fully = ((ms >= mm[LTS_MAX]) & (me <= mm[LTE_MIN])) | ((ms >= mm[UTS_MAX]) & (me <= mm[UTE_MIN]))
        part = ((ms < mm[LTE_MAX]) & (me > mm[LTS_MIN])) | ((ms < mm[UTE_MAX]) & (me > mm[UTS_MIN]))
    elif ncols == 2 and causal:
        fully = (ms >= mm[LTS_MAX]) & (me <= mm[LTE_MIN])
        part = (ms < mm[LTE_MAX]) & (me > mm[LTS_MIN])
    elif ncols == 2:
        fully = (ms >= mm[LTS_MAX]) | (me <= mm[UTE_MIN])
        part = (me > mm[LTS_MIN]) | (ms < mm[UTE_MAX])
    else:
        fully = ms >= mm[LTS_MAX]
        part = me > mm[LTS_MIN]
    return fully, part


def _n_block_max(me, Sq, Sk, tile_n, causal, nb):
    if not causal:
        return np.full_like(me, nb)
    right = me + Sk - Sq
    return np.clip((right + tile_n - 1) // tile_n, 0, nb)


def valid_block_count(minmax, B, Hm, Sq, Sk, ncols, causal, tile_m, tile_n):
    """[B, Hm, Tq] int32: K tiles n < n_block_max(t) that are not fully masked."""
    nb = (Sk + tile_n - 1) // tile_n
    tq = (Sq + tile_m - 1) // tile_m
    mm = [minmax[s].reshape(B, Hm, 1, -1)[..., :nb].astype(np.int64) for s in range(8)]
    ms = (np.arange(tq, dtype=np.int64) * tile_m)[None, None, :, None]
    me = np.minimum(ms + tile_m, Sq)
    fully, _ = _predicates(mm, ncols, causal, ms, me)
    nmax = _n_block_max(me, Sq, Sk, tile_n, causal, nb)
    n = np.arange(nb, dtype=np.int64)[None, None, None, :]
    return ((~fully) & (n < nmax)).sum(axis=-1).astype(np.int32)


def classify_tiles(minmax, B, Hm, Sq, Sk, ncols, causal, tile_m, tile_n):
    """[B, Hm, Tq, Tk] int8 in {TILE_SKIP, TILE_PARTIAL, TILE_FULL}.

    ``ncols == 0`` (no mask tensor) classifies on geometry alone."""
    nb = (Sk + tile_n - 1) // tile_n
    tq = (Sq + tile_m - 1) // tile_m
    ms = (np.arange(tq, dtype=np.int64) * tile_m)[None, None, :, None]
    me = np.minimum(ms + tile_m, Sq)
    ns = (np.arange(nb, dtype=np.int64) * tile_n)[None, None, None, :]
    ne = np.minimum(ns + tile_n, Sk)
    if ncols:
        mm = [minmax[s].reshape(B, Hm, 1, -1)[..., :nb].astype(np.int64) for s in range(8)]
        fully, part = _predicates(mm, ncols, causal, ms, me)
    else:
        fully = np.zeros((B, Hm, tq, nb), dtype=bool)
        part = np.zeros((B, Hm, tq, nb), dtype=bool)
    off = Sk - Sq
    if causal:
        c_empty = ns > (me - 1 + off)
        c_full = (ne - 1) <= (ms + off)
        c_part = (~c_empty) & (~c_full)
    else:
        c_empty = np.zeros((1, 1, tq, nb), dtype=bool)
        c_part = np.zeros((1, 1, tq, nb), dtype=bool)
    ragged = ne < ns + tile_n
    skip = c_empty | fully
    needs = c_part | ragged | part
    cls = np.where(skip, TILE_SKIP, np.where(needs, TILE_PARTIAL, TILE_FULL))
    return np.broadcast_to(cls, (B, Hm, tq, nb)).astype(np.int8)
