"""Context-parallel partitioner on the CPU (checker only).

Restates, in numpy / plain Python:
  * get_q_workload            flashmask/cp_balance/cp_balance.py:56-91 with the
    counting rule of reduce_workload_kernel, csrc/cp_balance_bridge.cu:91-127
    (non-causal predicates, 128-row blocks; real K blocks only, which equals the
    reference whenever S % 512 == 0 — its loop also visits uninitialised pads)
  * assign_tasks_heap         flashmask/cp_balance/cp_balance.py:96-174
  * indices_rerank_kernel     csrc/cp_balance_bridge.cu:185-216
  * indices_to_chunks_kernel  csrc/cp_balance_bridge.cu:153-183
No stored vector of the reference covers the heap partition: parity unpinned,
this restatement is the pin.  The rerank / localise / workload kernels are
additionally checked on the GPU against the reference's own CUDA source
compiled into oracle/_ref (see oracle/Makefile).
"""
from __future__ import annotations

import heapq

import numpy as np

from . import tiles


def chunk_workload(idx: np.ndarray, q_chunk_size: int, block: int = 128) -> np.ndarray:
    """[1, H, Tchunks, 2] int32 (workload, chunk index)."""
    B, H, S, ncols = idx.shape
    assert ncols in (2, 4)
    mm = tiles.scan_max_min(idx, block, False)
    cnt = tiles.valid_block_count(mm, B, H, S, S, ncols, False, block, block)   # [B,H,Tr]
    tr = cnt.shape[-1]
    bpc = q_chunk_size // block
    n_chunks = -(-tr // bpc)
    pad = np.zeros((B, H, n_chunks * bpc), dtype=np.int64)
    pad[..., :tr] = cnt
    per_chunk = pad.reshape(B, H, n_chunks, bpc).sum(axis=3).sum(axis=0)       # [H, Tchunks]
    out = np.zeros((1, H, n_chunks, 2), dtype=np.int32)
    out[0, :, :, 0] = per_chunk
    out[0, :, :, 1] = np.arange(n_chunks)
    return out


def assign_tasks_heap(tasks, num_buckets):
    """(buckets, bucket_weights, cuts); buckets[j] = [(weight, index), ...] sorted by index."""
    n = len(tasks)
    if n == 0:
        return [[] for _ in range(num_buckets)], [0] * num_buckets, 0
    cap = n // num_buckets
    order = sorted(tasks, key=lambda x: -x[0])          # stable: ties keep input order
    buckets = [[] for _ in range(num_buckets)]
    weights = [0] * num_buckets
    counts = [0] * num_buckets
    heap = [(0, i) for i in range(num_buckets)]
    for weight, idx in order:
        weight, idx = int(weight), int(idx)
        parked, placed = [], False
        while heap:
            load, b = heapq.heappop(heap)
            if counts[b] < cap:
                buckets[b].append((weight, idx)); weights[b] += weight; counts[b] += 1
                heapq.heappush(heap, (weights[b], b))
                placed = True
                break
            parked.append((load, b))
        for item in parked:
            heapq.heappush(heap, item)
        if not placed:
            load, b = heapq.heappop(heap)
            buckets[b].append((weight, idx)); weights[b] += weight; counts[b] += 1
            heapq.heappush(heap, (weights[b], b))
    buckets = [sorted(b, key=lambda x: x[1]) for b in buckets]
    all_idx = sorted(i for b in buckets for _, i in b)
    cuts = sum(1 for i in range(1, len(all_idx)) if all_idx[i] != all_idx[i - 1] + 1)
    return buckets, weights, cuts


def rerank(idx: np.ndarray, chunk_order, chunk_size: int) -> np.ndarray:
    B, H, S, D = idx.shape
    n_chunks = -(-S // chunk_size)
    out = np.zeros((B, H, n_chunks * chunk_size, D), dtype=np.int32)
    for c, src in enumerate(chunk_order):
        lo = int(src) * chunk_size
        hi = min(lo + chunk_size, S)
        if hi > lo:
            out[:, :, c * chunk_size:c * chunk_size + (hi - lo)] = idx[:, :, lo:hi]
    return out


def localize(idx: np.ndarray, local_chunks, chunk_size: int) -> np.ndarray:
    v = idx.astype(np.int64)
    best = None
    for k, c in enumerate(local_chunks):
        loc = np.clip(v - int(c) * chunk_size, 0, chunk_size)
        loc = np.where(loc > 0, loc + k * chunk_size, loc)
        best = loc if best is None else np.maximum(best, loc)
    return best.astype(np.int32)


def balance(idx: np.ndarray, cp_size: int, cp_rank: int, chunk_size: int):
    wl = chunk_workload(idx, chunk_size)
    buckets, _, _ = assign_tasks_heap(wl.reshape(-1, 2), cp_size)
    order = [i for b in buckets for _, i in b]
    rr = rerank(idx, order, chunk_size)
    return localize(rr, [i for _, i in buckets[cp_rank]], chunk_size), buckets
