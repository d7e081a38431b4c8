"""Mask-aware sequence partitioner for context parallelism.

Mirrors ``flashmask.cp_balance`` of the reference
(flashmask/cp_balance/cp_balance.py, cp_balance_cuda_kernels.py): the sequence
is cut into ``balance_chunk_size``-row chunks, each chunk is weighted by the
number of 128x128 tiles its rows keep, chunks are dealt to ranks so that the
heaviest rank is as light as possible, the mask's key axis is gathered into
rank order and its row bounds are rewritten into each rank's local row space.
All device work goes through the C ABI (fm_mask_prepare, fm_cp_*).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Sequence, Tuple

import numpy as np
import torch

from . import _lib
from .ops import _stream, prepare_mask

__all__ = ["get_q_workload", "assign_tasks_heap", "assign_tasks_ipo", "cp_balance_ipo_solve", "indices_rerank_cuda", "indices_to_chunks_cuda",
           "balance_flashmask_input", "scatter_by_buckets", "dual_chunk_buckets"]


def get_q_workload(startend_row_indices: torch.Tensor, q_chunk_size: int, m_block_size: int = 128,
                   n_block_size: int = 128) -> torch.Tensor:
    """int32 ``[1, Hm, Tchunks, 2]`` = (workload, chunk index) per balance chunk.

    Reference: get_q_workload, flashmask/cp_balance/cp_balance.py:11-93 — the
    mask must carry 2 or 4 bounds per column (non-causal forms), the count uses
    the non-causal fully-masked predicates on 128x128 tiles."""
    idx = startend_row_indices
    assert idx is not None and idx.dim() == 4 and idx.dtype == torch.int32
    assert idx.shape[-1] in (2, 4), "cp_balance needs a 2- or 4-column (non-causal) mask"
    assert q_chunk_size % m_block_size == 0, "q_chunk_size must be divisible by m_block_size"
    assert m_block_size == 128 and n_block_size == 128, "the workload estimate is defined on 128x128 tiles"
    B, H, S, _ = idx.shape
    info = prepare_mask(idx, S, False, m_block_size, n_block_size, want_count=True)
    tq = info.valid_block_count.shape[-1]
    bpc = q_chunk_size // m_block_size
    n_chunks = -(-tq // bpc)
    out = torch.empty((1, H, n_chunks, 2), dtype=torch.int32, device=idx.device)
    _lib.check(_lib.load().fm_cp_chunk_workload(info.valid_block_count.data_ptr(), B, H, tq, bpc,
                                                out.data_ptr(), _stream(idx)), "fm_cp_chunk_workload")
    return out


def assign_tasks_heap(tasks, num_buckets: int):
    """LPT heap partition.  ``tasks`` is ``(N, 2)`` rows ``[weight, index]``.
    Returns ``(buckets, bucket_weights, cuts)`` exactly as the reference
    (flashmask/cp_balance/cp_balance.py:96-174): each bucket is a list of
    ``(weight, index)`` sorted by index."""
    tasks = np.asarray(tasks.cpu() if hasattr(tasks, "cpu") else tasks)
    n = len(tasks)
    if n == 0:
        return [[] for _ in range(num_buckets)], [0] * num_buckets, 0
    w = np.ascontiguousarray(tasks[:, 0], dtype=np.int32)
    bucket_of = np.empty(n, dtype=np.int32)
    _lib.check(_lib.load().fm_cp_partition_heap(w.ctypes.data, n, int(num_buckets), bucket_of.ctypes.data),
               "fm_cp_partition_heap")
    buckets: List[List[Tuple[int, int]]] = [[] for _ in range(num_buckets)]
    for t in range(n):
        buckets[int(bucket_of[t])].append((int(tasks[t, 0]), int(tasks[t, 1])))
    buckets = [sorted(b, key=lambda x: x[1]) for b in buckets]
    weights = [sum(x[0] for x in b) for b in buckets]
    all_idx = sorted(i for b in buckets for _, i in b)
    cuts = sum(1 for i in range(1, len(all_idx)) if all_idx[i] != all_idx[i - 1] + 1)
    return buckets, weights, cuts


def cp_balance_ipo_solve(weights, num_buckets: int):
    """``(assign, max_load)``: ``assign`` is int32 ``[num_buckets, N // num_buckets]`` task indices.
    Reference: cp_balance_ipo_solve, flashmask/cp_balance/cp_balance_cuda_kernels.py, over
    CpBalanceSolver::solve_to (csrc/cp_balance_fast.hpp:86-100)."""
    w = np.ascontiguousarray(weights, dtype=np.int32)
    n = int(w.shape[0])
    assign = np.empty((int(num_buckets), n // int(num_buckets)), dtype=np.int32)
    best = C.c_int64(0)
    _lib.check(_lib.load().fm_cp_partition_ipo(w.ctypes.data, n, int(num_buckets), assign.ctypes.data,
                                               C.addressof(best)), "fm_cp_partition_ipo")
    return assign, int(best.value)


def assign_tasks_ipo(tasks, num_buckets: int):
    """Iterative pairwise/triple optimal partition with the interface of
    ``assign_tasks_heap``; falls back to the heap when ``N == 0``, ``N > 512`` or
    ``N % num_buckets != 0`` (reference: flashmask/cp_balance/cp_balance.py:177-228)
    and, where the reference solver's tables end, when ``num_buckets > 32``."""
    tasks = np.asarray(tasks.cpu() if hasattr(tasks, "cpu") else tasks)
    n = len(tasks)
    if n == 0 or n > 512 or n % num_buckets != 0 or num_buckets > 32:
        return assign_tasks_heap(tasks, num_buckets)
    assign, _ = cp_balance_ipo_solve(tasks[:, 0], num_buckets)
    buckets = [sorted(((int(tasks[i, 0]), int(tasks[i, 1])) for i in row), key=lambda x: x[1]) for row in assign]
    weights = [sum(x[0] for x in b) for b in buckets]
    all_idx = sorted(i for b in buckets for _, i in b)
    cuts = sum(1 for i in range(1, len(all_idx)) if all_idx[i] != all_idx[i - 1] + 1)
    return buckets, weights, cuts


def indices_rerank_cuda(startend_row_indices: torch.Tensor, indices: torch.Tensor,
                        balance_chunk_size: int = 2048) -> torch.Tensor:
    """Gather the key axis into chunk order ``indices``
    (reference: cp_balance_cuda_kernels.py:116-128)."""
    x = startend_row_indices.contiguous()
    ci = indices.to(device=x.device, dtype=torch.int32).contiguous()
    B, H, S, D = x.shape
    n_chunks = -(-S // balance_chunk_size)
    out = torch.empty((B, H, n_chunks * balance_chunk_size, D), dtype=torch.int32, device=x.device)
    _lib.check(_lib.load().fm_cp_rerank(x.data_ptr(), ci.data_ptr(), out.data_ptr(), B, H, S, D, n_chunks,
                                        balance_chunk_size, _stream(x)), "fm_cp_rerank")
    return out


def indices_to_chunks_cuda(startend_row_indices: torch.Tensor, bucket_idx: torch.Tensor,
                           chunksize: int = 2048) -> torch.Tensor:
    """Rewrite global row bounds into the local row space of the rank that owns
    chunks ``bucket_idx`` (reference: cp_balance_cuda_kernels.py:103-114)."""
    x = startend_row_indices.contiguous()
    bi = bucket_idx.to(device=x.device, dtype=torch.int32).contiguous()
    out = torch.empty_like(x)
    _lib.check(_lib.load().fm_cp_localize(x.data_ptr(), bi.data_ptr(), out.data_ptr(), x.numel(), bi.numel(),
                                          chunksize, _stream(x)), "fm_cp_localize")
    return out


def balance_flashmask_input(startend_row_indices: torch.Tensor, cp_size: int, cp_rank: int,
                            balance_chunk_size: int = 2048, q_block_size: int = 128, k_block_size: int = 128,
                            use_ipo: bool = False):
    """Returns ``(local_startend_row_indices, buckets)``.

    Reference: balance_flashmask_input, flashmask/cp_balance/cp_balance.py:360-430.
    ``buckets[r]`` lists the ``(workload, chunk)`` pairs rank ``r`` owns; q, k, v
    and dO are scattered with the same plan (``scatter_by_buckets``).  The local
    mask has its key axis in rank order over ALL ranks and its row bounds in
    this rank's local row space; run it with ``causal=False``."""
    workload = get_q_workload(startend_row_indices, balance_chunk_size, q_block_size, k_block_size)
    # one host synchronisation, as in the reference (cp_balance.py:400)
    tasks = workload[:, 0].reshape(-1, 2).cpu().numpy() if workload.shape[1] == 1 else \
        _sum_mask_heads(workload).cpu().numpy()
    buckets, _, _ = (assign_tasks_ipo if use_ipo else assign_tasks_heap)(tasks, cp_size)
    order = torch.tensor([i for b in buckets for _, i in b], dtype=torch.int32)
    reranked = indices_rerank_cuda(startend_row_indices, order, balance_chunk_size)
    local = torch.tensor([i for _, i in buckets[cp_rank]], dtype=torch.int32)
    return indices_to_chunks_cuda(reranked, local, balance_chunk_size), buckets


def _sum_mask_heads(workload: torch.Tensor) -> torch.Tensor:
    # several mask heads: one task per chunk with the workload summed over heads
    w = workload[0, :, :, 0].sum(dim=0, dtype=torch.int32)
    return torch.stack([w, workload[0, 0, :, 1]], dim=-1)


def scatter_by_buckets(x: torch.Tensor, buckets: Sequence[Sequence[Tuple[int, int]]], rank: int,
                       axis: int = 1) -> torch.Tensor:
    """This rank's share of ``x`` along ``axis``: its chunks concatenated in
    bucket order (reference harness: tests/torch/distributed/cp_utils.py:16-48)."""
    n_chunks = sum(len(b) for b in buckets)
    c = x.shape[axis] // n_chunks
    return torch.cat([x.narrow(axis, i * c, c) for _, i in buckets[rank]], dim=axis).contiguous()


def dual_chunk_buckets(n_chunks: int, cp_size: int):
    """The mask-agnostic baseline split: rank r owns block r from the front and
    block 2*cp-1-r from the back (tests/torch/distributed/cp_utils.py:29-37),
    expressed as buckets over ``n_chunks`` chunks."""
    assert n_chunks % (2 * cp_size) == 0
    per = n_chunks // (2 * cp_size)
    out = []
    for r in range(cp_size):
        front = list(range(r * per, (r + 1) * per))
        back = list(range(n_chunks - (r + 1) * per, n_chunks - r * per))
        out.append([(0, i) for i in front + back])
    return out
