"""Dense-mask attention in fp32 on the CPU (checker, not product code).

Restates tests/torch/attention_ref.py:44-226 (``attention_ref``) of the
reference together with the bias expander
tests/common/startend_row_indices.py:188-222, and adds what the reference's
eager path does not return: the log-sum-exp (kernel definition
flashmask/cute/flash_fwd_sm100.py:4873-4879) and hand-derived gradients
(the reference obtains them with autograd over the same graph).
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch


def dense_bias(idx: Optional[np.ndarray], Sq: int, Sk: int, causal: bool) -> Optional[np.ndarray]:
    """Additive bias [B, Hm, Sq, Sk] float32: 0 where visible, -inf where masked.

    Vectorised restatement of startend_row_indices_to_attn_bias
    (tests/common/startend_row_indices.py:188-222): per column j rows
    [LTS, LTE) (or [LTS, Sq) when the mask has no LTE) are masked; causal adds
    rows [0, j-(Sk-Sq)); non-causal adds [UTS, UTE) (or [0, UTE))."""
    if idx is None:
        if not causal:
            return None
        i = np.arange(Sq)[:, None]
        j = np.arange(Sk)[None, :]
        m = np.where(j > i + (Sk - Sq), -np.inf, 0.0).astype(np.float32)
        return m[None, None]
    a = np.asarray(idx).astype(np.int64)
    Bm, Hm, Sk_, n = a.shape
    assert Sk_ == Sk
    i = np.arange(Sq, dtype=np.int64)[None, None, :, None]
    j = np.arange(Sk, dtype=np.int64)[None, None, None, :]
    col = [a[..., t][:, :, None, :] for t in range(n)]
    has_end = (causal and n == 2) or ((not causal) and n == 4)
    if has_end:
        masked = (i >= col[0]) & (i < col[1])
    else:
        masked = i >= col[0]
    if causal:
        masked = masked | (i < np.maximum(0, j - (Sk - Sq)))
    elif has_end:
        masked = masked | ((i >= col[2]) & (i < col[3]))
    else:
        masked = masked | (i < col[1])
    return np.where(masked, -np.inf, 0.0).astype(np.float32)


def _expand_heads(x: torch.Tensor, H: int) -> torch.Tensor:
    # [B, h, ...] -> [B, H, ...] repeating each head H//h times (GQA order
    # "b h s d -> b (h g) s d", attention_ref.py:124-127)
    h = x.shape[1]
    if h == H:
        return x
    return x.repeat_interleave(H // h, dim=1)


def attention_forward(q, k, v, idx=None, causal=False, sink=None, softmax_scale=None):
    """Returns (out [B,Sq,Hq,dv] fp32, lse [B,Hq,Sq] fp32, P [B,Hq,Sq,Sk] fp32).

    q [B,Sq,Hq,d], k [B,Sk,Hkv,d], v [B,Sk,Hkv,dv]: torch CPU tensors (any float
    dtype; computed in fp32 as attention_ref does with upcast=True,
    attention_ref.py:98-106).  Rows with no visible key give out = 0
    (attention_ref.py:177-178,197) and lse = -inf (sink present: lse = sink)."""
    q = q.to(torch.float32); k = k.to(torch.float32); v = v.to(torch.float32)
    B, Sq, Hq, d = q.shape
    Sk = k.shape[1]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    qh = q.permute(0, 2, 1, 3)
    kh = _expand_heads(k.permute(0, 2, 1, 3), Hq)
    vh = _expand_heads(v.permute(0, 2, 1, 3), Hq)
    scores = torch.matmul(qh * scale, kh.transpose(-1, -2))
    bias = dense_bias(None if idx is None else np.asarray(idx), Sq, Sk, causal)
    if bias is not None:
        bt = torch.from_numpy(bias)
        if bt.shape[0] != B:
            bt = bt.expand(B, -1, -1, -1)
        scores = scores + _expand_heads(bt, Hq)
    if sink is not None:
        s = sink.to(torch.float32).reshape(1, Hq, 1, 1).expand(B, Hq, Sq, 1)
        full = torch.cat([scores, s], dim=-1)
    else:
        full = scores
    lse = torch.logsumexp(full, dim=-1)                      # -inf for empty rows
    safe = torch.where(torch.isinf(lse) & (lse < 0), torch.zeros_like(lse), lse)
    P = torch.exp(scores - safe[..., None])
    P = torch.where(torch.isinf(scores) & (scores < 0), torch.zeros_like(P), P)
    out = torch.matmul(P, vh).permute(0, 2, 1, 3).contiguous()
    return out, lse, P


def attention_forward_backward(q, k, v, d_out, idx=None, causal=False, sink=None,
                               softmax_scale=None):
    """Forward plus gradients.  Returns dict(out, lse, dq, dk, dv, dsink).

    dP = dO V^T, dS = P * (dP - rowsum(O * dO)), dQ = scale dS K,
    dK = scale dS^T Q, dV = P^T dO, dsink[h] = -sum_{b,i} p_sink * rowsum(O*dO)
    (flashmask/cute/flash_bwd_sm100.py:129-140, flash_bwd_sink.py:67-114); GQA
    gradients of k/v sum over the q heads of a group."""
    q32 = q.to(torch.float32); k32 = k.to(torch.float32); v32 = v.to(torch.float32)
    do = d_out.to(torch.float32)
    B, Sq, Hq, d = q32.shape
    Sk, Hkv, dv = k32.shape[1], k32.shape[2], v32.shape[3]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    out, lse, P = attention_forward(q32, k32, v32, idx, causal, sink, scale)
    doh = do.permute(0, 2, 1, 3)
    qh = q32.permute(0, 2, 1, 3)
    kh = _expand_heads(k32.permute(0, 2, 1, 3), Hq)
    vh = _expand_heads(v32.permute(0, 2, 1, 3), Hq)
    dpsum = (out.permute(0, 2, 1, 3) * doh).sum(-1)           # [B,Hq,Sq]
    dP = torch.matmul(doh, vh.transpose(-1, -2))
    dS = P * (dP - dpsum[..., None])
    dq = torch.matmul(dS, kh) * scale
    dk_full = torch.matmul(dS.transpose(-1, -2), qh) * scale  # [B,Hq,Sk,d]
    dv_full = torch.matmul(P.transpose(-1, -2), doh)
    g = Hq // Hkv
    dk = dk_full.reshape(B, Hkv, g, Sk, d).sum(2)
    dvv = dv_full.reshape(B, Hkv, g, Sk, dv).sum(2)
    res = dict(out=out, lse=lse,
               dq=dq.permute(0, 2, 1, 3).contiguous(),
               dk=dk.permute(0, 2, 1, 3).contiguous(),
               dv=dvv.permute(0, 2, 1, 3).contiguous(), dsink=None)
    if sink is not None:
        s = sink.to(torch.float32).reshape(1, Hq, 1)
        p_sink = torch.exp(s - lse)
        p_sink = torch.where(torch.isinf(lse), torch.zeros_like(p_sink), p_sink)
        res["dsink"] = -(p_sink * dpsum).sum(dim=(0, 2))
    return res


def block_logit_ref(q, k, idx=None, causal=False, softmax_scale=None, block_size=64,
                    num_blocks=None, block_bos=None):
    """Per (query row, block of key columns) maximum of the masked, scaled scores:
    [B, Hq, Sq, num_blocks] fp32, -inf where every column of the block is masked (or outside the
    sequence).

    Restates the checker of the reference's fused block-score epilogue
    (tests/paddle/test_block_score_fusion.py:62-87 ``ref_block_logit`` and :253-273 for GQA: scaled
    logit ``softmax_scale * q.k``, masked columns -inf, columns padded to whole blocks with -inf,
    max over each block) and extends it the way the kernel defines it
    (flashmask/cute/flash_fwd_sm100.py:4273-4371): the mask is the attention's own (column bounds
    and causal), and with ``block_bos`` ([B, Sq] int, first key column of the row's document) the
    block of column j for row i is ``floor((j - bos[i]) / block_size)``; blocks below 0 or at or
    past ``ceil(Sk / block_size)`` are dropped.  The reference's own test needs Paddle on an SM 10.x
    GPU and cannot run where this file is checked: parity unpinned beyond this restatement."""
    q = q.to(torch.float32); k = k.to(torch.float32)
    B, Sq, Hq, d = q.shape
    Sk = k.shape[1]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    qh = q.permute(0, 2, 1, 3)
    kh = _expand_heads(k.permute(0, 2, 1, 3), Hq)
    scores = torch.matmul(qh, kh.transpose(-1, -2)) * scale
    bias = dense_bias(None if idx is None else np.asarray(idx), Sq, Sk, causal)
    if bias is not None:
        bt = torch.from_numpy(bias)
        if bt.shape[0] != B:
            bt = bt.expand(B, -1, -1, -1)
        scores = scores + _expand_heads(bt, Hq)
    n_cols = -(-Sk // block_size)
    nb = n_cols if num_blocks is None else num_blocks
    out = torch.full((B, Hq, Sq, nb), float("-inf"), dtype=torch.float32)
    bos = torch.zeros((B, Sq), dtype=torch.int64) if block_bos is None else torch.as_tensor(block_bos).to(torch.int64)
    j = torch.arange(Sk, dtype=torch.int64)
    blk = torch.div(j[None, None, :] - bos[:, :, None], block_size, rounding_mode="floor")   # [B, Sq, Sk]
    ok = (blk >= 0) & (blk < n_cols)
    blk = blk.clamp(0, nb - 1)[:, None].expand(B, Hq, Sq, Sk)
    src = torch.where(ok[:, None].expand(B, Hq, Sq, Sk), scores, torch.full_like(scores, float("-inf")))
    out.scatter_reduce_(3, blk, src, reduce="amax", include_self=True)
    return out


# ---------------------------------------------------------------------------
# The same mathematics for ONE (batch, head) on a subset of query rows or key columns, so that
# the benchmark configurations can be checked at their full sequence lengths (8K-128K tokens),
# where a dense [Sq, Sk] score matrix of every head no longer fits the checker's memory or time.
# ---------------------------------------------------------------------------
def visible_block(bounds: Optional[np.ndarray], Sq: int, Sk: int, causal: bool,
                  rows: np.ndarray, cols: np.ndarray) -> np.ndarray:
    """bool [len(rows), len(cols)]: element (row, col) is unmasked.  ``bounds`` is the mask of one
    (batch, mask head), ``[Sk, ncols]`` int, or None.  Same predicate as ``dense_bias`` (restating
    tests/common/startend_row_indices.py:188-222), evaluated for the given global row / column
    indices only."""
    i = np.asarray(rows, dtype=np.int64)[:, None]
    j = np.asarray(cols, dtype=np.int64)[None, :]
    masked = np.zeros((i.shape[0], j.shape[1]), dtype=bool)
    if bounds is not None:
        a = np.asarray(bounds)[np.asarray(cols)].astype(np.int64)       # [C, n]
        n = a.shape[1]
        has_end = (causal and n == 2) or ((not causal) and n == 4)
        masked = ((i >= a[:, 0]) & (i < a[:, 1])) if has_end else (i >= a[:, 0])
        if not causal:
            masked = masked | (((i >= a[:, 2]) & (i < a[:, 3])) if has_end else (i < a[:, 1]))
    if causal:
        masked = masked | (j > i + (Sk - Sq))
    return ~masked


def candidate_columns(bounds: Optional[np.ndarray], Sq: int, Sk: int, causal: bool,
                      rmin: int, rmax: int) -> np.ndarray:
    """Key columns that are not masked for EVERY row of [rmin, rmax] (a superset of the columns
    some row of that range sees), from the bounds alone in O(Sk): a column is dropped when one of
    its masked row intervals covers the whole range, or when it lies in the causal future of rmax."""
    j = np.arange(Sk, dtype=np.int64)
    drop = np.zeros(Sk, dtype=bool)
    if bounds is not None:
        a = np.asarray(bounds).astype(np.int64)
        n = a.shape[1]
        has_end = (causal and n == 2) or ((not causal) and n == 4)
        drop = (a[:, 0] <= rmin) & ((a[:, 1] > rmax) if has_end else True)
        if not causal:
            drop = drop | (((a[:, 2] <= rmin) & (a[:, 3] > rmax)) if has_end else (a[:, 1] > rmax))
    if causal:
        drop = drop | (j > rmax + (Sk - Sq))
    return np.nonzero(~drop)[0]


def attention_rows(q, k, v, d_out, bounds, causal, sink=None, softmax_scale=None, rows=None,
                   chunk=1024, grads=True):
    """fp32 attention of ONE head restricted to the query rows ``rows`` (all rows when None).

    q ``[Sq, d]``, k ``[Sk, d]``, v ``[Sk, dv]``, d_out ``[Sq, dv]`` (torch CPU), ``bounds``
    ``[Sk, ncols]`` numpy or None, ``sink`` a python float or None.  Returns a dict with, for the
    selected rows in order, ``out [R, dv]``, ``lse [R]``, ``dpsum [R]``, ``dq [R, d]`` and the
    contribution of those rows to ``dk [Sk, d]`` / ``dv [Sk, dv]`` (the full gradient of this head
    when every row is selected).  Same formulas as ``attention_forward_backward``; rows are walked in
    chunks and each chunk only touches the key columns at least one of its rows can see."""
    q = q.to(torch.float32); k = k.to(torch.float32); v = v.to(torch.float32)
    do = d_out.to(torch.float32) if d_out is not None else None
    Sq, d = q.shape
    Sk, dv = v.shape
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    rows = np.arange(Sq, dtype=np.int64) if rows is None else np.asarray(rows, dtype=np.int64)
    R = rows.shape[0]
    res = dict(out=torch.zeros(R, dv), lse=torch.full((R,), float("-inf")), dpsum=torch.zeros(R))
    if grads:
        res.update(dq=torch.zeros(R, d), dk=torch.zeros(Sk, d), dv=torch.zeros(Sk, dv))
    for c0 in range(0, R, chunk):
        rr = rows[c0:c0 + chunk]
        cand = candidate_columns(bounds, Sq, Sk, causal, int(rr.min()), int(rr.max()))
        vis_np = visible_block(bounds, Sq, Sk, causal, rr, cand)
        keep = vis_np.any(axis=0)
        cols = cand[keep]
        sl = slice(c0, c0 + rr.shape[0])
        if sink is not None:
            res["lse"][sl] = float(sink)
        if cols.size == 0:
            continue
        vis = torch.from_numpy(vis_np[:, keep])
        ct = torch.from_numpy(cols)
        rt = torch.from_numpy(rr)
        kc, vc = k[ct], v[ct]
        s = torch.matmul(q[rt] * scale, kc.T)
        s = torch.where(vis, s, torch.full_like(s, float("-inf")))
        full = s if sink is None else torch.cat([s, torch.full((rr.shape[0], 1), float(sink))], dim=1)
        lse = torch.logsumexp(full, dim=-1)
        safe = torch.where(torch.isinf(lse) & (lse < 0), torch.zeros_like(lse), lse)
        P = torch.where(vis, torch.exp(s - safe[:, None]), torch.zeros_like(s))
        out = torch.matmul(P, vc)
        res["out"][sl] = out
        res["lse"][sl] = lse
        if do is None:
            continue
        dor = do[rt]
        dpsum = (out * dor).sum(-1)
        res["dpsum"][sl] = dpsum
        if not grads:
            continue
        dP = torch.matmul(dor, vc.T)
        dS = P * (dP - dpsum[:, None])
        res["dq"][sl] = torch.matmul(dS, kc) * scale
        res["dk"].index_add_(0, ct, torch.matmul(dS.T, q[rt]) * scale)
        res["dv"].index_add_(0, ct, torch.matmul(P.T, dor))
    return res


def attention_columns(q, k_cols, v_cols, d_out, lse, dpsum, bounds, causal, cols, Sk,
                      softmax_scale=None, chunk=2048):
    """fp32 dK / dV of the key columns ``cols`` of ONE kv head: ``dk [C, d]``, ``dv [C, dv]``.

    q ``[G, Sq, d]`` and d_out ``[G, Sq, dv]`` are the q heads of the kv head's group; ``lse`` and
    ``dpsum`` ``[G, Sq]`` their row statistics (natural-log LSE, rowsum(O * dO)); ``k_cols`` /
    ``v_cols`` the selected rows of k / v.  dV = P^T dO and dK = scale * dS^T Q summed over the
    group (flashmask/cute/flash_bwd_sm100.py:129-140), with P = exp(S - LSE) from the given LSE."""
    q = q.to(torch.float32); do = d_out.to(torch.float32)
    kc = k_cols.to(torch.float32); vc = v_cols.to(torch.float32)
    lse = lse.to(torch.float32); dpsum = dpsum.to(torch.float32)
    G, Sq, d = q.shape
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    cols = np.asarray(cols, dtype=np.int64)
    dk = torch.zeros(cols.shape[0], d)
    dvv = torch.zeros(cols.shape[0], vc.shape[1])
    for r0 in range(0, Sq, chunk):
        rr = np.arange(r0, min(r0 + chunk, Sq), dtype=np.int64)
        vis_np = visible_block(bounds, Sq, Sk, causal, rr, cols)
        if not vis_np.any():
            continue
        vis = torch.from_numpy(vis_np)
        for g in range(G):
            l = lse[g, r0:r0 + rr.shape[0]]
            dead = torch.isinf(l)
            s = torch.matmul(q[g, r0:r0 + rr.shape[0]] * scale, kc.T)
            P = torch.exp(s - torch.where(dead, torch.zeros_like(l), l)[:, None])
            P = torch.where(vis & ~dead[:, None], P, torch.zeros_like(P))
            dor = do[g, r0:r0 + rr.shape[0]]
            dS = P * (torch.matmul(dor, vc.T) - dpsum[g, r0:r0 + rr.shape[0]][:, None])
            dk += torch.matmul(dS.T, q[g, r0:r0 + rr.shape[0]]) * scale
            dvv += torch.matmul(P.T, dor)
    return dk, dvv
