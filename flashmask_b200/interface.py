"""Public operator: ``flashmask_attention`` and its autograd function.

Drop-in for the reference surface
``flashmask.flashmask_attention(q, k, v, startend_row_indices, *, causal,
softmax_scale, learnable_sink, return_lse, group)``
(flashmask/frontend/torch/__init__.py:37-102, autograd.py:32-103), plus the
Paddle-side keyword names ``window_size`` / ``return_softmax_lse``
(flashmask/frontend/paddle/__init__.py:30-82) and an explicit ``deterministic``
switch (the reference reads torch.are_deterministic_algorithms_enabled(),
frontend/torch/autograd.py:86; ``None`` keeps that behaviour).
"""
from __future__ import annotations

from typing import Optional, Tuple, Union

import torch

from .ops import _check_shapes, _flash_attn_bwd, _flash_attn_fwd, fwd_tile_shape, prepare_mask

__all__ = ["flashmask_attention", "FlashMaskFunc", "sliding_window_indices"]


class FlashMaskFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, startend_row_indices, softmax_scale, causal, learnable_sink,
                deterministic):
        # the mask is scanned once: forward and backward share its per-K-tile reductions and the
        # launch tables whenever their kernel variants tile the keys alike
        if not q.is_cuda:
            raise RuntimeError("flashmask_b200 runs on CUDA (sm_100a) tensors only; there is no CPU path")
        _check_shapes(q, k, v, startend_row_indices, causal)
        info = None
        if startend_row_indices is not None:
            tm, tn = fwd_tile_shape(q.shape[-1], v.shape[-1])
            info = prepare_mask(startend_row_indices, q.shape[1], causal, tm, tn)
        out, lse = _flash_attn_fwd(q, k, v, startend_row_indices, softmax_scale=softmax_scale,
                                   causal=causal, learnable_sink=learnable_sink, return_lse=True,
                                   mask_info=info)
        ctx.save_for_backward(q, k, v, startend_row_indices, out, lse, learnable_sink)
        ctx.mask_info = info
        ctx.softmax_scale = softmax_scale
        ctx.causal = causal
        ctx.deterministic = deterministic
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, dout, dlse):
        q, k, v, idx, out, lse, sink = ctx.saved_tensors
        det = ctx.deterministic
        if det is None:
            det = torch.are_deterministic_algorithms_enabled()
        dq, dk, dv, dsink = _flash_attn_bwd(q, k, v, out, dout, lse, idx, softmax_scale=ctx.softmax_scale,
                                            causal=ctx.causal, learnable_sink=sink, deterministic=det,
                                            mask_info=ctx.mask_info)
        return dq, dk, dv, None, None, None, dsink, None


def sliding_window_indices(Sq: int, Sk: int, window_size: Union[int, Tuple[int, int]], causal: bool,
                           batch: int, device) -> torch.Tensor:
    """Column bounds of a sliding window (the reference leaves ``window_size``
    unimplemented; its test generator builds the same bounds,
    tests/common/startend_row_indices.py:92-97).  An int ``w`` with ``causal=True`` is the reference
    generator's window: key j is visible to rows j .. j+w-1.  A ``(left, right)``
    pair follows the flash-attention convention: key j is visible to rows
    j - right .. j + left."""
    j = torch.arange(Sk, dtype=torch.int64, device=device)
    if causal:
        span = window_size if isinstance(window_size, int) else window_size[0] + 1
        lts = torch.clamp(j + span, max=Sq)
        idx = lts.view(1, 1, Sk, 1)
    else:
        left, right = (window_size, window_size) if isinstance(window_size, int) else window_size
        lts = torch.clamp(j + left + 1, max=Sq)
        ute = torch.clamp(j - right, min=0)
        idx = torch.stack([lts, ute], dim=-1).view(1, 1, Sk, 2)
    return idx.expand(batch, 1, Sk, idx.shape[-1]).to(torch.int32).contiguous()


def flashmask_attention(query, key, value, startend_row_indices: Optional[torch.Tensor] = None, *,
                        causal: bool = False, window_size=None, softmax_scale: Optional[float] = None,
                        sink: Optional[torch.Tensor] = None, learnable_sink: Optional[torch.Tensor] = None,
                        deterministic: Optional[bool] = None, return_softmax_lse: bool = False,
                        return_lse: bool = False, dropout: float = 0.0, group=None):
    """FlashMask attention: ``softmax(Q K^T * scale + M) V`` with the mask ``M``
    given column-wise by ``startend_row_indices`` ``[B, Hm, Sk, 1|2|4]`` int32.

    query ``[B, Sq, Hq, d]``, key ``[B, Sk, Hkv, d]``, value ``[B, Sk, Hkv, dv]``
    (bf16 / fp16, CUDA).  Returns ``out [B, Sq, Hq, dv]`` or ``(out, lse)`` when
    ``return_lse`` / ``return_softmax_lse`` is set (``lse [B, Hq, Sq]`` fp32).
    ``group``: a torch.distributed process group with more than one rank runs
    the context-parallel path (key/value are this rank's shards)."""
    assert dropout == 0.0, "dropout is not supported"
    if sink is not None and learnable_sink is not None:
        raise ValueError("pass either sink or learnable_sink, not both")
    sink = sink if sink is not None else learnable_sink
    if window_size is not None:
        if startend_row_indices is not None:
            raise ValueError("window_size cannot be combined with startend_row_indices")
        startend_row_indices = sliding_window_indices(query.shape[1], key.shape[1], window_size, causal,
                                                      query.shape[0], query.device)
    want_lse = return_lse or return_softmax_lse
    if group is not None and torch.distributed.is_initialized() and torch.distributed.get_world_size(group) > 1:
        from .cp import cp_flashmask_attention
        out, lse = cp_flashmask_attention(query, key, value, startend_row_indices, causal=causal,
                                          softmax_scale=softmax_scale, sink=sink,
                                          deterministic=deterministic, group=group)
    else:
        out, lse = FlashMaskFunc.apply(query, key, value, startend_row_indices, softmax_scale, causal,
                                       sink, deterministic)
    return (out, lse) if want_lse else out
