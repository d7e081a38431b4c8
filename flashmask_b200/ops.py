"""Host orchestration of the forward / backward operator.

Mirrors the reference's orchestration layer: ``_flash_attn_fwd`` /
``_flash_attn_bwd`` (flashmask/cute/ops/fwd.py:52-882, ops/bwd.py:56-1261) and
the mask-preprocessing entry points (flashmask/cute/flashmask_utils.py).  All
device work is done by libflashmask_b200.so through its C ABI; torch supplies
device memory and the current stream only.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple

import torch

from . import _lib

__all__ = ["FlashMaskInfo", "prepare_mask", "count_visible", "_flash_attn_fwd", "_flash_attn_bwd",
           "fwd_tile_shape", "bwd_tile_shape"]


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _lib.FM_DTYPE_BF16
    if t.dtype == torch.float16:
        return _lib.FM_DTYPE_FP16
    raise TypeError(f"flashmask_attention supports bfloat16 / float16, got {t.dtype}")


def fwd_tile_shape(d: int, dv: int) -> Tuple[int, int]:
    m, n = C.c_int(), C.c_int()
    _lib.check(_lib.load().fm_fwd_tile_shape(d, dv, C.byref(m), C.byref(n)), "fm_fwd_tile_shape")
    return m.value, n.value


def bwd_tile_shape(d: int, dv: int) -> Tuple[int, int]:
    m, n = C.c_int(), C.c_int()
    _lib.check(_lib.load().fm_bwd_tile_shape(d, dv, C.byref(m), C.byref(n)), "fm_bwd_tile_shape")
    return m.value, n.value


@dataclass
class FlashMaskInfo:
    """The mask plus its per-K-tile reductions (reference container:
    FlashMaskInfoPaddle, flashmask/cute/flashmask_utils.py:81-93)."""
    startend_row_indices: torch.Tensor          # [B, Hm, Sk, ncols] int32
    causal: bool
    tile_m: int
    tile_n: int
    minmax: torch.Tensor                        # [8, B*Hm, nblk_pad] int32
    valid_block_count: Optional[torch.Tensor]   # [B, Hm, Tq] int32
    tile_class: Optional[torch.Tensor]          # [B, Hm, Tq, Tk] int8
    # longest-work-first launch tables, built on first use: (which, d, dv, Sq, B, Hq, Hkv) -> int32 tensor or None
    orders: Dict[tuple, Optional[torch.Tensor]] = field(default_factory=dict)


def prepare_mask(idx: torch.Tensor, Sq: int, causal: bool, tile_m: int, tile_n: int,
                 want_count: bool = False, want_class: bool = False) -> FlashMaskInfo:
    """Per-K-tile min/max of every bound column and, on request, the surviving
    tile count and the (Q tile, K tile) class map."""
    assert idx.is_cuda and idx.dtype == torch.int32 and idx.dim() == 4
    idx = idx.contiguous()
    B, Hm, Sk, ncols = idx.shape
    lib = _lib.load()
    pad = lib.fm_mask_nblk_pad(Sk, tile_n)
    tq, tk = -(-Sq // tile_m), -(-Sk // tile_n)
    minmax = torch.empty((8, B * Hm, pad), dtype=torch.int32, device=idx.device)
    cnt = torch.empty((B, Hm, tq), dtype=torch.int32, device=idx.device) if want_count else None
    cls = torch.empty((B, Hm, tq, tk), dtype=torch.int8, device=idx.device) if want_class else None
    _lib.check(lib.fm_mask_prepare(idx.data_ptr(), B, Hm, Sq, Sk, ncols, int(causal), tile_m, tile_n,
                                   minmax.data_ptr(), cnt.data_ptr() if want_count else None,
                                   cls.data_ptr() if want_class else None, _stream(idx)),
               "fm_mask_prepare")
    return FlashMaskInfo(idx, causal, tile_m, tile_n, minmax, cnt, cls)


def _launch_order(a: "_lib.AttnArgs", info: FlashMaskInfo, which: int, ref: torch.Tensor) -> Optional[int]:
    """Device pointer of the launch table ``which`` (FM_ORDER_*) for this mask and kernel
    variant, or None when the variant takes none.  The tables of all three kernels are built
    together on first use, once per FlashMaskInfo (ONE small launch on the current stream).
    FLASHMASK_B200_ORDER=0 turns all tables off, a comma list out of fwd,dq,dkdv keeps only
    those (A/B runs)."""
    sel = os.environ.get("FLASHMASK_B200_ORDER", "1")
    names = ("fwd", "dq", "dkdv")
    wanted = [w for w in range(3) if sel == "1" or names[w] in sel.split(",")]
    if which not in wanted or info.tile_n != 128:
        return None     # the tables are counted in the 128-column tiles of the tcgen05 kernels, which alone read them
    geom = (a.d, a.dv, a.Sq, a.B, a.Hq, a.Hkv)
    if (which,) + geom not in info.orders:
        lib = _lib.load()
        bufs = [None, None, None]
        for w in wanted:
            if (w,) + geom in info.orders:
                continue
            n = lib.fm_launch_order_ints(C.byref(a), w)
            bufs[w] = torch.empty(n, dtype=torch.int32, device=ref.device) if n else None
            info.orders[(w,) + geom] = bufs[w]
        if any(t is not None for t in bufs):
            _lib.check(lib.fm_launch_orders(C.byref(a), *[None if t is None else t.data_ptr() for t in bufs],
                                            _stream(ref)), "fm_launch_orders")
    buf = info.orders[(which,) + geom]
    return None if buf is None else buf.data_ptr()


def count_visible(idx: torch.Tensor, Sq: int, causal: bool) -> torch.Tensor:
    """int64 [B, Hm]: exact number of unmasked (query, key) pairs."""
    idx = idx.contiguous()
    B, Hm, Sk, ncols = idx.shape
    out = torch.empty((B, Hm), dtype=torch.int64, device=idx.device)
    _lib.check(_lib.load().fm_mask_count_visible(idx.data_ptr(), B, Hm, Sq, Sk, ncols, int(causal),
                                                 out.data_ptr(), _stream(idx)), "fm_mask_count_visible")
    return out


def _last_dim_contiguous(t: torch.Tensor) -> torch.Tensor:
    return t if t.stride(-1) == 1 else t.contiguous()


def _strides(t: torch.Tensor):
    return _lib.I64x3(t.stride(0), t.stride(1), t.stride(2))


def _base_args(q, k, v, out, lse, idx, info, causal, softmax_scale, sink) -> _lib.AttnArgs:
    B, Sq, Hq, d = q.shape
    _, Sk, Hkv, dv = v.shape
    a = _lib.AttnArgs()
    a.B, a.Sq, a.Sk, a.Hq, a.Hkv = B, Sq, Sk, Hq, Hkv
    a.d, a.dv = d, dv
    a.causal = int(causal)
    a.dtype = _dtype_code(q)
    a.softmax_scale = softmax_scale
    a.q, a.k, a.v, a.o, a.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr()
    a.q_stride, a.k_stride, a.v_stride, a.o_stride = _strides(q), _strides(k), _strides(v), _strides(out)
    if idx is not None:
        a.ncols = idx.shape[-1]
        a.Hm = idx.shape[1]
        a.mask_B = idx.shape[0]
        a.mask = info.startend_row_indices.data_ptr()
        a.minmax = info.minmax.data_ptr()
        a.tile_m, a.tile_n = info.tile_m, info.tile_n
    else:
        a.ncols, a.Hm, a.mask_B = 0, 1, 1
    if sink is not None:
        a.sink = sink.data_ptr()
    return a


def _check_shapes(q, k, v, idx, causal):
    assert q.dim() == 4 and k.dim() == 4 and v.dim() == 4, "q/k/v must be [B, S, H, D]"
    B, Sq, Hq, d = q.shape
    Bk, Sk, Hkv, dk = k.shape
    assert (Bk, dk) == (B, d) and v.shape[:3] == k.shape[:3], "k/v shapes do not match q"
    assert Hq % Hkv == 0, "num q heads must be a multiple of num kv heads"
    assert q.dtype == k.dtype == v.dtype, "q/k/v must share a dtype"
    if idx is not None:
        assert idx.dtype == torch.int32, "startend_row_indices must be int32"
        assert idx.dim() == 4, "startend_row_indices must be [B, Hm, Sk, n]"
        assert idx.shape[0] in (B, 1), "startend_row_indices batch must match q"
        assert idx.shape[2] == Sk, "startend_row_indices seqlen must match k"
        assert idx.shape[1] in (1, Hkv), "startend_row_indices heads must be 1 or num kv heads"
        if causal:
            assert idx.shape[-1] in (1, 2), "causal masks carry 1 or 2 bounds per column"
        else:
            assert idx.shape[-1] in (2, 4), "non-causal masks carry 2 or 4 bounds per column"


# head-dim pairs for which the reference folds dV into dK when value aliases key
# (_LARGE_HDIMS, flashmask/cute/ops/bwd.py:136-139)
_KV_SHARED_HDIMS = ((512, 512), (576, 512))


def _kv_shared(k: torch.Tensor, v: torch.Tensor) -> bool:
    """True when ``v`` is ``k[..., :dv]`` on the same storage (MLA-style shared K/V) at one of the
    head-dim pairs for which the reference merges the two gradients; at every other head dim an
    aliased value keeps its own dV, as in the reference."""
    return ((k.shape[-1], v.shape[-1]) in _KV_SHARED_HDIMS
            and v.data_ptr() == k.data_ptr() and v.shape[:-1] == k.shape[:-1] and v.stride() == k.stride())


def _sink_fp32(sink, Hq, device):
    if sink is None:
        return None
    assert sink.numel() == Hq, "learnable_sink must have one logit per q head"
    return sink.detach().reshape(Hq).to(device=device, dtype=torch.float32).contiguous()


def _flash_attn_fwd(q, k, v, startend_row_indices=None, softmax_scale=None, causal=False,
                    learnable_sink=None, return_lse=True, mask_info: Optional[FlashMaskInfo] = None,
                    block_logit: Optional[torch.Tensor] = None, block_size: int = 64,
                    block_bos: Optional[torch.Tensor] = None, pack_gqa: Optional[bool] = False):
    """Forward.  Returns (out [B,Sq,Hq,dv], lse [B,Hq,Sq] fp32).

    With ``block_logit`` (fp32 ``[B, Hq, Sq, >= ceil(Sk / block_size)]``, filled with -inf by the
    caller) the kernel also merges into it, with fmax, the maximum of the masked, scaled scores of
    every (query row, block of ``block_size`` key columns); ``block_bos`` (int32 ``[B, Sq]``, first
    key of the row's document) makes the block ids document-relative.  Queries are never packed
    over the heads of a GQA group here, so ``pack_gqa`` must be False (or left at its default);
    the reference defaults it to True under GQA and rejects that combination.

    Reference: _flash_attn_fwd, flashmask/cute/ops/fwd.py:52-882 (same argument
    meaning; block-score arguments :75-77,605-658; split-KV and pack-GQA are not part of
    this operator surface)."""
    if not q.is_cuda:
        raise RuntimeError("flashmask_b200 runs on CUDA (sm_100a) tensors only; there is no CPU path")
    idx = startend_row_indices
    _check_shapes(q, k, v, idx, causal)
    q, k, v = _last_dim_contiguous(q), _last_dim_contiguous(k), _last_dim_contiguous(v)
    B, Sq, Hq, d = q.shape
    Sk, dv = k.shape[1], v.shape[3]
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(d)
    tm, tn = fwd_tile_shape(d, dv)
    info = mask_info
    if idx is not None and (info is None or info.tile_n != tn):
        info = prepare_mask(idx, Sq, causal, tm, tn)
    out = torch.empty((B, Sq, Hq, dv), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
    sink32 = _sink_fp32(learnable_sink, Hq, q.device)
    a = _base_args(q, k, v, out, lse, idx, info, causal, softmax_scale, sink32)
    if info is not None:
        a.fwd_order = _launch_order(a, info, _lib.FM_ORDER_FWD, q)
    if block_logit is None:
        assert block_bos is None, "block_bos requires block_logit (it drives its relative bucketing)"
        _lib.check(_lib.load().fm_fwd(C.byref(a), _stream(q)), "fm_fwd")
        return out, lse
    assert not pack_gqa, "block_logit requires pack_gqa=False: it is indexed by the query head and the query row"
    assert block_logit.dtype == torch.float32, f"block_logit must be float32; got {block_logit.dtype}"
    assert block_logit.is_cuda, "block_logit must be on CUDA"
    assert block_logit.ndim == 4, (
        f"block_logit must be [batch, num_heads, seqlen_q, num_blocks]; got ndim={block_logit.ndim}")
    nb_min = -(-Sk // block_size)
    assert tuple(block_logit.shape[:3]) == (B, Hq, Sq) and block_logit.is_contiguous(), (
        f"block_logit must be a contiguous [B={B}, H={Hq}, S={Sq}, num_blocks]; got {tuple(block_logit.shape)}")
    assert block_logit.shape[-1] >= nb_min, (
        f"block_logit num_blocks={block_logit.shape[-1]} < ceil(seqlen_k/block_size)={nb_min}")
    bos_ptr = None
    if block_bos is not None:
        assert block_bos.dtype == torch.int32, f"block_bos must be int32; got {block_bos.dtype}"
        assert block_bos.is_cuda, "block_bos must be on CUDA"
        assert tuple(block_bos.shape) == (B, Sq), f"block_bos must be [B={B}, S={Sq}]; got {tuple(block_bos.shape)}"
        block_bos = block_bos.contiguous()
        bos_ptr = block_bos.data_ptr()
    _lib.check(_lib.load().fm_fwd_block_score(C.byref(a), block_logit.data_ptr(), int(block_size),
                                              int(block_logit.shape[-1]), bos_ptr, _stream(q)),
               "fm_fwd_block_score")
    return out, lse


def _flash_attn_bwd(q, k, v, out, dout, lse, startend_row_indices=None, softmax_scale=None,
                    causal=False, learnable_sink=None, deterministic=False,
                    mask_info: Optional[FlashMaskInfo] = None, dq_chain: Optional[dict] = None):
    """Backward.  Returns (dq, dk, dv, dsink | None).

    ``dq_chain`` (context parallel): a dict shared by the backward calls over the same queries
    (``{"last": bool}`` set by the caller for each call).  When the one-kernel backward serves
    the calls, their dQ is summed in its fp32 accumulator and rounded once: every call but the
    last returns ``dq = None``.  When another variant serves them, every call returns its own dq
    and the caller adds them; ``dq_chain["summed"]`` tells which happened.

    Reference: _flash_attn_bwd, flashmask/cute/ops/bwd.py:56-1261."""
    idx = startend_row_indices
    _check_shapes(q, k, v, idx, causal)
    q, k, v = _last_dim_contiguous(q), _last_dim_contiguous(k), _last_dim_contiguous(v)
    out, dout = _last_dim_contiguous(out), _last_dim_contiguous(dout)
    B, Sq, Hq, d = q.shape
    Sk, Hkv, dv = k.shape[1], k.shape[2], v.shape[3]
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(d)
    tm, tn = bwd_tile_shape(d, dv)
    info = mask_info
    if idx is not None and (info is None or info.tile_n != tn):
        info = prepare_mask(idx, Sq, causal, tm, tn)
    dq = torch.empty_like(q)
    dk = torch.empty((B, Sk, Hkv, d), dtype=k.dtype, device=k.device)
    dvv = torch.empty((B, Sk, Hkv, dv), dtype=v.dtype, device=v.device)
    sink32 = _sink_fp32(learnable_sink, Hq, q.device)
    dsink32 = torch.empty(Hq, dtype=torch.float32, device=q.device) if sink32 is not None else None
    lse = lse.contiguous()
    a = _base_args(q, k, v, out, lse, idx, info, causal, softmax_scale, sink32)
    a.d_o, a.dq, a.dk, a.dv_out = dout.data_ptr(), dq.data_ptr(), dk.data_ptr(), dvv.data_ptr()
    a.do_stride, a.dq_stride, a.dk_stride, a.dv_stride = _strides(dout), _strides(dq), _strides(dk), _strides(dvv)
    a.deterministic = int(bool(deterministic))
    if dsink32 is not None:
        a.dsink = dsink32.data_ptr()
    lib = _lib.load()
    if info is not None:
        a.dq_order = _launch_order(a, info, _lib.FM_ORDER_BWD_DQ, q)
        a.dkdv_order = _launch_order(a, info, _lib.FM_ORDER_BWD_DKDV, q)
    nbytes = lib.fm_bwd_workspace_bytes(C.byref(a))
    chained = dq_chain is not None and bool(lib.fm_bwd_accumulates(C.byref(a)))
    if chained:
        # one workspace for the whole chain: the accumulator carries the sums from call to call
        if "ws" in dq_chain:
            a.bwd_flags |= _lib.FM_BWD_DQ_CARRY
        else:
            dq_chain["ws"] = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=q.device)
        if not dq_chain.get("last", False):
            a.bwd_flags |= _lib.FM_BWD_DQ_LEAVE
        ws = dq_chain["ws"]
        assert ws.numel() >= nbytes, "the backward calls of a chain must share one problem geometry"
    else:
        ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=q.device)
    if dq_chain is not None:
        dq_chain["summed"] = chained
    a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
    _lib.check(lib.fm_bwd(C.byref(a), _stream(q)), "fm_bwd")
    if chained and not dq_chain.get("last", False):
        dq = None
    if _kv_shared(k, v):
        # value is a view of key's leading dv columns on the same storage: the
        # gradient of that storage is dK with dV folded into its leading columns,
        # and the value slot returns zeros (reference convention,
        # flashmask/cute/ops/_common.py:52-88)
        dk[..., :dv] += dvv
        dvv.zero_()
    dsink = None
    if dsink32 is not None:
        dsink = dsink32.to(learnable_sink.dtype).reshape(learnable_sink.shape)
    return dq, dk, dvv, dsink
