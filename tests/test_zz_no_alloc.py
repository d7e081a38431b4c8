"""The allocation-free backward entry point (fm_bwd_static_scratch) against the
regular one (fm_bwd), through the C ABI.

Some hosts of this library may not allocate device memory when they call it —
a runtime whose memory arena is frozen after start-up, or a plug-in that owns
nothing but the tensors handed to it.  For them the backward keeps its row
scratch in a fixed array inside the library.  Two calls in a row, on different
problems, check that nothing left in that shared array by the first call leaks
into the second.  This file sorts last so that a run stopping at the first
failure has already been through every other test.
"""
import ctypes as C
import math

import numpy as np
import pytest
import torch

import flashmask_b200 as fm
from flashmask_b200 import _lib, ops, workloads as W

pytestmark = pytest.mark.gpu


def _problem(B, S, Hq, Hkv, d, seed, sink):
    rng = np.random.default_rng(seed)
    idx_np = np.concatenate([W.causal_document(1, S, S, W.uniform_doc_lengths(rng, S, 5))[0]
                             for _ in range(B)])
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, S, Hq, d, generator=g).bfloat16().cuda()
    k = torch.randn(B, S, Hkv, d, generator=g).bfloat16().cuda()
    v = torch.randn(B, S, Hkv, d, generator=g).bfloat16().cuda()
    do = torch.randn(B, S, Hq, d, generator=g).bfloat16().cuda()
    sk = torch.randn(Hq, generator=g).cuda() if sink else None
    return q, k, v, do, torch.from_numpy(np.ascontiguousarray(idx_np).copy()).cuda(), sk


def _bwd_both(q, k, v, do, idx, sink):
    """Returns (regular, static-scratch) gradients for the same saved forward."""
    out, lse = fm._flash_attn_fwd(q, k, v, idx, causal=True, learnable_sink=sink)
    ref = fm._flash_attn_bwd(q, k, v, out, do, lse, idx, causal=True, learnable_sink=sink, deterministic=True)

    B, S, Hq, d = q.shape
    Hkv = k.shape[2]
    tm, tn = fm.bwd_tile_shape(d, d)
    info = fm.prepare_mask(idx, S, True, tm, tn)
    sink32 = None if sink is None else sink.float().contiguous()
    a = ops._base_args(q, k, v, out, lse, idx, info, True, 1.0 / math.sqrt(d), sink32)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    dsink = torch.empty(Hq, dtype=torch.float32, device=q.device) if sink is not None else None
    a.d_o, a.dq, a.dk, a.dv_out = do.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.do_stride, a.dq_stride = ops._strides(do), ops._strides(dq)
    a.dk_stride, a.dv_stride = ops._strides(dk), ops._strides(dv)
    if dsink is not None:
        a.dsink = dsink.data_ptr()
    stream = torch.cuda.current_stream().cuda_stream
    # the regular backward above has already run the same kernels, so their code is resident;
    # from here to the end of the call the amount of free device memory must not move
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    _lib.check(_lib.load().fm_bwd_static_scratch(C.byref(a), stream), "fm_bwd_static_scratch")
    torch.cuda.synchronize()
    free_after = torch.cuda.mem_get_info()[0]
    return ref, (dq, dk, dv, dsink), (free_before, free_after)


def test_static_scratch_matches_regular_backward_twice():
    first = _problem(2, 640, 4, 2, 128, seed=31, sink=True)
    second = _problem(1, 300, 2, 2, 64, seed=32, sink=False)   # smaller: stale rows stay behind it
    for n, prob in enumerate((first, second, first)):
        ref, got, (free_before, free_after) = _bwd_both(*prob)
        # both entry points run the same kernels in the same fixed summation order: same bits
        for name, r, g_ in zip(("dq", "dk", "dv"), ref[:3], got[:3]):
            assert not torch.isnan(g_.float()).any(), name
            assert torch.equal(g_, r), (name, (g_.float() - r.float()).abs().max().item())
        if prob[5] is not None:
            assert torch.equal(got[3], ref[3].float())
        if n > 0:     # the first call may still look up the array's address; later ones touch no allocator
            assert free_after == free_before, (free_before, free_after)


def test_static_scratch_rejects_oversize_without_launching():
    q, k, v, do, idx, _ = _problem(1, 128, 2, 2, 64, seed=33, sink=False)
    out, lse = fm._flash_attn_fwd(q, k, v, idx, causal=True)
    info = fm.prepare_mask(idx, 128, True, *fm.bwd_tile_shape(64, 64))
    a = ops._base_args(q, k, v, out, lse, idx, info, True, 0.125, None)
    a.d_o, a.dq, a.dk, a.dv_out = do.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.do_stride, a.dq_stride = ops._strides(do), ops._strides(q)
    a.dk_stride, a.dv_stride = ops._strides(k), ops._strides(v)
    a.B = 4096          # 4096 * 2 * 128 rows = 1,048,576 fits exactly ...
    a.Hq = 4            # ... doubling the heads does not
    a.Hkv = 4
    rc = _lib.load().fm_bwd_static_scratch(C.byref(a), None)
    assert rc == 4 and b"exceeds the built-in scratch" in _lib.load().fm_last_error()
