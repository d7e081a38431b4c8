"""CPU-side checks: the shared library exports what the header declares, the
host helpers behave, the workload generators have the promised shapes."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import flashmask_b200 as fm
from flashmask_b200 import _lib, workloads as W

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = ""
    inc = os.path.join(ROOT, "include")
    for f in sorted(os.listdir(inc)):
        if f.endswith(".h"):
            text += open(os.path.join(inc, f)).read()
    return sorted(set(re.findall(r"FM_API\s+[\w\s\*]+?\b(fm_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = _declared()
    assert len(names) >= 10
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/*.h but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes binding and header disagree"


def test_version_and_pad_without_gpu():
    lib = _lib.load()
    assert b"sm_100a" in lib.fm_version()
    for sk, tn in [(1, 64), (8192, 128), (8193, 128), (333, 32)]:
        assert lib.fm_mask_nblk_pad(sk, tn) == ((sk + tn - 1) // tn + 3) & ~3


def test_argument_errors_need_no_gpu():
    lib = _lib.load()
    rc = lib.fm_mask_prepare(None, 1, 1, 8, 8, 3, 1, 64, 64, None, None, None, None)
    assert rc == 1 and b"ncols" in lib.fm_last_error()
    a = _lib.AttnArgs()
    assert lib.fm_fwd(ctypes.byref(a), None) == 1
    assert lib.fm_fwd_block_score(ctypes.byref(a), None, 64, 1, None, None) == 1
    assert b"block_logit is NULL" in lib.fm_last_error()
    with pytest.raises(NotImplementedError):
        fm.fwd_tile_shape(100, 300)
    with pytest.raises(RuntimeError):
        q = torch.zeros(1, 8, 1, 64, dtype=torch.bfloat16)
        fm.flashmask_attention(q, q, q)


def test_kernel_variant_routing_needs_no_gpu():
    """Tile shapes and launch tables by head dim: the tcgen05 variants (128-column K tiles; 64-query items in the
    backward) serve every head dim up to 128, 192 / 128 in both directions and the 256 / 256 forward; a launch
    table exists only where the variant walks one (not for the 256 forward, not for the 192 backward)."""
    for d, dv in [(8, 8), (64, 64), (96, 80), (128, 128), (192, 128), (256, 256)]:
        assert fm.fwd_tile_shape(d, dv) == (128, 128), (d, dv)
    for d, dv in [(64, 64), (128, 64), (128, 128), (192, 128)]:
        assert fm.bwd_tile_shape(d, dv) == (64, 128), (d, dv)
    assert fm.bwd_tile_shape(256, 256) != (64, 128) and fm.bwd_tile_shape(576, 512) != (64, 128)
    lib = _lib.load()
    a = _lib.AttnArgs()
    a.B, a.Sq, a.Sk, a.Hq, a.Hkv, a.Hm, a.mask_B, a.ncols = 2, 4096, 4096, 8, 2, 1, 2, 2
    want = {(128, 128): (True, True, True), (64, 64): (True, True, True), (192, 128): (True, False, False),
            (256, 256): (False, False, False), (576, 512): (False, False, False)}
    for (d, dv), has in want.items():
        a.d, a.dv = d, dv
        got = tuple(lib.fm_launch_order_ints(ctypes.byref(a), w) > 0 for w in
                    (_lib.FM_ORDER_FWD, _lib.FM_ORDER_BWD_DQ, _lib.FM_ORDER_BWD_DKDV))
        assert got == has, (d, dv, got)


def test_struct_layout_matches_header():
    # 18 int32/float + 15 pointers/size_t + 24 int64
    assert ctypes.sizeof(_lib.AttnArgs) == 18 * 4 + 15 * 8 + 24 * 8 + 3 * 8


def test_workload_shapes():
    w = W.make_workload("causal_doc_8k_gqa")
    assert w.idx.shape == (2, 1, 8192, 1) and w.idx.dtype == np.int32 and w.causal
    assert (w.idx[..., 0] > np.arange(8192)).all() and w.idx.max() == 8192
    fwd, bwd = w.flops()
    assert fwd * 5 == bwd * 2
    w5 = W.make_workload("cp_causal_doc_128k", S=8192)
    assert w5.idx.shape == (1, 1, 8192, 2) and not w5.causal
    # the non-causal 2-column form masks exactly what the causal 1-column form does
    lens = np.diff(np.concatenate([[0], np.unique(w5.idx[0, 0, :, 0])]))
    a = W.dense_visible(w5.idx[:, :, :512], 512, False)
    idx1 = np.minimum(w5.idx[:, :, :512, :1], 512)
    b = W.dense_visible(idx1, 512, True)
    assert np.array_equal(a[..., :512, :], b)
    for name in W.WORKLOADS:
        s = 2048 if "128k" in name or "32k" in name or "16k" in name else None
        wl = W.make_workload(name, S=s)
        assert 0.0 <= wl.sparsity() < 1.0


def test_sliding_window_kwarg_bounds():
    idx = fm.sliding_window_indices(16, 16, 4, True, 2, "cpu")
    ref, _ = W.sliding_window(2, 16, 16, 4)
    assert np.array_equal(idx.numpy(), ref)
    idx2 = fm.sliding_window_indices(16, 16, (3, 2), False, 1, "cpu")
    vis = W.dense_visible(idx2.numpy(), 16, False)[0, 0]
    i, j = np.indices((16, 16))
    assert np.array_equal(vis, (j - i <= 2) & (i - j <= 3))
