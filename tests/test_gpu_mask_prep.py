"""Bit-exact parity of the mask-preprocessing / tile-classification kernels
against the CPU restatement, through the C ABI."""
import numpy as np
import pytest
import torch

import oracle
from oracle import tiles
import flashmask_b200 as fm
from flashmask_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _masks(B, Sq, Sk, seed):
    rng = np.random.default_rng(seed)
    docs = W.uniform_doc_lengths(rng, Sk, min(7, Sk))
    yield "causal_doc", W.causal_document(B, Sq, Sk, docs)
    yield "bidir_doc", W.bidirectional_document(B, Sq, Sk, docs)
    yield "sliding_window", W.sliding_window(B, Sq, Sk, max(2, Sk // 9))
    yield "share_question", W.share_question(B, Sq, Sk, max(1, Sk // 6), max(1, Sk // 12), 3)
    yield "random_eviction", W.random_eviction(B, Sq, Sk, rng)
    yield "four_column", W.four_column_bands(B, Sq, Sk, rng)
    yield "cp_form", W.causal_document_noncausal_form(B, Sq, Sk, docs)
    yield "empty", W.empty_mask(B, Sq, Sk)


@pytest.mark.parametrize("Sq,Sk", [(1024, 1024), (300, 300), (203, 333), (4096, 4096), (1, 1), (129, 64)])
@pytest.mark.parametrize("tile_m,tile_n", [(128, 64), (64, 64), (128, 128), (256, 128), (64, 32)])
def test_prepare_bit_exact(Sq, Sk, tile_m, tile_n):
    B = 2
    for name, (idx_np, causal) in _masks(B, Sq, Sk, Sq * 7 + Sk):
        # give the two batches different content
        idx_np = idx_np.copy()
        idx_np[1] = np.minimum(idx_np[1] + (idx_np.shape[2] // 5), Sq) if Sq > 8 else idx_np[1]
        ncols = idx_np.shape[-1]
        info = fm.prepare_mask(torch.from_numpy(idx_np).cuda(), Sq, causal, tile_m, tile_n,
                               want_count=True, want_class=True)
        mm = tiles.scan_max_min(idx_np, tile_n, causal)
        got_mm = info.minmax.cpu().numpy()
        for smax, smin in tiles.column_slots(ncols, causal):
            assert np.array_equal(got_mm[smax], mm[smax]), (name, "max", smax)
            assert np.array_equal(got_mm[smin], mm[smin]), (name, "min", smin)
        cnt = tiles.valid_block_count(mm, B, 1, Sq, Sk, ncols, causal, tile_m, tile_n)
        cls = tiles.classify_tiles(mm, B, 1, Sq, Sk, ncols, causal, tile_m, tile_n)
        assert np.array_equal(info.valid_block_count.cpu().numpy(), cnt), name
        assert np.array_equal(info.tile_class.cpu().numpy(), cls), name


def test_classification_is_sound():
    """No skipped tile holds a visible element, no FULL tile a masked one."""
    Sq = Sk = 512
    for name, (idx_np, causal) in _masks(1, Sq, Sk, 5):
        info = fm.prepare_mask(torch.from_numpy(idx_np).cuda(), Sq, causal, 64, 64, want_class=True)
        cls = info.tile_class.cpu().numpy()[0, 0]
        vis = W.dense_visible(idx_np, Sq, causal)[0, 0].reshape(8, 64, 8, 64)
        assert not (vis.any(axis=(1, 3)) & (cls == 0)).any(), name
        assert not ((~vis.all(axis=(1, 3))) & (cls == 2)).any(), name


def test_count_visible_exact():
    for Sq, Sk in [(512, 512), (203, 333), (333, 203)]:
        for name, (idx_np, causal) in _masks(2, Sq, Sk, 3):
            got = fm.count_visible(torch.from_numpy(idx_np).cuda(), Sq, causal).cpu().numpy()
            ref = W.dense_visible(idx_np, Sq, causal).sum(axis=(2, 3))
            assert np.array_equal(got, ref), (name, Sq, Sk)
            assert np.array_equal(W.count_visible(idx_np, 2, Sq, Sk, causal), ref), (name, Sq, Sk)


def test_full_size_properties():
    """At benchmark size: counts agree with the host formula and the class map
    is consistent with the surviving-tile count (size-independent checks)."""
    w = W.make_workload("causal_doc_8k_gqa")
    idx = torch.from_numpy(w.idx).cuda()
    got = fm.count_visible(idx, w.Sq, w.causal).cpu().numpy()
    assert np.array_equal(got, W.count_visible(w.idx, w.B, w.Sq, w.Sk, w.causal))
    info = fm.prepare_mask(idx, w.Sq, w.causal, 128, 64, want_count=True, want_class=True)
    cls = info.tile_class.cpu().numpy()
    assert np.array_equal((cls != 0).sum(-1), info.valid_block_count.cpu().numpy())
    # every document diagonal tile is partial, far-away tiles are skipped
    assert (cls[:, :, np.arange(64), np.arange(64) * 2] == 1).all()
    assert (cls[:, :, 0, 2:] == 0).all()


def _expected_launch_table(work, n_units, Hm, mask_B, rep_h, rep_b, heads, buckets=8):
    """CPU restatement of the launch table: units in 8 work classes relative to the heaviest,
    class by class, inside a class repeat-major (batch repeat, head repeat) with units in index order."""
    mx = int(work.max()) if work.size else 0
    klass = ((mx - work.astype(np.int64)) * buckets) // (mx + 1)
    order = np.lexsort((np.arange(work.size), klass))
    table = []
    for k in range(buckets):
        ids = order[klass[order] == k]
        for rr in range(rep_h * rep_b):
            for i in ids:
                unit, hm, bm = i % n_units, (i // n_units) % Hm, i // (n_units * Hm)
                b = rr // rep_h if mask_B == 1 else bm
                table.append((unit, b * heads + hm * rep_h + rr % rep_h))
    return order, np.array(table, dtype=np.int32).reshape(-1, 2)


@pytest.mark.parametrize("Sq,Sk,mask_b,hm", [(4096, 4096, 2, 1), (1000, 1000, 1, 2), (384, 1333, 2, 2)])
def test_launch_order_bit_exact(Sq, Sk, mask_b, hm, monkeypatch):
    """fm_launch_order: work per unit equals the count of non-skipped tiles of the CPU
    classification; the table is the CPU restatement's, every CTA exactly once."""
    import ctypes as C
    from flashmask_b200 import _lib
    lib = _lib.load()
    B, Hq, Hkv = 2, 4, 2
    for name, (idx_np, causal) in _masks(mask_b * hm, Sq, Sk, Sq + 3 * Sk):
        idx_np = idx_np.copy()
        idx_np[-1] = np.minimum(idx_np[-1] + (Sk // 5), Sq)
        ncols = idx_np.shape[-1]
        idx_np = np.ascontiguousarray(idx_np.reshape(mask_b, hm, Sk, ncols))
        idx = torch.from_numpy(idx_np).cuda()
        info = fm.prepare_mask(idx, Sq, causal, 128, 128)
        mm = tiles.scan_max_min(idx_np, 128, causal)
        a = _lib.AttnArgs()
        a.B, a.Sq, a.Sk, a.Hq, a.Hkv, a.Hm, a.d, a.dv = B, Sq, Sk, Hq, Hkv, hm, 128, 128
        a.ncols, a.causal, a.mask_B, a.tile_m, a.tile_n = ncols, int(causal), mask_b, 128, 128
        a.mask, a.minmax = idx.data_ptr(), info.minmax.data_ptr()
        for which, rows, axis, heads in ((_lib.FM_ORDER_FWD, 256, 3, Hq), (_lib.FM_ORDER_BWD_DQ, 128, 3, Hq),
                                         (_lib.FM_ORDER_BWD_DKDV, 64, 2, Hkv)):
            cls = tiles.classify_tiles(mm, mask_b, hm, Sq, Sk, ncols, causal, rows, 128)
            work = (cls != 0).sum(axis=axis).reshape(-1)
            n_units = work.size // (mask_b * hm)
            rep_h, rep_b = heads // hm, B // mask_b
            n_cta = work.size * rep_h * rep_b
            n = lib.fm_launch_order_ints(C.byref(a), which)
            assert n == 2 * n_cta + 2 * work.size + 4, (name, which)
            out = torch.full((n,), -1, dtype=torch.int32, device="cuda")
            _lib.check(lib.fm_launch_order(C.byref(a), which, out.data_ptr(), None), "fm_launch_order")
            out = out.cpu().numpy()
            order, table = _expected_launch_table(work, n_units, hm, mask_b, rep_h, rep_b, heads)
            assert np.array_equal(out[2 * n_cta:2 * n_cta + work.size], work), (name, which)
            assert np.array_equal(out[2 * n_cta + work.size:2 * n_cta + 2 * work.size], order), (name, which)
            # behind the table: two counters at zero, the variant flag (persistent iff units are short), a pad
            assert out[-4] == 0 and out[-3] == 0 and out[-1] == 0 and out[-2] in (0, 1)
            if which != _lib.FM_ORDER_FWD:
                mult = 2 if which == _lib.FM_ORDER_BWD_DQ else Hq // Hkv
                assert out[-2] == int(int(work.sum()) * mult <= 96 * work.size), (name, which)
            got = out[:2 * n_cta].reshape(-1, 2)
            assert np.array_equal(got, table), (name, which)
            assert len({(int(u), int(h)) for u, h in got}) == n_cta == n_units * heads * B
    # all three tables in one launch are those of three single launches
    sizes = [lib.fm_launch_order_ints(C.byref(a), w) for w in range(3)]
    single = [torch.empty(n, dtype=torch.int32, device="cuda") for n in sizes]
    for w in range(3):
        _lib.check(lib.fm_launch_order(C.byref(a), w, single[w].data_ptr(), None), "fm_launch_order")
    fused = [torch.full((n,), -1, dtype=torch.int32, device="cuda") for n in sizes]
    _lib.check(lib.fm_launch_orders(C.byref(a), *[t.data_ptr() for t in fused], None), "fm_launch_orders")
    for w in range(3):
        assert torch.equal(single[w], fused[w]), w
    # no order where the kernel variant takes none, or without a mask tensor
    a.d = a.dv = 256
    assert lib.fm_launch_order_ints(C.byref(a), _lib.FM_ORDER_FWD) == 0
    a.d = a.dv = 64          # the 64-column tcgen05 variants read the same tables
    assert lib.fm_launch_order_ints(C.byref(a), _lib.FM_ORDER_FWD) == sizes[0]
    a.d = a.dv = 128
    a.ncols = 0
    assert lib.fm_launch_order_ints(C.byref(a), _lib.FM_ORDER_BWD_DKDV) == 0
