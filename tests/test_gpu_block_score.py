"""Fused block-score side output of the forward (``block_logit`` / ``block_size`` / ``block_bos``).

The cases follow the reference's own test of the feature
(tests/paddle/test_block_score_fusion.py: shapes, block sizes, corner cases, GQA, the pack_gqa
rejection, the probe tests of which entries are written) and add what that file does not cover:
column-bound masks and document-relative block ids.  Tolerance as there:
``0.06 * sqrt(d) * softmax_scale`` on the finite entries, identical -inf pattern.
"""
import math

import numpy as np
import pytest
import torch

import flashmask_b200 as fm
from flashmask_b200 import _lib
import oracle

pytestmark = pytest.mark.gpu

NEG_INF = float("-inf")
PROBE = -1e30          # very negative: the kernel merges with fmax, a positive probe would survive every write


def _inputs(b, s, sk, hq, hkv, d, dv, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(b, s, hq, d, generator=g).bfloat16()
    k = torch.randn(b, sk, hkv, d, generator=g).bfloat16()
    v = torch.randn(b, sk, hkv, dv, generator=g).bfloat16()
    return q, k, v


def _run(q, k, v, causal, block_size, idx=None, bos=None, fill=NEG_INF, extra_cols=0):
    b, s, hq, d = q.shape
    nb = -(-k.shape[1] // block_size) + extra_cols
    bl = torch.full((b, hq, s, nb), fill, dtype=torch.float32, device="cuda")
    out, lse = fm._flash_attn_fwd(q.cuda(), k.cuda(), v.cuda(), None if idx is None else idx.cuda(),
                                  causal=causal, block_logit=bl, block_size=block_size,
                                  block_bos=None if bos is None else bos.cuda(), pack_gqa=False)
    return out, lse, bl


def _check(got, ref, d, scale=None):
    got, ref = got.cpu().numpy(), ref.numpy()
    scale = scale or 1.0 / math.sqrt(d)
    gm, rm = got <= -1e30, ref <= -1e30
    assert int((gm != rm).sum()) == 0, f"masked pattern differs in {int((gm != rm).sum())} entries"
    if (~rm).any():
        diff = np.abs(got[~rm] - ref[~rm]).max()
        assert diff <= 0.06 * math.sqrt(d) * scale, diff


@pytest.fixture(params=["sm100", "mma"])
def variant(request, monkeypatch):
    """Head dims up to 128 have two forward kernel families, both with the side output."""
    monkeypatch.setenv("FLASHMASK_B200_FWD", request.param)
    _lib.reload_options()
    return request.param


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("b,s,sk,h,d", [(1, 256, 256, 8, 64), (2, 512, 512, 4, 128), (2, 640, 640, 6, 128),
                                        (1, 384, 384, 2, 96)])
def test_block_logit_shapes(b, s, sk, h, d, causal, variant):
    q, k, v = _inputs(b, s, sk, h, h, d, d, 0)
    _, _, bl = _run(q, k, v, causal, 64)
    _check(bl, oracle.block_logit_ref(q, k, None, causal, None, 64), d)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("b,s,sk,h,d,dv", [(1, 512, 512, 8, 256, 256), (1, 1024, 1024, 2, 256, 256),
                                           (1, 511, 513, 2, 256, 256), (1, 320, 320, 4, 192, 128)])
def test_block_logit_head_dims_above_128(b, s, sk, h, d, dv, causal):
    """Both head dims run the tcgen05 forward (d = 256 is the reference's HySparse full-attention configuration):
    the plain forward and the block-score variant must agree bitwise on O and LSE."""
    q, k, v = _inputs(b, s, sk, h, h, d, dv, 11)
    o0, l0 = fm._flash_attn_fwd(q.cuda(), k.cuda(), v.cuda(), causal=causal)
    o1, l1, bl = _run(q, k, v, causal, 64)
    assert torch.equal(o0, o1) and torch.equal(l0, l1)
    _check(bl, oracle.block_logit_ref(q, k, None, causal, None, 64), d)


@pytest.mark.parametrize("block_size", [32, 64, 128])
@pytest.mark.parametrize("causal", [True, False])
def test_block_logit_block_sizes(block_size, causal, variant):
    q, k, v = _inputs(1, 512, 512, 4, 4, 128, 128, 1)
    _, _, bl = _run(q, k, v, causal, block_size)
    assert tuple(bl.shape) == (1, 4, 512, 512 // block_size)
    _check(bl, oracle.block_logit_ref(q, k, None, causal, None, block_size), 128)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("b,s,sk", [(1, 250, 250), (1, 130, 130), (1, 63, 63), (1, 1, 1), (2, 300, 512), (2, 512, 300)])
def test_block_logit_corner_cases(b, s, sk, causal):
    q, k, v = _inputs(b, s, sk, 4, 4, 128, 128, 2)
    # two spare block columns: a row stride above ceil(Sk / block_size) must be honoured and stay untouched
    _, _, bl = _run(q, k, v, causal, 64, extra_cols=2)
    nb = -(-sk // 64)
    assert torch.isinf(bl[..., nb:]).all()
    _check(bl[..., :nb], oracle.block_logit_ref(q, k, None, causal, None, 64), 128)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("d", [64, 128])
def test_block_logit_does_not_change_output(causal, d):
    q, k, v = _inputs(1, 512, 512, 4, 4, d, d, 3)
    o0, l0 = fm._flash_attn_fwd(q.cuda(), k.cuda(), v.cuda(), causal=causal)
    o1, l1, _ = _run(q, k, v, causal, 64)
    assert torch.equal(o0, o1) and torch.equal(l0, l1)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("hq,hkv", [(8, 2), (8, 1), (4, 2)])
def test_block_logit_gqa(hq, hkv, causal):
    q, k, v = _inputs(1, 512, 512, hq, hkv, 128, 128, 5)
    _, _, bl = _run(q, k, v, causal, 64)
    _check(bl, oracle.block_logit_ref(q, k, None, causal, None, 64), 128)


def test_block_logit_rejects_pack_gqa_and_bad_arguments():
    q, k, v = _inputs(1, 128, 128, 8, 2, 128, 128, 6)
    bl = torch.full((1, 8, 128, 2), NEG_INF, dtype=torch.float32, device="cuda")
    with pytest.raises(AssertionError, match="pack_gqa"):
        fm._flash_attn_fwd(q.cuda(), k.cuda(), v.cuda(), block_logit=bl, pack_gqa=True)
    with pytest.raises(AssertionError, match="float32"):
        fm._flash_attn_fwd(q.cuda(), k.cuda(), v.cuda(), block_logit=bl.half())
    with pytest.raises(AssertionError, match="num_blocks"):
        fm._flash_attn_fwd(q.cuda(), k.cuda(), v.cuda(), block_logit=bl[..., :1].contiguous())
    with pytest.raises(AssertionError, match="requires block_logit"):
        fm._flash_attn_fwd(q.cuda(), k.cuda(), v.cuda(), block_bos=torch.zeros(1, 128, dtype=torch.int32).cuda())
    with pytest.raises(NotImplementedError, match="block_size must be 32, 64 or 128"):
        fm._flash_attn_fwd(q.cuda(), k.cuda(), v.cuda(),
                           block_logit=torch.full((1, 8, 128, 8), NEG_INF, device="cuda"), block_size=16)


@pytest.mark.parametrize("block_size", [32, 64, 128])
def test_block_logit_large_multitile_noncausal(block_size):
    """Sk >> 128: block id = tile * blocks per tile + slot; non-causal, so every entry is written."""
    q, k, v = _inputs(1, 2048, 2048, 2, 2, 128, 128, 7)
    _, _, bl = _run(q, k, v, False, block_size, fill=PROBE)
    assert int((bl == PROBE).sum()) == 0
    ref = oracle.block_logit_ref(q, k, None, False, None, block_size)
    assert (bl.cpu() - ref).abs().max().item() <= 0.06


def test_block_logit_unvisited_future_blocks_untouched_causal(variant):
    """Only visited K tiles are written: under causal the future tiles keep the caller's fill."""
    q, k, v = _inputs(1, 512, 512, 2, 2, 128, 128, 8)
    _, _, bl_inf = _run(q, k, v, True, 64)
    _, _, bl_probe = _run(q, k, v, True, 64, fill=PROBE)
    written = bl_probe != PROBE
    assert torch.equal(bl_inf[written], bl_probe[written])
    ref = oracle.block_logit_ref(q, k, None, True, None, 64)
    _check(bl_inf, ref, 128)
    assert (~written).any()
    assert (ref[~written.cpu()] <= -1e30).all()


def _doc_mask(B, S, cuts):
    """Causal document mask [B, 1, S, 1] and the first key of every row's document [B, S]."""
    idx = np.zeros((B, 1, S, 1), dtype=np.int32)
    bos = np.zeros((B, S), dtype=np.int32)
    for b in range(B):
        edges = [0] + list(cuts[b]) + [S]
        for lo, hi in zip(edges[:-1], edges[1:]):
            idx[b, 0, lo:hi, 0] = hi
            bos[b, lo:hi] = lo
    return torch.from_numpy(idx), torch.from_numpy(bos), cuts


@pytest.mark.parametrize("block_size", [32, 64, 128])
@pytest.mark.parametrize("with_bos", [False, True])
def test_block_logit_with_column_bound_mask(block_size, with_bos, variant):
    """The block maxima see the attention's own mask; with block_bos the ids are document-relative
    (documents start at columns that are multiples of nothing: every straddling case occurs)."""
    B, S = 2, 1000
    idx, bos, _ = _doc_mask(B, S, [[137, 451, 702], [333, 334, 900]])
    q, k, v = _inputs(B, S, S, 4, 2, 128, 128, 9)
    _, _, bl = _run(q, k, v, True, block_size, idx=idx, bos=bos if with_bos else None)
    ref = oracle.block_logit_ref(q, k, idx.numpy(), True, None, block_size, block_bos=bos if with_bos else None)
    _check(bl, ref, 128)


def test_block_logit_packed_equals_alone():
    """Pack equivalence: with block_bos, a document inside a packed sequence gets the block scores
    it gets when it is the whole sequence."""
    S = 900
    idx, bos, cuts = _doc_mask(1, S, [[201, 555]])
    q, k, v = _inputs(1, S, S, 2, 2, 64, 64, 10)
    _, _, packed = _run(q, k, v, True, 64, idx=idx, bos=bos)
    edges = [0] + cuts[0] + [S]
    for lo, hi in zip(edges[:-1], edges[1:]):
        _, _, alone = _run(q[:, lo:hi], k[:, lo:hi], v[:, lo:hi], True, 64)
        nb = alone.shape[-1]
        a, p = alone.cpu(), packed[:, :, lo:hi, :nb].cpu()
        assert torch.equal(torch.isinf(a), torch.isinf(p))
        fin = ~torch.isinf(a)
        assert (a[fin] - p[fin]).abs().max().item() <= 1e-5
        assert torch.isinf(packed[:, :, lo:hi, nb:]).all()
