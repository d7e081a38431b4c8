"""The benchmark configurations at their FULL sizes, checked through properties that need no
dense oracle (the CPU restatement would take hours at 8K-32K tokens):

  * rows of softmax sum to one: with V = 1 the output is 1 on every row that sees a key and 0 on the
    rows that see none, and those are exactly the rows whose LSE is -inf;
  * with V = 1 and dO = 1 the score gradient vanishes (dP - rowsum(dO*O) = 0), so dQ = dK = 0, and every
    column of dV sums to the number of rows that see a key (the columns of P^T dO add up the rows of P);
  * the forward is linear in V;
  * the tcgen05 kernels and the warp-MMA kernels, two independent implementations of tile skipping and
    masking, agree within the low-precision tolerance on random inputs;
  * two runs give the same bits.
"""
import os

import numpy as np
import pytest
import torch

import flashmask_b200 as fm
from flashmask_b200 import _lib
from flashmask_b200 import workloads as W

pytestmark = pytest.mark.gpu

FULL = ["causal_doc_8k_gqa", "sweep32k_sliding_window", "sweep32k_causal_doc", "sweep32k_share_question",
        "sweep32k_bidir_doc", "sweep32k_random_eviction"]


def _setup(name, seed=0, d=None):
    w = W.make_workload(name)
    d = d or w.d
    g = torch.Generator().manual_seed(seed)
    q, k, v, do = (torch.randn(w.B, s, h, d, generator=g).to(torch.bfloat16).cuda()
                   for s, h in ((w.Sq, w.Hq), (w.Sk, w.Hkv), (w.Sk, w.Hkv), (w.Sq, w.Hq)))
    idx = torch.from_numpy(np.ascontiguousarray(w.idx).copy()).cuda()
    return w, q, k, v, do, idx


def _fwd_bwd(w, q, k, v, do, idx):
    out, lse = fm._flash_attn_fwd(q, k, v, idx, causal=w.causal)
    dq, dk, dv, _ = fm._flash_attn_bwd(q, k, v, out, do, lse, idx, causal=w.causal, deterministic=True)
    return out, lse, dq, dk, dv


# the same masks at the head dims of the 64-column variants and of the zero-filled 128-column one
SMALL_D = [("causal_doc_8k_gqa", 64), ("causal_doc_8k_gqa", 96), ("sweep32k_share_question", 64),
           ("sweep32k_bidir_doc", 64)]


@pytest.mark.parametrize("name,d", [(n, None) for n in FULL] + SMALL_D)
def test_rows_sum_to_one_and_gradients_of_constant_values(name, d):
    w, q, k, v, do, idx = _setup(name, d=d)
    ones_v, ones_do = torch.ones_like(v), torch.ones_like(do)
    out, lse, dq, dk, dv = _fwd_bwd(w, q, k, ones_v, ones_do, idx)
    seen = torch.isfinite(lse)                                  # [B, Hq, Sq]
    o = out.float().permute(0, 2, 1, 3)                          # [B, Hq, Sq, dv]
    # P is rounded to bf16 before P V: a row of up to 32K weights sums to 1 within a few 2^-9 steps
    assert (o[seen] - 1.0).abs().max().item() < 2.0 ** -6
    assert (o[~seen] == 0).all()
    # the mask's own count of visible pairs says which (b, head) pairs can have empty rows at all
    n_vis = fm.count_visible(idx, w.Sq, w.causal)
    assert int(n_vis.min()) > 0
    # score gradient ~ 0: dP - rowsum(dO*O) = dv - dv*O is 0 wherever O rounded to exactly 1 and one bf16
    # step (0.5 or 1 at dv = 128) on the few rows where it did not
    assert dq.float().abs().max().item() < 1.0 and dk.float().abs().max().item() < 1.0
    assert dq.float().abs().mean().item() < 0.02 and dk.float().abs().mean().item() < 0.02
    # every column of dV adds up the rows of P of the q heads of its group: the rows that see a key
    G = w.Hq // w.Hkv
    rows = seen.view(w.B, w.Hkv, G, w.Sq).sum(dim=(2, 3)).double()          # [B, Hkv]
    col = dv.double().sum(dim=1)                                             # [B, Hkv, dv]
    rel = ((col - rows[..., None]).abs() / rows[..., None].clamp(min=1)).max().item()
    assert rel < 2e-3, rel


@pytest.mark.parametrize("name", FULL[:3])
def test_forward_is_linear_in_values(name):
    w, q, k, v, do, idx = _setup(name, seed=1)
    v2 = torch.randn_like(v)
    o1, _ = fm._flash_attn_fwd(q, k, v, idx, causal=w.causal)
    o2, _ = fm._flash_attn_fwd(q, k, v2, idx, causal=w.causal)
    o12, _ = fm._flash_attn_fwd(q, k, (v.float() + v2.float()).to(torch.bfloat16), idx, causal=w.causal)
    err = (o12.float() - (o1.float() + o2.float())).abs().max().item()
    assert err < 0.06, err          # three bf16 roundings of values of size ~1


@pytest.mark.parametrize("name,d", [("causal_doc_8k_gqa", None), ("sweep32k_causal_doc", None),
                                    ("sweep32k_random_eviction", None), ("causal_doc_8k_gqa", 64),
                                    ("causal_doc_8k_gqa", 80), ("sweep32k_random_eviction", 64)])
def test_tcgen05_and_warp_mma_kernels_agree(name, d, monkeypatch):
    w, q, k, v, do, idx = _setup(name, seed=2, d=d)
    a = _fwd_bwd(w, q, k, v, do, idx)
    monkeypatch.setenv("FLASHMASK_B200_FWD", "mma")
    monkeypatch.setenv("FLASHMASK_B200_BWD", "mma")
    _lib.reload_options()
    b = _fwd_bwd(w, q, k, v, do, idx)
    fin = torch.isfinite(a[1])
    assert torch.equal(fin, torch.isfinite(b[1]))
    assert (a[1][fin] - b[1][fin]).abs().max().item() < 2e-3
    for n, x, y in zip(("out", "dq", "dk", "dv"), (a[0], a[2], a[3], a[4]), (b[0], b[2], b[3], b[4])):
        d = (x.float() - y.float()).abs()
        scale = y.float().abs().max().item()
        # both sides round P / dS to bf16 at different points of differently ordered sums
        assert d.max().item() <= 2.0 ** -6 * max(scale, 1.0), (n, d.max().item(), scale)
        assert d.mean().item() <= 2.0 ** -5 * max(y.float().abs().mean().item(), 1e-3), n


@pytest.mark.parametrize("name", ["causal_doc_8k_gqa", "sweep32k_share_question"])
def test_full_size_runs_are_reproducible(name):
    w, q, k, v, do, idx = _setup(name, seed=3)
    a = _fwd_bwd(w, q, k, v, do, idx)
    b = _fwd_bwd(w, q, k, v, do, idx)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
