"""The CPU restatement (oracle/) against vectors produced by the reference's own
dense-mask attention and mask expander (tests/golden/make_golden.py)."""
import glob
import os

import numpy as np
import pytest
import torch

import oracle
from flashmask_b200 import workloads as W

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "attention_*.npz")))


def _case(path):
    z = np.load(path)
    return {k: z[k] for k in z.files}


def test_golden_present():
    assert len(GOLDEN) >= 14


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: os.path.basename(p)[10:-4])
def test_attention_oracle_matches_reference(path):
    c = _case(path)
    idx = c.get("idx")
    causal = bool(c["causal"])
    sink = torch.from_numpy(c["sink"]) if "sink" in c else None
    r = oracle.attention_forward_backward(
        torch.from_numpy(c["q"]), torch.from_numpy(c["k"]), torch.from_numpy(c["v"]),
        torch.from_numpy(c["do"]), idx, causal, sink)
    # fp32 on both sides, different association order only
    for name in ("out", "dq", "dk", "dv"):
        np.testing.assert_allclose(r[name].numpy(), c[name], rtol=2e-5, atol=2e-6, err_msg=name)
    if sink is not None:
        np.testing.assert_allclose(r["dsink"].numpy(), c["dsink"], rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: os.path.basename(p)[10:-4])
def test_visibility_matches_reference_bias(path):
    """dense_bias / dense_visible / count_visible are bit-exact against the
    reference's expander."""
    c = _case(path)
    if "visible" not in c:
        return
    Sq, Sk, causal = int(c["Sq"]), int(c["Sk"]), bool(c["causal"])
    ref_vis = np.unpackbits(c["visible"])[:Sq * Sk].reshape(Sq, Sk).astype(bool)
    idx = c.get("idx")
    bias = oracle.dense_bias(idx, Sq, Sk, causal)
    assert np.array_equal(np.isfinite(bias[0, 0]), ref_vis)
    if idx is not None:
        assert np.array_equal(W.dense_visible(idx, Sq, causal)[0, 0], ref_vis)
    assert int(W.count_visible(idx, 1, Sq, Sk, causal).sum()) == int(ref_vis.sum())


def test_lse_definition():
    """LSE = logsumexp over visible scores (and the sink logit); -inf for empty rows."""
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, 8, 1, 4, generator=g); k = torch.randn(1, 8, 1, 4, generator=g)
    v = torch.randn(1, 8, 1, 4, generator=g)
    idx = np.full((1, 1, 8, 1), 8, np.int32); idx[0, 0, :, 0] = [3, 3, 3, 8, 8, 8, 8, 8]
    out, lse, P = oracle.attention_forward(q, k, v, idx, True)
    s = (q[0, :, 0] @ k[0, :, 0].T) * 0.5
    for i in range(8):
        vis = [j for j in range(8) if j <= i and i < idx[0, 0, j, 0]]
        ref = torch.logsumexp(s[i, vis], 0) if vis else torch.tensor(-float("inf"))
        assert torch.allclose(lse[0, 0, i], ref, atol=1e-6)
    np.testing.assert_allclose(P.sum(-1)[0, 0].numpy(), 1.0, atol=1e-6)


def test_block_logit_restatement_matches_the_reference_checker_formula():
    """block_logit_ref against the literal formula of the reference's checker
    (tests/paddle/test_block_score_fusion.py:62-87: scaled logits, causal -inf, pad to whole
    blocks, reshape, max), and the document-relative ids against a per-row loop."""
    import torch
    g = torch.Generator().manual_seed(0)
    B, S, Sk, Hq, Hkv, d, bs = 2, 70, 90, 4, 2, 16, 32
    q = torch.randn(B, S, Hq, d, generator=g)
    k = torch.randn(B, Sk, Hkv, d, generator=g)
    scale = 1.0 / d ** 0.5
    s = torch.einsum("bihd,bjhd->bhij", q, k.repeat_interleave(Hq // Hkv, dim=2)) * scale
    i = torch.arange(S)[:, None]
    j = torch.arange(Sk)[None, :]
    s = s.masked_fill(j > i + (Sk - S), float("-inf"))
    nb = -(-Sk // bs)
    pad = torch.full((B, Hq, S, nb * bs - Sk), float("-inf"))
    want = torch.cat([s, pad], -1).reshape(B, Hq, S, nb, bs).amax(-1)
    got = oracle.block_logit_ref(q, k, None, True, None, bs)
    assert torch.allclose(got, want, atol=1e-6) and torch.equal(torch.isinf(got), torch.isinf(want))
    bos = torch.zeros(B, S, dtype=torch.int32)
    bos[:, 33:] = 41
    got = oracle.block_logit_ref(q, k, None, True, None, bs, block_bos=bos)
    for b, h, r in ((0, 0, 5), (1, 3, 40), (0, 2, 69)):
        for blk in range(nb):
            lo, hi = int(bos[b, r]) + blk * bs, min(int(bos[b, r]) + (blk + 1) * bs, Sk)
            w = s[b, h, r, lo:hi].max().item() if lo < hi else float("-inf")
            assert got[b, h, r, blk].item() == pytest.approx(w, abs=1e-6) or (w == float("-inf") and got[b, h, r, blk].item() == w)


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: os.path.basename(p)[10:-4])
def test_row_and_column_restrictions_agree_with_the_pinned_oracle(path):
    """attention_rows / attention_columns (the checker of the full-size configurations) against
    attention_forward_backward, which the golden vectors above pin: every row, a sample of rows,
    and a sample of key columns of one head group."""
    c = _case(path)
    idx = c.get("idx")
    causal = bool(c["causal"])
    q, k, v, do = (torch.from_numpy(c[n]) for n in ("q", "k", "v", "do"))
    sink = torch.from_numpy(c["sink"]) if "sink" in c else None
    B, Sq, Hq, d = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    G = Hq // Hkv
    full = oracle.attention_forward_backward(q, k, v, do, idx, causal, sink)
    b, hk = B - 1, Hkv - 1
    bounds = None if idx is None else idx[b if idx.shape[0] > 1 else 0, hk if idx.shape[1] > 1 else 0]
    rng = np.random.default_rng(0)
    some = np.unique(np.concatenate([[0, Sq - 1], rng.choice(Sq, min(Sq, 9), replace=False)]))
    dk = torch.zeros(Sk, d); dvv = torch.zeros(Sk, v.shape[3])
    lse_g, dps_g = [], []
    for g in range(G):
        h = hk * G + g
        s = None if sink is None else float(sink[h])
        r = oracle.attention_rows(q[b, :, h], k[b, :, hk], v[b, :, hk], do[b, :, h], bounds, causal, s,
                                  chunk=7)
        for name in ("out", "dq"):
            torch.testing.assert_close(r[name], full[name][b, :, h], rtol=2e-5, atol=2e-6)
        assert torch.equal(torch.isinf(r["lse"]), torch.isinf(full["lse"][b, h]))
        fin = torch.isfinite(r["lse"])
        torch.testing.assert_close(r["lse"][fin], full["lse"][b, h][fin], rtol=2e-5, atol=2e-6)
        dk += r["dk"]; dvv += r["dv"]
        lse_g.append(r["lse"]); dps_g.append(r["dpsum"])
        part = oracle.attention_rows(q[b, :, h], k[b, :, hk], v[b, :, hk], do[b, :, h], bounds, causal, s,
                                     rows=some, chunk=4)
        torch.testing.assert_close(part["out"], full["out"][b, some, h], rtol=2e-5, atol=2e-6)
        torch.testing.assert_close(part["dq"], full["dq"][b, some, h], rtol=2e-5, atol=2e-6)
    torch.testing.assert_close(dk, full["dk"][b, :, hk], rtol=2e-5, atol=4e-6)
    torch.testing.assert_close(dvv, full["dv"][b, :, hk], rtol=2e-5, atol=4e-6)
    cols = np.unique(np.concatenate([[0, Sk - 1], rng.choice(Sk, min(Sk, 11), replace=False)]))
    hs = slice(hk * G, hk * G + G)
    ck, cv = oracle.attention_columns(q[b, :, hs].permute(1, 0, 2), k[b, cols, hk], v[b, cols, hk],
                                      do[b, :, hs].permute(1, 0, 2), torch.stack(lse_g), torch.stack(dps_g),
                                      bounds, causal, cols, Sk, chunk=5)
    torch.testing.assert_close(ck, full["dk"][b, cols, hk], rtol=2e-5, atol=4e-6)
    torch.testing.assert_close(cv, full["dv"][b, cols, hk], rtol=2e-5, atol=4e-6)
