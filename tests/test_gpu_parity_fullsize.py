"""The benchmark configurations at their FULL sizes against the fp32 CPU checker.

A dense oracle of every head is out of reach at 8K-128K tokens, so each configuration is checked
on part of its output, at the tolerance rule of the reference's own tests
(tests/torch/test_flashmask.py:261,286,309-319: |got - ref| <= 2 |lowp - ref| + atol):

  * "group" cases: one kv head of one batch with ALL q heads of its group and ALL rows, i.e. the
    complete O, LSE and dQ of those heads and the complete dK / dV of that kv head;
  * "sampled" cases: O, LSE and dQ on sampled query rows (first / last rows, rows next to a
    document boundary, random rows) of two q heads, and dK / dV on sampled key columns of their kv
    head.  P of a key column needs the LSE of every row: it comes from a forward-only pass of the
    checker over all rows ("oracle" statistics) or, where even that is too slow for the CPU (16 q
    heads per kv head at d = 576; 128K rows), from the kernel's own LSE and O, which the sampled-row
    check of the same test has just compared with the checker ("gpu" statistics).
"""
import numpy as np
import pytest
import torch

import flashmask_b200 as fm
import oracle
from flashmask_b200 import workloads as W
from _util import assert_close_rule, lowp_columns, lowp_rows

pytestmark = pytest.mark.gpu


def _inputs(w):
    g = torch.Generator().manual_seed(100 + w.seed)
    q, k, v, do = (torch.randn(w.B, s, h, dd, generator=g).to(torch.bfloat16)
                   for s, h, dd in ((w.Sq, w.Hq, w.d), (w.Sk, w.Hkv, w.d), (w.Sk, w.Hkv, w.dv),
                                    (w.Sq, w.Hq, w.dv)))
    sink = torch.randn(w.Hq, generator=g) if w.sink else None
    idx = None if w.idx is None else torch.from_numpy(np.ascontiguousarray(w.idx).copy())
    return q, k, v, do, sink, idx


def _product(w, q, k, v, do, sink, idx):
    qd, kd, vd, dod = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    sd = None if sink is None else sink.cuda()
    idd = None if idx is None else idx.cuda()
    out, lse = fm._flash_attn_fwd(qd, kd, vd, idd, causal=w.causal, learnable_sink=sd)
    dq, dk, dv, dsink = fm._flash_attn_bwd(qd, kd, vd, out, dod, lse, idd, causal=w.causal,
                                           learnable_sink=sd, deterministic=w.deterministic)
    torch.cuda.synchronize()
    return dict(out=out, lse=lse, dq=dq, dk=dk, dv=dv, dsink=dsink), (qd, kd, vd, dod)


def _bounds(w, b):
    return None if w.idx is None else w.idx[b if w.idx.shape[0] > 1 else 0, 0]


def _check_lse(got, ref, label, tol=2e-2):
    g = got.float().cpu()
    fin = torch.isfinite(ref)
    assert torch.equal(torch.isfinite(g), fin), f"{label}: -inf pattern differs"
    if fin.any():
        err = (g[fin] - ref[fin]).abs().max().item()
        assert err <= tol, f"{label}: LSE err {err:.3e}"


def _sample_rows(rng, w, b, n):
    rows = [0, 1, w.Sq - 2, w.Sq - 1]
    bd = _bounds(w, b)
    if bd is not None:
        edges = np.unique(bd[:, 0])
        edges = edges[(edges > 0) & (edges < w.Sq)]
        pick = edges if edges.size <= 16 else rng.choice(edges, 16, replace=False)
        rows += [int(e) + o for e in pick for o in (-1, 0) if 0 <= int(e) + o < w.Sq]
    rows += list(rng.choice(w.Sq, n, replace=False))
    return np.unique(np.asarray(rows, dtype=np.int64))


GROUP = [("causal_doc_8k_gqa", 1, 5), ("sweep32k_sliding_window", 0, 3), ("sweep32k_causal_doc", 0, 7),
         ("sweep32k_share_question", 0, 11), ("sweep32k_bidir_doc", 0, 0)]


@pytest.mark.parametrize("name,b,hk", GROUP)
def test_one_head_group_complete(name, b, hk):
    w = W.make_workload(name)
    q, k, v, do, sink, idx = _inputs(w)
    got, (qd, kd, vd, dod) = _product(w, q, k, v, do, sink, idx)
    G = w.Hq // w.Hkv
    bd = _bounds(w, b)
    dk_ref = torch.zeros(w.Sk, w.d); dv_ref = torch.zeros(w.Sk, w.dv)
    dk_lp = torch.zeros(w.Sk, w.d); dv_lp = torch.zeros(w.Sk, w.dv)
    for g in range(G):
        h = hk * G + g
        s = None if sink is None else float(sink[h])
        ref = oracle.attention_rows(q[b, :, h], k[b, :, hk], v[b, :, hk], do[b, :, h], bd, w.causal, s)
        lp = lowp_rows(qd[b, :, h], kd[b, :, hk], vd[b, :, hk], dod[b, :, h], bd, w.causal, s)
        assert_close_rule(got["out"][b, :, h], ref["out"], lp["out"], f"{name} out h{h}")
        assert_close_rule(got["dq"][b, :, h], ref["dq"], lp["dq"], f"{name} dq h{h}")
        _check_lse(got["lse"][b, h], ref["lse"], f"{name} h{h}")
        dk_ref += ref["dk"]; dv_ref += ref["dv"]
        dk_lp += lp["dk"].float().cpu(); dv_lp += lp["dv"].float().cpu()
    assert_close_rule(got["dk"][b, :, hk], dk_ref, dk_lp, f"{name} dk")
    assert_close_rule(got["dv"][b, :, hk], dv_ref, dv_lp, f"{name} dv")


SAMPLED = [("sweep32k_random_eviction", 5, "oracle"), ("bigd16k_192_128", 2, "oracle"),
           ("bigd16k_576_512", 0, "gpu"), ("bigd16k_256_256", 9, "oracle"),
           ("cp_causal_doc_128k", 6, "gpu")]


@pytest.mark.parametrize("name,hk,stats", SAMPLED)
def test_sampled_rows_and_key_columns(name, hk, stats):
    w = W.make_workload(name)
    b = 0
    q, k, v, do, sink, idx = _inputs(w)
    got, (qd, kd, vd, dod) = _product(w, q, k, v, do, sink, idx)
    G = w.Hq // w.Hkv
    bd = _bounds(w, b)
    rng = np.random.default_rng(7)
    rows = _sample_rows(rng, w, b, 320)
    # the rule is applied to the sampled rows of both heads together, as the reference's test applies
    # it to whole tensors: the maxima of a few hundred rows of one head alone are too noisy a statistic
    parts = {n: ([], [], []) for n in ("out", "dq")}
    for g in sorted({0, G - 1}):
        h = hk * G + g
        s = None if sink is None else float(sink[h])
        ref = oracle.attention_rows(q[b, :, h], k[b, :, hk], v[b, :, hk], do[b, :, h], bd, w.causal, s,
                                    rows=rows)
        lp = lowp_rows(qd[b, :, h], kd[b, :, hk], vd[b, :, hk], dod[b, :, h], bd, w.causal, s, rows=rows)
        for n in parts:
            parts[n][0].append(got[n][b, rows, h].float().cpu())
            parts[n][1].append(ref[n])
            parts[n][2].append(lp[n].float().cpu())
        _check_lse(got["lse"][b, h, rows], ref["lse"], f"{name} h{h}")
    for n, (a, r_, l_) in parts.items():
        assert_close_rule(torch.cat(a), torch.cat(r_), torch.cat(l_), f"{name} {n}")
    # row statistics of every q head of the group, all rows
    hs = slice(hk * G, hk * G + G)
    if stats == "oracle":
        lse_g, dps_g = [], []
        for g in range(G):
            h = hk * G + g
            s = None if sink is None else float(sink[h])
            f = oracle.attention_rows(q[b, :, h], k[b, :, hk], v[b, :, hk], do[b, :, h], bd, w.causal, s,
                                      grads=False, chunk=2048)
            lse_g.append(f["lse"]); dps_g.append(f["dpsum"])
            _check_lse(got["lse"][b, h], f["lse"], f"{name} h{h} all rows")
        lse_g, dps_g = torch.stack(lse_g), torch.stack(dps_g)
    else:
        lse_g = got["lse"][b, hs].float().cpu()
        dps_g = (got["out"][b, :, hs].float() * dod[b, :, hs].float()).sum(-1).T.contiguous().cpu()
    cols = np.unique(np.concatenate([[0, 1, w.Sk - 2, w.Sk - 1], rng.choice(w.Sk, 160, replace=False)]))
    qg, dog = q[b, :, hs].permute(1, 0, 2), do[b, :, hs].permute(1, 0, 2)
    dk_ref, dv_ref = oracle.attention_columns(qg, k[b, cols, hk], v[b, cols, hk], dog, lse_g, dps_g, bd,
                                              w.causal, cols, w.Sk)
    ct = torch.from_numpy(cols).cuda()
    dk_lp, dv_lp = lowp_columns(qd[b, :, hs].permute(1, 0, 2), kd[b, ct, hk], vd[b, ct, hk],
                                dod[b, :, hs].permute(1, 0, 2), lse_g, dps_g, bd, w.causal, cols, w.Sk)
    assert_close_rule(got["dk"][b, ct, hk], dk_ref, dk_lp, f"{name} dk")
    assert_close_rule(got["dv"][b, ct, hk], dv_ref, dv_lp, f"{name} dv")
    if sink is not None:
        # dsink[h] = -sum_i p_sink(i) * rowsum(O dO)(i)  (flashmask/cute/flash_bwd_sink.py:67-114)
        s = sink[hs].float()[:, None]
        p_sink = torch.where(torch.isinf(lse_g), torch.zeros_like(lse_g), torch.exp(s - lse_g))
        ref_ds = -(p_sink * dps_g).sum(dim=1)
        err = (got["dsink"][hs].float().cpu() - ref_ds).abs().max().item()
        assert err <= 1e-2 + 2 * 2 ** -8 * (ref_ds.abs().max().item() + 1.0), f"{name} dsink err {err}"
