"""Shared helpers of the GPU parity tests."""
import math

import numpy as np
import torch

import oracle
import flashmask_b200 as fm


def make_inputs(B, Sq, Sk, Hq, Hkv, d, dv, seed, dtype=torch.bfloat16, device="cuda", sink=False):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Sq, Hq, d, generator=g).to(dtype)
    k = torch.randn(B, Sk, Hkv, d, generator=g).to(dtype)
    v = torch.randn(B, Sk, Hkv, dv, generator=g).to(dtype)
    do = torch.randn(B, Sq, Hq, dv, generator=g).to(dtype)
    s = torch.randn(Hq, generator=g) if sink else None
    return q, k, v, do, s


def naive_lowp(q, k, v, do, idx, causal, sink, scale=None):
    """The same mathematics evaluated in the inputs' low precision with torch
    ops on the GPU: the error yardstick of the reference's tolerance rule
    (tests/torch/test_flashmask.py:261,286,309-319: attention_ref(upcast=False))."""
    dt = q.dtype
    B, Sq, Hq, d = q.shape
    Sk, Hkv, dv = k.shape[1], k.shape[2], v.shape[3]
    scale = scale or 1.0 / math.sqrt(d)
    q = q.detach().clone().requires_grad_(True)
    k = k.detach().clone().requires_grad_(True)
    v = v.detach().clone().requires_grad_(True)
    g = Hq // Hkv
    qh = q.permute(0, 2, 1, 3)
    kh = k.permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vh = v.permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    scores = torch.matmul(qh * scale, kh.transpose(-1, -2))
    bias = oracle.dense_bias(None if idx is None else idx.cpu().numpy(), Sq, Sk, causal)
    if bias is not None:
        bt = torch.from_numpy(bias).to(q.device)
        bt = bt.expand(B, -1, -1, -1) if bt.shape[0] != B else bt
        bt = bt.repeat_interleave(Hq // bt.shape[1], dim=1)
        scores = scores + bt.to(scores.dtype)
        dead = torch.isinf(bt).all(dim=-1, keepdim=True)
        scores = torch.where(dead, torch.full_like(scores, -3e4), scores)
    sk = None
    if sink is not None:
        sk = sink.detach().clone().to(q.device).requires_grad_(True)
        s = sk.to(scores.dtype).reshape(1, Hq, 1, 1).expand(B, Hq, Sq, 1)
        att = torch.softmax(torch.cat([scores, s], dim=-1), dim=-1)[..., :-1].to(dt)
    else:
        att = torch.softmax(scores, dim=-1).to(dt)
    if bias is not None:
        att = torch.where(dead, torch.zeros_like(att), att)
    out = torch.matmul(att, vh).permute(0, 2, 1, 3)
    grads = torch.autograd.grad(out, [q, k, v] + ([sk] if sk is not None else []), do)
    return dict(out=out.detach(), dq=grads[0], dk=grads[1], dv=grads[2],
                dsink=grads[3] if sk is not None else None)


def run_product(q, k, v, do, idx, causal, sink, deterministic=None):
    q = q.detach().clone().requires_grad_(True)
    k = k.detach().clone().requires_grad_(True)
    v = v.detach().clone().requires_grad_(True)
    s = sink.detach().clone().to(q.device).requires_grad_(True) if sink is not None else None
    out, lse = fm.flashmask_attention(q, k, v, idx, causal=causal, sink=s, return_lse=True,
                                      deterministic=deterministic)
    grads = torch.autograd.grad(out, [q, k, v] + ([s] if s is not None else []), do)
    return dict(out=out.detach(), lse=lse.detach(), dq=grads[0], dk=grads[1], dv=grads[2],
                dsink=grads[3] if s is not None else None)


def run_oracle(q, k, v, do, idx, causal, sink):
    return oracle.attention_forward_backward(
        q.cpu(), k.cpu(), v.cpu(), do.cpu(), None if idx is None else idx.cpu().numpy(), causal,
        None if sink is None else sink.cpu())


def assert_parity(got, ref, lowp, names=("out", "dq", "dk", "dv"), label=""):
    """|got - ref| <= 2 |lowp - ref| + atol, atol = 2 |ref + 0.3 - 0.3 - ref|
    (tests/torch/test_flashmask.py:261,286,309-319 of the reference)."""
    for n in names:
        r = ref[n].float()
        gg = got[n].float().cpu()
        lp = lowp[n].float().cpu()
        atol = 2 * (r + 0.3 - 0.3 - r).abs().max().item()
        err = (gg - r).abs().max().item()
        yard = (lp - r).abs().max().item()
        assert not torch.isnan(gg).any(), f"{label}{n}: NaN"
        assert err <= 2 * yard + atol, f"{label}{n}: err {err:.3e} > 2*{yard:.3e} + {atol:.3e}"


def assert_lse(got, ref, tol=2e-2):
    g = got["lse"].float().cpu()
    r = ref["lse"].float()
    fin = torch.isfinite(r)
    assert torch.equal(torch.isfinite(g), fin), "LSE: -inf pattern differs"
    assert (g[fin] - r[fin]).abs().max().item() <= tol if fin.any() else True


# ---------------------------------------------------------------------------
# Full-size configurations: one head at a time, restricted to query rows or key columns.
# The low-precision yardsticks below mirror oracle.attention_rows / attention_columns with torch
# ops in the inputs' dtype on the GPU (the role attention_ref(upcast=False) plays in the
# reference's tolerance rule).
# ---------------------------------------------------------------------------
def lowp_rows(q, k, v, do, bounds, causal, sink, rows=None, scale=None, chunk=2048):
    """q [Sq,d], k [Sk,d], v [Sk,dv], do [Sq,dv] on the GPU (bf16 / fp16), one head.
    Returns out / dq for the rows and the rows' contribution to dk / dv."""
    dt = q.dtype
    Sq, d = q.shape
    Sk, dv = v.shape
    scale = scale or 1.0 / math.sqrt(d)
    rows = np.arange(Sq, dtype=np.int64) if rows is None else np.asarray(rows, dtype=np.int64)
    R = rows.shape[0]
    out = torch.zeros(R, dv, dtype=dt, device=q.device)
    dq = torch.zeros(R, d, dtype=dt, device=q.device)
    dk = torch.zeros(Sk, d, dtype=torch.float32, device=q.device)
    dvv = torch.zeros(Sk, dv, dtype=torch.float32, device=q.device)
    for c0 in range(0, R, chunk):
        rr = rows[c0:c0 + chunk]
        cand = oracle.candidate_columns(bounds, Sq, Sk, causal, int(rr.min()), int(rr.max()))
        vis_np = oracle.visible_block(bounds, Sq, Sk, causal, rr, cand)
        keep = vis_np.any(axis=0)
        cols = cand[keep]
        if cols.size == 0:
            continue
        vis = torch.from_numpy(vis_np[:, keep]).to(q.device)
        ct = torch.from_numpy(cols).to(q.device)
        rt = torch.from_numpy(rr).to(q.device)
        qr = q[rt].detach().clone().requires_grad_(True)
        kc = k[ct].detach().clone().requires_grad_(True)
        vc = v[ct].detach().clone().requires_grad_(True)
        s = torch.matmul(qr * scale, kc.T)
        dead = ~vis.any(dim=1, keepdim=True)
        s = torch.where(vis, s, torch.full_like(s, float("-inf")))
        s = torch.where(dead, torch.full_like(s, -3e4), s)
        if sink is not None:
            col = torch.full((rr.shape[0], 1), float(sink), dtype=s.dtype, device=s.device)
            att = torch.softmax(torch.cat([s, col], dim=-1), dim=-1)[:, :-1].to(dt)
        else:
            att = torch.softmax(s, dim=-1).to(dt)
        att = torch.where(dead, torch.zeros_like(att), att)
        o = torch.matmul(att, vc)
        gq, gk, gv = torch.autograd.grad(o, [qr, kc, vc], do[rt])
        sl = slice(c0, c0 + rr.shape[0])
        out[sl] = o.detach(); dq[sl] = gq
        dk.index_add_(0, ct, gk.float()); dvv.index_add_(0, ct, gv.float())
    return dict(out=out, dq=dq, dk=dk.to(dt), dv=dvv.to(dt))


def lowp_columns(q, k_cols, v_cols, do, lse, dpsum, bounds, causal, cols, Sk, scale=None, chunk=4096):
    """dK / dV of the key columns ``cols`` in the inputs' precision: q / do [G,Sq,*] on the GPU,
    lse / dpsum [G,Sq] fp32 (the same statistics the fp32 checker is given)."""
    dt = q.dtype
    G, Sq, d = q.shape
    scale = scale or 1.0 / math.sqrt(d)
    cols = np.asarray(cols, dtype=np.int64)
    dk = torch.zeros(cols.shape[0], d, dtype=torch.float32, device=q.device)
    dvv = torch.zeros(cols.shape[0], v_cols.shape[1], dtype=torch.float32, device=q.device)
    lse = lse.to(q.device); dpsum = dpsum.to(q.device)
    for r0 in range(0, Sq, chunk):
        rr = np.arange(r0, min(r0 + chunk, Sq), dtype=np.int64)
        vis_np = oracle.visible_block(bounds, Sq, Sk, causal, rr, cols)
        if not vis_np.any():
            continue
        vis = torch.from_numpy(vis_np).to(q.device)
        sl = slice(r0, r0 + rr.shape[0])
        for g in range(G):
            l = lse[g, sl]
            dead = torch.isinf(l)
            s = torch.matmul(q[g, sl] * scale, k_cols.T)
            P = torch.exp(s.float() - torch.where(dead, torch.zeros_like(l), l)[:, None]).to(dt)
            P = torch.where(vis & ~dead[:, None], P, torch.zeros_like(P))
            dS = (P * (torch.matmul(do[g, sl], v_cols.T) - dpsum[g, sl][:, None].to(dt))).to(dt)
            dk += (torch.matmul(dS.T, q[g, sl]) * scale).float()
            dvv += torch.matmul(P.T, do[g, sl]).float()
    return dk.to(dt), dvv.to(dt)


def assert_close_rule(got, ref, lowp, label):
    """The reference's tolerance rule on one tensor (see assert_parity)."""
    r = ref.float().cpu()
    gg = got.float().cpu()
    lp = lowp.float().cpu()
    atol = 2 * (r + 0.3 - 0.3 - r).abs().max().item()
    err = (gg - r).abs().max().item()
    yard = (lp - r).abs().max().item()
    assert not torch.isnan(gg).any(), f"{label}: NaN"
    assert err <= 2 * yard + atol, f"{label}: err {err:.3e} > 2*{yard:.3e} + {atol:.3e}"
    return err, yard
