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
