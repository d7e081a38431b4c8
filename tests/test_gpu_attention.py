"""GPU parity of forward / backward against the CPU oracle, through the public
operator (which calls the C ABI).  Tolerance: the reference's own rule."""
import glob
import math
import os

import numpy as np
import pytest
import torch

from flashmask_b200 import workloads as W
import flashmask_b200 as fm
from flashmask_b200 import _lib
from _util import (assert_lse, assert_parity, make_inputs, naive_lowp, run_oracle, run_product)

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["sm100", "split", "mma"])
def fwd_variant(request):
    """Head dims up to 128 have two kernel families, the tcgen05 ones (default) and the warp-MMA
    ones, and the tcgen05 backward has a one-kernel variant (default when the call does not ask for
    deterministic gradients) and a two-kernel one ("split"); FLASHMASK_B200_FWD / FLASHMASK_B200_BWD
    select them."""
    names = ("FLASHMASK_B200_FWD", "FLASHMASK_B200_BWD")
    old = {n: os.environ.get(n) for n in names}
    os.environ["FLASHMASK_B200_FWD"] = "mma" if request.param == "mma" else "sm100"
    os.environ["FLASHMASK_B200_BWD"] = request.param
    _lib.reload_options()
    yield request.param
    for n in names:
        if old[n] is None:
            os.environ.pop(n, None)
        else:
            os.environ[n] = old[n]
    _lib.reload_options()


def _kernel_status():
    import ctypes as C
    from flashmask_b200 import _lib
    v = C.c_int(0)
    _lib.check(_lib.load().fm_kernel_status(C.byref(v), 1), "fm_kernel_status")
    return v.value

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "attention_*.npz")))


def _docs(rng, S, n):
    return W.uniform_doc_lengths(rng, S, n)


def _mask(kind, B, Sq, Sk, seed):
    rng = np.random.default_rng(seed)
    if kind == "none_causal":
        return None, True
    if kind == "none_full":
        return None, False
    if kind == "causal_doc":
        m = [W.causal_document(1, Sq, Sk, _docs(rng, Sk, 5))[0] for _ in range(B)]
        return np.concatenate(m), True
    if kind == "bidir_doc":
        m = [W.bidirectional_document(1, Sq, Sk, _docs(rng, Sk, 4))[0] for _ in range(B)]
        return np.concatenate(m), False
    if kind == "sliding_window":
        return W.sliding_window(B, Sq, Sk, max(3, Sk // 7))
    if kind == "share_question":
        return W.share_question(B, Sq, Sk, Sk // 6, Sk // 12, 3)
    if kind == "random_eviction":
        return W.random_eviction(B, Sq, Sk, rng)
    if kind == "four_column":
        return W.four_column_bands(B, Sq, Sk, rng)
    if kind == "prefix_lm":
        third = Sk // 3
        return W.prefix_lm_document(B, Sq, Sk, [(third // 2, third), (third // 4, third), (5, Sk - 2 * third)])
    if kind == "cp_form":
        return W.causal_document_noncausal_form(B, Sq, Sk, _docs(rng, Sk, 6))
    if kind == "empty":
        return W.empty_mask(B, Sq, Sk)
    raise KeyError(kind)


MASKS = ["none_causal", "none_full", "causal_doc", "bidir_doc", "sliding_window", "share_question",
         "random_eviction", "four_column", "prefix_lm", "cp_form", "empty"]


def _run(kind, B, Sq, Sk, Hq, Hkv, d, dv, sink=False, seed=0, dtype=torch.bfloat16, hm=1):
    idx_np, causal = _mask(kind, B, Sq, Sk, seed)
    if idx_np is not None and hm > 1:
        rng = np.random.default_rng(seed + 99)
        per = [_mask(kind, B, Sq, Sk, seed + 1 + h)[0] for h in range(hm)]
        idx_np = np.ascontiguousarray(np.concatenate(per, axis=1))
    q, k, v, do, s = make_inputs(B, Sq, Sk, Hq, Hkv, d, dv, seed, dtype=dtype, sink=sink)
    idx = None if idx_np is None else torch.from_numpy(np.ascontiguousarray(idx_np).copy()).cuda()
    qc, kc, vc, doc = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    got = run_product(qc, kc, vc, doc, idx, causal, s)
    ref = run_oracle(q, k, v, do, idx, causal, s)
    lowp = naive_lowp(qc, kc, vc, doc, idx, causal, s)
    assert_parity(got, ref, lowp, label=f"{kind}: ")
    assert_lse(got, ref)
    if sink:
        scale = ref["dsink"].abs().max().item() + 1.0
        # the kernel against its own definition, evaluated on the tensors it read (the bf16 O and the LSE of this
        # forward): dsink[h] = -sum_{b,i} exp(sink[h] - lse[b,h,i]) * rowsum(O * dO)[b,i,h]
        dps = (got["out"].float() * doc.float()).sum(-1).permute(0, 2, 1)
        own = -(torch.exp(s.cuda()[None, :, None] - got["lse"].float()) * dps).sum((0, 2))
        err_own = (got["dsink"].float() - own).abs().max().item()
        assert err_own <= 1e-3 + 2 ** -10 * scale, f"dsink vs its definition: {err_own}"
        # and against the fp32 oracle: what is left is the rounding of O to 16 bits before rowsum(O * dO), which
        # the reference's preprocess kernel has too and which grows with the width of the row
        # (noise model: every element of O carries a relative rounding error of up to 2^-9, independent
        # between elements; four standard deviations of the resulting sum, per head)
        w2 = torch.exp(s[None, :, None] - ref["lse"].float()) ** 2
        var = (w2 * ((ref["out"].float() * do.float()) ** 2).sum(-1).permute(0, 2, 1)).sum((0, 2))
        tol = 1e-2 + 4 * 2 ** -9 * var.sqrt()
        err = (got["dsink"].float().cpu() - ref["dsink"]).abs()
        assert (err <= tol).all(), f"dsink err {err.tolist()} > {tol.tolist()}"
    return got, ref


@pytest.mark.parametrize("kind", MASKS)
def test_masks_d128_gqa(kind, fwd_variant):
    _run(kind, 2, 384, 384, 4, 2, 128, 128, seed=11)
    _run(kind, 1, 1024, 1024, 2, 1, 128, 128, seed=12)
    assert _kernel_status() == 0


@pytest.mark.parametrize("kind", ["causal_doc", "bidir_doc", "four_column", "none_causal"])
def test_ragged_shapes(kind, fwd_variant):
    # sequence lengths that are not multiples of any tile, Sq != Sk
    _run(kind, 1, 300, 300, 2, 2, 128, 128, seed=3)
    if kind in ("causal_doc", "none_causal"):
        _run(kind, 1, 203, 333, 2, 1, 64, 64, seed=4)
        _run(kind, 1, 203, 333, 2, 1, 128, 128, seed=4)
        _run(kind, 2, 333, 203, 2, 2, 128, 128, seed=4)
    assert _kernel_status() == 0


@pytest.mark.parametrize("d,dv,Hq,Hkv", [(64, 64, 2, 2), (80, 80, 2, 1), (128, 128, 4, 1),
                                         (192, 128, 4, 2), (256, 256, 2, 2), (576, 512, 2, 1),
                                         (512, 512, 2, 1)])
@pytest.mark.parametrize("kind", ["causal_doc", "bidir_doc"])
def test_head_dims(kind, d, dv, Hq, Hkv):
    _run(kind, 1, 320, 320, Hq, Hkv, d, dv, sink=True, seed=5)


@pytest.mark.parametrize("kind", MASKS)
def test_masks_d192(kind):
    """Every mask family through the 192 / 128 variants of the tcgen05 kernels (forward: two-slot K/V ring,
    twelve k-steps per score GEMM; backward: three-slot ring, single dP buffer, operands written over the
    score buffer): GQA, ragged sizes, rows long enough to wrap the rings many times."""
    _run(kind, 2, 384, 384, 4, 2, 192, 128, seed=31)
    _run(kind, 1, 1411, 1411, 2, 1, 192, 128, sink=True, seed=32)
    assert _kernel_status() == 0


@pytest.mark.parametrize("d,dv", [(192, 128), (256, 256)])
@pytest.mark.parametrize("kind", ["causal_doc", "none_causal", "bidir_doc"])
def test_ragged_shapes_big_head_dims(kind, d, dv):
    """Sq != Sk and lengths that are no multiple of any tile through the 192 / 128 and 256 / 256 variants."""
    _run(kind, 1, 300, 300, 2, 2, d, dv, seed=61)
    if kind != "bidir_doc":
        _run(kind, 1, 203, 333, 2, 1, d, dv, sink=True, seed=62)
        _run(kind, 2, 333, 203, 4, 2, d, dv, seed=63)
    assert _kernel_status() == 0


@pytest.mark.parametrize("kind", MASKS)
def test_masks_d256(kind):
    """Every mask family through the 256 / 256 forward variant of the tcgen05 kernel (128 query rows per CTA, the
    two warpgroups own the two 128-column halves of V / O); the backward of this head dim is the warp-MMA one."""
    _run(kind, 2, 384, 384, 4, 2, 256, 256, seed=51)
    _run(kind, 1, 1411, 1411, 2, 1, 256, 256, sink=True, seed=52)
    assert _kernel_status() == 0


@pytest.mark.parametrize("kind", MASKS)
def test_masks_d64(kind, fwd_variant):
    """Every mask family through the 64-column variants: GQA, rows long enough to wrap the K/V ring."""
    _run(kind, 2, 384, 384, 4, 2, 64, 64, seed=21)
    _run(kind, 1, 1280, 1280, 2, 1, 64, 64, seed=22)
    assert _kernel_status() == 0


@pytest.mark.parametrize("d,dv", [(32, 32), (64, 32), (96, 96), (64, 128), (128, 64), (8, 8)])
def test_padded_head_dims(d, dv, fwd_variant):
    """Head dims below a variant's width: the columns past the end of a head must read as zeros and stay unwritten."""
    _run("causal_doc", 1, 333, 333, 2, 1, d, dv, sink=True, seed=23)
    _run("bidir_doc", 2, 256, 256, 2, 2, d, dv, seed=24)
    assert _kernel_status() == 0


@pytest.mark.parametrize("kind", ["none_causal", "causal_doc", "random_eviction"])
def test_sink(kind, fwd_variant):
    _run(kind, 2, 256, 256, 4, 2, 128, 128, sink=True, seed=7)


def test_mask_heads_per_kv_head(fwd_variant):
    _run("causal_doc", 2, 256, 256, 4, 2, 128, 128, seed=8, hm=2)


def test_fp16(fwd_variant):
    _run("causal_doc", 1, 256, 256, 2, 2, 128, 128, seed=9, dtype=torch.float16)
    _run("bidir_doc", 1, 384, 384, 4, 2, 64, 64, seed=10, dtype=torch.float16)


def test_long_rows_many_tiles(fwd_variant):
    """Enough K tiles per Q tile to wrap the K/V ring and the bounds slots many times."""
    _run("random_eviction", 1, 2048, 2048, 2, 1, 128, 128, seed=13)
    _run("sliding_window", 1, 2048, 2048, 1, 1, 128, 128, seed=14)
    assert _kernel_status() == 0


def test_cpu_config_shape():
    """The CPU-runnable configuration: B=1, H=2, S=1024, d=64, 4 documents."""
    w = W.make_workload("cpu_causal_doc_1k")
    q, k, v, do, _ = make_inputs(w.B, w.Sq, w.Sk, w.Hq, w.Hkv, w.d, w.dv, w.seed)
    idx = torch.from_numpy(w.idx).cuda()
    got = run_product(q.cuda(), k.cuda(), v.cuda(), do.cuda(), idx, w.causal, None)
    ref = run_oracle(q, k, v, do, idx, w.causal, None)
    lowp = naive_lowp(q.cuda(), k.cuda(), v.cuda(), do.cuda(), idx, w.causal, None)
    assert_parity(got, ref, lowp)
    assert_lse(got, ref)


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: os.path.basename(p)[10:-4])
def test_against_reference_golden(path):
    """Vectors produced by the reference's own dense-mask attention (fp32).
    Head dim 16 is padded to the 64 bucket by the kernels."""
    z = np.load(path)
    c = {k_: z[k_] for k_ in z.files}
    causal = bool(c["causal"])
    dt = torch.bfloat16
    q, k, v, do = (torch.from_numpy(c[n]).to(dt) for n in ("q", "k", "v", "do"))
    sink = torch.from_numpy(c["sink"]) if "sink" in c else None
    idx = torch.from_numpy(c["idx"]).cuda() if "idx" in c else None
    got = run_product(q.cuda(), k.cuda(), v.cuda(), do.cuda(), idx, causal, sink)
    ref = run_oracle(q, k, v, do, idx, causal, sink)       # oracle on the bf16-rounded inputs
    lowp = naive_lowp(q.cuda(), k.cuda(), v.cuda(), do.cuda(), idx, causal, sink)
    assert_parity(got, ref, lowp)
    # and against the stored reference outputs themselves (fp32 inputs there, bf16 here)
    for n in ("out", "dq", "dk", "dv"):
        err = (got[n].float().cpu() - torch.from_numpy(c[n])).abs().max().item()
        assert err < 0.15, (n, err)


def test_deterministic_bitwise(fwd_variant):
    idx_np, causal = _mask("causal_doc", 2, 512, 512, 21)
    q, k, v, do, s = make_inputs(2, 512, 512, 8, 2, 128, 128, 21, sink=True)
    idx = torch.from_numpy(np.ascontiguousarray(idx_np).copy()).cuda()
    a = run_product(q.cuda(), k.cuda(), v.cuda(), do.cuda(), idx, causal, s, deterministic=True)
    for _ in range(3):
        b = run_product(q.cuda(), k.cuda(), v.cuda(), do.cuda(), idx, causal, s, deterministic=True)
        for n in ("out", "lse", "dq", "dk", "dv", "dsink"):
            assert torch.equal(a[n], b[n]), n


def test_d192_deterministic_bitwise_and_fp16():
    """The 192 / 128 backward is the two-kernel variant whatever `deterministic` says: repeated runs are
    bitwise equal (sink gradient included); fp16 inputs run the same kernels."""
    idx_np, causal = _mask("share_question", 2, 640, 640, 41)
    q, k, v, do, s = make_inputs(2, 640, 640, 8, 2, 192, 128, 41, sink=True)
    idx = torch.from_numpy(np.ascontiguousarray(idx_np).copy()).cuda()
    a = run_product(q.cuda(), k.cuda(), v.cuda(), do.cuda(), idx, causal, s, deterministic=True)
    for det in (True, False, True):
        b = run_product(q.cuda(), k.cuda(), v.cuda(), do.cuda(), idx, causal, s, deterministic=det)
        for n in ("out", "lse", "dq", "dk", "dv", "dsink"):
            assert torch.equal(a[n], b[n]), (n, det)
    _run("causal_doc", 1, 448, 448, 4, 2, 192, 128, seed=42, dtype=torch.float16)
    assert _kernel_status() == 0


@pytest.mark.parametrize("persist", ["0", "1"])
@pytest.mark.parametrize("kind,mask_b,hm", [("causal_doc", 2, 1), ("four_column", 1, 2), ("share_question", 2, 2),
                                            ("bidir_doc", 1, 1)])
def test_launch_order_changes_no_bit(kind, mask_b, hm, persist, monkeypatch):
    """The longest-work-first launch order only permutes which CTA runs which tile, and the
    persistent backward variant only changes which CTA runs which unit: results are bitwise
    those of the index order, for every mask batch / head broadcast and both backward variants."""
    monkeypatch.setenv("FLASHMASK_B200_PERSIST", persist)
    _lib.reload_options()
    B, S, Hq, Hkv = 2, 1024, 8, 2
    idx_np, causal = _mask(kind, B, S, S, 33)
    idx_np = np.ascontiguousarray(idx_np[:mask_b]).copy()
    if hm > 1:   # distinct masks per mask head
        other = np.clip(idx_np + np.array(S // 7, dtype=np.int32), 0, S).astype(np.int32)
        idx_np = np.concatenate([idx_np, other], axis=1)
    q, k, v, do, s = make_inputs(B, S, S, Hq, Hkv, 128, 128, 33, sink=True)
    idx = torch.from_numpy(idx_np).cuda()
    monkeypatch.setenv("FLASHMASK_B200_ORDER", "0")
    a = run_product(q.cuda(), k.cuda(), v.cuda(), do.cuda(), idx, causal, s, deterministic=True)
    monkeypatch.setenv("FLASHMASK_B200_ORDER", "1")
    b = run_product(q.cuda(), k.cuda(), v.cuda(), do.cuda(), idx, causal, s, deterministic=True)
    for n in ("out", "lse", "dq", "dk", "dv", "dsink"):
        assert torch.equal(a[n], b[n]), n


def test_launch_tables_are_reusable():
    """One FlashMaskInfo (one set of launch tables, whose unit counters the persistent backward
    advances and rewinds) serves many launches: every repeat gives the first result."""
    B, S, Hq, Hkv = 1, 2048, 4, 2
    idx_np, causal = _mask("causal_doc", B, S, S, 9)
    q, k, v, do, _ = make_inputs(B, S, S, Hq, Hkv, 128, 128, 9)
    q, k, v, do = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    idx = torch.from_numpy(np.ascontiguousarray(idx_np).copy()).cuda()
    info = fm.prepare_mask(idx, S, causal, 128, 128)
    out, lse = fm._flash_attn_fwd(q, k, v, idx, causal=causal, mask_info=info)
    first = fm._flash_attn_bwd(q, k, v, out, do, lse, idx, causal=causal, mask_info=info)
    assert any(t is not None for t in info.orders.values())
    for _ in range(4):
        out2, lse2 = fm._flash_attn_fwd(q, k, v, idx, causal=causal, mask_info=info)
        again = fm._flash_attn_bwd(q, k, v, out, do, lse, idx, causal=causal, mask_info=info)
        assert torch.equal(out, out2) and torch.equal(lse, lse2)
        for a, b in zip(first[:3], again[:3]):
            assert torch.equal(a, b)
    # the counters behind the backward tables are back at zero
    torch.cuda.synchronize()
    for key, t in info.orders.items():
        if t is not None and key[0] != 0:
            assert t[-4:-2].tolist() == [0, 0], key


def test_layout_invariance(fwd_variant):
    """Contiguous vs permuted storage of q/k/v give bitwise equal results
    (reference: tests/torch/test_flashmask.py:354-396)."""
    idx_np, causal = _mask("causal_doc", 1, 256, 256, 5)
    q, k, v, do, _ = make_inputs(1, 256, 256, 4, 2, 128, 128, 5)
    idx = torch.from_numpy(np.ascontiguousarray(idx_np).copy()).cuda()
    a = run_product(q.cuda(), k.cuda(), v.cuda(), do.cuda(), idx, causal, None, deterministic=True)

    def bhsd(t):  # same values, [B,H,S,D] storage viewed as [B,S,H,D]
        return t.cuda().permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
    b = run_product(bhsd(q), bhsd(k), bhsd(v), bhsd(do), idx, causal, None, deterministic=True)
    for n in ("out", "dq", "dk", "dv"):
        assert torch.equal(a[n], b[n]), n


def test_window_size_kwarg():
    q, k, v, do, _ = make_inputs(1, 256, 256, 2, 2, 64, 64, 1)
    out = fm.flashmask_attention(q.cuda(), k.cuda(), v.cuda(), causal=True, window_size=32)
    idx, causal = W.sliding_window(1, 256, 256, 32)
    ref = fm.flashmask_attention(q.cuda(), k.cuda(), v.cuda(), torch.from_numpy(idx).cuda(), causal=True)
    assert torch.equal(out, ref)


def test_errors():
    q, k, v, do, _ = make_inputs(1, 64, 64, 2, 2, 64, 64, 1)
    with pytest.raises(RuntimeError):
        fm.flashmask_attention(q, k, v)  # CPU tensors: no fallback
    with pytest.raises(AssertionError):
        fm.flashmask_attention(q.cuda(), k.cuda(), v.cuda(),
                               torch.zeros(1, 1, 64, 4, dtype=torch.int32).cuda(), causal=True)
    with pytest.raises(NotImplementedError):
        fm.flashmask_attention(q.cuda()[..., :40].contiguous().repeat(1, 1, 1, 8),
                               k.cuda()[..., :40].contiguous().repeat(1, 1, 1, 8),
                               v.cuda()[..., :40].contiguous().repeat(1, 1, 1, 8))


def test_bounded_wait_reports_timeout_without_fault():
    """A wait on a barrier nothing arrives on gives up after its budget, the kernel
    returns, the status word says FM_ERR_TIMEOUT and the context keeps working."""
    from flashmask_b200 import _lib
    assert _kernel_status() == 0
    _lib.check(_lib.load().fm_selftest_bounded_wait(2000, torch.cuda.current_stream().cuda_stream),
               "fm_selftest_bounded_wait")
    torch.cuda.synchronize()
    assert _kernel_status() == 5          # FM_ERR_TIMEOUT, and the read cleared it
    assert _kernel_status() == 0
    x = torch.ones(8, device="cuda")
    assert float(x.sum()) == 8.0          # the context is still usable
    _run("causal_doc", 1, 256, 256, 2, 2, 128, 128, seed=2)


def test_shared_kv_convention():
    """value = key[..., :dv] on the same storage (576/512): dv comes back zero and dk
    carries dK + dV (reference: flashmask/cute/ops/_common.py:52-88)."""
    B, S, Hq, Hkv, d, dv = 1, 256, 2, 1, 576, 512
    g = torch.Generator().manual_seed(3)
    q = torch.randn(B, S, Hq, d, generator=g).bfloat16().cuda()
    kv = torch.randn(B, S, Hkv, d, generator=g).bfloat16().cuda()
    do = torch.randn(B, S, Hq, dv, generator=g).bfloat16().cuda()
    k, v = kv, kv[..., :dv]
    out, lse = fm._flash_attn_fwd(q, k, v, None, causal=True)
    dq, dk, dvv, _ = fm._flash_attn_bwd(q, k, v, out, do, lse, None, causal=True)
    assert float(dvv.abs().max()) == 0.0
    v2 = v.contiguous()                    # separate storage: plain gradients
    dq2, dk2, dv2, _ = fm._flash_attn_bwd(q, k, v2, out, do, lse, None, causal=True)
    want = dk2.float()
    want[..., :dv] += dv2.float()
    assert torch.equal(dq, dq2)
    assert (dk.float() - want).abs().max().item() <= 2 ** -6 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("deterministic", [True, False])
def test_four_column_mask_long_lists_both_backward_variants(deterministic):
    """A 4-column mask whose units carry far more than 64 work items (S = 8192: up to 128 half
    tiles per unit and q head), through the two-kernel and the one-kernel backward: the case on
    which an MMA issue order that let the second score GEMM of item k+2 overwrite the P^T / dS^T
    of item k once gave wrong gradients."""
    B, S, Hq, Hkv, d = 1, 8192, 2, 1, 128
    rng = np.random.default_rng(77)
    idx_np, causal = W.four_column_bands(B, S, S, rng)
    q, k, v, do, _ = make_inputs(B, S, S, Hq, Hkv, d, d, 77)
    idx = torch.from_numpy(np.ascontiguousarray(idx_np).copy()).cuda()
    got = run_product(q.cuda(), k.cuda(), v.cuda(), do.cuda(), idx, causal, None, deterministic=deterministic)
    import oracle
    from _util import assert_close_rule, lowp_rows
    bd = idx_np[0, 0]
    dk_ref = torch.zeros(S, d); dv_ref = torch.zeros(S, d); dk_lp = torch.zeros(S, d); dv_lp = torch.zeros(S, d)
    for h in range(Hq):
        ref = oracle.attention_rows(q[0, :, h], k[0, :, 0], v[0, :, 0], do[0, :, h], bd, causal)
        lp = lowp_rows(q[0, :, h].cuda(), k[0, :, 0].cuda(), v[0, :, 0].cuda(), do[0, :, h].cuda(), bd, causal, None)
        assert_close_rule(got["dq"][0, :, h], ref["dq"], lp["dq"], f"dq h{h}")
        assert_close_rule(got["out"][0, :, h], ref["out"], lp["out"], f"out h{h}")
        dk_ref += ref["dk"]; dv_ref += ref["dv"]
        dk_lp += lp["dk"].float().cpu(); dv_lp += lp["dv"].float().cpu()
    assert_close_rule(got["dk"][0, :, 0], dk_ref, dk_lp, "dk")
    assert_close_rule(got["dv"][0, :, 0], dv_ref, dv_lp, "dv")
    assert _kernel_status() == 0


def test_aliased_value_keeps_its_own_gradient_below_the_shared_head_dims():
    """The merge of dV into dK is the reference's convention for (512, 512) and (576, 512) only
    (flashmask/cute/ops/bwd.py:136-139); at d = 128 a value that aliases the key still gets its dV."""
    B, S, H, d = 1, 256, 2, 128
    g = torch.Generator().manual_seed(4)
    q = torch.randn(B, S, H, d, generator=g).bfloat16().cuda()
    kv = torch.randn(B, S, H, d, generator=g).bfloat16().cuda()
    do = torch.randn(B, S, H, d, generator=g).bfloat16().cuda()
    out, lse = fm._flash_attn_fwd(q, kv, kv, None, causal=True)
    dq, dk, dv, _ = fm._flash_attn_bwd(q, kv, kv, out, do, lse, None, causal=True)
    dq2, dk2, dv2, _ = fm._flash_attn_bwd(q, kv, kv.clone(), out, do, lse, None, causal=True)
    assert float(dv.abs().max()) > 0.0
    assert torch.equal(dk, dk2) and torch.equal(dv, dv2) and torch.equal(dq, dq2)


@pytest.mark.parametrize("d", [64, 128])
def test_forward_and_backward_replay_from_a_cuda_graph(d):
    """fm_fwd / fm_bwd synchronise nothing and allocate nothing: with the mask prepared and the launch
    tables built beforehand, forward + backward capture into one CUDA graph, and a replay on new input
    values gives the bits of an eager run (the persistent kernels rewind their own table counters)."""
    B, S, Hq, Hkv = 2, 1024, 4, 2
    idx_np, causal = _mask("causal_doc", B, S, S, 41)
    idx = torch.from_numpy(np.ascontiguousarray(idx_np).copy()).cuda()
    a = [t.cuda() for t in make_inputs(B, S, S, Hq, Hkv, d, d, 42)[:4]]
    b = [t.cuda() for t in make_inputs(B, S, S, Hq, Hkv, d, d, 43)[:4]]
    info = fm.prepare_mask(idx, S, causal, *fm.fwd_tile_shape(d, d))

    def step(q, k, v, do):
        out, lse = fm._flash_attn_fwd(q, k, v, idx, causal=causal, mask_info=info)
        dq, dk, dv, _ = fm._flash_attn_bwd(q, k, v, out, do, lse, idx, causal=causal, mask_info=info)
        return out, lse, dq, dk, dv

    want = [t.clone() for t in step(*b)]            # eager; also builds the launch tables
    static = [t.clone() for t in a]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step(*static)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        got = step(*static)
    for s_, n_ in zip(static, b):
        s_.copy_(n_)
    graph.replay()
    graph.replay()                                   # a second replay: the table counters were rewound
    torch.cuda.synchronize()
    for g_, w_ in zip(got, want):
        assert torch.equal(g_, w_)
    assert _kernel_status() == 0
