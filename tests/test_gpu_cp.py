"""Context parallel on the GPU: partitioner kernels bit-exact against the CPU
restatement and against the reference's own CUDA source (oracle/_ref), and the
full schedule (all ranks emulated in one process on one GPU) against the
single-GPU operator."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import oracle.cp as ocp
import flashmask_b200 as fm
from flashmask_b200 import cp, cp_balance, workloads as W

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libcpbalance_ref.so")


def _masks(S, seed):
    rng = np.random.default_rng(seed)
    docs = W.uniform_doc_lengths(rng, S, 11)
    yield "causal_doc_cp_form", W.causal_document_noncausal_form(1, S, S, docs)[0]
    yield "bidir_doc", W.bidirectional_document(1, S, S, docs)[0]
    yield "four_column", W.four_column_bands(1, S, S, rng)[0]
    lens = W.lognormal_doc_lengths(rng, S, np.log(S / 16), 1.5, 64, S // 2)
    yield "heavy_tail_docs", W.causal_document_noncausal_form(1, S, S, lens)[0]


@pytest.mark.parametrize("S,chunk,cpn", [(8192, 1024, 4), (16384, 2048, 8), (4096, 512, 2)])
def test_partition_bit_exact_vs_restatement(S, chunk, cpn):
    for name, idx_np in _masks(S, S + cpn):
        idx_np = np.concatenate([idx_np, idx_np[:, :, ::-1][:, :, ::-1]], axis=0)   # B = 2
        idx = torch.from_numpy(np.ascontiguousarray(idx_np)).cuda()
        wl = cp_balance.get_q_workload(idx, chunk).cpu().numpy()
        assert np.array_equal(wl, ocp.chunk_workload(idx_np, chunk)), name
        for r in range(cpn):
            local, buckets = cp_balance.balance_flashmask_input(idx, cpn, r, balance_chunk_size=chunk)
            ref_local, ref_buckets = ocp.balance(idx_np, cpn, r, chunk)
            assert buckets == ref_buckets, name
            assert np.array_equal(local.cpu().numpy(), ref_local), (name, r)
        flat = sorted(i for b in buckets for _, i in b)
        assert flat == list(range(S // chunk)) and all(len(b) == S // chunk // cpn for b in buckets)


@pytest.mark.skipif(not os.path.exists(REF_SO), reason="oracle/_ref not built (needs the reference checkout)")
def test_partition_kernels_vs_reference_cuda_source():
    """The reference's own cp_balance CUDA bridge (compiled from its sources into
    oracle/_ref) as the oracle for workload, rerank and localise."""
    lib = C.CDLL(REF_SO)
    S, chunk, cpn = 8192, 1024, 4       # S % 512 == 0: the reference's pads do not exist
    stream = torch.cuda.current_stream().cuda_stream
    for name, idx_np in _masks(S, 7):
        idx = torch.from_numpy(np.ascontiguousarray(idx_np)).cuda()
        B, H, _, n = idx.shape
        cols = [idx[..., c].contiguous() for c in range(n)]
        nblk = ((S + 127) // 128 + 3) & ~3
        mm = []
        for c in cols:
            mx = torch.empty((B * H, nblk), dtype=torch.int32, device="cuda")
            mn = torch.empty((B * H, nblk), dtype=torch.int32, device="cuda")
            lib.fm_cpb_scan_max_min(C.c_uint64(c.data_ptr()), B * H, S, 128, C.c_uint64(mx.data_ptr()),
                                    C.c_uint64(mn.data_ptr()), C.c_uint64(stream))
            mm += [mx, mn]
        if n == 2:      # [LTS, UTE]
            ptrs = [mm[0], mm[1], None, None, None, None, mm[2], mm[3]]
        else:
            ptrs = mm
        ref_wl = torch.empty((B, H, S // 128, 1), dtype=torch.int32, device="cuda")
        lib.fm_cpb_reduce_workload(*[C.c_uint64(t.data_ptr() if t is not None else 0) for t in ptrs],
                                   C.c_uint64(ref_wl.data_ptr()), B * H, S // 128, nblk, S, 128, 0, 128,
                                   C.c_uint64(stream))
        ref_chunks = ref_wl.reshape(B, H, S // chunk, chunk // 128).sum(3).sum(0)
        got = cp_balance.get_q_workload(idx, chunk)
        assert torch.equal(got[0, :, :, 0], ref_chunks.to(torch.int32)), name
        # rerank + localise
        tasks = got.reshape(-1, 2).cpu().numpy()
        buckets, _, _ = cp_balance.assign_tasks_heap(tasks, cpn)
        order = torch.tensor([i for b in buckets for _, i in b], dtype=torch.int32, device="cuda")
        mine = cp_balance.indices_rerank_cuda(idx, order, chunk)
        ref_rr = torch.empty_like(mine)
        lib.fm_cpb_indices_rerank(C.c_uint64(idx.data_ptr()), C.c_uint64(order.data_ptr()),
                                  C.c_uint64(ref_rr.data_ptr()), B, H, S, n, S // chunk, chunk, C.c_uint64(stream))
        assert torch.equal(mine, ref_rr), name
        local_idx = torch.tensor([i for _, i in buckets[1]], dtype=torch.int32, device="cuda")
        loc = cp_balance.indices_to_chunks_cuda(mine, local_idx, chunk)
        ref_loc = torch.empty_like(loc)
        lib.fm_cpb_indices_to_chunks(C.c_uint64(ref_rr.data_ptr()), C.c_uint64(local_idx.data_ptr()),
                                     C.c_uint64(ref_loc.data_ptr()), ref_rr.numel(), local_idx.numel(), chunk,
                                     C.c_uint64(stream))
        assert torch.equal(loc, ref_loc), name


def _global_problem(S, Hq, Hkv, seed, kind):
    rng = np.random.default_rng(seed)
    if kind == "causal_doc":
        idx = W.causal_document_noncausal_form(1, S, S, W.lognormal_doc_lengths(rng, S, np.log(S / 8), 1.2, 64, S))[0]
    elif kind == "bidir_doc":
        idx = W.bidirectional_document(1, S, S, W.uniform_doc_lengths(rng, S, 6))[0]
    else:
        idx = W.four_column_bands(1, S, S, rng)[0]
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(1, S, Hq, 128, generator=g).bfloat16().cuda()
    k = torch.randn(1, S, Hkv, 128, generator=g).bfloat16().cuda()
    v = torch.randn(1, S, Hkv, 128, generator=g).bfloat16().cuda()
    do = torch.randn(1, S, Hq, 128, generator=g).bfloat16().cuda()
    return torch.from_numpy(np.ascontiguousarray(idx)).cuda(), q, k, v, do


def _unscatter(parts, buckets, chunk, axis=1):
    """Inverse of scatter_by_buckets over all ranks."""
    n_chunks = sum(len(b) for b in buckets)
    pieces = [None] * n_chunks
    for r, b in enumerate(buckets):
        for pos, (_, i) in enumerate(b):
            pieces[i] = parts[r].narrow(axis, pos * chunk, chunk)
    return torch.cat(pieces, dim=axis)


@pytest.mark.parametrize("kind", ["causal_doc", "bidir_doc", "four_column"])
@pytest.mark.parametrize("cpn", [2, 4])
def test_emulated_cp_matches_single_gpu(kind, cpn):
    S, chunk, Hq, Hkv = 4096, 256, 4, 2
    idx, q, k, v, do = _global_problem(S, Hq, Hkv, 11 + cpn, kind)
    sink = torch.randn(Hq, generator=torch.Generator().manual_seed(1)).cuda()
    # single GPU, whole sequence
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
    sg = sink.clone().requires_grad_(True)
    out_ref, lse_ref = fm.flashmask_attention(qg, kg, vg, idx, causal=False, sink=sg, return_lse=True)
    out_ref.backward(do)
    # context parallel, all ranks in this process
    locals_, buckets = zip(*[cp_balance.balance_flashmask_input(idx, cpn, r, balance_chunk_size=chunk)
                             for r in range(cpn)])
    buckets = buckets[0]
    sc = lambda t: [cp_balance.scatter_by_buckets(t, buckets, r) for r in range(cpn)]
    outs, lses, dqs, dks, dvs, dsink = cp.emulate_cp(sc(q), sc(k), sc(v), sc(do), list(locals_), sink=sink)
    out = _unscatter(outs, buckets, chunk)
    lse = _unscatter(lses, buckets, chunk, axis=2)
    dq, dk, dv = (_unscatter(x, buckets, chunk) for x in (dqs, dks, dvs))
    assert torch.equal(torch.isfinite(lse), torch.isfinite(lse_ref))
    fin = torch.isfinite(lse_ref)
    assert (lse[fin] - lse_ref[fin]).abs().max().item() < 1e-3
    # every element is a sum of at most `cpn` bf16-rounded partials of the single-GPU value
    for name, a, b in (("out", out, out_ref), ("dq", dq, qg.grad), ("dk", dk, kg.grad), ("dv", dv, vg.grad)):
        err = (a.float() - b.float()).abs().max().item()
        tol = 2 ** -7 * cpn * max(1.0, b.float().abs().max().item())
        assert err <= tol, (name, err, tol)
    assert torch.allclose(dsink, sg.grad.float(), rtol=2e-2, atol=2e-2)
    # bitwise reproducible
    again = cp.emulate_cp(sc(q), sc(k), sc(v), sc(do), list(locals_), sink=sink)
    for x, y in zip(dks + dvs + dqs + outs, again[3] + again[4] + again[2] + again[0]):
        assert torch.equal(x, y)


def test_skipped_shards_and_balance_quality():
    """With well separated documents most (rank, shard) pairs hold nothing visible
    and are skipped; the heap partition keeps the heaviest rank within 4/3 of the mean + one chunk."""
    S, chunk, cpn = 16384, 1024, 8
    rng = np.random.default_rng(2)
    idx_np = W.causal_document_noncausal_form(1, S, S, W.lognormal_doc_lengths(rng, S, np.log(1024), 1.5, 128, 8192))[0]
    idx = torch.from_numpy(np.ascontiguousarray(idx_np)).cuda()
    wl = cp_balance.get_q_workload(idx, chunk)[0, 0, :, 0].cpu().numpy()
    need = []
    for r in range(cpn):
        local, buckets = cp_balance.balance_flashmask_input(idx, cpn, r, balance_chunk_size=chunk)
        need.append(cp.shard_need_row(local, S // cpn, False, cpn).cpu().tolist())
        vis = W.dense_visible(local.cpu().numpy()[:, :, :, :], S // cpn, False)[0, 0]
        per_shard = vis.reshape(S // cpn, cpn, S // cpn).any(axis=(0, 2))
        assert per_shard.tolist() == need[-1]
    loads = [sum(w for w, _ in b) for b in buckets]
    assert max(loads) <= sum(loads) / cpn * 4 / 3 + wl.max()
    assert sum(map(sum, need)) < cpn * cpn      # something was skipped


@pytest.mark.parametrize("cpn", [2, 4, 8])
def test_ipo_partition_end_to_end(cpn):
    """use_ipo=True: same contract as the heap path (every chunk once, equal counts, local
    masks consistent with the CPU localisation), never a heavier heaviest rank."""
    S, chunk = 16384, 512
    rng = np.random.default_rng(40 + cpn)
    lens = W.lognormal_doc_lengths(rng, S, np.log(S / 16), 1.5, 64, S // 2)
    idx_np = W.causal_document_noncausal_form(1, S, S, lens)[0]
    idx = torch.from_numpy(np.ascontiguousarray(idx_np)).cuda()
    heap_buckets = cp_balance.balance_flashmask_input(idx, cpn, 0, balance_chunk_size=chunk)[1]
    for r in range(cpn):
        local, buckets = cp_balance.balance_flashmask_input(idx, cpn, r, balance_chunk_size=chunk, use_ipo=True)
        order = [i for b in buckets for _, i in b]
        ref_local = ocp.localize(ocp.rerank(idx_np, order, chunk), [i for _, i in buckets[r]], chunk)
        assert np.array_equal(local.cpu().numpy(), ref_local), r
    assert sorted(order) == list(range(S // chunk)) and all(len(b) == S // chunk // cpn for b in buckets)
    load = lambda bs: max(sum(w for w, _ in b) for b in bs)
    assert load(buckets) <= load(heap_buckets)


def test_unneeded_shards_are_never_read_nan_poisoned_buffers():
    """A shard no row of a rank sees is masked by a MIX of columns (LTS = 0 next to UTE = Sq), so
    the per-tile reductions alone cannot prove its tiles empty (lts_max = Sq, ute_min = 0) and the
    attention kernel would run them with the element mask: P = 0 times whatever the buffer holds.
    The remote buffer therefore has no place for such a shard at all.  The receive buffers are
    filled with NaN before the pulled shards are copied in; nothing of it may reach the outputs,
    and the result is the single-GPU operator's."""
    cpn, S_l, Hq, Hkv = 4, 512, 4, 2
    S = cpn * S_l
    # Column c of shard o is visible to the rows [UTE, LTS) (non-causal 2-column form):
    #   odd columns: the rows of rank o;  even columns of shards 2, 3: the rows of rank 0;
    #   even columns of shard 0: the rows of ranks 0 and 1;  even columns of shard 1: rank 1.
    # Ranks 1 and 2 then see shards 2 / 3 (rank 2: shard 3) as a mix of columns masked from
    # below (visible rows lie before theirs) and from above (after theirs), and need none of them.
    idx_np = np.zeros((1, 1, S, 2), dtype=np.int32)
    for c in range(S):
        o = c // S_l
        if c % 2 == 0 and o >= 2:
            lo, hi = 0, S_l
        elif c % 2 == 0 and o == 0:
            lo, hi = 0, 2 * S_l
        else:
            lo, hi = o * S_l, (o + 1) * S_l
        idx_np[0, 0, c] = (hi, lo)
    want_need = [[True, False, True, True], [True, True, False, False], [False, False, True, False],
                 [False, False, False, True]]
    idx = torch.from_numpy(idx_np).cuda()
    g = torch.Generator().manual_seed(5)
    q, k, v, do = (torch.randn(1, S, h, 128, generator=g).bfloat16().cuda() for h in (Hq, Hkv, Hkv, Hq))
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
    out_ref, lse_ref = fm.flashmask_attention(qg, kg, vg, idx, causal=False, return_lse=True)
    out_ref.backward(do)
    # identity partition (rank r owns rows / keys [r*S_l, (r+1)*S_l)); local masks: row bounds
    # shifted into the rank's local rows and clamped
    sc = lambda t: [t[:, r * S_l:(r + 1) * S_l].contiguous() for r in range(cpn)]
    locals_ = []
    for r in range(cpn):
        loc = np.clip(idx_np.astype(np.int64) - r * S_l, 0, S_l).astype(np.int32)
        locals_.append(torch.from_numpy(loc).cuda())
        assert cp.shard_need_row(locals_[-1], S_l, False, cpn).cpu().tolist() == want_need[r], r
    far = locals_[1][0, 0, 2 * S_l:3 * S_l].cpu().numpy()      # rank 1's view of shard 2: mixed
    assert (far[0::2] == 0).all() and (far[1::2] == S_l).all()
    outs, lses, dqs, dks, dvs, _ = cp.emulate_cp(sc(q), sc(k), sc(v), sc(do), locals_, poison=float("nan"))
    for name, parts, ref in (("out", outs, out_ref), ("dq", dqs, qg.grad), ("dk", dks, kg.grad), ("dv", dvs, vg.grad)):
        a = torch.cat(parts, dim=1)
        assert not torch.isnan(a.float()).any(), name
        err = (a.float() - ref.float()).abs().max().item()
        assert err <= 2 ** -7 * cpn * max(1.0, ref.float().abs().max().item()), (name, err)
