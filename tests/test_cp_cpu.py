"""CPU checks of the context-parallel host logic: the heap partitioner (C++ in
the library) against the Python restatement of the reference, the plan's
send/recv pairing, and a 2-rank gloo run of the plan exchange."""
import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest

import oracle.cp as ocp
from flashmask_b200 import cp, cp_balance, workloads as W

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("n,m", [(8, 2), (64, 4), (64, 8), (10, 4), (7, 3), (512, 8), (1, 1), (3, 4)])
def test_heap_partition_matches_restatement(n, m):
    rng = np.random.default_rng(n * 31 + m)
    for trial in range(5):
        w = rng.integers(0, 50 if trial % 2 else 5000, size=n)      # many ties / few ties
        tasks = np.stack([w, np.arange(n)], axis=1).astype(np.int32)
        got = cp_balance.assign_tasks_heap(tasks, m)
        ref = ocp.assign_tasks_heap(tasks, m)
        assert got[0] == ref[0] and got[1] == ref[1] and got[2] == ref[2]
        flat = sorted(i for b in got[0] for _, i in b)
        assert flat == list(range(n))
        if n % m == 0:
            assert all(len(b) == n // m for b in got[0])


def test_heap_known_answer():
    tasks = np.array([[100, 0], [80, 1], [60, 2], [40, 3], [30, 4], [20, 5], [15, 6], [10, 7]], dtype=np.int32)
    buckets, weights, _ = cp_balance.assign_tasks_heap(tasks, 2)
    # LPT with capacity 4: 100->b0, 80->b1, 60->b1, 40->b0, 30->b0(140<=140 tie: bucket 0 first), ...
    assert sorted(weights) == sorted(ocp.assign_tasks_heap(tasks, 2)[1])
    assert sum(weights) == 355 and max(weights) <= 180


def test_heap_partition_matches_reference_vectors():
    """fm_cp_partition_heap and the restatement against assignments computed by the reference's own
    assign_tasks_heap (tests/golden/make_heap_golden.py lifts the function out of
    flashmask/cp_balance/cp_balance.py:96-174 and runs it)."""
    z = np.load(os.path.join(ROOT, "tests", "golden", "heap_partition.npz"))
    n_cases = int(z["n_cases"])
    assert n_cases >= 72
    for k in range(n_cases):
        w, m, want = z[f"w_{k}"], int(z[f"m_{k}"]), z[f"b_{k}"]
        tasks = np.stack([w, np.arange(len(w))], axis=1).astype(np.int32)
        for impl in (cp_balance.assign_tasks_heap, ocp.assign_tasks_heap):
            buckets, bw, cuts = impl(tasks, m)
            got = np.full(len(w), -1, dtype=np.int32)
            for r, items in enumerate(buckets):
                assert [i for _, i in items] == sorted(i for _, i in items)
                got[[int(i) for _, i in items]] = r
            assert np.array_equal(got, want), (k, impl.__module__)
            assert [int(x) for x in bw] == [int(x) for x in z[f"bw_{k}"]]
            assert int(cuts) == int(z[f"cuts_{k}"])


def test_reference_ipo_solver_oracle_if_built():
    """oracle/_ref/libcpsolver_ref.so is the reference's own IPO solver header; the
    heap partition may never beat it and must stay within 4/3 of it (LPT bound)."""
    path = os.path.join(ROOT, "oracle", "_ref", "libcpsolver_ref.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref not built (needs the reference checkout)")
    lib = ctypes.CDLL(path)
    w = np.array([100, 80, 60, 40, 30, 20, 15, 10], dtype=np.int32)
    out = np.empty(8, dtype=np.int32)
    assert lib.ref_ipo_solve(w.ctypes.data, 8, 2, out.ctypes.data) == 180
    rng = np.random.default_rng(0)
    for _ in range(10):
        w = rng.integers(1, 3000, size=64).astype(np.int32)
        out = np.empty(64, dtype=np.int32)
        best = lib.ref_ipo_solve(w.ctypes.data, 64, 8, out.ctypes.data)
        tasks = np.stack([w, np.arange(64)], axis=1)
        _, weights, _ = cp_balance.assign_tasks_heap(tasks, 8)
        assert best <= max(weights) <= best * 4 / 3 + 1
        assert sorted(out.tolist()) == list(range(64))


def test_ipo_partition_matches_reference_vectors():
    """fm_cp_partition_ipo against assignments computed by the reference's own solver
    (tests/golden/make_ipo_golden.py): the same chunk in the same slot of the same rank."""
    g = np.load(os.path.join(ROOT, "tests", "golden", "ipo_partition.npz"))
    for k in range(int(g["n_cases"])):
        w, m = g[f"w_{k}"], int(g[f"m_{k}"])
        a, best = cp_balance.cp_balance_ipo_solve(w, m)
        assert best == int(g[f"best_{k}"]), k
        assert np.array_equal(a, g[f"a_{k}"]), k
        assert best == max(int(w[row].sum()) for row in a)


def test_ipo_partition_matches_reference_solver_if_built():
    path = os.path.join(ROOT, "oracle", "_ref", "libcpsolver_ref.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref not built (needs the reference checkout)")
    lib = ctypes.CDLL(path)
    rng = np.random.default_rng(11)
    for m, per in [(2, 6), (4, 8), (8, 8), (8, 10), (4, 11), (16, 3), (5, 7)]:
        for hi in (6, 300, 100000):
            n = m * per
            w = rng.integers(0, hi, size=n).astype(np.int32)
            ref = np.zeros((m, per), dtype=np.int32)
            best_ref = lib.ref_ipo_solve(w.ctypes.data, n, m, ref.ctypes.data)
            a, best = cp_balance.cp_balance_ipo_solve(w, m)
            assert best == best_ref and np.array_equal(a, ref)


def test_assign_tasks_ipo_interface_and_fallbacks():
    rng = np.random.default_rng(5)
    w = rng.integers(1, 3000, size=64)
    tasks = np.stack([w, np.arange(64)], axis=1).astype(np.int32)
    buckets, weights, cuts = cp_balance.assign_tasks_ipo(tasks, 8)
    heap = cp_balance.assign_tasks_heap(tasks, 8)
    assert sorted(i for b in buckets for _, i in b) == list(range(64))
    assert all(len(b) == 8 and b == sorted(b, key=lambda x: x[1]) for b in buckets)
    assert weights == [sum(x[0] for x in b) for b in buckets]
    lower = max(-(-int(w.sum()) // 8), int(w.max()))
    assert lower <= max(weights) <= max(heap[1])
    # the cases the reference hands to the heap: n not a multiple of the ranks, n > 512, no tasks
    for n, m in [(10, 4), (1024, 8)]:
        t = np.stack([rng.integers(0, 99, size=n), np.arange(n)], axis=1).astype(np.int32)
        assert cp_balance.assign_tasks_ipo(t, m) == cp_balance.assign_tasks_heap(t, m)
    assert cp_balance.assign_tasks_ipo(np.zeros((0, 2), np.int32), 4)[1] == [0, 0, 0, 0]
    # the C entry point refuses what it cannot solve instead of guessing
    lib = cp_balance._lib.load()
    big = np.ones(1024, np.int32)
    out = np.zeros(1024, np.int32)
    assert lib.fm_cp_partition_ipo(big.ctypes.data, 1024, 8, out.ctypes.data, None) == 2
    assert lib.fm_cp_partition_ipo(big.ctypes.data, 10, 4, out.ctypes.data, None) == 1


def test_plan_pairs_are_consistent():
    rng = np.random.default_rng(3)
    for world in (2, 4, 8):
        need = (rng.random((world, world)) < 0.5).tolist()
        plans = [cp.CPPlan(world, r, need) for r in range(world)]
        for r in range(world):
            for o in plans[r].pulls():
                assert r in plans[o].pushes()
            for t in plans[r].pushes():
                assert r in plans[t].pulls()
        # at every ring distance the sends and receives pair up
        for s in range(1, world):
            for r in range(world):
                dst = (r + s) % world
                assert (dst in plans[r].pushes()) == (r in plans[dst].pulls())


def test_rerank_localize_restatement_properties():
    S, C, cpn = 4096, 512, 4
    rng = np.random.default_rng(5)
    idx, _ = W.causal_document_noncausal_form(1, S, S, W.uniform_doc_lengths(rng, S, 9))
    locals_, buckets = zip(*[ocp.balance(idx, cpn, r, C) for r in range(cpn)])
    assert all(b == buckets[0] for b in buckets)
    order = [i for b in buckets[0] for _, i in b]
    assert sorted(order) == list(range(S // C))
    full = W.dense_visible(idx, S, False)[0, 0]
    rows_of = lambda r: np.concatenate([np.arange(i * C, (i + 1) * C) for _, i in buckets[0][r]])
    cols = np.concatenate([np.arange(i * C, (i + 1) * C) for i in order])
    for r in range(cpn):
        vis = W.dense_visible(locals_[r], S // cpn, False)[0, 0]      # [S_local, S]
        assert np.array_equal(vis, full[np.ix_(rows_of(r), cols)]), r


_GLOO_SCRIPT = r"""
import os, sys
sys.path.insert(0, {root!r})
import torch, torch.distributed as dist
from flashmask_b200 import cp
rank, world = int(sys.argv[1]), 2
os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT={port!r})
dist.init_process_group("gloo", rank=rank, world_size=world)
ex = cp.TorchDistExchange(None)
row = torch.tensor([rank == 0, True])
need = ex.all_gather_need(row)
assert need == [[True, True], [False, True]], need
plan = cp.CPPlan(world, rank, need)
assert plan.pulls() == ([1] if rank == 0 else []) and plan.pushes() == ([] if rank == 0 else [0])
# shard round trip with gloo point-to-point in the order the plan dictates
x = torch.full((4,), float(rank))
if rank == 1:
    dist.send(x, 0)
else:
    y = torch.empty(4); dist.recv(y, 1); assert float(y[0]) == 1.0
dist.barrier(); dist.destroy_process_group()
print("rank", rank, "ok")
"""


_GLOO_REPLAN = r"""
import os, sys
sys.path.insert(0, {root!r})
import numpy as np, torch, torch.distributed as dist
from flashmask_b200 import cp, workloads as W
rank, world = int(sys.argv[1]), 2
os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT={port!r})
dist.init_process_group("gloo", rank=rank, world_size=world)
S = 64                                     # rows per rank = keys per shard
def need_row(mask, Sq, causal, world):     # CPU stand-in of the device kernel: exact visibility per shard
    vis = W.dense_visible(mask.numpy(), Sq, causal)[0, 0]
    return torch.from_numpy(vis.reshape(Sq, world, -1).any(axis=(0, 2)))
def mask_all():                            # every key visible to every row
    m = np.zeros((1, 1, world * S, 2), np.int32); m[..., 0] = S; return m
def mask_own_only():                       # only the own shard visible
    m = np.zeros((1, 1, world * S, 2), np.int32); m[..., 1] = S
    m[:, :, rank * S:(rank + 1) * S, 0] = S; m[:, :, rank * S:(rank + 1) * S, 1] = 0; return m
ex = cp.TorchDistExchange(None)
gathers = [0]
orig = ex.all_gather_need
def counted(row):
    gathers[0] += 1
    return orig(row)
ex.all_gather_need = counted
state = lambda t: cp.mask_state(t, S, S, 128, 128, ex, need_row_fn=need_row)
buf = torch.from_numpy(mask_all())
st1 = state(buf)
assert st1.plan.need == [[True, True], [True, True]] and st1.owners == [1 - rank] and gathers[0] == 1
assert state(buf) is st1 and gathers[0] == 1          # same tensor, unchanged: no second all-gather
# a different mask of the same shape written into the SAME buffer: the plan is rebuilt on every rank
buf.copy_(torch.from_numpy(mask_own_only()))
st2 = state(buf)
assert gathers[0] == 2 and st2.plan.need == [[True, False], [False, True]] and st2.owners == []
assert st2.rest_mask is None
# a new tensor object that aliases that storage (what the caching allocator hands to the next step's mask)
alias = buf.view(buf.shape)
alias.copy_(torch.from_numpy(mask_all()))
st3 = state(alias)
assert gathers[0] == 3 and st3.plan.need == [[True, True], [True, True]]
# ... and the old tensor object, whose version counter the write moved too, no longer hits its stale entry
st4 = state(buf)
assert gathers[0] == 4 and st4.plan.need == [[True, True], [True, True]]
del alias
import gc; gc.collect()
assert all(e[0]() is not None for e in cp._STATE_CACHE.values())   # entries die with their tensors
dist.barrier(); dist.destroy_process_group()
print("rank", rank, "ok")
"""


def test_plan_is_rebuilt_when_the_mask_changes_two_ranks_gloo(tmp_path):
    script = tmp_path / "gloo_replan.py"
    script.write_text(_GLOO_REPLAN.format(root=ROOT, port=str(31500 + os.getpid() % 2000)))
    procs = [subprocess.Popen([sys.executable, str(script), str(r)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=120)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, o


def test_plan_exchange_two_ranks_gloo(tmp_path):
    script = tmp_path / "gloo_cp.py"
    script.write_text(_GLOO_SCRIPT.format(root=ROOT, port=str(29500 + os.getpid() % 2000)))
    procs = [subprocess.Popen([sys.executable, str(script), str(r)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=120)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, o
        assert f"rank {r} ok" in o
