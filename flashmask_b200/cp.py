"""Context-parallel ``flashmask_attention``: queries, keys and values are
sharded along the sequence; every rank attends its local queries to the key
shards it needs.

Semantics of the ``group=`` entry (reference: flashmask/overlap/overlap_runtime.py:175-232,
flashmask/cute/ops/fwd.py:282-313, ops/bwd.py:87-89): ``key`` / ``value`` are
this rank's shards, the mask's key axis spans all ranks in group-rank order,
its row bounds are local rows, and ``dk`` / ``dv`` come back reduced onto the
owner of each shard.

Schedule (one NVSwitch domain, every peer at full bandwidth): a rank pulls the
shards it needs straight from their owners with ONE grouped NCCL send/recv on a
high-priority side stream, into one local K/V buffer that holds the pulled
shards concatenated in rank order of their owners.  The forward is two attention calls
whatever the group size: local queries x own shard (overlaps with the
exchange) and local queries x that remote buffer (one launch; tile skipping
drops the parts of shards that nothing sees), merged by log-sum-exp in
fp32.  A (rank, shard) pair whose part of the mask holds no visible element is
neither transferred nor given a place in the buffer; all ranks derive the same
need matrix from one small all-gather, once per mask tensor (the split masks,
their tile reductions and launch tables are kept with it).  The backward runs the remote call first, sends each owner the
bf16 dK/dV slice of its shard while the own-shard call runs, and every owner
sums the contributions in rank order in fp32 and rounds once: bitwise
reproducible.  Remote data is only ever consumed from local HBM.
"""
from __future__ import annotations

import ctypes as C
import math
import weakref
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import torch

from . import _lib
from .ops import (FlashMaskInfo, _dtype_code, _flash_attn_bwd, _flash_attn_fwd, _stream, bwd_tile_shape,
                  prepare_mask)

__all__ = ["cp_flashmask_attention", "CPPlan", "CPMaskState", "TorchDistExchange", "RemoteKV", "mask_state",
           "invalidate_mask_state", "cp_forward", "emulate_cp", "shard_need_row", "profile_phases",
           "phase_report"]


# ---------------------------------------------------------------------------
# optional per-phase device timing (CUDA events on the compute stream)
# ---------------------------------------------------------------------------
_PHASES: Optional[list] = None


def profile_phases(on: bool) -> None:
    """Start (or stop and drop) the recording of phase marks: every phase boundary of the
    context-parallel forward / backward records a CUDA event on the current stream."""
    global _PHASES
    _PHASES = [] if on else None


def _mark(name: str) -> None:
    if _PHASES is not None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        _PHASES.append((name, ev))


def phase_report() -> Dict[str, float]:
    """Milliseconds per phase since profile_phases(True), summed over calls: the time between a
    mark and the one before it on the compute stream (idle time of the stream, e.g. waiting for
    the host or for a transfer, counts towards the phase it precedes).  Clears the marks."""
    global _PHASES
    out: Dict[str, float] = {}
    if not _PHASES:
        return out
    torch.cuda.synchronize()
    for (n0, e0), (n1, e1) in zip(_PHASES[:-1], _PHASES[1:]):
        # the stretch that ends at a ":begin" mark is what lies between two calls (host work, other
        # kernels of the step): reported as "gap_before_fwd" / "gap_before_bwd"
        name = "gap_before_" + n1[:-6] if n1.endswith(":begin") else n1
        out[name] = out.get(name, 0.0) + e0.elapsed_time(e1)
    _PHASES = []
    return out


# ---------------------------------------------------------------------------
# plan: who needs which shard
# ---------------------------------------------------------------------------
@dataclass
class CPPlan:
    world: int
    rank: int
    need: List[List[bool]]      # need[r][o]: rank r attends to the shard owned by rank o

    def pulls(self) -> List[int]:
        """Owners whose shard this rank pulls, nearest first (ring distance)."""
        return [o for s in range(1, self.world) for o in [(self.rank - s) % self.world]
                if self.need[self.rank][o]]

    def pushes(self) -> List[int]:
        """Ranks that pull this rank's shard, in the order they ask for it."""
        return [t for s in range(1, self.world) for t in [(self.rank + s) % self.world]
                if self.need[t][self.rank]]

    def pull_order(self) -> List[int]:
        """The pulled owners in rank order: the order of their shards in the remote K/V buffer."""
        return sorted(self.pulls())


def shard_need_row(local_mask: Optional[torch.Tensor], Sq: int, causal: bool, world: int) -> torch.Tensor:
    """bool [world] on the device: which key shards hold a visible element for
    this rank's rows."""
    if local_mask is None:
        return torch.ones(world, dtype=torch.bool, device="cuda")
    m = local_mask.contiguous()
    B, Hm, Sk, ncols = m.shape
    out = torch.empty((B * Hm, world), dtype=torch.int64, device=m.device)
    _lib.check(_lib.load().fm_cp_shard_visible(m.data_ptr(), B, Hm, Sq, Sk, ncols, int(causal), world,
                                               out.data_ptr(), _stream(m)), "fm_cp_shard_visible")
    return out.sum(dim=0) > 0


# ---------------------------------------------------------------------------
# exchange over a torch.distributed group
# ---------------------------------------------------------------------------
class TorchDistExchange:
    """NCCL point-to-point over a torch.distributed group.  One grouped
    send/recv (a single NCCL launch for all peers) per direction, issued from a
    side stream before the compute it overlaps with is enqueued."""

    def __init__(self, group):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.comm_stream = torch.cuda.Stream(priority=-1) if torch.cuda.is_available() else None

    def _global(self, r):
        return self.dist.get_global_rank(self.group, r) if self.group is not None else r

    def all_gather_need(self, row: torch.Tensor) -> List[List[bool]]:
        rows = [torch.empty_like(row) for _ in range(self.world)]
        self.dist.all_gather(rows, row, group=self.group)
        return [[bool(v) for v in r.cpu().tolist()] for r in rows]

    def exchange(self, send: Dict[int, List[torch.Tensor]], recv: Dict[int, List[torch.Tensor]]):
        """Post all sends and receives as one group on the side stream (ordered
        after the work already enqueued on the current stream).  Returns a CUDA
        event that fires when every receive has landed."""
        dist = self.dist
        cur = torch.cuda.current_stream()
        self.comm_stream.wait_stream(cur)
        ev = torch.cuda.Event()
        with torch.cuda.stream(self.comm_stream):
            ops = []
            for s in range(1, self.world):        # same peer order on every rank
                for peer, table, fn in (((self.rank + s) % self.world, send, dist.isend),
                                        ((self.rank - s) % self.world, recv, dist.irecv)):
                    if peer in table:
                        ops += [dist.P2POp(fn, t, self._global(peer), self.group) for t in table[peer]]
            if ops:
                for w in dist.batch_isend_irecv(ops):
                    w.wait()
            ev.record(self.comm_stream)
        for ts in list(send.values()) + list(recv.values()):
            for t in ts:
                t.record_stream(self.comm_stream)
        return ev


# ---------------------------------------------------------------------------
# numerics helpers through the C ABI
# ---------------------------------------------------------------------------
def _merge(acc, lse_run, o_s, lse_s, first):
    B, S, H, dv = o_s.shape
    _lib.check(_lib.load().fm_cp_merge_partial(acc.data_ptr(), lse_run.data_ptr(), o_s.data_ptr(), lse_s.data_ptr(),
                                               B, S, H, dv, _dtype_code(o_s), int(first), _stream(o_s)),
               "fm_cp_merge_partial")


def _accumulate(acc, x, first):
    _lib.check(_lib.load().fm_cp_accumulate(acc.data_ptr(), x.data_ptr(), x.numel(), _dtype_code(x), int(first),
                                            _stream(x)), "fm_cp_accumulate")


def _cast(acc, like):
    out = torch.empty(acc.shape, dtype=like.dtype, device=acc.device)
    _lib.check(_lib.load().fm_cp_cast(acc.data_ptr(), out.data_ptr(), acc.numel(), _dtype_code(like), _stream(acc)),
               "fm_cp_cast")
    return out


def _reduce_partials(parts: List[torch.Tensor]) -> torch.Tensor:
    parts = [p.contiguous() for p in parts]
    out = torch.empty_like(parts[0])
    arr = (C.c_void_p * len(parts))(*[p.data_ptr() for p in parts])
    _lib.check(_lib.load().fm_cp_reduce_partials(arr, len(parts), out.data_ptr(), out.numel(),
                                                 _dtype_code(out), _stream(out)), "fm_cp_reduce_partials")
    return out


# ---------------------------------------------------------------------------
# per-rank forward / backward: two attention calls whatever the group size
#   "own"    local queries x this rank's own K/V shard (needs no transfer and
#            overlaps with the exchange)
#   "remote" local queries x every pulled shard, concatenated in rank order in
#            ONE K/V buffer with the matching mask columns: one launch, tile
#            skipping takes care of the parts of shards nothing sees
# ---------------------------------------------------------------------------
def _split_mask(local_mask, rank, S_shard, owners):
    """(mask of the own shard's columns, mask of the columns of the shards owned by ``owners``,
    concatenated in that order)."""
    if local_mask is None:
        return None, None
    lo, hi = rank * S_shard, (rank + 1) * S_shard
    own = local_mask[:, :, lo:hi].contiguous()
    rest = None
    if owners:
        rest = torch.cat([local_mask[:, :, o * S_shard:(o + 1) * S_shard] for o in owners], dim=2).contiguous()
    return own, rest


class RemoteKV:
    """K/V of the shards this rank pulls, concatenated along the sequence in rank order of their
    owners.  Only pulled shards have a place in it, so every byte of the buffer is written by a
    transfer before a kernel reads it.  For batch 1 the receive buffers ARE slices of the
    concatenation; larger batches receive per owner and are copied into place."""

    def __init__(self, k, v, owners: List[int]):
        B, S, H, d = k.shape
        self.B, self.S, self.owners = B, S, list(owners)
        self.pos = {o: i for i, o in enumerate(self.owners)}
        n = len(self.owners)
        self.k = torch.empty((B, n * S, H, d), dtype=k.dtype, device=k.device)
        self.v = torch.empty((B, n * S, v.shape[2], v.shape[3]), dtype=v.dtype, device=v.device)
        self.tmp = {}

    def recv_buffers(self, owner):
        pos = self.pos[owner]
        ks, vs = self.k[:, pos * self.S:(pos + 1) * self.S], self.v[:, pos * self.S:(pos + 1) * self.S]
        if self.B == 1:
            return [ks, vs]
        self.tmp[owner] = (torch.empty_like(ks.contiguous()), torch.empty_like(vs.contiguous()), ks, vs)
        return list(self.tmp[owner][:2])

    def finalize(self):
        for tk, tv, ks, vs in self.tmp.values():
            ks.copy_(tk); vs.copy_(tv)
        self.tmp = {}

    def slice_of(self, t, owner):
        pos = self.pos[owner]
        return t[:, pos * self.S:(pos + 1) * self.S]


# ---------------------------------------------------------------------------
# what depends on the mask only: built once per mask, reused by every forward and backward
# ---------------------------------------------------------------------------
@dataclass
class CPMaskState:
    plan: CPPlan
    owners: List[int]                         # pulled owners in rank order
    own_mask: Optional[torch.Tensor]
    rest_mask: Optional[torch.Tensor]
    own_info: Optional[FlashMaskInfo] = None  # per-K-tile reductions + launch tables of the two calls
    rest_info: Optional[FlashMaskInfo] = None


def _build_state(local_mask, Sq, S_shard, d, dv, plan: CPPlan) -> CPMaskState:
    owners = plan.pull_order()
    own, rest = _split_mask(local_mask, plan.rank, S_shard, owners)
    st = CPMaskState(plan, owners, own, rest)
    if local_mask is not None and local_mask.is_cuda:
        tm, tn = bwd_tile_shape(d, dv)
        if plan.need[plan.rank][plan.rank]:
            st.own_info = prepare_mask(own, Sq, False, tm, tn)
        if rest is not None:
            st.rest_info = prepare_mask(rest, Sq, False, tm, tn)
    return st


# id(mask) -> (weak reference to the mask, its version counter, geometry key, state)
_STATE_CACHE: Dict[int, tuple] = {}


def invalidate_mask_state(local_mask=None) -> None:
    """Forget the cached plan of ``local_mask`` (of every mask when None).  Needed only after a
    mask tensor has been rewritten in place behind torch's back (through a raw pointer): tensor
    identity and torch's version counter, which the cache is keyed on, do not see such a write."""
    if local_mask is None:
        _STATE_CACHE.clear()
    else:
        _STATE_CACHE.pop(id(local_mask), None)


def mask_state(local_mask, Sq, S_shard, d, dv, ex, need_row_fn: Optional[Callable] = None) -> CPMaskState:
    """Plan, split masks and their tile reductions for ``local_mask`` on this rank.

    The need matrix costs one small all-gather and a device->host read, the split two copies of
    the mask and the reductions two kernel launches; all of it depends on the mask only.  The
    state is kept on the mask TENSOR: the cache entry is found by the tensor's identity, is valid
    only while that very tensor object is alive (weak reference) and unchanged (torch version
    counter), and never by its storage address, which the caching allocator hands out again for the
    next step's mask.  A new mask tensor therefore always rebuilds the plan, on every rank alike."""
    geom = (Sq, S_shard, d, dv, ex.world, ex.rank, id(ex.group))
    if local_mask is not None:
        ent = _STATE_CACHE.get(id(local_mask))
        if ent is not None and ent[0]() is local_mask and ent[1] == local_mask._version and ent[2] == geom:
            return ent[3]
    row = (need_row_fn or shard_need_row)(local_mask, Sq, False, ex.world)
    plan = CPPlan(ex.world, ex.rank, ex.all_gather_need(row))
    st = _build_state(local_mask, Sq, S_shard, d, dv, plan)
    if local_mask is not None:
        key = id(local_mask)
        ref = weakref.ref(local_mask, lambda _r, key=key: _STATE_CACHE.pop(key, None))
        _STATE_CACHE[key] = (ref, local_mask._version, geom, st)
    return st


_EXCHANGES: Dict[int, "TorchDistExchange"] = {}


def _exchange_for(group) -> "TorchDistExchange":
    """One exchange object (and one side stream) per process group."""
    ex = _EXCHANGES.get(id(group))
    if ex is None or ex.group is not group:
        ex = TorchDistExchange(group)
        _EXCHANGES[id(group)] = ex
    return ex


def cp_forward(q, k, v, remote: Optional[RemoteKV], st: CPMaskState, softmax_scale, sink, ready=None):
    """Returns (out, lse).  ``ready``: CUDA event after which ``remote`` is complete."""
    plan = st.plan
    need_own = plan.need[plan.rank][plan.rank]
    need_remote = remote is not None and len(st.owners) > 0
    parts = []
    _mark("fwd:begin")
    if need_own:
        parts.append(_flash_attn_fwd(q, k, v, st.own_mask, softmax_scale=softmax_scale, causal=False,
                                     learnable_sink=sink, mask_info=st.own_info))
        _mark("fwd_own")
    if need_remote:
        if ready is not None:
            torch.cuda.current_stream().wait_event(ready)
        remote.finalize()
        _mark("fwd_wait_kv")
        # the sink logit joins the softmax once: with the first partial only
        parts.append(_flash_attn_fwd(q, remote.k, remote.v, st.rest_mask, softmax_scale=softmax_scale,
                                     causal=False, learnable_sink=None if need_own else sink,
                                     mask_info=st.rest_info))
        _mark("fwd_remote")
    if len(parts) == 1:
        return parts[0]
    B, Sq, Hq, _ = q.shape
    dv = v.shape[-1]
    if not parts:
        return (torch.zeros((B, Sq, Hq, dv), dtype=q.dtype, device=q.device),
                torch.full((B, Hq, Sq), float("-inf"), dtype=torch.float32, device=q.device))
    (o_a, lse_a), (o_b, lse_b) = parts
    lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
    # both partials are contiguous [B, Sq, Hq, dv]; the merged rows overwrite the first one
    _lib.check(_lib.load().fm_cp_merge_two(o_a.data_ptr(), lse_a.data_ptr(), o_b.data_ptr(), lse_b.data_ptr(),
                                           o_a.data_ptr(), lse.data_ptr(), B, Sq, Hq, dv, _dtype_code(o_a),
                                           _stream(o_a)), "fm_cp_merge_two")
    _mark("fwd_merge")
    return o_a, lse


def cp_backward_remote(q, remote, out, dout, lse, st: CPMaskState, softmax_scale, deterministic, dq_chain=None):
    """Gradients of the remote call: (dq_remote, dk_all_remote, dv_all_remote).  With ``dq_chain``
    (and the own-shard call still to come) dq may stay in the chain's accumulator: dq_remote is None."""
    dq, dk, dv, _ = _flash_attn_bwd(q, remote.k, remote.v, out, dout, lse, st.rest_mask, softmax_scale=softmax_scale,
                                    causal=False, deterministic=deterministic, mask_info=st.rest_info,
                                    dq_chain=dq_chain)
    return dq, dk, dv


def cp_backward_own(q, k, v, out, dout, lse, st: CPMaskState, softmax_scale, sink, deterministic, dq_chain=None):
    return _flash_attn_bwd(q, k, v, out, dout, lse, st.own_mask, softmax_scale=softmax_scale, causal=False,
                           learnable_sink=sink, deterministic=deterministic, mask_info=st.own_info,
                           dq_chain=dq_chain)


def _dq_chain(n_calls: int):
    """Chain record for the backward calls of one rank: with two calls (pulled shards, then own shard) the
    first leaves its dQ in the fp32 accumulator of the one-kernel backward and the second rounds the sum."""
    return {"last": False} if n_calls == 2 else None


def _sum_dq(dq_a, dq_b):
    if dq_a is None:
        return dq_b
    if dq_b is None:
        return dq_a
    return _reduce_partials([dq_a, dq_b])      # fp32 sum of the two, rounded once


def _dsink_only(q, k, v, out, dout, lse, sink, softmax_scale):
    # no shard of this rank's own keys is visible: the sink gradient still needs
    # rowsum(O*dO) and LSE; run the own call on an all-masked single column set
    idx = torch.zeros((q.shape[0], 1, k.shape[1], 2), dtype=torch.int32, device=q.device)
    idx[..., 1] = q.shape[1]
    return _flash_attn_bwd(q, k, v, out, dout, lse, idx, softmax_scale=softmax_scale, causal=False,
                           learnable_sink=sink, deterministic=True)[3]


# ---------------------------------------------------------------------------
# autograd entry for real process groups
# ---------------------------------------------------------------------------
class _CPFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, local_mask, softmax_scale, sink, deterministic, group):
        ex = _exchange_for(group)
        k, v = k.contiguous(), v.contiguous()
        st = mask_state(local_mask, q.shape[1], k.shape[1], q.shape[3], v.shape[3], ex)
        plan = st.plan
        remote = RemoteKV(k, v, st.owners)
        recv = {o: remote.recv_buffers(o) for o in plan.pulls()}
        send = {t: [k, v] for t in plan.pushes()}
        ready = ex.exchange(send, recv)                     # overlaps with the own-shard call below
        out, lse = cp_forward(q, k, v, remote, st, softmax_scale, sink, ready)
        torch.cuda.current_stream().wait_stream(ex.comm_stream)
        ctx.save_for_backward(q, k, v, out, lse, sink)
        ctx.remote, ctx.st, ctx.ex = remote, st, ex          # pulled shards are kept for the backward
        ctx.softmax_scale, ctx.deterministic = softmax_scale, deterministic
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, dout, dlse):
        q, k, v, out, lse, sink = ctx.saved_tensors
        st, ex, remote = ctx.st, ctx.ex, ctx.remote
        plan = st.plan
        det = ctx.deterministic
        if det is None:
            det = torch.are_deterministic_algorithms_enabled()
        dout = dout.contiguous()
        need_own = plan.need[plan.rank][plan.rank]
        dq_r = None
        send, ready = {}, None
        recv = {t: [torch.empty_like(k), torch.empty_like(v)] for t in plan.pushes()}
        chain = _dq_chain(int(bool(st.owners)) + int(need_own))
        _mark("bwd:begin")
        if st.owners:
            dq_r, dk_all, dv_all = cp_backward_remote(q, remote, out, dout, lse, st, ctx.softmax_scale, det, chain)
            send = {o: [remote.slice_of(dk_all, o).contiguous(), remote.slice_of(dv_all, o).contiguous()]
                    for o in plan.pulls()}
            _mark("bwd_remote")
        if send or recv:
            ready = ex.exchange_reverse(send, recv)          # overlaps with the own-shard call below
        dq_o = dsink = None
        own = None
        if need_own:
            if chain is not None:
                chain["last"] = True
            dq_o, dk_o, dv_o, dsink = cp_backward_own(q, k, v, out, dout, lse, st, ctx.softmax_scale, sink, det, chain)
            own = (dk_o, dv_o)
            _mark("bwd_own")
        elif sink is not None:
            dsink = _dsink_only(q, k, v, out, dout, lse, sink, ctx.softmax_scale)
        dq = _sum_dq(dq_o, dq_r)
        if dq is None:
            dq = torch.zeros_like(q)
        _mark("bwd_dq_sum")
        if ready is not None:
            torch.cuda.current_stream().wait_event(ready)
        _mark("bwd_wait_dkv")
        by_rank = {t: ts for t, ts in recv.items()}
        if own is not None:
            by_rank[plan.rank] = list(own)
        ranks = sorted(by_rank)                              # fixed summation order: by rank
        if ranks:
            dk = _reduce_partials([by_rank[r][0] for r in ranks])
            dv = _reduce_partials([by_rank[r][1] for r in ranks])
        else:
            dk, dv = torch.zeros_like(k), torch.zeros_like(v)
        _mark("bwd_reduce_dkv")
        torch.cuda.current_stream().wait_stream(ex.comm_stream)
        return dq, dk, dv, None, None, dsink, None, None


def _exchange_reverse(self, send, recv):
    """Gradient direction: partials go to the shard owners (the ranks this rank
    pulled from), contributions come from the ranks that pulled this shard."""
    dist = self.dist
    cur = torch.cuda.current_stream()
    self.comm_stream.wait_stream(cur)
    ev = torch.cuda.Event()
    with torch.cuda.stream(self.comm_stream):
        ops = []
        for s in range(1, self.world):
            for peer, table, fn in (((self.rank - s) % self.world, send, dist.isend),
                                    ((self.rank + s) % self.world, recv, dist.irecv)):
                if peer in table:
                    ops += [dist.P2POp(fn, t, self._global(peer), self.group) for t in table[peer]]
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        ev.record(self.comm_stream)
    for ts in list(send.values()) + list(recv.values()):
        for t in ts:
            t.record_stream(self.comm_stream)
    return ev


TorchDistExchange.exchange_reverse = _exchange_reverse


def cp_flashmask_attention(query, key, value, startend_row_indices=None, *, causal=False, softmax_scale=None,
                           sink=None, deterministic=None, group=None):
    """Context-parallel attention over ``group``; returns ``(out, lse)`` for the
    local queries.  Masks must be in the non-causal 2- or 4-column form with
    local row bounds (``balance_flashmask_input`` produces exactly that)."""
    if causal:
        raise NotImplementedError("context parallel takes non-causal 2/4-column masks (express a causal mask "
                                  "with UTE[j] = j), as the reference does (cp_balance.py:43-48)")
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(query.shape[-1])
    return _CPFunc.apply(query, key, value, startend_row_indices, softmax_scale, sink, deterministic, group)


# ---------------------------------------------------------------------------
# single-process emulation (all ranks on one GPU)
# ---------------------------------------------------------------------------
def emulate_cp(qs, ks, vs, douts, local_masks, softmax_scale=None, sink=None, deterministic=True, poison=None):
    """Run the context-parallel schedule for ``world = len(qs)`` ranks inside
    one process (tests of the arithmetic and of the schedule without several
    GPUs): plans, forward, backward partials, owner reductions, with exchanges
    replaced by copies.  ``poison``: value the receive buffers are filled with before the copies
    (a test passes NaN to show that nothing a kernel reads is left unwritten).  Returns per-rank
    lists (out, lse, dq, dk, dv) and dsink."""
    world = len(qs)
    Sq = qs[0].shape[1]
    S = ks[0].shape[1]
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(qs[0].shape[-1])
    need = [[bool(x) for x in shard_need_row(local_masks[r], Sq, False, world).cpu().tolist()]
            for r in range(world)]
    plans = [CPPlan(world, r, need) for r in range(world)]
    ks = [k.contiguous() for k in ks]
    vs = [v.contiguous() for v in vs]
    d, dvd = qs[0].shape[3], vs[0].shape[3]
    states = [_build_state(local_masks[r], Sq, S, d, dvd, plans[r]) for r in range(world)]
    remotes, outs, lses = [], [], []
    for r in range(world):
        rem = RemoteKV(ks[r], vs[r], states[r].owners)
        if poison is not None:
            rem.k.fill_(poison); rem.v.fill_(poison)
        for o in plans[r].pulls():
            bufs = rem.recv_buffers(o)
            bufs[0].copy_(ks[o]); bufs[1].copy_(vs[o])
        remotes.append(rem)
        out, lse = cp_forward(qs[r], ks[r], vs[r], rem, states[r], softmax_scale, sink)
        outs.append(out); lses.append(lse)
    dqs, contrib, dsinks = [], {o: {} for o in range(world)}, []
    for r in range(world):
        dq_r = dq_o = ds = None
        chain = _dq_chain(int(bool(states[r].owners)) + int(need[r][r]))
        if states[r].owners:
            dq_r, dk_all, dv_all = cp_backward_remote(qs[r], remotes[r], outs[r], douts[r], lses[r], states[r],
                                                      softmax_scale, deterministic, chain)
            for o in plans[r].pulls():
                contrib[o][r] = (remotes[r].slice_of(dk_all, o), remotes[r].slice_of(dv_all, o))
        if need[r][r]:
            if chain is not None:
                chain["last"] = True
            dq_o, dk_o, dv_o, ds = cp_backward_own(qs[r], ks[r], vs[r], outs[r], douts[r], lses[r], states[r],
                                                   softmax_scale, sink, deterministic, chain)
            contrib[r][r] = (dk_o, dv_o)
        elif sink is not None:
            ds = _dsink_only(qs[r], ks[r], vs[r], outs[r], douts[r], lses[r], sink, softmax_scale)
        dq = _sum_dq(dq_o, dq_r)
        dqs.append(dq if dq is not None else torch.zeros_like(qs[r]))
        dsinks.append(ds)
    dks, dvs = [], []
    for o in range(world):
        ranks = sorted(contrib[o])
        if ranks:
            dks.append(_reduce_partials([contrib[o][r][0] for r in ranks]))
            dvs.append(_reduce_partials([contrib[o][r][1] for r in ranks]))
        else:
            dks.append(torch.zeros_like(ks[o])); dvs.append(torch.zeros_like(vs[o]))
    dsink = None
    if sink is not None:
        dsink = torch.stack([d.float() for d in dsinks]).sum(0)
    return outs, lses, dqs, dks, dvs, dsink
