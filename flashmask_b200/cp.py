"""Context-parallel ``flashmask_attention``: queries, keys and values are
sharded along the sequence; every rank attends its local queries to the key
shards it needs.

Semantics of the ``group=`` entry (reference: flashmask/overlap/overlap_runtime.py:175-232,
flashmask/cute/ops/fwd.py:282-313, ops/bwd.py:87-89): ``key`` / ``value`` are
this rank's shards, the mask's key axis spans all ranks in group-rank order,
its row bounds are local rows, and ``dk`` / ``dv`` come back reduced onto the
owner of each shard.

Schedule (one NVSwitch domain, every peer at full bandwidth): a rank pulls the
shards it needs straight from their owners with NCCL send/recv pairs on a side
stream, all posted up front into separate local buffers, and computes step by
step as shards land (CUDA events gate each step).  A (rank, shard) pair whose
tile of the mask holds no visible element is skipped: no transfer, no compute;
all ranks derive the same need matrix from one small all-gather.  Forward
partials are merged by log-sum-exp in fp32.  Backward sends the bf16 dK/dV
partial of every needed shard to its owner, which sums all partials in rank
order in fp32 and rounds once: bitwise reproducible.  Remote data is only ever
consumed from local HBM.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from . import _lib
from .ops import _dtype_code, _flash_attn_bwd, _flash_attn_fwd, _stream

__all__ = ["cp_flashmask_attention", "CPPlan", "TorchDistExchange", "InProcessExchange", "build_plan",
           "cp_forward", "cp_backward"]


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
# exchanges
# ---------------------------------------------------------------------------
class TorchDistExchange:
    """NCCL point-to-point over a torch.distributed group, on a side stream."""

    def __init__(self, group):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.comm_stream = torch.cuda.Stream() if torch.cuda.is_available() else None

    def _global(self, r):
        return self.dist.get_global_rank(self.group, r) if self.group is not None else r

    def all_gather_need(self, row: torch.Tensor) -> List[List[bool]]:
        rows = [torch.empty_like(row) for _ in range(self.world)]
        self.dist.all_gather(rows, row, group=self.group)
        return [[bool(v) for v in r.cpu().tolist()] for r in rows]

    def exchange(self, send: Dict[int, List[torch.Tensor]], recv: Dict[int, List[torch.Tensor]], order: List[int]):
        """Post every send / recv on the side stream, paired per ring distance so
        both ends issue matching operations in the same order.  Returns one CUDA
        event per source rank in ``recv``."""
        dist = self.dist
        cur = torch.cuda.current_stream()
        self.comm_stream.wait_stream(cur)
        events = {}
        with torch.cuda.stream(self.comm_stream):
            for s in range(1, self.world):
                src, dst = (self.rank - s) % self.world, (self.rank + s) % self.world
                ops = []
                if dst in send:
                    ops += [dist.P2POp(dist.isend, t, self._global(dst), self.group) for t in send[dst]]
                if src in recv:
                    ops += [dist.P2POp(dist.irecv, t, self._global(src), self.group) for t in recv[src]]
                if ops:
                    for w in dist.batch_isend_irecv(ops):
                        w.wait()
                if src in recv:
                    ev = torch.cuda.Event()
                    ev.record(self.comm_stream)
                    events[src] = ev
                    for t in recv[src]:
                        t.record_stream(cur)
        for ts in send.values():
            for t in ts:
                t.record_stream(self.comm_stream)
        return events

    def finish(self):
        torch.cuda.current_stream().wait_stream(self.comm_stream)


class InProcessExchange:
    """All ranks live in one process on one GPU (tests of the schedule and of the
    merge / reduce arithmetic without a multi-GPU box).  Ranks are driven in
    lock-step phases by ``emulate_cp``; an exchange is a dictionary lookup."""

    def __init__(self, world: int):
        self.world = world
        self.mail: Dict[tuple, List[torch.Tensor]] = {}


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
    out = torch.empty_like(parts[0])
    arr = (C.c_void_p * len(parts))(*[p.data_ptr() for p in parts])
    _lib.check(_lib.load().fm_cp_reduce_partials(arr, len(parts), out.data_ptr(), out.numel(),
                                                 _dtype_code(out), _stream(out)), "fm_cp_reduce_partials")
    return out


def _mask_slice(local_mask, owner, S_shard):
    if local_mask is None:
        return None
    return local_mask[:, :, owner * S_shard:(owner + 1) * S_shard, :].contiguous()


# ---------------------------------------------------------------------------
# per-rank forward / backward given the shards
# ---------------------------------------------------------------------------
def cp_forward(q, shards: Dict[int, tuple], local_mask, causal, softmax_scale, sink, plan: CPPlan,
               events: Optional[Dict[int, torch.cuda.Event]] = None):
    """Attend local ``q`` to every needed shard (own shard first, then the pulled
    ones in ring-distance order) and merge.  Returns (out, lse)."""
    B, Sq, Hq, d = q.shape
    S_shard = shards[plan.rank][0].shape[1]
    dv = shards[plan.rank][1].shape[-1]
    acc = torch.empty((B, Sq, Hq, dv), dtype=torch.float32, device=q.device)
    lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
    order = ([plan.rank] if plan.need[plan.rank][plan.rank] else []) + plan.pulls()
    first = True
    for o in order:
        if events is not None and o in events:
            torch.cuda.current_stream().wait_event(events[o])
        k_o, v_o = shards[o]
        # the sink logit joins the softmax once: with the first partial only
        o_s, lse_s = _flash_attn_fwd(q, k_o, v_o, _mask_slice(local_mask, o, S_shard), softmax_scale=softmax_scale,
                                     causal=False, learnable_sink=sink if first else None)
        _merge(acc, lse, o_s, lse_s, first)
        first = False
    if first:  # nothing visible at all
        acc.zero_()
        lse.fill_(float("-inf"))
    return _cast(acc, q), lse


def cp_backward(q, shards, out, dout, lse, local_mask, causal, softmax_scale, sink, deterministic, plan: CPPlan,
                events=None):
    """Returns (dq, partials, dsink): ``partials[o] = (dk_o, dv_o)`` are this
    rank's contributions to the gradients of shard ``o``."""
    S_shard = shards[plan.rank][0].shape[1]
    order = ([plan.rank] if plan.need[plan.rank][plan.rank] else []) + plan.pulls()
    dq_acc = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    partials = {}
    dsink = None
    first = True
    for o in order:
        if events is not None and o in events:
            torch.cuda.current_stream().wait_event(events[o])
        k_o, v_o = shards[o]
        dq_s, dk_o, dv_o, ds = _flash_attn_bwd(q, k_o, v_o, out, dout, lse, _mask_slice(local_mask, o, S_shard),
                                               softmax_scale=softmax_scale, causal=False,
                                               learnable_sink=sink if first else None, deterministic=deterministic)
        if first:
            dsink = ds
        _accumulate(dq_acc, dq_s, first)
        partials[o] = (dk_o, dv_o)
        first = False
    if first:
        dq_acc.zero_()
    return _cast(dq_acc, q), partials, dsink


# ---------------------------------------------------------------------------
# autograd entry for real process groups
# ---------------------------------------------------------------------------
_PLAN_CACHE: Dict[tuple, CPPlan] = {}


def build_plan(local_mask, Sq, causal, ex: TorchDistExchange) -> CPPlan:
    """The need matrix costs one small all-gather and a device->host read; it
    depends on the mask only, so it is kept per (mask storage, version, group)."""
    key = None
    if local_mask is not None:
        key = (local_mask.data_ptr(), local_mask._version, tuple(local_mask.shape), Sq, ex.world, ex.rank,
               id(ex.group))
        if key in _PLAN_CACHE:
            return _PLAN_CACHE[key]
    row = shard_need_row(local_mask, Sq, causal, ex.world)
    plan = CPPlan(ex.world, ex.rank, ex.all_gather_need(row))
    if key is not None:
        if len(_PLAN_CACHE) > 64:
            _PLAN_CACHE.clear()
        _PLAN_CACHE[key] = plan
    return plan


class _CPFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, local_mask, softmax_scale, sink, deterministic, group):
        ex = TorchDistExchange(group)
        plan = build_plan(local_mask, q.shape[1], False, ex)
        k, v = k.contiguous(), v.contiguous()
        recv = {o: [torch.empty_like(k), torch.empty_like(v)] for o in plan.pulls()}
        send = {t: [k, v] for t in plan.pushes()}
        events = ex.exchange(send, recv, plan.pulls())
        shards = {plan.rank: (k, v)}
        shards.update({o: tuple(ts) for o, ts in recv.items()})
        out, lse = cp_forward(q, shards, local_mask, False, softmax_scale, sink, plan, events)
        ex.finish()
        ctx.save_for_backward(q, k, v, local_mask, out, lse, sink)
        ctx.shards_remote = {o: ts for o, ts in shards.items() if o != plan.rank}
        ctx.plan, ctx.ex = plan, ex
        ctx.softmax_scale, ctx.deterministic = softmax_scale, deterministic
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, dout, dlse):
        q, k, v, local_mask, out, lse, sink = ctx.saved_tensors
        plan, ex = ctx.plan, ctx.ex
        shards = {plan.rank: (k, v)}
        shards.update(ctx.shards_remote)          # pulled shards are kept from the forward
        det = ctx.deterministic
        if det is None:
            det = torch.are_deterministic_algorithms_enabled()
        dq, partials, dsink = cp_backward(q, shards, out, dout.contiguous(), lse, local_mask, False,
                                          ctx.softmax_scale, sink, det, plan)
        # partials travel back to the owners; what this rank receives are the
        # contributions of the ranks that pulled its shard
        send = {o: list(partials[o]) for o in plan.pulls()}
        recv = {t: [torch.empty_like(k), torch.empty_like(v)] for t in plan.pushes()}
        # directions are mirrored with respect to the forward exchange
        events = _exchange_reverse(ex, send, recv)
        torch.cuda.current_stream().wait_stream(ex.comm_stream)
        own = partials.get(plan.rank)
        by_rank = dict(recv)
        if own is not None:
            by_rank[plan.rank] = list(own)
        ranks = sorted(by_rank)
        if ranks:
            dk = _reduce_partials([by_rank[r][0] for r in ranks])
            dv = _reduce_partials([by_rank[r][1] for r in ranks])
        else:
            dk, dv = torch.zeros_like(k), torch.zeros_like(v)
        return dq, dk, dv, None, None, dsink, None, None


def _exchange_reverse(ex: TorchDistExchange, send, recv):
    """Like ``TorchDistExchange.exchange`` with the ring directions swapped:
    at distance s this rank sends to (rank - s) and receives from (rank + s)."""
    dist = ex.dist
    cur = torch.cuda.current_stream()
    ex.comm_stream.wait_stream(cur)
    with torch.cuda.stream(ex.comm_stream):
        for s in range(1, ex.world):
            dst, src = (ex.rank - s) % ex.world, (ex.rank + s) % ex.world
            ops = []
            if dst in send:
                ops += [dist.P2POp(dist.isend, t, ex._global(dst), ex.group) for t in send[dst]]
            if src in recv:
                ops += [dist.P2POp(dist.irecv, t, ex._global(src), ex.group) for t in recv[src]]
            if ops:
                for w in dist.batch_isend_irecv(ops):
                    w.wait()
    for ts in list(send.values()) + list(recv.values()):
        for t in ts:
            t.record_stream(ex.comm_stream)
    return None


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
def emulate_cp(qs, ks, vs, douts, local_masks, softmax_scale=None, sink=None, deterministic=True):
    """Run the context-parallel schedule for ``world = len(qs)`` ranks inside
    one process, in lock-step phases: plans, forward, backward partials, owner
    reductions.  Returns per-rank lists (out, lse, dq, dk, dv) and dsink."""
    world = len(qs)
    Sq = qs[0].shape[1]
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(qs[0].shape[-1])
    need = [[bool(x) for x in shard_need_row(local_masks[r], Sq, False, world).cpu().tolist()]
            for r in range(world)]
    plans = [CPPlan(world, r, need) for r in range(world)]
    shards = {o: (ks[o].contiguous(), vs[o].contiguous()) for o in range(world)}
    outs, lses, dqs, parts, dsinks = [], [], [], [], []
    for r in range(world):
        mine = {o: shards[o] for o in [r] + plans[r].pulls()}
        out, lse = cp_forward(qs[r], mine, local_masks[r], False, softmax_scale, sink, plans[r])
        outs.append(out); lses.append(lse)
    for r in range(world):
        mine = {o: shards[o] for o in [r] + plans[r].pulls()}
        dq, p_r, ds = cp_backward(qs[r], mine, outs[r], douts[r], lses[r], local_masks[r], False, softmax_scale,
                                  sink, deterministic, plans[r])
        dqs.append(dq); parts.append(p_r); dsinks.append(ds)
    dks, dvs = [], []
    for o in range(world):
        contrib = [parts[r][o] for r in range(world) if o in parts[r]]
        if contrib:
            dks.append(_reduce_partials([c[0] for c in contrib]))
            dvs.append(_reduce_partials([c[1] for c in contrib]))
        else:
            dks.append(torch.zeros_like(ks[o])); dvs.append(torch.zeros_like(vs[o]))
    dsink = None
    if sink is not None:
        dsink = torch.stack([d.float() for d in dsinks]).sum(0)
    return outs, lses, dqs, dks, dvs, dsink
