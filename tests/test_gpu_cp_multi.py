"""Context parallel over real GPUs (NCCL point-to-point on a side stream).
Needs at least two visible GPUs; child processes, NVLS off, no rank leaves
with work in flight."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_WORKER = r"""
import os, sys
sys.path.insert(0, {root!r})
import numpy as np, torch, torch.distributed as dist
import flashmask_b200 as fm
from flashmask_b200 import cp, cp_balance, workloads as W
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
S, chunk, Hq, Hkv = 8192, 512, 8, 2
rng = np.random.default_rng(5)
idx_np = W.causal_document_noncausal_form(1, S, S, W.lognormal_doc_lengths(rng, S, np.log(1024), 1.2, 64, S))[0]
idx = torch.from_numpy(np.ascontiguousarray(idx_np)).cuda()
g = torch.Generator().manual_seed(0)
q, k, v, do = (torch.randn(1, S, h, 128, generator=g).bfloat16().cuda() for h in (Hq, Hkv, Hkv, Hq))
local, buckets = cp_balance.balance_flashmask_input(idx, world, rank, balance_chunk_size=chunk)
ql, kl, vl, dol = (cp_balance.scatter_by_buckets(t, buckets, rank) for t in (q, k, v, do))
ql, kl, vl = (t.requires_grad_(True) for t in (ql, kl, vl))
out, lse = fm.flashmask_attention(ql, kl, vl, local, causal=False, return_lse=True, group=dist.group.WORLD,
                                  deterministic=True)
out.backward(dol)
torch.cuda.synchronize()
# single-GPU answer on every rank, scattered the same way
qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
o_ref, lse_ref = fm.flashmask_attention(qg, kg, vg, idx, causal=False, return_lse=True)
o_ref.backward(do)
ok = True
for name, a, b in (("out", out, o_ref), ("dq", ql.grad, qg.grad), ("dk", kl.grad, kg.grad), ("dv", vl.grad, vg.grad)):
    bl = cp_balance.scatter_by_buckets(b.detach(), buckets, rank)
    err = (a.float() - bl.float()).abs().max().item()
    tol = 2 ** -7 * world * max(1.0, bl.float().abs().max().item())
    if not err <= tol:
        ok = False
        print(f"rank {{rank}} {{name}} err {{err}} tol {{tol}}", flush=True)
flag = torch.tensor([1 if ok else 0], device="cuda")
dist.all_reduce(flag, op=dist.ReduceOp.MIN)
dist.barrier()
dist.destroy_process_group()
assert flag.item() == 1
print("rank", rank, "ok", flush=True)
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_cp_real_ranks(tmp_path):
    world = min(4, torch.cuda.device_count())
    script = tmp_path / "cp_worker.py"
    script.write_text(_WORKER.format(root=ROOT))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1", MASTER_PORT="29611",
               WORLD_SIZE=str(world))
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            outs.append(p.communicate(timeout=600)[0])
        except subprocess.TimeoutExpired:
            p.kill()
            outs.append("timeout")
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, o[-3000:]
