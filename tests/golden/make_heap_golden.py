"""Generates tests/golden/heap_partition.npz: chunk-to-rank assignments computed by the
reference's own ``assign_tasks_heap`` (flashmask/cp_balance/cp_balance.py:96-174).

    python tests/golden/make_heap_golden.py [path-to-reference-checkout]

The reference module cannot be imported here (its package pulls in the GPU kernels), but the
function body uses only ``heapq`` and numpy: the one ``FunctionDef`` is lifted out of the
reference file with ``ast``, compiled and run with those names in scope.  Nothing of the
reference is copied into this repository; only its outputs are stored.

Each case k stores w_k (int32 weights in chunk order), m_k (ranks), b_k (int32 [n]: the rank
of every chunk), bw_k (int64 [m]: rank loads) and cuts_k.  Weight families as for the IPO
vectors: uniform, many ties, log-normal tile counts, sorted ramps, constants, mostly empty.
"""
import ast
import heapq
import os
import sys
from typing import List, Tuple

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference_function(ref_root: str):
    path = os.path.join(ref_root, "flashmask", "cp_balance", "cp_balance.py")
    tree = ast.parse(open(path, encoding="utf-8").read(), filename=path)
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "assign_tasks_heap")
    mod = ast.Module(body=[fn], type_ignores=[])
    scope = {"heapq": heapq, "np": np, "List": List, "Tuple": Tuple}
    exec(compile(mod, path, "exec"), scope)
    return scope["assign_tasks_heap"]


def weights(rng, family, n):
    if family == 0:
        w = rng.integers(0, 1000, n)
    elif family == 1:
        w = rng.integers(0, 8, n)
    elif family == 2:
        w = np.round(np.exp(rng.normal(5, 1.5, n)))
    elif family == 3:
        w = np.sort(rng.integers(0, 4000, n))
    elif family == 4:
        w = np.full(n, 7)
    else:
        w = (rng.integers(0, 3, n) == 0) * rng.integers(1, 100000, n)
    return np.ascontiguousarray(w, dtype=np.int32)


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
    ref = load_reference_function(ref_root)
    rng = np.random.default_rng(2027)
    out = {}
    k = 0
    # (ranks, chunks): even deals, uneven deals (the overflow branch), fewer chunks than ranks
    for m, n in [(2, 8), (2, 64), (4, 64), (8, 64), (8, 512), (4, 10), (3, 7), (8, 61), (4, 3), (1, 5),
                 (16, 64), (8, 8)]:
        for family in range(6):
            w = weights(rng, family, n)
            tasks = np.stack([w, np.arange(n, dtype=np.int32)], axis=1)
            buckets, bw, cuts = ref(tasks, m)
            b = np.full(n, -1, dtype=np.int32)
            for r, items in enumerate(buckets):
                idxs = [int(i) for _, i in items]
                assert idxs == sorted(idxs)
                b[idxs] = r
            assert (b >= 0).all()
            out[f"w_{k}"], out[f"m_{k}"], out[f"b_{k}"] = w, np.int32(m), b
            out[f"bw_{k}"], out[f"cuts_{k}"] = np.asarray(bw, dtype=np.int64), np.int64(cuts)
            k += 1
    out["n_cases"] = np.int32(k)
    np.savez_compressed(os.path.join(HERE, "heap_partition.npz"), **out)
    print("wrote", k, "cases")


if __name__ == "__main__":
    main()
