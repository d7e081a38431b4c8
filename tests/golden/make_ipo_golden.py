"""Generates tests/golden/ipo_partition.npz: chunk-to-rank assignments computed by
the reference's own IPO solver header (compiled from the reference checkout into
oracle/_ref/libcpsolver_ref.so by oracle/Makefile).

    make -C oracle && python tests/golden/make_ipo_golden.py

Each case k stores w_k (int32 weights), m_k (ranks), a_k (int32 [m, n/m]
assignment in the solver's order) and best_k (heaviest rank).  The weight
families follow what the partitioner sees: tile counts of document masks
(log-normal), many ties, sorted ramps, constants, mostly-empty chunks.
"""
import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


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
    lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libcpsolver_ref.so"))
    lib.ref_ipo_solve.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    rng = np.random.default_rng(2026)
    out = {}
    k = 0
    # (ranks, chunks per rank): meet-in-the-middle (<=10), search (11..16), LPT only (17),
    # with and without the 3-way phase (per rank <= 8, ranks >= 3)
    for m, per in [(2, 4), (2, 10), (2, 12), (3, 3), (4, 8), (4, 9), (8, 8), (8, 4), (8, 16), (16, 4),
                   (8, 17), (32, 2), (32, 16), (4, 1), (1, 8)]:
        for family in range(6):
            n = m * per
            w = weights(rng, family, n)
            a = np.zeros((m, per), dtype=np.int32)
            best = lib.ref_ipo_solve(w.ctypes.data, n, m, a.ctypes.data)
            out[f"w_{k}"], out[f"m_{k}"], out[f"a_{k}"], out[f"best_{k}"] = w, np.int32(m), a, np.int64(best)
            k += 1
    out["n_cases"] = np.int32(k)
    np.savez_compressed(os.path.join(HERE, "ipo_partition.npz"), **out)
    print("wrote", k, "cases")


if __name__ == "__main__":
    main()
