#!/usr/bin/env python
"""Generates the golden fixtures tests/golden/*.npz by running the REFERENCE's own code
(oracle/_ref/ref_harness, built by `make -C oracle` where the reference tree exists) on small seeded
graphs.  Run from the repository root:  python tests/golden/make_golden.py

Each fixture holds the inputs (edge list in .edge file order, seeds, fanout in hop order, F), the
reference's whole-graph CSC, and for every block of the sampled batch (index 0 = input side) the
reference's arrays (destination, source, column_offset, row_indices, row_offset, column_indices,
edge_weight_forward, edge_weight_backward) plus MiniBatchFuseOp forward/backward on seeded tensors
(x, y, gy, gx).  The raw sampled edge list of a hop is source[row_indices] of its block, so a test can
feed the identical edges to another implementation.
"""
import os
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from neutronbench_b200 import synth  # noqa: E402

HARNESS = os.path.join(ROOT, "oracle", "_ref", "ref_harness")

CASES = {
    # name: (edges, V, number of seeds, fanout in hop order, F)
    "rmat300_f4x3": (lambda: synth.rmat_numpy(300, 3000, (0.57, 0.19, 0.19), 11), 300, 32, [4, 3], 8),
    "uniform500_f25x10": (lambda: synth.uniform_undirected_numpy(500, 1500, 5), 500, 48, [25, 10], 16),
    "rmat1500_f5x4x3": (lambda: synth.rmat_numpy(1500, 12000, (0.45, 0.22, 0.22), 7), 1500, 64, [5, 4, 3], 4),
    "dups_and_isolated": (lambda: np.array([[1, 0], [1, 0], [1, 0], [0, 0], [2, 1], [2, 1], [63, 1], [5, 5], [7, 9],
                                            [9, 7], [9, 7], [40, 9]], dtype=np.int32), 64, 6, [2, 2], 3),
}


def run_case(name, make_edges, V, n_seeds, fanout, F):
    edges = make_edges().astype("<u4")
    rng = np.random.RandomState(len(name))
    seeds = rng.choice(V, n_seeds, replace=False).astype("<u4")
    with tempfile.TemporaryDirectory() as tmp:
        edges.tofile(os.path.join(tmp, "g.edge"))
        seeds.tofile(os.path.join(tmp, "seeds.u32"))
        out = os.path.join(tmp, "out")
        os.makedirs(out)
        subprocess.check_call([HARNESS, os.path.join(tmp, "g.edge"), str(V), os.path.join(tmp, "seeds.u32"),
                               ",".join(map(str, fanout)), str(F), out], stdout=subprocess.DEVNULL)
        arrays = {"edges": edges, "seeds": seeds, "fanout": np.array(fanout, dtype=np.int32),
                  "V": np.array([V], dtype=np.int64), "F": np.array([F], dtype=np.int64)}
        for line in open(os.path.join(out, "index.txt")):
            n, t, _ = line.split()
            arrays[n] = np.fromfile(os.path.join(out, n + ".bin"), dtype={"u32": "<u4", "f32": "<f4"}[t])
    path = os.path.join(ROOT, "tests", "golden", name + ".npz")
    np.savez_compressed(path, **arrays)
    print(f"{name}: {os.path.getsize(path) / 1024:.1f} KB")


if __name__ == "__main__":
    if not os.path.exists(HARNESS):
        sys.exit("oracle/_ref/ref_harness is missing: run `make -C oracle` in a container that has the reference tree")
    for name, (mk, V, n, fan, F) in CASES.items():
        run_case(name, mk, V, n, fan, F)
