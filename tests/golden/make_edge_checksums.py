"""Generates tests/golden/full_size_edge_checksums.json: for the 1,000,000-atom disordered solid (uniform random placement
with a 1.8 A minimum distance, cutoff 5 A) the number of directed edges of the periodic radius graph and an
order-independent checksum of the (centre, neighbour, lattice shift) set, from the CPU oracle (explicit periodic images,
then the edge search over real centres), with the edge count confirmed by an independent k-d tree count; and, for the
2 x 2 x 2 brick decomposition with a cutoff-wide halo, the owned and ghost atom counts of every brick.
Run from the repository root:

    make -C oracle && python tests/golden/make_edge_checksums.py

Inputs are not stored: the tests regenerate them from the same seed (deepscalemd_b200.synthetic.disordered_solid).
"""
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

from deepscalemd_b200 import synthetic as syn  # noqa: E402
from oracle import cpu_oracle as co  # noqa: E402
from pair_checksum import checksum_numpy  # noqa: E402


def edge_code(dst, shift):
    """Neighbour index and lattice shift (each component -1, 0 or 1) as one integer."""
    shift = np.asarray(shift, dtype=np.int64)
    return np.asarray(dst, dtype=np.int64) * 27 + (shift[:, 0] + 1) * 9 + (shift[:, 1] + 1) * 3 + (shift[:, 2] + 1)


def main():
    from scipy.spatial import cKDTree
    s = syn.disordered_solid(1_000_000)
    L = s.box[0]
    t0 = time.time()
    reach = s.cutoff + 1e-8
    im = co.images(s.pos[:, 0], s.pos[:, 1], s.pos[:, 2], s.box, np.zeros(3), -np.full(3, reach), s.box + reach,
                   np.ones(3, dtype=np.int32))
    idx, sh = co.edges(im["x"], im["y"], im["z"], s.cutoff, n_centers=s.n, owner=im["owner"], shift=im["shift"])
    lattice = np.rint(sh / L).astype(np.int64)
    assert np.abs(lattice).max() <= 1
    count, s1, s2 = checksum_numpy(idx[0], edge_code(idx[1], lattice))
    t1 = time.time()
    wrapped = s.pos - s.box * np.floor(s.pos / s.box)
    tree = cKDTree(wrapped, boxsize=L)
    by_tree = int(tree.count_neighbors(tree, s.cutoff)) - s.n
    assert by_tree == count, (by_tree, count)
    bricks = syn.brick_decompose(s.pos, s.box, (2, 2, 2), s.cutoff)
    out = dict(case="disordered_solid(1_000_000), seed 99", atoms=int(s.n), cutoff=s.cutoff, edges=count, sum1=str(s1),
               sum2=str(s2), image_atoms=int(len(im["x"]) - s.n), source="oracle (edge count equal to a k-d tree count)",
               bricks=[dict(owned=int(len(b["owned"])), ghosts=int(len(b["ghost_src"]))) for b in bricks])
    print(out, "oracle %.1f s, tree %.1f s" % (t1 - t0, time.time() - t1))
    with open(os.path.join(HERE, "full_size_edge_checksums.json"), "w") as f:
        json.dump(out, f, indent=1)


if __name__ == "__main__":
    main()
