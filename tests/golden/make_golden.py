"""Generates the committed golden fixtures by running the REFERENCE's own CPU code (oracle/_ref, compiled in place from
the reference tree) on seeded synthetic inputs. Run from the repository root, where the reference tree is present:

    make -C oracle && python tests/golden/make_golden.py

Inputs are not stored: the tests regenerate them from the same seeds (deepscalemd_b200.synthetic). Stored per case:
the reference's forces, potential energy (real-space part), virial and its diagonal, the pair counts inside the list
radius and inside the cutoff, and a checksum of the canonical pair list.
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from deepscalemd_b200 import synthetic as syn  # noqa: E402
from oracle import cpu_oracle as co  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def cases():
    """name -> (system, switch distance)."""
    ka = syn.kob_andersen(4096, seed=5)
    return {
        "lj_fcc_864": (syn.fcc_lj(6, seed=1), -1.0),
        "lj_fcc_4000_switch": (syn.fcc_lj(10, seed=2), 2.0),
        "kob_andersen_4096": (ka, -1.0),
        "water_3993": (syn.water_box(11, seed=3), -1.0),
    }


def pair_checksum(pairs):
    canon = co.canonical_pairs(pairs).astype(np.int64)
    return hashlib.sha256(canon.tobytes()).hexdigest()


def main():
    if not co.ref_available():
        raise SystemExit("oracle/_ref is not built (the reference tree is needed): run `make -C oracle`")
    for name, (s, switch) in cases().items():
        x, y, z = (np.ascontiguousarray(s.pos[:, k]) for k in range(3))
        ref = co.RefCase(x, y, z, s.n, s.box, s.cutoff, s.skin, charge=s.charge, types=s.types, eps=s.eps, sig=s.sig,
                         switch=switch, exclusions=s.exclusions)
        ref.build_list()
        pairs = ref.list_pairs()
        in_list, in_cut = ref.pair_counts()
        forces, sc = ref.compute(do_lj=True, do_coulomb=s.coulomb, tensor=True)
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"), forces=forces, pe_real=sc["pe_real"], virial=sc["virial"],
            virial_diag=sc["virial_diag"], alpha=sc["alpha"], pairs_in_list=in_list, pairs_in_cutoff=in_cut,
            pair_sha256=pair_checksum(pairs), switch=switch, simd_width=ref.simd_width())
        print(name, s.n, "atoms", in_list, "listed pairs", in_cut, "in cutoff; PE", sc["pe_real"])
        ref.close()


if __name__ == "__main__":
    main()
