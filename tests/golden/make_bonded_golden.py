"""Generates tests/golden/chains_bonded_512.npz: forces, potential energy, virial and its diagonal of the bonded terms and
scaled special pairs of 64 flexible chains (deepscalemd_b200.synthetic.chain_fluid(4, 8, seed=11)) from the REFERENCE's own
compute_bond_forces / compute_angle_forces / compute_torsion_forces / compute_special_pair_forces (oracle/_ref, compiled in
place from the reference tree), all kinds together and each kind alone. Run from the repository root:

    make -C oracle && python tests/golden/make_bonded_golden.py

Inputs are not stored: the tests regenerate them from the same seed.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from deepscalemd_b200 import synthetic as syn  # noqa: E402
from oracle import cpu_oracle as co  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

KINDS = dict(all=None, bonds=("bonds", "bond_k", "bond_r0"), angles=("angles", "angle_k", "angle_theta0"),
             torsions=("torsions", "torsion_k", "torsion_phi0", "torsion_n", "n_dihedrals"),
             specials=("specials", "special_sigma", "special_epsilon", "special_lj_scale", "special_coulomb_scale"))


def main():
    if not co.ref_available():
        raise SystemExit("oracle/_ref is not built (the reference tree is needed): run `make -C oracle`")
    s = syn.chain_fluid(4, 8, seed=11)
    out = {}
    for kind, keys in KINDS.items():
        terms = co.BondedTerms(**(s.bonded if keys is None else {k: s.bonded[k] for k in keys}))
        ref = co.RefCase(s.pos[:, 0], s.pos[:, 1], s.pos[:, 2], s.n, s.box, s.cutoff, s.skin, charge=s.charge, types=s.types,
                         eps=s.eps, sig=s.sig)
        f, sc = ref.bonded(terms)
        ref.close()
        out[f"f_{kind}"] = f
        out[f"scalars_{kind}"] = np.array([sc["pe"], sc["virial"], *sc["virial_diag"]])
        print(kind, out[f"scalars_{kind}"])
    np.savez_compressed(os.path.join(HERE, "chains_bonded_512.npz"), **out)


if __name__ == "__main__":
    main()
