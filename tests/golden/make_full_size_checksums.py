"""Generates tests/golden/full_size_pair_checksums.json and tests/golden/full_size_<case>.npz: for the full-size systems
(LJ 4,000,000 atoms, the 1,048,576-atom binary mixture, the 648,000-atom water box) the number of pairs inside the list
radius and an order-independent checksum of the pair set, computed by the CPU oracle and by the REFERENCE's own
SpatialVerletList (oracle/_ref, compiled in place) - the two must agree before anything is written - and the potential
energy, virial and the forces on every SAMPLE-th atom from the oracle (exact erfc) and from the reference's
ForceCalculatorCPU.
Run from the repository root, where the reference tree is present:

    make -C oracle && python tests/golden/make_full_size_checksums.py

Inputs are not stored: the tests regenerate them from the same seeds (deepscalemd_b200.synthetic).
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


def cases():
    return {
        "lj_4m": lambda: syn.fcc_lj(100, seed=12345),
        "kob_andersen_1m": lambda: syn.kob_andersen(1_048_576, seed=5),
        "water_648k": lambda: syn.water_box(60, seed=3),
    }


SAMPLES = 4096


def undirected(p):
    a = np.minimum(p[:, 0], p[:, 1])
    b = np.maximum(p[:, 0], p[:, 1])
    return a, b


def main():
    out = {}
    for name, make in cases().items():
        s = make()
        x, y, z = (np.ascontiguousarray(s.pos[:, k]) for k in range(3))
        t0 = time.time()
        p = co.pairs(x, y, z, s.n, s.box, search=s.cutoff + s.skin)
        got = checksum_numpy(*undirected(p))
        c6, c12 = co.lj_tables(s.eps, s.sig)
        alpha = co.ewald_alpha(s.cutoff) if s.coulomb else 0.0
        f, sc = co.forces(x, y, z, s.n, s.box, p, c6, c12, s.cutoff, charge=s.charge, types=s.types, do_coulomb=s.coulomb,
                          alpha=alpha, ewald_mode=1, exclusions=s.exclusions)
        sample = np.arange(0, s.n, max(1, s.n // SAMPLES), dtype=np.int64)
        fixture = dict(sample=sample, f_oracle=f[sample], f_rms_oracle=np.sqrt((f * f).sum(1).mean()),
                       pe_oracle=sc["pe"], virial_oracle=sc["virial"])
        del f
        t1 = time.time()
        del p
        entry = dict(atoms=int(s.n), pairs=got[0], sum1=str(got[1]), sum2=str(got[2]), source="oracle")
        if co.ref_available():
            ref = co.RefCase(x, y, z, s.n, s.box, s.cutoff, s.skin, charge=s.charge, types=s.types, eps=s.eps,
                             sig=s.sig, exclusions=s.exclusions)
            ref.build_list()
            rp = ref.list_pairs()
            ref_sum = checksum_numpy(*undirected(rp))
            del rp
            fr, rsc = ref.compute(do_coulomb=bool(s.coulomb))
            fixture.update(f_reference=fr[sample], f_rms_reference=np.sqrt((fr * fr).sum(1).mean()),
                           pe_reference=rsc["pe_real"], virial_reference=rsc["virial"])
            del fr
            ref.close()
            assert ref_sum == got, (name, ref_sum, got)
            entry["source"] = "oracle and reference SpatialVerletList (equal)"
        print(name, entry, "oracle %.1f s, reference %.1f s" % (t1 - t0, time.time() - t1), flush=True)
        out[name] = entry
        np.savez(os.path.join(HERE, "full_size_%s.npz" % name), **fixture)
    with open(os.path.join(HERE, "full_size_pair_checksums.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
        f.write("\n")


if __name__ == "__main__":
    main()
