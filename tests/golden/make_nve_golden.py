"""Energy-drift fixture: the REFERENCE's own CPU code (oracle/_ref) integrates the 32,000-atom LJ system (FCC 20^3,
density 0.8442, T* = 1.44, cutoff 2.5 plain truncation, skin 0.3, dt 0.005) with velocity Verlet for 2,000 equilibration
steps and then 10,000 measured steps, rebuilding its list when SpatialVerletList::needs_rebuild says so. Stored: total
energy per atom every 100 measured steps. Run from the repository root where the reference tree is present:

    make -C oracle && python tests/golden/make_nve_golden.py          (about two minutes on 8 cores)
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from deepscalemd_b200 import synthetic as syn  # noqa: E402
from oracle import cpu_oracle as co  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
DT, EQUIL, STEPS, EVERY = 0.005, 2000, 10000, 100


def main():
    s = syn.fcc_lj(20, seed=12345)
    pos = [np.ascontiguousarray(s.pos[:, k]) for k in range(3)]
    vel = [np.ascontiguousarray(s.vel[:, k]) for k in range(3)]
    ref = co.RefCase(*pos, s.n, s.box, s.cutoff, s.skin, eps=s.eps, sig=s.sig)
    ref.build_list()

    def force():
        f, sc = ref.compute(tensor=False)
        return [np.ascontiguousarray(f[:, k]) for k in range(3)], sc["pe"]

    def energy(pe):
        return (pe + 0.5 * sum((s.mass * v * v).sum() for v in vel)) / s.n

    frc, pe = force()
    rebuilds = 0
    trace = []
    for step in range(EQUIL + STEPS + 1):
        if step >= EQUIL and (step - EQUIL) % EVERY == 0:
            trace.append(energy(pe))
            print(step - EQUIL, trace[-1], flush=True)
        if step == EQUIL + STEPS:
            break
        co.vv_half(True, DT, 1.0, pos, vel, frc, s.mass)
        ref.update_positions(*pos)
        if ref.needs_rebuild():
            # The reference wraps atoms into the box when it migrates them, i.e. on rebuild steps only
            # (src/md_simulation.cpp:1310-1316); between rebuilds positions run on, so the list's per-tile-pair periodic
            # shifts stay valid. Its CPU list builder bins by clamping, so it must be given wrapped positions.
            for k in range(3):
                pos[k] -= s.box[k] * np.floor(pos[k] / s.box[k])
            ref.update_positions(*pos)
            ref.build_list()
            rebuilds += 1
        frc, pe = force()
        co.vv_half(False, DT, 1.0, pos, vel, frc, s.mass)
    np.savez(os.path.join(HERE, "nve_lj_32000.npz"), energy_per_atom=np.array(trace), dt=DT, equilibration=EQUIL,
             steps=STEPS, every=EVERY, rebuilds=rebuilds)
    print("rebuilds", rebuilds, "drift per atom", trace[-1] - trace[0])


if __name__ == "__main__":
    main()
