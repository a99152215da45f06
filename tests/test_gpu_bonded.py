"""GPU tests of the bonded terms (bonds, angles, proper and improper torsions, scaled special pairs) against the CPU
oracle's restatement of the reference's routines (itself equal to the reference's compiled code, tests/test_oracle.py)."""
import numpy as np
import pytest

from deepscalemd_b200 import capi
from deepscalemd_b200 import synthetic as syn
from oracle import cpu_oracle as co

pytestmark = pytest.mark.gpu


def chain_context(s, pos=None, n_owned=None, gid=None, atom=None, lo=(0, 0, 0), hi=(0, 0, 0), halo=0.0, pair=True):
    """pair=False: Lennard-Jones strengths zero and no Coulomb, so that the pair kernel leaves exact zeros and the bonded
    forces can be read off without cancellation (the seeded chains overlap here and there, with huge pair forces)."""
    pos = s.pos if pos is None else pos
    atom = np.arange(s.n) if atom is None else atom
    ctx = capi.Context(len(pos))
    ctx.set_box(s.box, (1, 1, 1), lo, hi, halo)
    ctx.set_pair_params(s.eps if pair else 0.0 * s.eps, s.sig, s.cutoff, s.skin)
    ctx.set_coulomb(bool(pair))
    ctx.set_exclusions(s.n, s.exclusions)
    ctx.set_bonded(s.n, s.bonded)
    ctx.upload(pos, n_owned=n_owned, vel=None if s.vel is None else s.vel[atom], mass=s.mass[atom], types=s.types[atom],
               charge=s.charge[atom], gid=gid)
    return ctx


def forces_by_gid(ctx, n_owned):
    gid = ctx.download("global_id", n_owned)
    f = np.stack([ctx.download(k, n_owned) for k in ("fx", "fy", "fz")], axis=1)
    return gid, f


def test_bonded_forces_energy_and_virial_equal_the_oracle(cuda_device):
    """The bonded kernel ADDS to the forces of the pair kernel: the difference equals the oracle's bonded forces to 1e-10
    of their RMS, energy and virial to 1e-12; two evaluations give the same bits (fixed summation order)."""
    s = syn.chain_fluid(6, 8, seed=11)                       # 216 chains of 8 atoms, box 54 A
    want_f, want = co.bonded(s.pos, s.n, s.box, co.BondedTerms(**s.bonded), charge=s.charge)
    scale = np.sqrt((want_f * want_f).sum(1).mean())
    ctx = chain_context(s, pair=False)
    ctx.build_neighbor_list()
    ctx.compute_forces(capi.PHASE_FULL)
    gid, f_pair = forces_by_gid(ctx, s.n)
    assert not f_pair.any()
    ctx.compute_bonded()
    _, f_all = forces_by_gid(ctx, s.n)
    got = ctx.read_bonded_scalars()
    f_bonded = np.empty_like(f_all)
    f_bonded[gid] = f_all
    assert np.abs(f_bonded - want_f).max() <= 1e-10 * scale
    assert abs(got["pe"] - want["pe"]) <= 1e-12 * abs(want["pe"])
    assert abs(got["virial"] - want["virial"]) <= 1e-11 * abs(want["virial"])
    assert np.abs(got["virial_diag"] - want["virial_diag"]).max() <= 1e-11 * np.abs(want["virial_diag"]).max()
    ctx.compute_forces(capi.PHASE_FULL)
    ctx.compute_bonded()
    _, again = forces_by_gid(ctx, s.n)
    assert np.array_equal(again, f_all)
    assert ctx.read_bonded_scalars()["pe"] == got["pe"]
    # no terms: nothing is added
    ctx.set_bonded(s.n, None)
    ctx.compute_forces(capi.PHASE_FULL)
    ctx.compute_bonded()
    assert np.array_equal(forces_by_gid(ctx, s.n)[1], f_pair)
    ctx.close()


def test_bonded_terms_across_a_brick_boundary(cuda_device):
    """Two bricks emulated on one device, each with its owned atoms and image-shifted ghost atoms and the WHOLE term table:
    a term is evaluated where one of its atoms is owned, forces go to owned atoms only (they equal the undivided
    system's), energy and virial are counted once (the two bricks add up to the whole)."""
    s = syn.chain_fluid(6, 8, seed=12)
    want_f, want = co.bonded(s.pos, s.n, s.box, co.BondedTerms(**s.bonded), charge=s.charge)
    scale = np.sqrt((want_f * want_f).sum(1).mean())
    halo = s.cutoff + s.skin
    wrapped = s.pos - s.box * np.floor(s.pos / s.box)
    pe = 0.0
    diag = np.zeros(3)
    seen = np.zeros(s.n, dtype=bool)
    for brick in syn.brick_decompose(s.pos, s.box, (2, 1, 1), halo):
        own, src, img = brick["owned"], brick["ghost_src"], brick["ghost_image"]
        pos = np.concatenate([wrapped[own], wrapped[src] + img * s.box])
        atom = np.concatenate([own, src])
        ctx = chain_context(s, pos=pos, n_owned=len(own), gid=atom.astype(np.int32), atom=atom, lo=brick["lo"], hi=brick["hi"],
                            halo=halo, pair=False)
        ctx.build_neighbor_list()
        ctx.compute_forces(capi.PHASE_FULL)
        gid, f_pair = forces_by_gid(ctx, len(own))
        ctx.compute_bonded()
        _, f_all = forces_by_gid(ctx, len(own))
        got = ctx.read_bonded_scalars()
        assert np.abs((f_all - f_pair) - want_f[gid]).max() <= 1e-10 * scale
        assert not seen[gid].any()
        seen[gid] = True
        pe += got["pe"]
        diag += got["virial_diag"]
        ctx.close()
    assert seen.all()
    assert abs(pe - want["pe"]) <= 1e-12 * abs(want["pe"])
    assert np.abs(diag - want["virial_diag"]).max() <= 1e-10 * np.abs(want["virial_diag"]).max()


def test_a_term_whose_partner_is_not_on_the_rank_is_reported(cuda_device):
    """A brick whose halo is narrower than its chains are long: the bonded call reports the missing partners."""
    s = syn.chain_fluid(6, 8, seed=13)
    halo = s.cutoff + s.skin
    wrapped = s.pos - s.box * np.floor(s.pos / s.box)
    brick = syn.brick_decompose(s.pos, s.box, (2, 1, 1), halo)[0]
    own = brick["owned"]
    ctx = chain_context(s, pos=wrapped[own], n_owned=len(own), gid=own.astype(np.int32), atom=own, lo=brick["lo"],
                        hi=brick["hi"], halo=halo)      # no ghosts at all
    ctx.build_neighbor_list()
    ctx.compute_forces(capi.PHASE_FULL)
    ctx.compute_bonded()
    with pytest.raises(capi.DsmdError) as err:
        ctx.read_bonded_scalars()
    assert err.value.code == capi.ERR_STATE and "partner is not on this rank" in str(err.value)
    ctx.close()


def test_flexible_chains_conserve_energy(cuda_device):
    """Velocity Verlet over pair and bonded forces: 400 steps of 0.5 fs on flexible chains keep kinetic + pair + bonded
    energy to a small fraction of the kinetic energy."""
    s = syn.chain_fluid(4, 8, spacing=14.0, seed=14)        # 64 chains, box 56 A, well separated
    ctx = chain_context(s)
    ctx.build_neighbor_list()

    def total():
        ctx.compute_forces(capi.PHASE_FULL, want_energy=True)
        ctx.compute_bonded()
        return ctx.kinetic_energy() / s.force_to_accel, ctx.read_scalars()["pe"], ctx.read_bonded_scalars()["pe"]

    ke0, pair0, bonded0 = total()
    assert ke0 > 0 and bonded0 > 0
    energies = []
    for _ in range(8):
        ctx.run_nve(50, 0.5, s.force_to_accel, 0.5, 0, False)
        energies.append(sum(total()))
    e0 = ke0 + pair0 + bonded0
    assert max(abs(e - e0) for e in energies) < 0.02 * ke0
    ke1, _, bonded1 = total()
    assert abs(bonded1 - bonded0) > 0.05 * ke0              # energy does move between the terms
    ctx.close()
