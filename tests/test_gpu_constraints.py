"""GPU tests of the rigid-group constraints (SHAKE after the drift, RATTLE after the second velocity half) against the
CPU oracle's restatement of the reference's ConstraintSolver, and a constrained MD run of the rigid-water geometry box."""
import numpy as np
import pytest

from deepscalemd_b200 import capi
from deepscalemd_b200 import synthetic as syn
from oracle import cpu_oracle as co

pytestmark = pytest.mark.gpu


def water_context(s):
    ctx = capi.Context(s.n)
    ctx.set_box(s.box)
    ctx.set_pair_params(s.eps, s.sig, s.cutoff, s.skin)
    ctx.set_coulomb(True)
    ctx.set_exclusions(s.n, s.exclusions)
    ctx.set_constraints(s.n, s.constraints)
    return ctx


def by_gid(ctx, names, n):
    gid = ctx.download("global_id", n)
    out = np.empty((n, len(names)))
    out[gid] = np.stack([ctx.download(k, n) for k in names], axis=1)
    return out


def test_shake_and_rattle_equal_the_oracle(cuda_device):
    """One velocity-Verlet step with zero forces: half 1 drifts the molecules out of shape and SHAKE puts them back, half 2
    is followed by RATTLE; positions and velocities equal the oracle's to 1e-10 (the same sweeps, in the same order)."""
    s = syn.water_box(11, seed=9)                  # 1,331 molecules (the smallest box the list radius of 12 A fits)
    rng = np.random.default_rng(4)
    vel = rng.normal(scale=0.02, size=(s.n, 3))   # A / fs: thermal-ish, enough to break the geometry by 1e-3 per step
    dt = 2.0
    ctx = water_context(s)
    ctx.upload(s.pos, vel=vel, mass=s.mass, types=s.types, charge=s.charge)
    ctx.build_neighbor_list()                      # forces stay zero: the step below is pure drift + constraints
    ctx.integrate(1, dt, 4.184e-4)
    pos1, vel1 = by_gid(ctx, "xyz", s.n), by_gid(ctx, ("vx", "vy", "vz"), s.n)
    # the oracle: drift, then SHAKE with the positions from before the drift
    pre = [np.ascontiguousarray(s.pos[:, k]) for k in range(3)]
    p = [np.ascontiguousarray(s.pos[:, k] + dt * vel[:, k]) for k in range(3)]
    v = [np.ascontiguousarray(vel[:, k]) for k in range(3)]
    assert co.shake(s.constraints, p, v, s.mass, pre, s.box, dt)
    want_p, want_v = np.stack(p, axis=1), np.stack(v, axis=1)
    assert np.abs(pos1 - want_p).max() <= 1e-10 * np.abs(want_p).max()
    assert np.abs(vel1 - want_v).max() <= 1e-10 * np.abs(want_v).max() + 1e-14
    # the geometry is back
    c = np.asarray(s.constraints)
    i, j, d = c[:, 0].astype(int), c[:, 1].astype(int), c[:, 2]
    r = np.linalg.norm(pos1[i] - pos1[j], axis=1)
    assert np.abs(r * r - d * d).max() <= 1e-8 * (d * d).max()
    ctx.integrate(2, dt, 4.184e-4)                 # zero forces: the kick does nothing, RATTLE projects the velocities
    vel2 = by_gid(ctx, ("vx", "vy", "vz"), s.n)
    ok, _ = co.rattle(s.constraints, p, v, s.mass, s.box, dt, 4.184e-4)
    assert ok
    want_v = np.stack(v, axis=1)
    assert np.abs(vel2 - want_v).max() <= 1e-10 * np.abs(want_v).max() + 1e-14
    along = ((pos1[i] - pos1[j]) * (vel2[i] - vel2[j])).sum(1)
    assert np.abs(along).max() < 1e-8
    assert ctx.constraint_failures() == 0
    ctx.close()


def test_constrained_water_run_keeps_the_geometry_and_the_energy(cuda_device):
    """The rigid-water geometry box as MD (real-space forces only): 200 steps of 2 fs through the library's own loop with
    SHAKE / RATTLE inside the integration halves. Bond lengths stay at their targets, no group fails to converge, and
    the total energy does not run away (real-space Ewald alone with a plain cutoff is not a conserving force field, so
    the bound is loose)."""
    s = syn.water_box(11, seed=3)                  # 1,331 molecules
    ctx = water_context(s)
    ctx.upload(s.pos, vel=s.vel, mass=s.mass, types=s.types, charge=s.charge)             # 300 K, A / fs
    ctx.build_neighbor_list()
    ctx.compute_forces(want_energy=True)
    # the start velocities have components along the bonds: one RATTLE-like projection by a zero-length step is not
    # available, so the first steps remove them; compare energies from step 20 on
    out = ctx.run_nve(20, 2.0, 4.184e-4, 0.5, 0, True)
    ctx.compute_forces(want_energy=True)
    e0 = ctx.read_scalars()["pe"] + ctx.kinetic_energy() * 2390.0574
    out = ctx.run_nve(200, 2.0, 4.184e-4, 0.5, 0, True)
    ctx.compute_forces(want_energy=True)
    e1 = ctx.read_scalars()["pe"] + ctx.kinetic_energy() * 2390.0574
    pos = by_gid(ctx, "xyz", s.n)
    c = np.asarray(s.constraints)
    i, j, d = c[:, 0].astype(int), c[:, 1].astype(int), c[:, 2]
    r = np.linalg.norm(pos[i] - pos[j], axis=1)
    assert np.abs(r * r - d * d).max() <= 2e-8 * (d * d).max()
    assert ctx.constraint_failures() == 0
    ke = ctx.kinetic_energy() * 2390.0574
    assert np.isfinite(e1) and abs(e1 - e0) < 0.5 * ke
    assert out["rebuilds"] >= 1
    ctx.close()
