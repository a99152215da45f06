"""The MD driver executable end to end on a GPU: the reference's input files in, status lines out."""
import os
import re
import subprocess

import numpy as np
import pytest

from deepscalemd_b200 import build, input_api, input_files
from deepscalemd_b200 import synthetic as syn
from oracle import cpu_oracle as co

pytestmark = pytest.mark.gpu

LINE = re.compile(r"^Step: (\d+), T: ([-\d.eE+]+), KE: ([-\d.eE+]+), PE: ([-\d.eE+]+), Etot: ([-\d.eE+]+)$")


def run_driver(yaml_path, timeout=300):
    r = subprocess.run([build.build_driver(), str(yaml_path)], capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stderr + r.stdout
    rows = [tuple(float(v) for v in m.groups()) for m in map(LINE.match, r.stdout.splitlines()) if m]
    return np.array(rows), r.stdout


def test_nve_run_from_input_files(cuda_device, tmp_path):
    """864 argon atoms from XYZ + legacy .top + run description: start energies equal the oracle's for the same positions,
    the total energy is conserved, the list is rebuilt on the way, the closing lines are the reference's."""
    s = syn.fcc_lj(6, seed=1)
    path, scale = input_files.argon_files(str(tmp_path), s, total_steps=200, output_freq=50, update_freq=1000)
    rows, out = run_driver(path)
    assert [int(r[0]) for r in rows] == [0, 50, 100, 150, 200]
    n = s.n
    target_t = 1.44 * scale["epsilon"] / input_files.KB
    assert rows[0][2] == pytest.approx(0.5 * (3 * n - 3) * input_files.KB * target_t, abs=2e-6)    # Maxwell-Boltzmann start (six decimals are printed)
    assert rows[0][1] == pytest.approx(target_t * (3 * n - 3) / (3 * n), abs=2e-6)                 # printed T uses 3N
    # potential energy of the start configuration: the oracle's, in kcal/mol
    x, y, z = (np.ascontiguousarray(s.pos[:, k]) for k in range(3))
    c6, c12 = co.lj_tables(s.eps, s.sig)
    _, sc = co.forces(x, y, z, n, s.box, co.pairs(x, y, z, n, s.box, search=s.cutoff), c6, c12, s.cutoff)
    assert rows[0][3] == pytest.approx(sc["pe"] * scale["epsilon"], rel=2e-6)
    etot = rows[:, 4]
    # Plain truncation (the reference's LJ has no energy shift, src/force_calculator_cpu.cpp:81-98): while the lattice
    # melts, the number of pairs inside the cutoff grows from 54 to about 55.3 per atom and each new pair brings
    # u(rc) = -0.0163 epsilon with it, so the total energy steps down once (about -2.2 kcal/mol for 864 argon atoms)
    # and is conserved from then on, with noise from pairs crossing the cutoff.
    ke0 = rows[0][2]
    settled = etot[1:]
    assert np.abs(settled - settled.mean()).max() < 3e-3 * ke0
    u_rc = 4.0 * (2.5 ** -12 - 2.5 ** -6) * scale["epsilon"]
    melt_step = settled.mean() - etot[0]
    assert 3.0 * 0.5 * n * u_rc < melt_step < 0.0          # at most three more neighbours per atom inside the cutoff
    assert rows[-1][1] < 0.75 * rows[0][1]           # the lattice start gives half its kinetic energy to the potential
    builds = int(re.search(r"Neighbor list builds = (\d+)", out).group(1))
    assert builds >= 5
    assert re.search(r"Performance: [\d.]+ Matom-step/s, [\d.]+ ms/step, [\d.]+ ns/day \(md_loop only, dt=[\d.]+ fs\)", out)


def test_nose_hoover_holds_the_target_temperature(cuda_device, tmp_path):
    s = syn.fcc_lj(6, seed=1)
    path, scale = input_files.argon_files(str(tmp_path), s, total_steps=3000, output_freq=100, update_freq=1000,
                                          thermostat="nose_hoover", tau_t=200.0)
    rows, _ = run_driver(path)
    target_t = 1.44 * scale["epsilon"] / input_files.KB
    late = rows[rows[:, 0] >= 1500][:, 1]
    assert abs(late.mean() - target_t) < 0.05 * target_t


def test_restart_continues_the_run(cuda_device, tmp_path):
    s = syn.fcc_lj(6, seed=1)
    whole, _ = input_files.argon_files(str(tmp_path / "whole"), s, total_steps=100, output_freq=50, update_freq=1000)
    rows_whole, _ = run_driver(whole)
    first, _ = input_files.argon_files(str(tmp_path / "first"), s, total_steps=50, output_freq=50, update_freq=1000,
                                       restart_output=str(tmp_path / "half.restart"), restart_output_freq=50)
    rows_first, out_first = run_driver(first)
    assert "[restart] wrote" in out_first and os.path.exists(tmp_path / "half.restart")
    second, scale = input_files.argon_files(str(tmp_path / "second"), s, total_steps=50, output_freq=50, update_freq=1000,
                                            restart_file=str(tmp_path / "half.restart"))
    rows_second, _ = run_driver(second)
    assert [int(r[0]) for r in rows_second] == [50, 100]                    # the step counter goes on
    # same state as where the first half stopped (the list is rebuilt at the restart, so fp32 sums run in another order)
    assert rows_second[0][2:] == pytest.approx(rows_first[-1][2:], rel=1e-6)
    assert rows_second[-1][2:] == pytest.approx(rows_whole[-1][2:], rel=1e-5)  # and the same end as the uninterrupted run
    # the file itself: the layout the reference reads
    raw = open(tmp_path / "half.restart", "rb").read()
    assert raw[:8] == b"DSMDRST1" and raw[-8:] == b"DSMDEND1" and len(raw) == 8 + 16 + 32 + 12 + (4 + 4) + 4 + (4 + 4) + 4 + \
        48 * s.n + 8
    sys_ = input_api.System(coordinate_file=str(tmp_path / "first" / "argon.xyz"), box=scale["box"])
    info = sys_.read_restart(tmp_path / "half.restart")
    assert info["step"] == 50 and info["thermostat"] == "none"


def test_velocity_scaling_entry_point(cuda_device):
    from deepscalemd_b200 import capi
    s = syn.fcc_lj(4, seed=3)
    ctx = capi.Context(s.n)
    ctx.set_box(s.box, (1, 1, 1), (0, 0, 0), (0, 0, 0), 0.0)
    ctx.set_pair_params(s.eps, s.sig, s.cutoff, s.skin)
    ctx.upload(s.pos, vel=s.vel, mass=s.mass, types=s.types)
    before = ctx.kinetic_energy()
    v_before = np.stack([ctx.download(k, s.n) for k in ("vx", "vy", "vz")], axis=1)
    ctx.scale_velocities(0.75)
    v_after = np.stack([ctx.download(k, s.n) for k in ("vx", "vy", "vz")], axis=1)
    assert np.array_equal(v_after, v_before * 0.75)
    assert ctx.kinetic_energy() == pytest.approx(before * 0.5625, rel=1e-13)
    ctx.close()


def test_rigid_water_runs_as_md_from_the_reference_input_files(cuda_device, tmp_path):
    """The rigid-water geometry box through the driver: a dsMD_input folder (manifest, .xyz, .dsMDtop with exclusions and
    constraints, .dsMDprm with the explicit pair table) and a run description with real_space_only: true. The run
    finishes; the seeded start (random orientations on a jittered lattice) is far from equilibrium and heats up as it
    relaxes, but stays finite and bounded with the molecules held rigid by SHAKE / RATTLE (the printed temperature counts
    the constraints in its degrees of freedom: 450 K at step 0 for velocities drawn at 300 K); the total energy moves by a
    fraction of the kinetic energy only; the list is rebuilt on the way."""
    s = syn.water_box(11, seed=3)
    sigma = [[3.166, 1.583], [1.583, 0.0]]
    epsilon = [[0.1553, 0.0], [0.0, 0.0]]
    pos = s.pos - s.box * np.floor(s.pos / s.box)
    pos = pos + (s.box / 2.0 - pos.mean(0))
    manifest = input_files.write_dsmd_input(str(tmp_path / "water"), "water", pos, ["O", "H", "H"] * (s.n // 3), s.types,
                                            ["OW", "HW"], s.mass, s.charge, sigma, epsilon, exclusions=s.exclusions,
                                            constraints=s.constraints)
    path = input_files.write_run_yaml(tmp_path / "water.yaml", box=s.box, total_steps=100, timestep=2.0, temperature=300.0,
                                      cutoff=s.cutoff, skin=s.skin, input_system=manifest, force_type="lj, PME",
                                      output_freq=25, update_freq=1000, extra={"real_space_only": "true"})
    rows, out = run_driver(path)
    assert [int(r[0]) for r in rows] == [0, 25, 50, 75, 100]
    assert np.all(np.isfinite(rows)) and np.all(rows[:, 1] > 100.0) and np.all(rows[:, 1] < 3000.0)
    assert rows[0][1] == pytest.approx(300.0 * 9.0 / 6.0, rel=0.05)
    assert np.abs(rows[1:, 4] - rows[1, 4]).max() < 0.25 * rows[-1][2]
    assert int(re.search(r"Neighbor list builds = (\d+)", out).group(1)) >= 2


def test_flexible_chains_run_from_dsmd_input_files(cuda_device, tmp_path):
    """Bonded terms through the driver: flexible chains as a dsMD_input folder (bonds, angles, dihedrals, impropers and
    special pairs with their parameter sections), force_calculation.type naming every kind. The potential energy printed
    at step 0 is the pair energy plus the oracle's bonded energy, and the total energy holds over 200 steps of 0.5 fs."""
    from deepscalemd_b200 import capi
    from oracle import cpu_oracle as co
    s = syn.chain_fluid(4, 8, spacing=14.0, seed=14)
    pos = s.pos + (s.box / 2.0 - s.pos.mean(0))             # the reader centres the atoms in the box: write them so
    manifest = input_files.write_dsmd_input(str(tmp_path / "chains"), "chains", pos, ["C"] * s.n, s.types, ["CH3", "CH2"],
                                            s.mass, s.charge, s.sig, s.eps, bonded=s.bonded)
    path = input_files.write_run_yaml(tmp_path / "chains.yaml", box=s.box, total_steps=200, timestep=0.5, temperature=300.0,
                                      cutoff=s.cutoff, skin=s.skin, input_system=manifest,
                                      force_type="lj, PME, bonds, angles, dihedrals", output_freq=50, update_freq=1000,
                                      extra={"real_space_only": "true", "velocity_seed": "7"})
    rows, out = run_driver(path)
    assert [int(r[0]) for r in rows] == [0, 50, 100, 150, 200] and np.all(np.isfinite(rows))
    _, bonded = co.bonded(pos, s.n, s.box, co.BondedTerms(**s.bonded), charge=s.charge)
    ctx = capi.Context(s.n)
    ctx.set_box(s.box)
    ctx.set_pair_params(s.eps, s.sig, s.cutoff, s.skin)
    ctx.set_coulomb(True)
    ctx.set_exclusions(s.n, s.exclusions)
    ctx.upload(pos, mass=s.mass, types=s.types, charge=s.charge)
    ctx.build_neighbor_list()
    ctx.compute_forces(capi.PHASE_FULL, want_energy=True)
    pair = ctx.read_scalars()["pe"]
    ctx.close()
    assert bonded["pe"] > 10.0
    assert rows[0][3] == pytest.approx(pair + bonded["pe"], rel=1e-5)
    assert np.abs(rows[:, 4] - rows[0, 4]).max() < 0.02 * rows[0][2]
    assert np.abs(rows[1:, 3] - rows[0, 3]).max() > 0.05 * rows[0][2]      # energy moves between kinetic and potential
