"""Host-side input layer (libdsmd_input.so, no GPU): the reference's run-description grammar, coordinate / topology /
parameter readers against the reference's own Topology reader (golden fixture, and live when oracle/_ref holds it),
restart files against a byte-level restatement of the layout, start velocities and the Nose-Hoover scale."""
import json
import os
import struct
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import input_cases  # noqa: E402

from deepscalemd_b200 import input_api, input_files
from deepscalemd_b200 import synthetic as syn

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_library_exports_every_declared_symbol():
    import re
    header = open(os.path.join(os.path.dirname(GOLDEN), "..", "include", "dsmd_input.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(dsmd_(?:input|host)_[a-z_0-9]+)\s*\(", header))
    assert declared == set(input_api.SYMBOLS)
    L = input_api.lib()
    for name in declared:
        assert hasattr(L, name), name


# ---------------------------------------------------------------------------------------------------------------------
# run description
# ---------------------------------------------------------------------------------------------------------------------
BASE = """
# a comment line
coordinate_file: "coords.xyz"     # the quotes go, and so does this comment
topology_file: system.top
target_temperature: 300
timestep: 2.0
total_steps: 1000
box_x: 30.0
box_y: 31.5
box_z: 33
periodic_x: true
periodic_y: True
periodic_z: true
cutoff: 10.0
verlet_skin: 2.0
thermostat_damping: 250
thermostat: nose_hoover
force_calculation:
  mode: builtin
  type: lj, PME
  precision: mixed
  nonbonded_kernel: list
output_freq: 50
mode: mlip
advanced:
  timing_trace: off
  decomposition:
    grid_policy: cubic
  tf32: false
"""


def read(tmp_path, text, name="run.yaml"):
    p = tmp_path / name
    p.write_text(text)
    return input_api.Config(p).values


def test_run_description_rules(tmp_path):
    v = read(tmp_path, BASE)
    assert v["coordinate_file"] == "coords.xyz" and v["topology_file"] == "system.top"
    assert v["target_temperature"] == 300.0 and v["timestep"] == 2.0 and v["total_steps"] == 1000
    assert v["box"] == [30.0, 31.5, 33.0]
    assert v["periodic"] == [True, False, True]          # only the exact text "true"
    assert v["cutoff_distance"] == 10.0                  # alias
    assert v["tau_t"] == 250.0 and v["thermostat"] == "nose_hoover"
    assert v["force_mode"] == "builtin"                  # the top-level "mode: mlip" belongs in the section: ignored
    assert v["enable_lennard_jones"] and v["enable_coulomb"] and not v["enable_bonded"]
    assert v["force_precision"] == "mixed" and v["nonbonded_kernel"] == "list"
    assert v["output_freq"] == 50                        # an unindented key closes the section before it
    assert v["neighbor_list_update_freq"] == 10 and v["lj_switch_distance"] == -1.0 and v["integrator"] == "verlet"
    assert v["restart_output"] == "md_output.restart"
    entries = dict(map(tuple, v["entries"]))
    assert entries["advanced.decomposition.grid_policy"] == "cubic" and entries["advanced.tf32"] == "false"
    assert v["unsupported"] == []


def test_run_description_defaults_errors_and_unsupported(tmp_path):
    with pytest.raises(input_api.InputError, match="run description .* cannot be opened"):
        input_api.Config(tmp_path / "absent.yaml")
    with pytest.raises(input_api.InputError, match="lacks required keys: coordinate_file, timestep"):
        read(tmp_path, "target_temperature: 1\ntotal_steps: 5\n")
    with pytest.raises(input_api.InputError, match="timestep"):
        read(tmp_path, BASE.replace("timestep: 2.0", "timestep: fast"))
    with pytest.raises(input_api.InputError, match="force_calculation.mode: 'ase' is not a force provider"):
        read(tmp_path, BASE.replace("mode: builtin", "mode: ase"))
    with pytest.raises(input_api.InputError, match="total_steps must be positive"):
        read(tmp_path, BASE.replace("total_steps: 1000", "total_steps: 0"))
    # without "type" the enable_* keys apply, and only the exact text "true" keeps a term on
    v = read(tmp_path, BASE.replace("  type: lj, PME\n", "  enable_coulomb: false\n  enable_lennard_jones: true\n"))
    assert v["enable_lennard_jones"] and not v["enable_coulomb"] and v["enable_bonded"]
    # a section name outside the grammar captures nothing: its keys count as top-level keys
    v = read(tmp_path, BASE.replace("output_freq: 50", "my_notes:\n  output_freq: 7"))
    assert v["output_freq"] == 7
    v = read(tmp_path, BASE.replace("thermostat: nose_hoover", "thermostat: langevin") + "barostat: berendsen\n"
             "integrator: leap_frog\n")
    assert len(v["unsupported"]) == 3


def test_manifest_fills_the_missing_file_names(tmp_path):
    cases = input_cases.topology_cases(str(tmp_path))
    manifest = cases["dsmd_binary"]["manifest"]
    text = f"input_system: {manifest}\ntarget_temperature: 1\ntimestep: 1\ntotal_steps: 1\n"
    v = read(tmp_path, text)
    assert v["coordinate_file"] == cases["dsmd_binary"]["coordinate_file"]
    assert v["topology_file"] == cases["dsmd_binary"]["topology_file"]
    assert v["parameter_file"] == cases["dsmd_binary"]["parameter_file"]
    v = read(tmp_path, text + "coordinate_file: other.xyz\n")
    assert v["coordinate_file"] == "other.xyz"           # what the YAML names itself wins
    bad = tmp_path / "bad_manifest.yaml"
    bad.write_text("schema_version: 2\nformat: dsMD_input\n")
    with pytest.raises(input_api.InputError, match="schema_version must be 1"):
        read(tmp_path, f"input_system: {bad}\ntarget_temperature: 1\ntimestep: 1\ntotal_steps: 1\n")


# ---------------------------------------------------------------------------------------------------------------------
# coordinates, topology, parameters
# ---------------------------------------------------------------------------------------------------------------------
def compare_with_reference(system, want):
    c = system.counts()
    assert c["atoms"] == want["atoms"]
    assert np.array_equal(system.types(), np.array(want["type"], dtype=np.int32))
    assert np.array_equal(system.real("mass"), np.array(want["mass"]))
    assert np.array_equal(system.real("charge"), np.array(want["charge"]))
    eps, sig, n, m = system.pair_table()
    assert [n, m] == want["mie"]
    types = system.types()
    assert np.array_equal(sig[types, types], np.array(want["sigma"]))       # per-atom sigma = the diagonal of the table
    assert np.array_equal(eps[types, types], np.array(want["epsilon"]))
    if want["pair_sigma"]:
        assert c["explicit_pairs"]
        assert np.array_equal(sig.ravel(), np.array(want["pair_sigma"]))
        assert np.array_equal(eps.ravel(), np.array(want["pair_epsilon"]))
    else:   # Lorentz-Berthelot from the per-type rows
        assert not c["explicit_pairs"]
        d_s, d_e = np.diag(sig), np.diag(eps)
        assert np.array_equal(sig, 0.5 * (d_s[:, None] + d_s[None, :]))
        assert np.array_equal(eps, np.sqrt(d_e[:, None] * d_e[None, :]))
    assert np.array_equal(system.exclusions().ravel(), np.array(want["exclusions"], dtype=np.int32))
    ci, cj, cd = system.constraints()
    assert np.array_equal(ci, np.array(want["constraint_i"], dtype=np.int32))
    assert np.array_equal(cj, np.array(want["constraint_j"], dtype=np.int32))
    assert np.array_equal(cd, np.array(want["constraint_d"]))
    if c["explicit_pairs"] and "bonded" in want:      # dsMD_input: every bonded term with the parameters resolved for it
        b, got = want["bonded"], system.bonded()
        assert [len(got["bonds"]), len(got["angles"]), len(got["torsions"]), got["n_dihedrals"], len(got["specials"])] == b["counts"]
        for mine, atoms in (("bonds", "bond_atoms"), ("angles", "angle_atoms"), ("torsions", "torsion_atoms"),
                            ("specials", "special_atoms")):
            assert np.array_equal(got[mine].ravel(), np.array(b[atoms], dtype=np.int32)), mine
        assert np.array_equal(np.stack([got["bond_k"], got["bond_r0"]], 1).ravel(), np.array(b["bond_par"]))
        assert np.array_equal(np.stack([got["angle_k"], got["angle_theta0"]], 1).ravel(), np.array(b["angle_par"]))
        assert np.array_equal(np.stack([got["torsion_k"], got["torsion_phi0"]], 1).ravel(), np.array(b["torsion_par"]))
        assert np.array_equal(got["torsion_n"], np.array(b["torsion_n"], dtype=np.int32))
        assert np.array_equal(np.stack([got["special_sigma"], got["special_epsilon"], got["special_lj_scale"],
                                        got["special_coulomb_scale"]], 1).ravel(), np.array(b["special_par"]))


@pytest.mark.parametrize("name", ["legacy_argon", "legacy_mixed", "dsmd_binary", "dsmd_water", "dsmd_chains"])
def test_topology_readers_match_the_reference_reader(tmp_path, name):
    case = input_cases.topology_cases(str(tmp_path))[name]
    system = input_api.System(coordinate_file=case["coordinate_file"], topology_file=case["topology_file"],
                              parameter_file=case["parameter_file"], box=case["box"])
    with open(os.path.join(GOLDEN, "input_topology.json")) as f:
        compare_with_reference(system, json.load(f)[name])
    if input_cases.reference_available():     # live, where the reference tree was compiled in place
        compare_with_reference(system, input_cases.reference_topology(case["topology_file"], case["parameter_file"]))
    if name == "legacy_mixed":                # type ids follow first appearance among the atoms, not the alphabet
        first = open(case["coordinate_file"]).read().split("\n")[2].split()[0]
        assert system.types()[0] == 0 and first in ("Zn", "C", "Ar")
    if name == "dsmd_water":
        c = system.counts()
        assert c["exclusions"] == 81 and c["constraints"] == 81
    if name == "dsmd_chains":
        assert len(system.bonded()["bonds"]) == 27 * 7 and len(system.bonded()["specials"]) == 27 * 5


def test_coordinates_are_recentred_into_the_box(tmp_path):
    rng = np.random.default_rng(1)
    pos = rng.normal(5.0, 2.0, (50, 3))
    input_files.write_xyz(tmp_path / "c.xyz", pos, ["X"] * 50, comment="50 is not the count on this line")
    box = np.array([40.0, 50.0, 60.0])
    s = input_api.System(coordinate_file=tmp_path / "c.xyz", box=box)
    got = s.positions()
    assert np.allclose(got.mean(0), box / 2, atol=1e-12)
    assert np.allclose(got - got[0], pos - pos[0], atol=1e-12)        # a rigid shift
    assert np.array_equal(s.real("mass"), np.ones(50)) and np.array_equal(s.types(), np.zeros(50, dtype=np.int32))
    (tmp_path / "short.xyz").write_text("3\ncomment\nAr 0 0 0\nAr 1 1 1\nnot a record\n")
    with pytest.raises(input_api.InputError, match="announces 3 atoms, 2 usable"):
        input_api.System(coordinate_file=tmp_path / "short.xyz", box=box)
    with pytest.raises(input_api.InputError, match="coordinate file .* cannot be opened"):
        input_api.System(coordinate_file=tmp_path / "none.xyz", box=box)


def test_reader_errors_name_file_and_line(tmp_path):
    cases = input_cases.topology_cases(str(tmp_path))
    case = cases["dsmd_water"]
    text = open(case["parameter_file"]).read()
    broken = tmp_path / "broken.dsMDprm"
    broken.write_text(text.replace("lj 0 1 ", "lj 0 7 "))
    with pytest.raises(input_api.InputError, match="invalid atom type ID"):
        input_api.System(coordinate_file=case["coordinate_file"], topology_file=case["topology_file"], parameter_file=broken,
                         box=case["box"])
    broken.write_text(text.replace("[pair_parameters]", "[pear_parameters]"))
    with pytest.raises(input_api.InputError, match=r"broken.dsMDprm:\d+: unknown parameter section \[pear_parameters\]"):
        input_api.System(coordinate_file=case["coordinate_file"], topology_file=case["topology_file"], parameter_file=broken,
                         box=case["box"])
    top = open(case["topology_file"]).read()
    broken_top = tmp_path / "broken.dsMDtop"
    broken_top.write_text(top.replace("atom_count 81", "atom_count 80"))
    with pytest.raises(input_api.InputError, match="atom_count is 80 but \\[atoms\\] contains 81"):
        input_api.System(coordinate_file=case["coordinate_file"], topology_file=broken_top,
                         parameter_file=case["parameter_file"], box=case["box"])
    if input_cases.reference_available():    # the reference's reader refuses the same files
        assert input_cases.reference_topology(str(broken_top), case["parameter_file"]) is None
        assert input_cases.reference_topology(case["topology_file"], str(broken)) is None
    other = cases["legacy_argon"]
    with pytest.raises(input_api.InputError, match="describes 108 atoms, the coordinate file has 81"):
        input_api.System(coordinate_file=case["coordinate_file"], topology_file=other["topology_file"], box=case["box"])


# ---------------------------------------------------------------------------------------------------------------------
# restart files, velocities, thermostat
# ---------------------------------------------------------------------------------------------------------------------
def test_restart_files_have_the_reference_layout(tmp_path):
    rng = np.random.default_rng(2)
    n = 37
    pos, vel = rng.uniform(0, 30, (n, 3)), rng.normal(0, 0.01, (n, 3))
    box = [30.0, 31.0, 32.0]
    path = tmp_path / "a.restart"
    input_api.write_restart(path, 1234, 2.0, box, (True, False, True), "nose_hoover", [0.125], pos, vel)
    want = input_files.pack_restart(1234, 2.0, box, (True, False, True), "nose_hoover", [0.125], pos, vel)
    assert path.read_bytes() == want
    assert not os.path.exists(str(path) + ".tmp")
    # header fields at the documented offsets
    raw = path.read_bytes()
    assert raw[:8] == b"DSMDRST1" and raw[-8:] == b"DSMDEND1"
    assert struct.unpack("<qq", raw[8:24]) == (1234, n)
    assert struct.unpack("<4d", raw[24:56]) == (2.0, 30.0, 31.0, 32.0)
    assert struct.unpack("<3i", raw[56:68]) == (1, 0, 1)
    # read back into a system with as many atoms
    input_files.write_xyz(tmp_path / "c.xyz", rng.uniform(0, 30, (n, 3)), ["Ar"] * n)
    s = input_api.System(coordinate_file=tmp_path / "c.xyz", box=box)
    info = s.read_restart(path)
    assert (info["step"], info["timestep"], info["thermostat"], info["xi"]) == (1234, 2.0, "nose_hoover", 0.125)
    assert np.array_equal(info["box"], np.array(box))
    assert np.array_equal(s.positions(), pos) and np.array_equal(s.velocities(), vel)
    # damaged files
    (tmp_path / "cut.restart").write_bytes(raw[:-20])
    with pytest.raises(input_api.InputError, match="truncated|ends early"):
        s.read_restart(tmp_path / "cut.restart")
    (tmp_path / "bad.restart").write_bytes(b"NOTARST1" + raw[8:])
    with pytest.raises(input_api.InputError, match="is not a dsMD restart file"):
        s.read_restart(tmp_path / "bad.restart")
    input_files.write_xyz(tmp_path / "d.xyz", rng.uniform(0, 30, (n + 1, 3)), ["Ar"] * (n + 1))
    with pytest.raises(input_api.InputError, match=f"has {n} atoms, the coordinate file has {n + 1}"):
        input_api.System(coordinate_file=tmp_path / "d.xyz", box=box).read_restart(path)


def test_start_velocities_and_nose_hoover(tmp_path):
    cases = input_cases.topology_cases(str(tmp_path))
    case = cases["dsmd_water"]
    s = input_api.System(coordinate_file=case["coordinate_file"], topology_file=case["topology_file"],
                         parameter_file=case["parameter_file"], box=case["box"])
    s.init_velocities(300.0, 7)
    v, m = s.velocities(), s.real("mass")
    assert np.abs((m[:, None] * v).sum(0)).max() < 1e-12
    ke = 0.5 * (m[:, None] * v * v).sum() * input_files.MVV2E
    assert ke == pytest.approx(0.5 * (3 * len(m) - 3) * input_files.KB * 300.0, rel=1e-12)
    light, heavy = v[m < 2.0], v[m > 2.0]
    assert (light ** 2).mean() > 4.0 * (heavy ** 2).mean()        # variance kT / m: hydrogens move faster
    s.init_velocities(300.0, 7)
    assert np.array_equal(s.velocities(), v)                      # the same seed gives the same velocities
    s.init_velocities(300.0, 8)
    assert not np.array_equal(s.velocities(), v)
    # Nose-Hoover: two half updates of xi around the scaling
    n, T, tau, dt, xi = 1000, 300.0, 100.0, 2.0, 0.01
    target2 = 3 * n * input_files.KB * T
    q = target2 * tau * tau
    ke = 0.6 * target2
    xi1 = xi + 0.5 * dt * (2 * ke - target2) / q
    scale = np.exp(-xi1 * dt)
    xi2 = xi1 + 0.5 * dt * (2 * ke * scale * scale - target2) / q
    got_scale, got_xi = input_api.nose_hoover_scale(ke, n, T, tau, dt, xi)
    assert got_scale == pytest.approx(scale, rel=1e-15) and got_xi == pytest.approx(xi2, rel=1e-15)
    assert input_api.nose_hoover_scale(ke, n, 0.0, tau, dt, xi) == (1.0, xi)


def test_ewald_table_equals_the_reference_builders_coefficient_by_coefficient():
    """The product's real-space Ewald table builder (Newton divided differences on the Chebyshev nodes) against the
    reference's own (include/ewald_real_table.h:41-105, a 4 x 4 elimination), compiled from the reference header where
    it lies: same intervals, and the same cubic in every interval, for the water box's alpha and two others."""
    import ctypes
    from tests.input_cases import REF_TOPOLOGY
    if not os.path.exists(REF_TOPOLOGY):
        pytest.skip("oracle/_ref is not built")
    ref = ctypes.CDLL(REF_TOPOLOGY)
    if not hasattr(ref, "dsmd_ref_ewald_table"):
        pytest.skip("oracle/_ref predates the Ewald table hook: make -C oracle ref")
    for alpha, cutoff in ((0.3123, 10.0), (0.25, 12.0), (1.1, 2.5)):
        mine = input_api.ewald_table(alpha, cutoff)
        n = ref.dsmd_ref_ewald_table(ctypes.c_double(alpha), ctypes.c_double(cutoff * cutoff), None, ctypes.c_int(0))
        assert n == mine.shape[0]
        theirs = np.zeros((n, 2, 4), dtype=np.float32)
        ref.dsmd_ref_ewald_table(ctypes.c_double(alpha), ctypes.c_double(cutoff * cutoff),
                                 theirs.ctypes.data_as(ctypes.c_void_p), ctypes.c_int(n))
        # the cubics are the same polynomial found two ways: equal to a few ulp of the interval's largest coefficient
        scale = np.abs(theirs).max(axis=2, keepdims=True)
        assert np.all(np.abs(mine - theirs) <= 4e-6 * scale + 1e-30)
        # and they evaluate to the same values across every interval
        t = np.linspace(0.0, 1.0, 9, dtype=np.float32)[None, None, :]
        ev = lambda c: ((c[..., 3:4] * t + c[..., 2:3]) * t + c[..., 1:2]) * t + c[..., 0:1]
        va, vb = ev(mine.astype(np.float64)), ev(theirs.astype(np.float64))
        assert np.all(np.abs(va - vb) <= 2e-6 * np.abs(vb) + 1e-30)


def test_dart_throw_keeps_the_minimum_distance_and_repeats_for_a_seed():
    """The disordered-solid generator: n points in the periodic cube, none closer than the minimum distance to another
    (images included), the same points for the same seed, other points for another; a density past saturation fails."""
    from scipy.spatial import cKDTree
    from deepscalemd_b200 import synthetic as syn
    s = syn.disordered_solid(20000, seed=5)
    L = s.box[0]
    assert s.pos.shape == (20000, 3) and s.pos.min() >= 0.0 and s.pos.max() < L
    assert abs(20000 / L ** 3 - 0.05) < 1e-12
    nearest = cKDTree(s.pos, boxsize=L).query(s.pos, k=2)[0][:, 1]
    assert nearest.min() >= 1.8 and nearest.min() < 1.9          # rejection at work: without it the minimum is ~0.05 A
    assert np.array_equal(s.pos, syn.disordered_solid(20000, seed=5).pos)
    assert not np.array_equal(s.pos, syn.disordered_solid(20000, seed=6).pos)
    assert np.bincount(s.types, minlength=3).tolist() == pytest.approx([10000, 6000, 4000], abs=300)
    with pytest.raises(input_api.InputError):
        input_api.dart_throw(1000, 10.0, 1.8, 1)                 # 1000 spheres of 1.8 A do not fit a 10 A cube
    assert input_api.dart_throw(50, 10.0, 0.0, 1).shape == (50, 3)


def test_bonded_sections_of_a_dsmd_input_system_come_back_term_by_term(tmp_path):
    """Flexible chains written as a dsMD_input folder: the reader returns every bond, angle, dihedral, improper and special
    pair with its own parameters (angles and phases converted to radians, a harmonic improper as multiplicity 0), in the
    form the device library takes; 1-2, 1-3 and 1-4 pairs become exclusions; a special pair whose parameter id is not
    listed takes the pair matrix of its two atom types."""
    s = syn.chain_fluid(3, 8, seed=5)
    elements = ["C"] * s.n
    manifest = input_files.write_dsmd_input(str(tmp_path / "chains"), "chains", s.pos, elements, s.types, ["CH3", "CH2"], s.mass,
                                            s.charge, s.sig, s.eps, bonded=s.bonded)
    folder = os.path.dirname(manifest)
    files = dict(coordinate_file=os.path.join(folder, "chains.xyz"), topology_file=os.path.join(folder, "chains.dsMDtop"),
                 parameter_file=os.path.join(folder, "chains.dsMDprm"), box=s.box)
    system = input_api.System(**files)
    got = system.bonded()
    want = s.bonded
    assert got["n_dihedrals"] == want["n_dihedrals"] == 27 * 5
    for key in ("bonds", "angles", "torsions", "specials", "torsion_n"):
        assert np.array_equal(got[key], np.asarray(want[key])), key
    for key in ("bond_k", "bond_r0", "angle_k", "torsion_k", "special_sigma", "special_epsilon", "special_lj_scale",
                "special_coulomb_scale"):
        assert np.array_equal(got[key], want[key]), key
    for key in ("angle_theta0", "torsion_phi0"):
        assert np.abs(got[key] - want[key]).max() < 1e-14, key
    assert (len(got["bonds"]), len(got["angles"]), len(got["torsions"]), len(got["specials"])) == (
        27 * 7, 27 * 6, len(want["torsions"]), 27 * 5)
    excl = {tuple(sorted(p)) for p in s.exclusions.tolist()}
    assert {tuple(p) for p in system.exclusions().tolist()} == excl
    # unlisted special-pair parameter id: the pair matrix stands in
    text = open(os.path.join(folder, "chains.dsMDprm")).read()
    head, tail = text.split("[special_pair_parameters]\n")
    open(os.path.join(folder, "chains.dsMDprm"), "w").write(head + "[special_pair_parameters]\n" + "\n".join(tail.split("\n")[1:]))
    again = input_api.System(**files).bonded()
    i, j = want["specials"][0]
    assert again["special_sigma"][0] == s.sig[s.types[i], s.types[j]] and again["special_epsilon"][0] == s.eps[s.types[i], s.types[j]]
    assert np.array_equal(again["special_sigma"][1:], want["special_sigma"][1:])
