"""Writers of the reference's input formats for the synthetic systems (run description, XYZ coordinates, legacy ``.top``,
``dsMD_input`` folder with manifest / ``.dsMDtop`` / ``.dsMDprm``, ``DSMDRST1`` restart files), so that the same seeded
systems that feed the kernels directly can also be fed through files, the way ``bin/dsMD`` takes them
(docs/03_Input_Reference.md, docs/04_Preparing_a_System.md of the reference; restart layout src/md_restart.cpp:3-12).

Reduced Lennard-Jones systems are written in the reference's real units as argon (sigma 3.405 A, epsilon 0.238 kcal/mol,
mass 39.948 g/mol; one reduced time unit = 2156 fs).
"""
from __future__ import annotations

import os
import struct

import numpy as np

ARGON = dict(sigma=3.405, epsilon=0.238, mass=39.948)
KB = 0.0019872041            # kcal / (mol K)
MVV2E = 48.88821291 ** 2     # (g/mol)(A/fs)^2 -> kcal/mol


def reduced_time_fs(sigma=ARGON["sigma"], epsilon=ARGON["epsilon"], mass=ARGON["mass"]) -> float:
    """One reduced LJ time unit sigma * sqrt(m / epsilon) in fs."""
    return sigma * np.sqrt(mass / (epsilon * 1.0 / MVV2E))


def write_xyz(path, pos, elements, comment="generated"):
    pos = np.asarray(pos, dtype=np.float64)
    with open(path, "w") as f:
        f.write(f"{len(pos)}\n{comment}\n")
        for e, p in zip(elements, pos):
            f.write(f"{e} {p[0]:.17g} {p[1]:.17g} {p[2]:.17g}\n")


def write_legacy_top(path, type_rows, atom_types):
    """type_rows: name -> (mass, charge, sigma, epsilon); atom_types: the type name of every atom (ids are 1-based)."""
    with open(path, "w") as f:
        f.write("; legacy topology\n[ atomtypes ]\n; name mass charge sigma epsilon\n")
        for name, (mass, charge, sigma, eps) in type_rows.items():
            f.write(f"{name} {mass:.17g} {charge:.17g} {sigma:.17g} {eps:.17g}\n")
        f.write("\n[ atoms ]\n")
        for i, name in enumerate(atom_types):
            f.write(f"{i + 1} {name}\n")


def write_dsmd_input(folder, name, pos, elements, type_ids, type_names, mass, charge, pair_sigma, pair_epsilon,
                     exclusions=None, constraints=None, bonded=None):
    """A dsMD_input folder: manifest.yaml, <name>.xyz, <name>.dsMDtop, <name>.dsMDprm. pair_sigma / pair_epsilon:
    [ntypes, ntypes] symmetric (the upper triangle is written). bonded: the mapping synthetic.chain_fluid() makes (every
    term gets a parameter id of its own; angles and phases are written in degrees, as the format wants them)."""
    os.makedirs(folder, exist_ok=True)
    write_xyz(os.path.join(folder, name + ".xyz"), pos, elements)
    nt = len(type_names)
    with open(os.path.join(folder, name + ".dsMDprm"), "w") as f:
        f.write("[meta]\nschema_version 1\nlength_unit angstrom\nenergy_unit kcal_per_mol\ncharge_unit elementary_charge\n\n")
        f.write("[nonbonded]\ncomponent lj mie n=12 m=6\n\n[atom_types]\n")
        for t, tn in enumerate(type_names):
            f.write(f"{t} {tn}\n")
        f.write("\n[pair_parameters]\n; component type_i type_j sigma epsilon\n")
        for a in range(nt):
            for b in range(a, nt):
                f.write(f"lj {a} {b} {pair_sigma[a][b]:.17g} {pair_epsilon[a][b]:.17g}\n")
        if bonded is not None:
            nd = int(bonded["n_dihedrals"])
            f.write("\n[bond_parameters]\n")
            for k, (kk, r0) in enumerate(zip(bonded["bond_k"], bonded["bond_r0"])):
                f.write(f"{k} harmonic {kk:.17g} {r0:.17g}\n")
            f.write("\n[angle_parameters]\n")
            for k, (kk, th) in enumerate(zip(bonded["angle_k"], np.rad2deg(bonded["angle_theta0"]))):
                f.write(f"{k} harmonic {kk:.17g} {th:.17g}\n")
            f.write("\n[torsion_parameters]\n")
            for k in range(nd):
                f.write(f"{k} periodic {bonded['torsion_k'][k]:.17g} {np.rad2deg(bonded['torsion_phi0'][k]):.17g} "
                        f"{int(bonded['torsion_n'][k])}\n")
            f.write("\n[improper_parameters]\n")
            for k in range(nd, len(bonded["torsions"])):
                form = "harmonic" if int(bonded["torsion_n"][k]) == 0 else "periodic"
                tail = "" if form == "harmonic" else f" {int(bonded['torsion_n'][k])}"
                f.write(f"{k - nd} {form} {bonded['torsion_k'][k]:.17g} {np.rad2deg(bonded['torsion_phi0'][k]):.17g}{tail}\n")
            f.write("\n[special_pair_parameters]\n")
            for k, (sg, ep) in enumerate(zip(bonded["special_sigma"], bonded["special_epsilon"])):
                f.write(f"{k} {sg:.17g} {ep:.17g}\n")
    with open(os.path.join(folder, name + ".dsMDtop"), "w") as f:
        f.write(f"[meta]\nschema_version 1\natom_count {len(pos)}\n\n[atoms]\n; atom_id element type_id mass charge\n")
        for i in range(len(pos)):
            f.write(f"{i} {elements[i]} {int(type_ids[i])} {mass[i]:.17g} {charge[i]:.17g}\n")
        if exclusions is not None and len(exclusions):
            f.write("\n[exclusions]\n")
            for a, b in exclusions:
                f.write(f"{int(a)} {int(b)}\n")
        if constraints is not None and len(constraints):
            f.write("\n[constraints]\n")
            for a, b, d in constraints:
                f.write(f"{int(a)} {int(b)} {d:.17g}\n")
        if bonded is not None:
            nd = int(bonded["n_dihedrals"])
            f.write("\n[bonds]\n")
            for k, (a, b) in enumerate(bonded["bonds"]):
                f.write(f"{int(a)} {int(b)} {k}\n")
            f.write("\n[angles]\n")
            for k, (a, b, c) in enumerate(bonded["angles"]):
                f.write(f"{int(a)} {int(b)} {int(c)} {k}\n")
            f.write("\n[dihedrals]\n")
            for k, (a, b, c, d) in enumerate(bonded["torsions"][:nd]):
                f.write(f"{int(a)} {int(b)} {int(c)} {int(d)} {k}\n")
            f.write("\n[impropers]\n")
            for k, (a, b, c, d) in enumerate(bonded["torsions"][nd:]):
                f.write(f"{int(a)} {int(b)} {int(c)} {int(d)} {k}\n")
            f.write("\n[special_pairs]\n")
            for k, (a, b) in enumerate(bonded["specials"]):
                f.write(f"{int(a)} {int(b)} {k} {bonded['special_lj_scale'][k]:.17g} {bonded['special_coulomb_scale'][k]:.17g}\n")
    with open(os.path.join(folder, "manifest.yaml"), "w") as f:
        f.write("schema_version: 1\nformat: dsMD_input\n")
        f.write(f"coordinate_file: {name}.xyz\ntopology_file: {name}.dsMDtop\nparameter_file: {name}.dsMDprm\n")
    return os.path.join(folder, "manifest.yaml")


def write_run_yaml(path, *, box, total_steps, timestep, temperature, cutoff, skin, coordinate_file=None, topology_file=None,
                   parameter_file=None, input_system=None, periodic=(True, True, True), force_type="lj", thermostat="none",
                   tau_t=100.0, output_freq=10, output_info="STEP, T, KE, PE, ETOTAL", switch=None, update_freq=10,
                   restart_file=None, restart_output=None, restart_output_freq=0, output_prefix="md_output",
                   trajectory_output_freq=0, extra=None):
    lines = ["# generated run description"]
    if input_system:
        lines.append(f"input_system: {input_system}")
    if coordinate_file:
        lines.append(f"coordinate_file: {coordinate_file}")
    if topology_file:
        lines.append(f"topology_file: {topology_file}")
    if parameter_file:
        lines.append(f"parameter_file: {parameter_file}")
    lines += [f"target_temperature: {temperature:.17g}", f"timestep: {timestep:.17g}", f"total_steps: {total_steps}",
              f"box_x: {box[0]:.17g}", f"box_y: {box[1]:.17g}", f"box_z: {box[2]:.17g}"]
    for axis, p in zip("xyz", periodic):
        lines.append(f"periodic_{axis}: {'true' if p else 'false'}")
    lines += [f"cutoff_distance: {cutoff:.17g}", f"verlet_skin: {skin:.17g}", f"neighbor_list_update_freq: {update_freq}",
              "integrator: velocity_verlet", f"thermostat: {thermostat}", f"tau_t: {tau_t:.17g}", "barostat: none",
              f"output_freq: {output_freq}", f"output_info: {output_info}", f"output_prefix: {output_prefix}",
              f"trajectory_output_freq: {trajectory_output_freq}"]
    if switch is not None:
        lines.append(f"lj_switch_distance: {switch:.17g}")
    if restart_file:
        lines.append(f"restart_file: {restart_file}")
    if restart_output:
        lines.append(f"restart_output: {restart_output}")
    if restart_output_freq:
        lines.append(f"restart_output_freq: {restart_output_freq}")
    for k, v in (extra or {}).items():
        lines.append(f"{k}: {v}")
    lines += ["force_calculation:", "  mode: builtin", f"  type: {force_type}", "  precision: mixed", "  nonbonded_kernel: list"]
    with open(path, "w") as f:
        f.write("\n".join(lines) + "\n")
    return path


def pack_restart(step, timestep, box, periodic, thermostat, thermostat_state, pos, vel, barostat="none", barostat_state=()):
    """The bytes of a DSMDRST1 file (positions [N, 3] in A, velocities [N, 3] in A/fs, both in global atom id order)."""
    pos = np.asarray(pos, dtype="<f8")
    vel = np.asarray(vel, dtype="<f8")

    def text(s):
        b = s.encode()
        return struct.pack("<i", len(b)) + b

    def reals(v):
        return struct.pack("<i", len(v)) + np.asarray(v, dtype="<f8").tobytes()

    out = b"DSMDRST1" + struct.pack("<qq", int(step), len(pos)) + struct.pack("<4d", timestep, *box)
    out += struct.pack("<3i", *[1 if p else 0 for p in periodic])
    out += text(thermostat) + reals(thermostat_state) + text(barostat) + reals(barostat_state)
    for a in (pos[:, 0], pos[:, 1], pos[:, 2], vel[:, 0], vel[:, 1], vel[:, 2]):
        out += np.ascontiguousarray(a).tobytes()
    return out + b"DSMDEND1"


def argon_files(folder, s, *, total_steps=100, temperature_reduced=1.44, thermostat="none", dt_reduced=0.005, **yaml_kw):
    """Writes a reduced-unit LJ system as argon: <folder>/argon.xyz, argon.top, run.yaml. Returns (yaml path, scale)."""
    os.makedirs(folder, exist_ok=True)
    sig, eps, mass = ARGON["sigma"], ARGON["epsilon"], ARGON["mass"]
    box = np.asarray(s.box) * sig
    pos = np.asarray(s.pos) * sig
    pos = pos - box * np.floor(pos / box)
    pos = pos + (box / 2.0 - pos.mean(0))       # mean at the box centre: the reader's recentring moves nothing
    write_xyz(os.path.join(folder, "argon.xyz"), pos, ["Ar"] * s.n)
    write_legacy_top(os.path.join(folder, "argon.top"), {"Ar": (mass, 0.0, sig, eps)}, ["Ar"] * s.n)
    tau = reduced_time_fs()
    path = write_run_yaml(os.path.join(folder, "run.yaml"), box=box, total_steps=total_steps, timestep=dt_reduced * tau,
                          temperature=temperature_reduced * eps / KB, cutoff=s.cutoff * sig, skin=s.skin * sig,
                          coordinate_file=os.path.join(folder, "argon.xyz"), topology_file=os.path.join(folder, "argon.top"),
                          thermostat=thermostat, **yaml_kw)
    return path, dict(sigma=sig, epsilon=eps, mass=mass, tau_fs=tau, positions=pos, box=box)
