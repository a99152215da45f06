"""The MD driver executable (deepscalemd_b200/bin/dsmd_b200_run): what runs without a GPU - input checking, refusals,
usage errors."""
import json
import os
import subprocess
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import input_cases  # noqa: E402

from deepscalemd_b200 import build, input_files
from deepscalemd_b200 import synthetic as syn


@pytest.fixture(scope="module")
def driver():
    if not os.path.exists(build.LIBRARY):
        pytest.skip("libdsmd_b200.so is not built")
    return build.build_driver()


def run(driver, *args):
    return subprocess.run([driver, *map(str, args)], capture_output=True, text=True, timeout=120)


def test_check_input_reports_configuration_and_system(driver, tmp_path):
    path, scale = input_files.argon_files(str(tmp_path), syn.fcc_lj(3, seed=4), total_steps=50)
    r = run(driver, path, "--check-input")
    assert r.returncode == 0, r.stderr
    out = json.loads(r.stdout)
    assert out["refused"] == []
    assert out["system"]["atoms"] == 108 and out["system"]["types"] == 1
    assert out["system"]["total_mass"] == pytest.approx(108 * 39.948)
    assert out["config"]["total_steps"] == 50 and out["config"]["enable_lennard_jones"] and not out["config"]["enable_coulomb"]
    assert out["config"]["box"] == pytest.approx(list(scale["box"]))


def test_refuses_what_the_path_does_not_cover(driver, tmp_path):
    case = input_cases.topology_cases(str(tmp_path))["dsmd_water"]
    common = dict(box=case["box"], total_steps=10, timestep=2.0, temperature=300.0, cutoff=4.0, skin=0.5,
                  input_system=case["manifest"])
    y = input_files.write_run_yaml(tmp_path / "water.yaml", force_type="lj, PME", **common)
    r = run(driver, y, "--check-input")
    assert r.returncode == 3
    refused = json.loads(r.stdout)["refused"]
    # constraints are solved on the device (SHAKE / RATTLE) and no longer refused; reciprocal-space PME still is
    assert not any("constraints" in t for t in refused) and any("reciprocal-space PME" in t for t in refused)
    r = run(driver, y)                      # refused before any device work
    assert r.returncode == 3 and "does not cover" in r.stderr
    y = input_files.write_run_yaml(tmp_path / "langevin.yaml", force_type="lj", thermostat="langevin", **common)
    assert any("langevin" in t for t in json.loads(run(driver, y, "--check-input").stdout)["refused"])


def test_usage_and_input_errors(driver, tmp_path):
    assert run(driver).returncode == 2
    assert run(driver, "--no-such-flag").returncode == 2
    r = run(driver, tmp_path / "absent.yaml")
    assert r.returncode == 1 and "cannot be opened" in r.stderr
    (tmp_path / "incomplete.yaml").write_text("timestep: 1.0\n")
    r = run(driver, tmp_path / "incomplete.yaml", "--check-input")
    assert r.returncode == 1 and "lacks required keys: coordinate_file, target_temperature, total_steps" in r.stderr


def test_bonded_terms_of_a_dsmd_input_system_are_accepted_and_those_of_a_legacy_topology_refused(driver, tmp_path):
    s = syn.chain_fluid(3, 8, seed=5)
    manifest = input_files.write_dsmd_input(str(tmp_path / "chains"), "chains", s.pos, ["C"] * s.n, s.types, ["CH3", "CH2"],
                                            s.mass, s.charge, s.sig, s.eps, bonded=s.bonded)
    common = dict(box=s.box, total_steps=10, timestep=0.5, temperature=300.0, cutoff=s.cutoff, skin=s.skin,
                  extra={"real_space_only": "true"})
    y = input_files.write_run_yaml(tmp_path / "chains.yaml", input_system=manifest,
                                   force_type="lj, PME, bonds, angles, dihedrals", **common)
    r = run(driver, y, "--check-input")
    assert r.returncode == 0, r.stderr
    out = json.loads(r.stdout)
    assert out["refused"] == [] and out["system"]["bonds"] == 27 * 7
    assert out["config"]["enable_bonds"] and out["config"]["enable_angles"] and out["config"]["enable_dihedrals"]
    y = input_files.write_run_yaml(tmp_path / "bonds_only.yaml", input_system=manifest, force_type="lj, bonds", **common)
    cfg = json.loads(run(driver, y, "--check-input").stdout)["config"]
    assert cfg["enable_bonds"] and not cfg["enable_angles"] and not cfg["enable_dihedrals"] and not cfg["enable_coulomb"]
    legacy = input_cases.topology_cases(str(tmp_path / "cases"))["legacy_mixed"]       # a legacy .top with a [bonds] section
    y = input_files.write_run_yaml(tmp_path / "legacy.yaml", coordinate_file=legacy["coordinate_file"],
                                   topology_file=legacy["topology_file"], force_type="lj, bonds", **dict(common, box=legacy["box"]))
    refused = json.loads(run(driver, y, "--check-input").stdout)["refused"]
    assert any("legacy topology" in t for t in refused)
