"""The MD driver's host logic on the CPU: the driver's own sources linked against a host-side test double of the device
library (tests/mock_device), so that step order, rebuild policy, output, thermostat and restart handling run end to end
without a GPU. The GPU tests run the real executable (tests/test_gpu_driver.py)."""
import os
import re
import subprocess

import numpy as np
import pytest

from deepscalemd_b200 import build, input_api, input_files
from deepscalemd_b200 import synthetic as syn
from oracle import cpu_oracle as co

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
LINE = re.compile(r"^Step: (\d+), T: ([-\d.eE+]+), KE: ([-\d.eE+]+), PE: ([-\d.eE+]+), Etot: ([-\d.eE+]+)$")


@pytest.fixture(scope="module")
def driver(tmp_path_factory):
    out = tmp_path_factory.mktemp("mock_driver")
    lib = out / "libdsmd_b200.so"
    subprocess.run(["/usr/bin/g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-I", os.path.join(ROOT, "include"), "-o", str(lib),
                    os.path.join(HERE, "mock_device", "mock_dsmd_b200.cpp")], check=True)
    host = os.path.join(ROOT, "deepscalemd_b200", "csrc", "host")
    srcs = [os.path.join(host, "dsmd_run.cpp")] + [os.path.join(ROOT, "deepscalemd_b200", s) for s in build.HOST_SOURCES[:-1]]
    exe = out / "dsmd_b200_run"
    subprocess.run(["/usr/bin/g++", "-std=c++17", "-O2", "-I", os.path.join(ROOT, "include"), "-I", host, "-o", str(exe), *srcs,
                    "-L", str(out), "-l:libdsmd_b200.so", f"-Wl,-rpath,{out}"], check=True)
    return str(exe)


def run_driver(driver, yaml_path):
    r = subprocess.run([driver, str(yaml_path)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr + r.stdout
    rows = [tuple(float(v) for v in m.groups()) for m in map(LINE.match, r.stdout.splitlines()) if m]
    return np.array(rows), r.stdout


def test_nve_run(driver, tmp_path):
    s = syn.fcc_lj(4, seed=1)
    path, scale = input_files.argon_files(str(tmp_path), s, total_steps=200, output_freq=50, update_freq=1000)
    rows, out = run_driver(driver, path)
    assert [int(r[0]) for r in rows] == [0, 50, 100, 150, 200]
    n = s.n
    target_t = 1.44 * scale["epsilon"] / input_files.KB
    assert rows[0][2] == pytest.approx(0.5 * (3 * n - 3) * input_files.KB * target_t, abs=2e-6)
    assert rows[0][1] == pytest.approx(target_t * (3 * n - 3) / (3 * n), abs=2e-6)
    x, y, z = (np.ascontiguousarray(s.pos[:, k]) for k in range(3))
    c6, c12 = co.lj_tables(s.eps, s.sig)
    _, sc = co.forces(x, y, z, n, s.box, co.pairs(x, y, z, n, s.box, search=s.cutoff), c6, c12, s.cutoff)
    assert rows[0][3] == pytest.approx(sc["pe"] * scale["epsilon"], rel=1e-8)
    etot = rows[:, 4]
    assert np.abs(etot - etot[0]).max() < 5e-3 * rows[0][2]
    assert rows[-1][1] < 0.75 * rows[0][1]
    assert int(re.search(r"Neighbor list builds = (\d+)", out).group(1)) >= 5
    assert re.search(r"Performance: [\d.]+ Matom-step/s, [\d.]+ ms/step, [\d.]+ ns/day \(md_loop only, dt=[\d.]+ fs\)", out)


def test_periodic_rebuilds_follow_the_step_counter(driver, tmp_path):
    s = syn.fcc_lj(4, seed=1)
    path, _ = input_files.argon_files(str(tmp_path), s, total_steps=40, output_freq=1, update_freq=5, temperature_reduced=0.01)
    _, out = run_driver(driver, path)      # cold: nothing moves half a skin in 40 steps, only the counter rebuilds
    assert int(re.search(r"Neighbor list builds = (\d+)", out).group(1)) == 1 + 7    # first build + steps 5, 10, .. 35


def test_nose_hoover(driver, tmp_path):
    s = syn.fcc_lj(4, seed=1)
    path, scale = input_files.argon_files(str(tmp_path), s, total_steps=3000, output_freq=100, update_freq=1000,
                                          thermostat="nose_hoover", tau_t=200.0)
    rows, _ = run_driver(driver, path)
    target_t = 1.44 * scale["epsilon"] / input_files.KB
    late = rows[rows[:, 0] >= 1500][:, 1]
    assert abs(late.mean() - target_t) < 0.06 * target_t
    nve, _ = input_files.argon_files(str(tmp_path / "nve"), s, total_steps=3000, output_freq=100, update_freq=1000)
    rows_nve, _ = run_driver(driver, nve)
    assert rows_nve[rows_nve[:, 0] >= 1500][:, 1].mean() < 0.8 * target_t      # without it the lattice start stays cold


def test_restart_continues_the_run(driver, tmp_path):
    s = syn.fcc_lj(4, seed=1)
    kw = dict(output_freq=25, update_freq=1000, thermostat="nose_hoover", tau_t=200.0)
    whole, _ = input_files.argon_files(str(tmp_path / "whole"), s, total_steps=100, **kw)
    rows_whole, _ = run_driver(driver, whole)
    first, _ = input_files.argon_files(str(tmp_path / "first"), s, total_steps=50, restart_output=str(tmp_path / "half.restart"),
                                       restart_output_freq=50, **kw)
    rows_first, out_first = run_driver(driver, first)
    assert "[restart] wrote" in out_first
    second, scale = input_files.argon_files(str(tmp_path / "second"), s, total_steps=50,
                                            restart_file=str(tmp_path / "half.restart"), **kw)
    rows_second, _ = run_driver(driver, second)
    assert [int(r[0]) for r in rows_second] == [50, 75, 100]
    assert rows_second[0][1:] == pytest.approx(rows_first[-1][1:], abs=2e-6)
    # positions, velocities and the thermostat variable all came through the file: the same trajectory to rounding
    assert rows_second[-1][1:] == pytest.approx(rows_whole[-1][1:], rel=1e-9)
    sys_ = input_api.System(coordinate_file=str(tmp_path / "first" / "argon.xyz"), box=scale["box"])
    info = sys_.read_restart(tmp_path / "half.restart")
    assert info["step"] == 50 and info["thermostat"] == "nose_hoover" and info["xi"] != 0.0


def test_binary_mixture_from_a_dsmd_input_folder(driver, tmp_path):
    """Two atom types with an explicit pair table (not Lorentz-Berthelot), read through input_system -> manifest ->
    .dsMDtop / .dsMDprm: the start energy equals the oracle's for the same table, and the run conserves energy."""
    ka = syn.kob_andersen(256, seed=5)
    sig, eps, mass = 3.405, 0.238, 39.948
    box = np.asarray(ka.box) * sig
    pos = ka.pos * sig
    pos = pos - box * np.floor(pos / box)
    pos = pos + (box / 2 - pos.mean(0))
    manifest = input_files.write_dsmd_input(str(tmp_path / "ka"), "ka", pos, ["Ar" if t == 0 else "Kr" for t in ka.types],
                                            ka.types, ["A", "B"], ka.mass * mass, ka.charge, np.asarray(ka.sig) * sig,
                                            np.asarray(ka.eps) * eps)
    tau = input_files.reduced_time_fs()
    # cutoff 2.2 sigma_AA: the 256-atom box is 5.98 sigma wide, the test double needs twice the list radius
    path = input_files.write_run_yaml(tmp_path / "ka.yaml", box=box, total_steps=100, timestep=0.0002 * tau,
                                      temperature=0.8 * eps / input_files.KB, cutoff=2.2 * sig, skin=0.3 * sig,
                                      input_system=manifest, output_freq=50, update_freq=1000)
    rows, _ = run_driver(driver, path)
    x, y, z = (np.ascontiguousarray(ka.pos[:, k]) for k in range(3))
    c6, c12 = co.lj_tables(ka.eps, ka.sig)
    _, sc = co.forces(x, y, z, ka.n, ka.box, co.pairs(x, y, z, ka.n, ka.box, search=2.2), c6, c12, 2.2, types=ka.types)
    assert rows[0][3] == pytest.approx(sc["pe"] * eps, rel=1e-8)
    # (the start configuration is unrelaxed, with strongly repulsive contacts: hence the short time step)
    assert abs(rows[-1][4] - rows[0][4]) < 1e-3 * abs(rows[0][3])


def test_xyz_frames_have_the_reference_layout(driver, tmp_path):
    s = syn.fcc_lj(4, seed=1)
    prefix = str(tmp_path / "traj")
    path, scale = input_files.argon_files(str(tmp_path), s, total_steps=20, output_freq=10, update_freq=1000,
                                          trajectory_output_freq=10, output_prefix=prefix,
                                          extra={"trajectory_include_velocities": "true"})
    rows, _ = run_driver(driver, path)
    frames = sorted(f for f in os.listdir(tmp_path) if f.startswith("traj_") and f.endswith(".xyz"))
    assert frames == ["traj_0.xyz", "traj_10.xyz", "traj_20.xyz"]
    lines = open(tmp_path / "traj_10.xyz").read().splitlines()
    assert lines[0] == str(s.n) and len(lines) == s.n + 2
    m = re.match(r"^Step 10 Time ([\d.]+) fs KE=([-\d.]+) PE=([-\d.]+) Total=([-\d.]+)$", lines[1])
    assert m and float(m.group(1)) == pytest.approx(10 * 0.005 * scale["tau_fs"], abs=1e-3)
    assert float(m.group(2)) == pytest.approx(rows[1][2], abs=2e-6) and float(m.group(3)) == pytest.approx(rows[1][3], abs=2e-6)
    first = lines[2].split()
    assert first[0] == "Ar" and len(first) == 7 and all(re.match(r"^-?\d+\.\d{6}$", v) for v in first[1:])
    # frame 0 holds the start positions in coordinate-file order
    start = np.array([[float(v) for v in l.split()[1:4]] for l in open(tmp_path / "traj_0.xyz").read().splitlines()[2:]])
    assert np.abs(start - scale["positions"]).max() < 1e-6
