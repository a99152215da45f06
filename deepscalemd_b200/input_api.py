"""ctypes binding of the host-side input layer (``include/dsmd_input.h``, ``libdsmd_input.so``): the reference's run
description, coordinate, topology / parameter and restart files read by the C++ readers of ``csrc/host``."""
from __future__ import annotations

import ctypes
import json
import os
from ctypes import POINTER, byref, c_char_p, c_double, c_int, c_int32, c_int64, c_uint64, c_void_p

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY = os.path.join(_HERE, "libdsmd_input.so")

SYMBOLS = [
    "dsmd_input_last_error", "dsmd_input_config_read", "dsmd_input_config_destroy", "dsmd_input_config_json",
    "dsmd_input_system_load", "dsmd_input_system_load_files", "dsmd_input_system_destroy", "dsmd_input_system_counts",
    "dsmd_input_system_real", "dsmd_input_system_types", "dsmd_input_system_pair_table", "dsmd_input_system_exclusions",
    "dsmd_input_system_constraints", "dsmd_input_system_bonded", "dsmd_input_system_velocities", "dsmd_input_restart_read", "dsmd_input_restart_write",
    "dsmd_input_nose_hoover_scale", "dsmd_host_brick_plan", "dsmd_host_counts_verdict", "dsmd_host_wait_probe", "dsmd_host_ewald_table", "dsmd_host_dart_throw",
]

_lib = None


class InputError(RuntimeError):
    pass


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIBRARY):
            raise InputError(f"{LIBRARY} has not been built (python -m deepscalemd_b200.build)")
        L = ctypes.CDLL(LIBRARY)
        L.dsmd_input_last_error.restype = c_char_p
        for name in SYMBOLS[1:]:
            getattr(L, name).restype = c_int
        L.dsmd_input_config_destroy.restype = None
        L.dsmd_input_system_destroy.restype = None
        _lib = L
    return _lib


def _check(rc):
    if rc != 0:
        raise InputError(lib().dsmd_input_last_error().decode())


class Config:
    """A run description read by the C++ reader; ``values`` is the resolved configuration."""

    def __init__(self, path):
        self.h = c_void_p()
        _check(lib().dsmd_input_config_read(str(path).encode(), byref(self.h)))
        text = c_char_p()
        _check(lib().dsmd_input_config_json(self.h, byref(text)))
        self.values = json.loads(text.value.decode())

    def close(self):
        if self.h:
            lib().dsmd_input_config_destroy(self.h)
            self.h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class System:
    """Coordinates + topology (+ parameters) read by the C++ readers."""

    def __init__(self, config=None, *, coordinate_file=None, topology_file=None, parameter_file=None, box=None):
        self.h = c_void_p()
        if config is not None:
            _check(lib().dsmd_input_system_load(config.h, byref(self.h)))
        else:
            b = (c_double * 3)(*box)
            _check(lib().dsmd_input_system_load_files(str(coordinate_file).encode(),
                                                      str(topology_file).encode() if topology_file else None,
                                                      str(parameter_file).encode() if parameter_file else None, b,
                                                      byref(self.h)))

    def counts(self):
        atoms, excl, cons = c_int64(), c_int64(), c_int64()
        types, explicit = c_int32(), c_int32()
        _check(lib().dsmd_input_system_counts(self.h, byref(atoms), byref(types), byref(excl), byref(cons), byref(explicit)))
        return dict(atoms=atoms.value, types=types.value, exclusions=excl.value, constraints=cons.value,
                    explicit_pairs=bool(explicit.value))

    def real(self, field):
        index = ["x", "y", "z", "vx", "vy", "vz", "mass", "charge"].index(field)
        p = POINTER(c_double)()
        _check(lib().dsmd_input_system_real(self.h, c_int(index), byref(p)))
        return np.ctypeslib.as_array(p, shape=(self.counts()["atoms"],)).copy()

    def positions(self):
        return np.stack([self.real(k) for k in "xyz"], axis=1)

    def velocities(self):
        return np.stack([self.real(k) for k in ("vx", "vy", "vz")], axis=1)

    def types(self):
        p = POINTER(c_int32)()
        _check(lib().dsmd_input_system_types(self.h, byref(p)))
        return np.ctypeslib.as_array(p, shape=(self.counts()["atoms"],)).copy()

    def pair_table(self):
        e, s = POINTER(c_double)(), POINTER(c_double)()
        n, m = c_int32(), c_int32()
        _check(lib().dsmd_input_system_pair_table(self.h, byref(e), byref(s), byref(n), byref(m)))
        nt = self.counts()["types"]
        return (np.ctypeslib.as_array(e, shape=(nt, nt)).copy(), np.ctypeslib.as_array(s, shape=(nt, nt)).copy(), n.value,
                m.value)

    def exclusions(self):
        n = self.counts()["exclusions"]
        if n == 0:
            return np.zeros((0, 2), dtype=np.int32)
        p = POINTER(c_int32)()
        _check(lib().dsmd_input_system_exclusions(self.h, byref(p)))
        return np.ctypeslib.as_array(p, shape=(n, 2)).copy()

    def constraints(self):
        n = self.counts()["constraints"]
        if n == 0:
            return np.zeros(0, dtype=np.int32), np.zeros(0, dtype=np.int32), np.zeros(0)
        i, j, d = POINTER(c_int32)(), POINTER(c_int32)(), POINTER(c_double)()
        _check(lib().dsmd_input_system_constraints(self.h, byref(i), byref(j), byref(d)))
        return (np.ctypeslib.as_array(i, shape=(n,)).copy(), np.ctypeslib.as_array(j, shape=(n,)).copy(),
                np.ctypeslib.as_array(d, shape=(n,)).copy())

    def bonded(self):
        """The bonded terms with per-term parameters as a mapping of arrays (the keys Context.set_bonded reads), plus
        n_dihedrals: how many of the torsions are proper dihedrals (they come first)."""
        counts = (c_int64 * 5)()
        atom_ptrs = [POINTER(c_int32)() for _ in range(4)]
        par_ptrs = [POINTER(c_double)() for _ in range(10)]
        mult = POINTER(c_int32)()
        atoms = (POINTER(POINTER(c_int32)) * 4)(*[ctypes.pointer(p) for p in atom_ptrs])
        pars = (POINTER(POINTER(c_double)) * 10)(*[ctypes.pointer(p) for p in par_ptrs])
        _check(lib().dsmd_input_system_bonded(self.h, counts, atoms, pars, byref(mult)))
        nb, na, nt, nd, ns = (int(v) for v in counts)

        def ints(k, n, width):
            if n == 0:
                return np.zeros((0, width), dtype=np.int32)
            return np.ctypeslib.as_array(atom_ptrs[k], shape=(n * width,)).copy().reshape(n, width)

        def reals(k, n):
            return np.ctypeslib.as_array(par_ptrs[k], shape=(n,)).copy() if n else np.zeros(0)
        return dict(bonds=ints(0, nb, 2), bond_k=reals(0, nb), bond_r0=reals(1, nb),
                    angles=ints(1, na, 3), angle_k=reals(2, na), angle_theta0=reals(3, na),
                    torsions=ints(2, nt, 4), torsion_k=reals(4, nt), torsion_phi0=reals(5, nt),
                    torsion_n=(np.ctypeslib.as_array(mult, shape=(nt,)).copy() if nt else np.zeros(0, np.int32)),
                    n_dihedrals=nd, specials=ints(3, ns, 2), special_sigma=reals(6, ns), special_epsilon=reals(7, ns),
                    special_lj_scale=reals(8, ns), special_coulomb_scale=reals(9, ns))

    def init_velocities(self, temperature, seed):
        _check(lib().dsmd_input_system_velocities(self.h, c_double(temperature), c_uint64(seed)))

    def read_restart(self, path):
        step, dt, xi = c_int64(), c_double(), c_double()
        box = (c_double * 3)()
        name = ctypes.create_string_buffer(64)
        _check(lib().dsmd_input_restart_read(str(path).encode(), self.h, byref(step), box, byref(dt), name, byref(xi)))
        return dict(step=step.value, timestep=dt.value, box=np.array(list(box)), thermostat=name.value.decode(), xi=xi.value)

    def close(self):
        if self.h:
            lib().dsmd_input_system_destroy(self.h)
            self.h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def write_restart(path, step, timestep, box, periodic, thermostat, thermostat_state, pos, vel):
    pos = np.ascontiguousarray(pos, dtype=np.float64)
    vel = np.ascontiguousarray(vel, dtype=np.float64)
    cols = [np.ascontiguousarray(a) for a in (pos[:, 0], pos[:, 1], pos[:, 2], vel[:, 0], vel[:, 1], vel[:, 2])]
    state = np.ascontiguousarray(thermostat_state, dtype=np.float64)
    ptr = lambda a: a.ctypes.data_as(POINTER(c_double))
    _check(lib().dsmd_input_restart_write(str(path).encode(), c_int64(step), c_double(timestep), (c_double * 3)(*box),
                                          (c_int32 * 3)(*[int(bool(p)) for p in periodic]), thermostat.encode(),
                                          ptr(state) if len(state) else None, c_int32(len(state)), c_int64(len(pos)),
                                          *[ptr(c) for c in cols]))


def nose_hoover_scale(kinetic_kcal, atoms, target_temperature, tau, dt, xi, dof_fraction=1.0):
    """Returns (scale, new xi)."""
    x, s = c_double(xi), c_double()
    _check(lib().dsmd_input_nose_hoover_scale(c_double(kinetic_kcal), c_int64(atoms), c_double(target_temperature),
                                              c_double(tau), c_double(dt), c_double(dof_fraction), byref(x), byref(s)))
    return s.value, x.value


# ---- host logic of the multi-GPU domain code (no GPU needed) ----------------------------------------------------------

BINS = 29          # counts a rank publishes: stays, 26 directions, lost atoms, room


def brick_plan(dims, rank):
    """Neighbour directions (destination rank of each, ordered by destination), distinct neighbour ranks and how many of
    each neighbour's directions point back at `rank`."""
    d = (ctypes.c_int32 * 3)(*[int(v) for v in dims])
    n_dirs, n_peers = ctypes.c_int32(0), ctypes.c_int32(0)
    dest, peers, back = (ctypes.c_int32 * 26)(), (ctypes.c_int32 * 26)(), (ctypes.c_int32 * 26)()
    _check(lib().dsmd_host_brick_plan(d, ctypes.c_int32(rank), ctypes.byref(n_dirs), dest, ctypes.byref(n_peers), peers, back))
    return dict(dir_dest=[dest[k] for k in range(n_dirs.value)], peers=[peers[k] for k in range(n_peers.value)],
                from_count=[back[k] for k in range(n_peers.value)])


def counts_verdict(dims, counts, scratch_capacity=1 << 30):
    """The status every rank derives from the gathered counts ([world, 29] int32) and the messages each rank posts."""
    d = (ctypes.c_int32 * 3)(*[int(v) for v in dims])
    world = int(np.prod(dims))
    c = np.ascontiguousarray(counts, dtype=np.int32).reshape(world, BINS)
    code, about = ctypes.c_int32(0), ctypes.c_int32(-1)
    messages = (ctypes.c_int32 * 64)()
    _check(lib().dsmd_host_counts_verdict(d, c.ctypes.data_as(ctypes.c_void_p), c_int64(scratch_capacity), ctypes.byref(code),
                                          ctypes.byref(about), messages))
    return dict(code=code.value, rank=about.value, text=lib().dsmd_input_last_error().decode(),
                messages=[messages[r] for r in range(min(world, 64))])


def wait_probe(limit_s, ready_after=-1, fail_after=-1):
    return lib().dsmd_host_wait_probe(c_double(limit_s), c_int64(ready_after), c_int64(fail_after))


def dart_throw(n, box, min_dist, seed):
    """[n, 3] points drawn uniformly in a periodic cube, each at least min_dist from all earlier ones (seeded)."""
    out = np.zeros((int(n), 3), dtype=np.float64)
    _check(lib().dsmd_host_dart_throw(c_int64(int(n)), c_double(box), c_double(min_dist), ctypes.c_uint64(int(seed)),
                                      out.ctypes.data_as(ctypes.c_void_p), None))
    return out


def ewald_table(alpha, cutoff):
    """[intervals, 2, 4] float32: force and energy cubic of every interval of the table the pair kernel evaluates."""
    n = lib().dsmd_host_ewald_table(c_double(alpha), c_double(cutoff * cutoff), None, ctypes.c_int32(0))
    out = np.zeros((n, 2, 4), dtype=np.float32)
    lib().dsmd_host_ewald_table(c_double(alpha), c_double(cutoff * cutoff), out.ctypes.data_as(ctypes.c_void_p), ctypes.c_int32(n))
    return out

