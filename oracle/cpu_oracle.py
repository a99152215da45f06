"""ctypes front end of the CPU oracle. TEST INFRASTRUCTURE ONLY.

Two libraries sit behind it:

* ``libdsmd_oracle.so`` - this repository's fp64 restatement (``dsmd_oracle.cpp``), always available after ``make``;
* ``_ref/libdsmd_ref*.so`` - the reference's own CPU sources compiled in place (``ref_build/``), available where the
  reference tree was present at build time (the built file travels with the repository snapshot).

Only the test-suite, the smoke check and the benchmark's CPU-baseline legs may import this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_dp = ctypes.POINTER(ctypes.c_double)
_ip = ctypes.POINTER(ctypes.c_int)


def _ptr(a, ctype):
    if a is None:
        return None
    return a.ctypes.data_as(ctypes.POINTER(ctype))


def _f64(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float64)


def _i32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.int32)


def build(quiet: bool = True) -> None:
    """Compile the oracle (and the reference build when the reference tree is present)."""
    subprocess.run(["make", "-C", _HERE, "all"], check=True,
                   stdout=subprocess.DEVNULL if quiet else None)


_oracle = None


def lib():
    global _oracle
    if _oracle is None:
        path = os.path.join(_HERE, "libdsmd_oracle.so")
        if not os.path.exists(path):
            build()
        L = ctypes.CDLL(path)
        L.dsmd_oracle_pairs.restype = ctypes.c_long
        L.dsmd_oracle_edges.restype = ctypes.c_long
        L.dsmd_oracle_images.restype = ctypes.c_long
        L.dsmd_oracle_ghosts.restype = ctypes.c_long
        L.dsmd_oracle_ewald_alpha.restype = ctypes.c_double
        L.dsmd_oracle_ewald_alpha.argtypes = [ctypes.c_double]
        _oracle = L
    return _oracle


def threads() -> int:
    return lib().dsmd_oracle_threads()


# ---------------------------------------------------------------------------------------------------------------------
# restatement
# ---------------------------------------------------------------------------------------------------------------------

def pairs(x, y, z, n_local, box, periodic=(1, 1, 1), split=(0, 0, 0), search=None):
    """Half pair list (i owned, j) with r < search, as an [P, 2] int32 array sorted by (i, j)."""
    x, y, z = _f64(x), _f64(y), _f64(z)
    n = len(x)
    Lv = _f64(box)
    per = _i32(periodic)
    spl = _i32(split)
    args = (ctypes.c_long(n), ctypes.c_long(n_local), _ptr(x, ctypes.c_double), _ptr(y, ctypes.c_double),
            _ptr(z, ctypes.c_double), _ptr(Lv, ctypes.c_double), _ptr(per, ctypes.c_int), _ptr(spl, ctypes.c_int),
            ctypes.c_double(search))
    count = lib().dsmd_oracle_pairs(*args, None, None, ctypes.c_long(0))
    pi = np.zeros(count, dtype=np.int32)
    pj = np.zeros(count, dtype=np.int32)
    lib().dsmd_oracle_pairs(*args, _ptr(pi, ctypes.c_int), _ptr(pj, ctypes.c_int), ctypes.c_long(count))
    return np.stack([pi, pj], axis=1)


def ewald_alpha(cutoff: float) -> float:
    return lib().dsmd_oracle_ewald_alpha(cutoff)


def lj_tables(eps, sig):
    """c6 = 4 eps sig^6, c12 = c6 sig^6 for full [nt, nt] matrices."""
    eps = np.asarray(eps, dtype=np.float64)
    sig = np.asarray(sig, dtype=np.float64)
    s6 = (sig * sig) ** 3
    c6 = 4.0 * eps * s6
    return c6, 4.0 * eps * s6 * s6


def exclusion_keys(pairs_gid):
    if pairs_gid is None or len(pairs_gid) == 0:
        return np.zeros(0, dtype=np.uint64)
    p = np.asarray(pairs_gid, dtype=np.uint64)
    lo = np.minimum(p[:, 0], p[:, 1])
    hi = np.maximum(p[:, 0], p[:, 1])
    return np.unique((lo << np.uint64(32)) | hi)


def forces(x, y, z, n_local, box, pair_list, c6, c12, rc, *, charge=None, types=None, gid=None, periodic=(1, 1, 1),
           split=(0, 0, 0), switch=-1.0, do_lj=True, do_coulomb=False, alpha=0.0, ewald_mode=1, exclusions=None):
    """Forces on the owned atoms and {pe, virial, virial_diag, pairs_in_cutoff} for the listed pairs."""
    x, y, z = _f64(x), _f64(y), _f64(z)
    n = len(x)
    c6 = _f64(np.atleast_2d(c6))
    c12 = _f64(np.atleast_2d(c12))
    nt = c6.shape[0]
    q = _f64(charge if charge is not None else np.zeros(n))
    t = _i32(types if types is not None else np.zeros(n, dtype=np.int32))
    g = _i32(gid if gid is not None else np.arange(n, dtype=np.int32))
    keys = np.ascontiguousarray(exclusion_keys(exclusions))
    pl = np.ascontiguousarray(pair_list, dtype=np.int32)
    pi = np.ascontiguousarray(pl[:, 0])
    pj = np.ascontiguousarray(pl[:, 1])
    fx = np.zeros(n_local)
    fy = np.zeros(n_local)
    fz = np.zeros(n_local)
    sc = np.zeros(6)
    Lv, per, spl = _f64(box), _i32(periodic), _i32(split)
    lib().dsmd_oracle_forces(
        ctypes.c_long(n), ctypes.c_long(n_local), _ptr(x, ctypes.c_double), _ptr(y, ctypes.c_double),
        _ptr(z, ctypes.c_double), _ptr(q, ctypes.c_double), _ptr(t, ctypes.c_int), _ptr(g, ctypes.c_int),
        _ptr(Lv, ctypes.c_double), _ptr(per, ctypes.c_int), _ptr(spl, ctypes.c_int), ctypes.c_long(len(pi)),
        _ptr(pi, ctypes.c_int), _ptr(pj, ctypes.c_int), ctypes.c_int(nt), _ptr(c6, ctypes.c_double),
        _ptr(c12, ctypes.c_double), ctypes.c_double(rc), ctypes.c_double(switch), ctypes.c_int(int(do_lj)),
        ctypes.c_int(int(do_coulomb)), ctypes.c_double(alpha), ctypes.c_int(ewald_mode), ctypes.c_long(len(keys)),
        _ptr(keys, ctypes.c_uint64), _ptr(fx, ctypes.c_double), _ptr(fy, ctypes.c_double), _ptr(fz, ctypes.c_double),
        _ptr(sc, ctypes.c_double))
    return np.stack([fx, fy, fz], axis=1), dict(pe=sc[0], virial=sc[1], virial_diag=sc[2:5].copy(),
                                                pairs_in_cutoff=int(sc[5]))


def cubic_table(alpha, cutoff_sq):
    n = lib().dsmd_oracle_cubic_table(ctypes.c_double(alpha), ctypes.c_double(cutoff_sq), None, None)
    fc = np.zeros(4 * n, dtype=np.float32)
    ec = np.zeros(4 * n, dtype=np.float32)
    lib().dsmd_oracle_cubic_table(ctypes.c_double(alpha), ctypes.c_double(cutoff_sq), _ptr(fc, ctypes.c_float),
                                  _ptr(ec, ctypes.c_float))
    return fc.reshape(n, 4), ec.reshape(n, 4)


def cubic_eval(coef, r2):
    v = ctypes.c_float(0.0)
    c = np.ascontiguousarray(coef, dtype=np.float32)
    ok = lib().dsmd_oracle_cubic_eval(_ptr(c, ctypes.c_float), ctypes.c_int(c.shape[0]), ctypes.c_float(r2),
                                      ctypes.byref(v))
    return v.value if ok else None


def edges(x, y, z, cutoff, *, n_centers=None, owner=None, shift=None, receiver_ok=None, row=1):
    """Directed edges as (index [2, E] int64, shift [E, 3] float64), ordered by (centre, found atom)."""
    x, y, z = _f64(x), _f64(y), _f64(z)
    n = len(x)
    nc = n if n_centers is None else n_centers
    own = _i32(owner)
    sx = sy = sz = None
    if shift is not None:
        shift = np.asarray(shift, dtype=np.float64)
        sx, sy, sz = (_f64(shift[:, k]) for k in range(3))
    ok = None if receiver_ok is None else np.ascontiguousarray(receiver_ok, dtype=np.uint8)

    def call(oi, oj, osh, cap):
        return lib().dsmd_oracle_edges(
            ctypes.c_long(n), _ptr(x, ctypes.c_double), _ptr(y, ctypes.c_double), _ptr(z, ctypes.c_double),
            ctypes.c_double(cutoff), ctypes.c_long(nc), _ptr(own, ctypes.c_int), _ptr(sx, ctypes.c_double),
            _ptr(sy, ctypes.c_double), _ptr(sz, ctypes.c_double), _ptr(ok, ctypes.c_ubyte), ctypes.c_int(row),
            _ptr(oi, ctypes.c_longlong), _ptr(oj, ctypes.c_longlong), _ptr(osh, ctypes.c_double), ctypes.c_long(cap))

    count = call(None, None, None, 0)
    oi = np.zeros(count, dtype=np.int64)
    oj = np.zeros(count, dtype=np.int64)
    osh = np.zeros((count, 3), dtype=np.float64)
    call(oi, oj, osh, count)
    return np.stack([oi, oj]), osh


def images(x, y, z, box, origin, region_lo, region_hi, shells):
    x, y, z = _f64(x), _f64(y), _f64(z)
    n = len(x)
    b, o, rl, rh, sh = _f64(box), _f64(origin), _f64(region_lo), _f64(region_hi), _i32(shells)

    def call(arrs, cap):
        ptrs = [None] * 7 if arrs is None else [
            _ptr(arrs[0], ctypes.c_double), _ptr(arrs[1], ctypes.c_double), _ptr(arrs[2], ctypes.c_double),
            _ptr(arrs[3], ctypes.c_int), _ptr(arrs[4], ctypes.c_double), _ptr(arrs[5], ctypes.c_double),
            _ptr(arrs[6], ctypes.c_double)]
        return lib().dsmd_oracle_images(
            ctypes.c_long(n), _ptr(x, ctypes.c_double), _ptr(y, ctypes.c_double), _ptr(z, ctypes.c_double),
            _ptr(b, ctypes.c_double), _ptr(o, ctypes.c_double), _ptr(rl, ctypes.c_double), _ptr(rh, ctypes.c_double),
            _ptr(sh, ctypes.c_int), *ptrs, ctypes.c_long(cap))

    total = call(None, 0)
    arrs = [np.zeros(total), np.zeros(total), np.zeros(total), np.zeros(total, dtype=np.int32), np.zeros(total),
            np.zeros(total), np.zeros(total)]
    call(arrs, total)
    return dict(x=arrs[0], y=arrs[1], z=arrs[2], owner=arrs[3], shift=np.stack(arrs[4:7], axis=1))


def fold_image_forces(f, n, owner, target, n_out=None, with_images=True):
    """target[:n_out] += f[:n_out] + the forces on each atom's images (slots n..; owner[slot] = the atom copied), added in
    slot order. f: [n_all, 3]; owner: [n_all]; target: [n, 3]. Returns the new target."""
    f = np.ascontiguousarray(f, dtype=np.float64)
    n_out = n if n_out is None else n_out
    own = np.asarray(owner[n:], dtype=np.int64)
    count = np.bincount(own, minlength=n).astype(np.int64)
    first = np.concatenate([[0], np.cumsum(count)[:-1]]).astype(np.int64)
    assert np.array_equal(own, np.repeat(np.arange(n), count)), "images must be stored atom after atom"
    cols = [np.ascontiguousarray(f[:, k]) for k in range(3)]
    out = [np.ascontiguousarray(target[:, k], dtype=np.float64).copy() for k in range(3)]
    cl = ctypes.POINTER(ctypes.c_long)
    lib().dsmd_oracle_fold_image_forces(
        ctypes.c_long(n_out), ctypes.c_long(n), *[_ptr(c, ctypes.c_double) for c in cols],
        first.ctypes.data_as(cl), count.ctypes.data_as(cl) if with_images else None,
        *[_ptr(o, ctypes.c_double) for o in out])
    return np.stack(out, axis=1)


def virial_from_forces(pos, f):
    """{sum r.F, sum x Fx, sum y Fy, sum z Fz} over all rows of pos / f ([n, 3] each)."""
    p = [np.ascontiguousarray(pos[:, k], dtype=np.float64) for k in range(3)]
    g = [np.ascontiguousarray(f[:, k], dtype=np.float64) for k in range(3)]
    out = np.zeros(4)
    lib().dsmd_oracle_virial_from_forces(ctypes.c_long(len(p[0])), *[_ptr(a, ctypes.c_double) for a in p + g],
                                         _ptr(out, ctypes.c_double))
    return out


def _i64(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.int64)


class BondedTerms:
    """Plain arrays of the bonded terms of a system: bonds [nb, 2] + k, r0; angles [na, 3] + k, theta0 (radians);
    torsions [nt, 4] + k, phi0 (radians), n (dihedrals first, impropers behind: n_dihedrals tells where they start);
    specials [ns, 2] + sigma, epsilon, lj_scale, coulomb_scale. Atom numbers are indices into the arrays handed to the
    evaluation (for the device library: global ids)."""

    def __init__(self, bonds=None, bond_k=None, bond_r0=None, angles=None, angle_k=None, angle_theta0=None, torsions=None,
                 torsion_k=None, torsion_phi0=None, torsion_n=None, n_dihedrals=None, specials=None, special_sigma=None,
                 special_epsilon=None, special_lj_scale=None, special_coulomb_scale=None):
        def table(a, width):
            return np.zeros((0, width), dtype=np.int64) if a is None else _i64(np.asarray(a).reshape(-1, width))

        def column(a, n, dtype=np.float64):
            return np.zeros(n, dtype=dtype) if a is None else np.ascontiguousarray(a, dtype=dtype)
        self.bonds = table(bonds, 2)
        self.bond_k, self.bond_r0 = column(bond_k, len(self.bonds)), column(bond_r0, len(self.bonds))
        self.angles = table(angles, 3)
        self.angle_k, self.angle_theta0 = column(angle_k, len(self.angles)), column(angle_theta0, len(self.angles))
        self.torsions = table(torsions, 4)
        self.torsion_k, self.torsion_phi0 = column(torsion_k, len(self.torsions)), column(torsion_phi0, len(self.torsions))
        self.torsion_n = column(torsion_n, len(self.torsions), np.int32)
        self.n_dihedrals = len(self.torsions) if n_dihedrals is None else int(n_dihedrals)
        self.specials = table(specials, 2)
        ns = len(self.specials)
        self.special_sigma, self.special_epsilon = column(special_sigma, ns), column(special_epsilon, ns)
        self.special_lj_scale, self.special_coulomb_scale = column(special_lj_scale, ns), column(special_coulomb_scale, ns)


def bonded(pos, n_local, box, terms, *, periodic=(1, 1, 1), gid=None, charge=None):
    """Forces [n_local, 3] of the bonded terms and scaled special pairs on the owned atoms, and {pe, virial, virial_diag}:
    the restatement of the reference's bond / angle / torsion / special-pair routines with the ownership rule of its
    GPU kernels (a term with no owned atom is skipped; energy where the lowest global id is owned)."""
    x, y, z = (_f64(pos[:, k]) for k in range(3))
    f = [np.zeros(len(x)) for _ in range(3)]
    out = np.zeros(5)
    Lv, per, g, q = _f64(box), _i32(periodic), _i32(gid), _f64(charge)
    t = terms
    lib().dsmd_oracle_bonded(
        ctypes.c_long(n_local), _ptr(x, ctypes.c_double), _ptr(y, ctypes.c_double), _ptr(z, ctypes.c_double),
        _ptr(g, ctypes.c_int), _ptr(Lv, ctypes.c_double), _ptr(per, ctypes.c_int),
        ctypes.c_long(len(t.bonds)), _ptr(t.bonds, ctypes.c_long), _ptr(t.bond_k, ctypes.c_double), _ptr(t.bond_r0, ctypes.c_double),
        ctypes.c_long(len(t.angles)), _ptr(t.angles, ctypes.c_long), _ptr(t.angle_k, ctypes.c_double),
        _ptr(t.angle_theta0, ctypes.c_double),
        ctypes.c_long(len(t.torsions)), _ptr(t.torsions, ctypes.c_long), _ptr(t.torsion_k, ctypes.c_double),
        _ptr(t.torsion_phi0, ctypes.c_double), _ptr(t.torsion_n, ctypes.c_int),
        ctypes.c_long(len(t.specials)), _ptr(t.specials, ctypes.c_long), _ptr(t.special_sigma, ctypes.c_double),
        _ptr(t.special_epsilon, ctypes.c_double), _ptr(t.special_lj_scale, ctypes.c_double),
        _ptr(t.special_coulomb_scale, ctypes.c_double), _ptr(q, ctypes.c_double),
        *[_ptr(a, ctypes.c_double) for a in f], _ptr(out, ctypes.c_double))
    return np.stack(f, axis=1)[:n_local], dict(pe=out[0], virial=out[1], virial_diag=out[2:5].copy())


def mark_receivers(x, y, z, lo, hi, reach):
    x, y, z = _f64(x), _f64(y), _f64(z)
    ok = np.zeros(len(x), dtype=np.uint8)
    lo, hi = _f64(lo), _f64(hi)
    lib().dsmd_oracle_mark_receivers(ctypes.c_long(len(x)), _ptr(x, ctypes.c_double), _ptr(y, ctypes.c_double),
                                     _ptr(z, ctypes.c_double), _ptr(lo, ctypes.c_double), _ptr(hi, ctypes.c_double),
                                     ctypes.c_double(reach), _ptr(ok, ctypes.c_ubyte))
    return ok


def ghosts(x, y, z, box, periodic, dims, coords, halo):
    """(source index [G], image shift [G, 3]) of the ghost atoms of brick `coords` in a `dims` grid."""
    x, y, z = _f64(x), _f64(y), _f64(z)
    n = len(x)
    Lv, per, dm, co = _f64(box), _i32(periodic), _i32(dims), _i32(coords)

    def call(src, img, cap):
        return lib().dsmd_oracle_ghosts(
            ctypes.c_long(n), _ptr(x, ctypes.c_double), _ptr(y, ctypes.c_double), _ptr(z, ctypes.c_double),
            _ptr(Lv, ctypes.c_double), _ptr(per, ctypes.c_int), _ptr(dm, ctypes.c_int), _ptr(co, ctypes.c_int),
            ctypes.c_double(halo), _ptr(src, ctypes.c_int), _ptr(img, ctypes.c_int), ctypes.c_long(cap))

    count = call(None, None, 0)
    src = np.zeros(count, dtype=np.int32)
    img = np.zeros((count, 3), dtype=np.int32)
    call(src, img, count)
    return src, img


def vv_half(first_half, dt, force_to_accel, pos, vel, frc, mass):
    """In-place velocity-Verlet half step on [N, 3] arrays given as three contiguous columns each."""
    n = len(mass)
    lib().dsmd_oracle_vv_half(
        ctypes.c_long(n), ctypes.c_double(dt), ctypes.c_double(force_to_accel), ctypes.c_int(int(first_half)),
        *[_ptr(a, ctypes.c_double) for a in pos], *[_ptr(a, ctypes.c_double) for a in vel],
        *[_ptr(a, ctypes.c_double) for a in frc], _ptr(mass, ctypes.c_double))


def _constraint_arrays(constraints):
    a = np.ascontiguousarray([c[0] for c in constraints], dtype=np.int64)
    b = np.ascontiguousarray([c[1] for c in constraints], dtype=np.int64)
    d = np.ascontiguousarray([c[2] for c in constraints], dtype=np.float64)
    return a, b, d


def shake(constraints, pos, vel, mass, pre, box, dt, periodic=(1, 1, 1), max_iterations=500, tolerance=1e-8):
    """SHAKE in place on pos / vel (three contiguous columns each); pre = the positions before the drift. Returns True
    when converged."""
    a, b, d = _constraint_arrays(constraints)
    rc = lib().dsmd_oracle_shake(
        ctypes.c_long(len(a)), _ptr(a, ctypes.c_long), _ptr(b, ctypes.c_long), _ptr(d, ctypes.c_double),
        *[_ptr(c, ctypes.c_double) for c in pos], *[_ptr(c, ctypes.c_double) for c in vel], _ptr(_f64(mass), ctypes.c_double),
        *[_ptr(c, ctypes.c_double) for c in pre], _ptr(_f64(box), ctypes.c_double), _ptr(_i32(periodic), ctypes.c_int),
        ctypes.c_double(dt), ctypes.c_int(max_iterations), ctypes.c_double(tolerance))
    return bool(rc)


def rattle(constraints, pos, vel, mass, box, dt, force_to_accel, periodic=(1, 1, 1), gid=None, n_local=None,
           max_iterations=500, tolerance=1e-8):
    """RATTLE in place on vel. Returns (converged, diagonal of the constraint virial)."""
    a, b, _ = _constraint_arrays(constraints)
    n = len(mass)
    virial = np.zeros(3)
    g = None if gid is None else _i32(gid)
    rc = lib().dsmd_oracle_rattle(
        ctypes.c_long(len(a)), _ptr(a, ctypes.c_long), _ptr(b, ctypes.c_long), *[_ptr(c, ctypes.c_double) for c in pos],
        *[_ptr(c, ctypes.c_double) for c in vel], _ptr(_f64(mass), ctypes.c_double),
        _ptr(g, ctypes.c_int) if g is not None else None, ctypes.c_long(n if n_local is None else n_local),
        _ptr(_f64(box), ctypes.c_double), _ptr(_i32(periodic), ctypes.c_int), ctypes.c_double(dt),
        ctypes.c_double(force_to_accel), ctypes.c_int(max_iterations), ctypes.c_double(tolerance),
        _ptr(virial, ctypes.c_double))
    return bool(rc), virial


def ref_constrain(which, constraints, pos, vel, mass, box, dt, pre=None, periodic=(1, 1, 1), max_iterations=500,
                  tolerance=1e-8):
    """The REFERENCE's ConstraintSolver (src/constraint_solver.cpp, compiled in place) on the same arrays, in place.
    which = "shake" or "rattle". Returns (converged, virial diagonal)."""
    a, b, d = _constraint_arrays(constraints)
    n = len(mass)
    virial = np.zeros(3)
    pre = pos if pre is None else pre
    L = ref_lib()
    rc = L.dsmd_ref_constrain(
        ctypes.c_int(0 if which == "shake" else 1), ctypes.c_long(n), ctypes.c_long(n), *[_ptr(c, ctypes.c_double) for c in pos],
        *[_ptr(c, ctypes.c_double) for c in vel], _ptr(_f64(mass), ctypes.c_double), None, _ptr(_f64(box), ctypes.c_double),
        _ptr(_i32(periodic), ctypes.c_int), ctypes.c_long(len(a)), _ptr(a, ctypes.c_long), _ptr(b, ctypes.c_long),
        _ptr(d, ctypes.c_double), ctypes.c_double(dt), *[_ptr(c, ctypes.c_double) for c in pre], ctypes.c_int(max_iterations),
        ctypes.c_double(tolerance), _ptr(virial, ctypes.c_double))
    return bool(rc), virial


# ---------------------------------------------------------------------------------------------------------------------
# brute force (pure numpy, O(N^2): small cases only)
# ---------------------------------------------------------------------------------------------------------------------

def brute_pairs(pos, box, search):
    pos = np.asarray(pos, dtype=np.float64)
    d = pos[:, None, :] - pos[None, :, :]
    d -= np.asarray(box) * np.round(d / np.asarray(box))
    r2 = (d * d).sum(-1)
    iu = np.triu_indices(len(pos), 1)
    m = r2[iu] < search * search
    return np.stack([iu[0][m], iu[1][m]], axis=1).astype(np.int32)


def brute_edges(pos, cutoff):
    pos = np.asarray(pos, dtype=np.float64)
    d = pos[None, :, :] - pos[:, None, :]
    r2 = (d * d).sum(-1)
    m = r2 < cutoff * cutoff
    np.fill_diagonal(m, False)
    i, j = np.nonzero(m)
    return np.stack([i, j]).astype(np.int64)


# ---------------------------------------------------------------------------------------------------------------------
# the reference's own CPU code (oracle/_ref)
# ---------------------------------------------------------------------------------------------------------------------

def _cpu_has_avx512() -> bool:
    try:
        with open("/proc/cpuinfo") as fh:
            for line in fh:
                if line.startswith("flags"):
                    flags = line.split()
                    return all(f in flags for f in ("avx512f", "avx512dq", "avx512vl", "avx512bw", "avx512cd"))
    except OSError:
        pass
    return False


_ref = None


def ref_available() -> bool:
    return os.path.exists(os.path.join(_HERE, "_ref", "libdsmd_ref.so"))


def ref_lib():
    global _ref
    if _ref is None:
        name = "libdsmd_ref_avx512.so" if _cpu_has_avx512() else "libdsmd_ref.so"
        path = os.path.join(_HERE, "_ref", name)
        if not os.path.exists(path):
            path = os.path.join(_HERE, "_ref", "libdsmd_ref.so")
        L = ctypes.CDLL(path)
        L.dsmd_ref_create.restype = ctypes.c_void_p
        L.dsmd_ref_build_list.restype = ctypes.c_long
        L.dsmd_ref_list_pairs.restype = ctypes.c_long
        L.dsmd_ref_pairs_inside_list.restype = ctypes.c_ulonglong
        L.dsmd_ref_pairs_inside_cutoff.restype = ctypes.c_ulonglong
        _ref = L
    return _ref


class RefCase:
    """One system held by the reference's CPU code (SpatialVerletList + ForceCalculatorCPU)."""

    def __init__(self, x, y, z, n_local, box, cutoff, skin, *, periodic=(1, 1, 1), lo=(0, 0, 0), hi=(0, 0, 0),
                 charge=None, types=None, gid=None, eps=((1.0,),), sig=((1.0,),), switch=-1.0, exclusions=None,
                 n_global=None):
        L = ref_lib()
        self.L = L
        self.h = ctypes.c_void_p(L.dsmd_ref_create())
        self.n = len(x)
        self.n_local = n_local
        x, y, z = _f64(x), _f64(y), _f64(z)
        Lv, per, lo, hi = _f64(box), _i32(periodic), _f64(lo), _f64(hi)
        L.dsmd_ref_set_box(self.h, _ptr(Lv, ctypes.c_double), _ptr(per, ctypes.c_int), _ptr(lo, ctypes.c_double),
                           _ptr(hi, ctypes.c_double))
        q, t, g = _f64(charge), _i32(types), _i32(gid)
        L.dsmd_ref_set_particles(self.h, ctypes.c_long(self.n), ctypes.c_long(n_local), _ptr(x, ctypes.c_double),
                                 _ptr(y, ctypes.c_double), _ptr(z, ctypes.c_double), _ptr(q, ctypes.c_double),
                                 _ptr(t, ctypes.c_int), _ptr(g, ctypes.c_int))
        eps = _f64(np.atleast_2d(eps))
        sig = _f64(np.atleast_2d(sig))
        L.dsmd_ref_set_force_field(self.h, ctypes.c_int(eps.shape[0]), _ptr(eps, ctypes.c_double),
                                   _ptr(sig, ctypes.c_double), ctypes.c_double(switch))
        if exclusions is not None and len(exclusions):
            e = np.asarray(exclusions, dtype=np.int32)
            a, b = _i32(e[:, 0]), _i32(e[:, 1])
            ng = n_global if n_global is not None else (int(np.max(g)) + 1 if g is not None else self.n)
            L.dsmd_ref_set_exclusions(self.h, ctypes.c_int(ng), ctypes.c_long(len(a)), _ptr(a, ctypes.c_int),
                                      _ptr(b, ctypes.c_int))
        L.dsmd_ref_set_cutoff(self.h, ctypes.c_double(cutoff), ctypes.c_double(skin))

    def threads(self):
        return self.L.dsmd_ref_threads()

    def simd_width(self):
        return self.L.dsmd_ref_simd_width()

    def build_list(self):
        return self.L.dsmd_ref_build_list(self.h)

    def update_positions(self, x, y, z):
        x, y, z = _f64(x), _f64(y), _f64(z)
        self.L.dsmd_ref_update_positions(self.h, _ptr(x, ctypes.c_double), _ptr(y, ctypes.c_double),
                                         _ptr(z, ctypes.c_double))

    def needs_rebuild(self):
        return bool(self.L.dsmd_ref_needs_rebuild(self.h))

    def pair_counts(self):
        return int(self.L.dsmd_ref_pairs_inside_list(self.h)), int(self.L.dsmd_ref_pairs_inside_cutoff(self.h))

    def list_pairs(self):
        count = self.L.dsmd_ref_list_pairs(self.h, None, None, ctypes.c_long(0))
        pi = np.zeros(count, dtype=np.int32)
        pj = np.zeros(count, dtype=np.int32)
        self.L.dsmd_ref_list_pairs(self.h, _ptr(pi, ctypes.c_int), _ptr(pj, ctypes.c_int), ctypes.c_long(count))
        return np.stack([pi, pj], axis=1)

    def compute(self, *, do_lj=True, do_coulomb=False, tensor=True, mixed=False):
        fx, fy, fz = np.zeros(self.n_local), np.zeros(self.n_local), np.zeros(self.n_local)
        sc = np.zeros(7)
        rc = self.L.dsmd_ref_compute_forces(self.h, int(do_lj), int(do_coulomb), int(tensor), int(mixed),
                                            _ptr(fx, ctypes.c_double), _ptr(fy, ctypes.c_double),
                                            _ptr(fz, ctypes.c_double), _ptr(sc, ctypes.c_double))
        if rc != 0:
            raise RuntimeError("reference compute_forces failed")
        return np.stack([fx, fy, fz], axis=1), dict(pe=sc[0], virial=sc[1], virial_diag=sc[2:5].copy(), alpha=sc[5],
                                                    self_energy=sc[6], pe_real=sc[0] - sc[6])

    def bonded(self, terms, *, do_lj=True, do_coulomb=True):
        """The reference's own bond / angle / dihedral / improper / special-pair routines on this case's atoms."""
        fx, fy, fz = np.zeros(self.n_local), np.zeros(self.n_local), np.zeros(self.n_local)
        sc = np.zeros(5)
        t = terms
        rc = self.L.dsmd_ref_bonded(
            self.h, ctypes.c_long(len(t.bonds)), _ptr(t.bonds, ctypes.c_long), _ptr(t.bond_k, ctypes.c_double),
            _ptr(t.bond_r0, ctypes.c_double), ctypes.c_long(len(t.angles)), _ptr(t.angles, ctypes.c_long),
            _ptr(t.angle_k, ctypes.c_double), _ptr(t.angle_theta0, ctypes.c_double), ctypes.c_long(len(t.torsions)),
            ctypes.c_long(t.n_dihedrals), _ptr(t.torsions, ctypes.c_long), _ptr(t.torsion_k, ctypes.c_double),
            _ptr(t.torsion_phi0, ctypes.c_double), _ptr(t.torsion_n, ctypes.c_int), ctypes.c_long(len(t.specials)),
            _ptr(t.specials, ctypes.c_long), _ptr(t.special_sigma, ctypes.c_double), _ptr(t.special_epsilon, ctypes.c_double),
            _ptr(t.special_lj_scale, ctypes.c_double), _ptr(t.special_coulomb_scale, ctypes.c_double), int(do_lj),
            int(do_coulomb), _ptr(fx, ctypes.c_double), _ptr(fy, ctypes.c_double), _ptr(fz, ctypes.c_double),
            _ptr(sc, ctypes.c_double))
        if rc != 0:
            raise RuntimeError("reference bonded routines failed")
        return np.stack([fx, fy, fz], axis=1), dict(pe=sc[0], virial=sc[1], virial_diag=sc[2:5].copy())

    def close(self):
        if self.h:
            self.L.dsmd_ref_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def canonical_pairs(p):
    """Unordered pairs as a sorted [P, 2] array (min, max)."""
    p = np.asarray(p)
    lo = np.minimum(p[:, 0], p[:, 1])
    hi = np.maximum(p[:, 0], p[:, 1])
    key = np.lexsort((hi, lo))
    return np.stack([lo[key], hi[key]], axis=1)
