"""Seeded synthetic systems with the shapes, sizes and value distributions of the benchmark configurations.

Everything is generated from a seed with numpy; no external dataset is read. Units: the LJ systems are in reduced units
(sigma = epsilon = mass = 1); the water and radius-graph systems are in Angstrom / kcal/mol / e.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


@dataclass
class System:
    """Host-side description of one input: positions and parameters in the caller's atom order."""
    name: str
    pos: np.ndarray                      # [N, 3] float64
    box: np.ndarray                      # [3]
    types: np.ndarray                    # [N] int32
    charge: np.ndarray                   # [N] float64
    mass: np.ndarray                     # [N] float64
    eps: np.ndarray                      # [nt, nt] pair epsilon
    sig: np.ndarray                      # [nt, nt] pair sigma
    cutoff: float
    skin: float
    vel: np.ndarray | None = None        # [N, 3]
    exclusions: np.ndarray | None = None  # [X, 2] global ids
    constraints: np.ndarray | None = None  # [C, 3] global id, global id, distance
    bonded: dict | None = None           # bonds / angles / torsions / specials with their parameters (chain_fluid)
    coulomb: bool = False
    dt: float = 0.005
    force_to_accel: float = 1.0          # 4.184e-4 in the reference's real units, 1 in reduced units
    meta: dict = field(default_factory=dict)

    @property
    def n(self) -> int:
        return len(self.pos)


def lorentz_berthelot(eps_t, sig_t):
    eps_t = np.asarray(eps_t, dtype=np.float64)
    sig_t = np.asarray(sig_t, dtype=np.float64)
    return np.sqrt(np.outer(eps_t, eps_t)), 0.5 * (sig_t[:, None] + sig_t[None, :])


def maxwell_boltzmann(n, temperature, mass, rng, kb=1.0):
    """Velocities N(0, sqrt(kT/m)), zero net momentum, rescaled to the exact temperature with 3N - 3 degrees of freedom."""
    v = rng.standard_normal((n, 3)) * np.sqrt(kb * temperature / mass)[:, None]
    v -= (v * mass[:, None]).sum(0) / mass.sum()
    ke2 = (mass[:, None] * v * v).sum()
    t_now = ke2 / (kb * (3 * n - 3))
    return v * np.sqrt(temperature / t_now)


def fcc_lj(cells: int, *, density=0.8442, temperature=1.44, jitter=0.05, cutoff=2.5, skin=0.3, seed=12345) -> System:
    """Single-species LJ fluid started from an FCC lattice of cells^3 unit cells (4 atoms each) with a small seeded
    jitter (a perfect lattice has many exactly degenerate distances). cells=20 -> 32,000 atoms, cells=100 -> 4,000,000."""
    rng = np.random.default_rng(seed)
    a = (4.0 / density) ** (1.0 / 3.0)
    g = np.arange(cells, dtype=np.float64)
    cell = np.stack(np.meshgrid(g, g, g, indexing="ij"), axis=-1).reshape(-1, 1, 3)
    basis = np.array([[0.0, 0.0, 0.0], [0.5, 0.5, 0.0], [0.5, 0.0, 0.5], [0.0, 0.5, 0.5]])
    pos = ((cell + basis[None]) * a).reshape(-1, 3) + 0.25 * a
    n = len(pos)
    pos += rng.uniform(-jitter, jitter, pos.shape)
    box = np.full(3, cells * a)
    pos %= box
    mass = np.ones(n)
    vel = maxwell_boltzmann(n, temperature, mass, rng)
    return System(name=f"lj_fcc_{n}", pos=pos, box=box, types=np.zeros(n, dtype=np.int32), charge=np.zeros(n),
                  mass=mass, eps=np.ones((1, 1)), sig=np.ones((1, 1)), cutoff=cutoff, skin=skin, vel=vel,
                  meta=dict(seed=seed, cells=cells, density=density, temperature=temperature))


def kob_andersen(n_target=1_048_576, *, density=1.2, temperature=0.8, cutoff=2.5, skin=0.3, seed=777) -> System:
    """80:20 binary LJ mixture. Atoms sit on a seeded random subset of a jittered simple-cubic lattice (uniformly random
    placement at this density overlaps and gives infinite forces), types are shuffled."""
    rng = np.random.default_rng(seed)
    m = int(np.ceil(n_target ** (1.0 / 3.0)))
    while m ** 3 < n_target:
        m += 1
    L = (n_target / density) ** (1.0 / 3.0)
    a = L / m
    sites = rng.permutation(m ** 3)[:n_target]
    sites.sort()
    ix, iy, iz = np.unravel_index(sites, (m, m, m))
    pos = (np.stack([ix, iy, iz], axis=1) + 0.5) * a
    pos += rng.uniform(-0.12, 0.12, pos.shape)
    box = np.full(3, L)
    pos %= box
    types = np.zeros(n_target, dtype=np.int32)
    types[rng.permutation(n_target)[: n_target // 5]] = 1
    eps = np.array([[1.0, 1.5], [1.5, 0.5]])
    sig = np.array([[1.0, 0.8], [0.8, 0.88]])
    mass = np.ones(n_target)
    vel = maxwell_boltzmann(n_target, temperature, mass, rng)
    return System(name=f"kob_andersen_{n_target}", pos=pos, box=box, types=types, charge=np.zeros(n_target), mass=mass,
                  eps=eps, sig=sig, cutoff=cutoff, skin=skin, vel=vel, meta=dict(seed=seed, density=density))


def _random_rotations(n, rng):
    q = rng.standard_normal((n, 4))
    q /= np.linalg.norm(q, axis=1, keepdims=True)
    w, x, y, z = q.T
    return np.stack([
        np.stack([1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w)], axis=1),
        np.stack([2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w)], axis=1),
        np.stack([2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)], axis=1)], axis=1)


def water_box(cells: int = 60, *, cutoff=10.0, skin=2.0, seed=4242) -> System:
    """Rigid three-site water geometry (O-H 1.0 A, H-O-H 109.47 deg, charges -0.8476 / +0.4238 e) with seeded random
    orientations on a jittered cubic lattice at 1.0 g/cm^3; LJ on O-O only; O-H and H-H of a molecule are excluded.
    cells=60 -> 216,000 molecules, 648,000 atoms. Atom order: O, H, H per molecule."""
    rng = np.random.default_rng(seed)
    spacing = (18.01528 / 6.02214076e23 / 1.0e-24) ** (1.0 / 3.0)   # cube root of the volume per molecule in A^3
    nm = cells ** 3
    g = np.arange(cells, dtype=np.float64)
    centre = (np.stack(np.meshgrid(g, g, g, indexing="ij"), axis=-1).reshape(-1, 3) + 0.5) * spacing
    centre += rng.uniform(-0.3, 0.3, centre.shape)
    half = np.deg2rad(109.47) / 2.0
    local = np.array([[0.0, 0.0, 0.0], [np.sin(half), 0.0, np.cos(half)], [-np.sin(half), 0.0, np.cos(half)]])
    rot = _random_rotations(nm, rng)
    pos = (centre[:, None, :] + np.einsum("mij,aj->mai", rot, local)).reshape(-1, 3)
    box = np.full(3, cells * spacing)
    n = 3 * nm
    types = np.tile(np.array([0, 1, 1], dtype=np.int32), nm)
    charge = np.tile(np.array([-0.8476, 0.4238, 0.4238]), nm)
    mass = np.tile(np.array([15.9994, 1.008, 1.008]), nm)
    eps = np.array([[0.1553, 0.0], [0.0, 0.0]])
    sig = np.array([[3.166, 1.583], [1.583, 0.0]])
    o = 3 * np.arange(nm, dtype=np.int32)
    excl = np.concatenate([np.stack([o, o + 1], 1), np.stack([o, o + 2], 1), np.stack([o + 1, o + 2], 1)])
    kb = 0.0019872041
    vel = maxwell_boltzmann(n, 300.0, mass, rng, kb=kb / (48.88821291 ** 2))
    # the rigid geometry as distance constraints, molecule after molecule: O-H, O-H, H-H
    hh = 2.0 * np.sin(half)
    cons = np.stack([np.stack([o, o + 1, np.full(nm, 1.0)], 1), np.stack([o, o + 2, np.full(nm, 1.0)], 1),
                     np.stack([o + 1, o + 2, np.full(nm, hh)], 1)], axis=1).reshape(-1, 3)
    return System(name=f"water_{n}", pos=pos, box=box, types=types, charge=charge, mass=mass, eps=eps, sig=sig,
                  cutoff=cutoff, skin=skin, vel=vel, exclusions=excl, constraints=cons, coulomb=True, dt=2.0, force_to_accel=4.184e-4,
                  meta=dict(seed=seed, molecules=nm))


def _torsion_angle(p0, p1, p2, p3):
    """The torsion angle the bonded kernels use (atan2 form over the normals of the two planes), for arrays of points."""
    ij, jk, kl = p0 - p1, p1 - p2, p2 - p3
    n1, n2 = np.cross(ij, jk), np.cross(jk, kl)
    jkm = np.linalg.norm(jk, axis=-1)
    return np.arctan2((np.cross(n1, n2) * jk).sum(-1), (n1 * n2).sum(-1) * jkm)


def chain_fluid(cells: int = 6, length: int = 8, *, spacing=9.0, cutoff=9.0, skin=1.5, seed=77) -> System:
    """Flexible chain molecules for the bonded terms: cells^3 chains of `length` united atoms (bond 1.53 A, bend near
    112 degrees, torsions within 35 degrees of trans, so that a chain does not fold onto itself) grown roughly along x
    from the sites of a cubic lattice and wrapped into the periodic box, so that terms cross the box boundary. With the
    default spacing neighbouring chains overlap here and there (fine for force parity with the pair terms switched off);
    spacing >= 14 keeps them apart for dynamics. Two atom types (chain ends and inner atoms), small alternating charges,
    and every kind of bonded term the reference evaluates: harmonic bonds and angles, periodic dihedrals of multiplicity
    1 to 3, harmonic (n = 0) impropers on every other quadruple with a rest angle near the actual one, and 1-4 special
    pairs with scaled Lennard-Jones and Coulomb parts. 1-2, 1-3 and 1-4 pairs are excluded from the nonbonded list."""
    rng = np.random.default_rng(seed)
    nm = cells ** 3
    g = np.arange(cells, dtype=np.float64)
    start = (np.stack(np.meshgrid(g, g, g, indexing="ij"), axis=-1).reshape(-1, 3) + 0.15) * spacing
    start += rng.uniform(-0.5, 0.5, start.shape)
    pos = np.zeros((nm, length, 3))
    bond = 1.53
    for m in range(nm):
        d = np.array([1.0, 0.0, 0.0]) + rng.uniform(-0.25, 0.25, 3)
        d /= np.linalg.norm(d)
        p = [start[m], start[m] + bond * d]
        for k in range(2, length):
            c_, b_ = p[-1], p[-2]
            bc = (c_ - b_) / np.linalg.norm(c_ - b_)
            if k == 2:
                ref = rng.normal(size=3)
            else:
                ref = b_ - p[-3]
            n = np.cross(ref, bc)
            n /= np.linalg.norm(n)
            mvec = np.cross(n, bc)
            theta = np.deg2rad(112.0 + rng.uniform(-10.0, 10.0))
            phi = np.pi + np.deg2rad(rng.uniform(-35.0, 35.0)) if k > 2 else 0.0
            step = -np.cos(theta) * bc + np.sin(theta) * (np.cos(phi) * mvec + np.sin(phi) * n)
            p.append(c_ + bond * step)
        pos[m] = np.array(p)
    box = np.full(3, cells * spacing)
    unwrapped = pos.reshape(-1, 3).copy()
    pos = unwrapped - box * np.floor(unwrapped / box)
    n = nm * length
    first = (np.arange(nm) * length)[:, None]
    k = np.arange(length)
    ids = first + k[None, :]
    types = np.tile(np.where((k == 0) | (k == length - 1), 0, 1).astype(np.int32), nm)
    charge = np.tile(np.where(k % 2 == 0, 0.12, -0.12) * (1.0 if length % 2 == 0 else 0.0), nm)
    mass = np.tile(np.where((k == 0) | (k == length - 1), 15.035, 14.027), nm)
    eps, sig = lorentz_berthelot([0.175, 0.118], [3.905, 3.905])
    bonds = np.stack([ids[:, :-1], ids[:, 1:]], axis=-1).reshape(-1, 2)
    angles = np.stack([ids[:, :-2], ids[:, 1:-1], ids[:, 2:]], axis=-1).reshape(-1, 3)
    quads = np.stack([ids[:, :-3], ids[:, 1:-2], ids[:, 2:-1], ids[:, 3:]], axis=-1).reshape(-1, 4)
    impropers = quads[::2]
    nd, ni = len(quads), len(impropers)
    actual = _torsion_angle(*(unwrapped[impropers[:, q]] for q in range(4)))
    rest = actual + rng.uniform(-0.3, 0.3, ni)
    rest = rest - 2.0 * np.pi * np.round(rest / (2.0 * np.pi))
    bonded = dict(
        bonds=bonds, bond_k=rng.uniform(400.0, 640.0, len(bonds)), bond_r0=rng.uniform(1.50, 1.56, len(bonds)),
        angles=angles, angle_k=rng.uniform(80.0, 130.0, len(angles)),
        angle_theta0=np.deg2rad(rng.uniform(107.0, 117.0, len(angles))),
        torsions=np.concatenate([quads, impropers]),
        torsion_k=np.concatenate([rng.uniform(0.2, 2.5, nd), rng.uniform(5.0, 40.0, ni)]),
        torsion_phi0=np.concatenate([rng.choice([0.0, np.pi], nd), rest]),
        torsion_n=np.concatenate([rng.integers(1, 4, nd), np.zeros(ni, dtype=np.int64)]).astype(np.int32),
        n_dihedrals=nd,
        specials=np.stack([quads[:, 0], quads[:, 3]], axis=1), special_sigma=np.full(nd, 3.905),
        special_epsilon=rng.uniform(0.05, 0.2, nd), special_lj_scale=np.full(nd, 0.5),
        special_coulomb_scale=np.full(nd, 0.8333))
    excl = np.concatenate([bonds, angles[:, [0, 2]], quads[:, [0, 3]]]).astype(np.int32)
    kb = 0.0019872041
    vel = maxwell_boltzmann(n, 300.0, mass, rng, kb=kb / (48.88821291 ** 2))
    return System(name=f"chains_{n}", pos=pos, box=box, types=types, charge=charge, mass=mass, eps=eps, sig=sig,
                  cutoff=cutoff, skin=skin, vel=vel, exclusions=excl, coulomb=True, dt=1.0, force_to_accel=4.184e-4,
                  bonded=bonded, meta=dict(seed=seed, molecules=nm, length=length))


def disordered_solid(n_target=1_000_000, *, density=0.05, min_dist=1.8, cutoff=5.0, seed=99) -> System:
    """Three-species disordered periodic solid for the radius-graph build: uniform random positions with a minimum
    distance (seeded dart throwing over a cell grid in the host library: a draw is kept only when it lies min_dist or
    more from every point kept before it). A million atoms take about a second."""
    from . import input_api
    L = (n_target / density) ** (1.0 / 3.0)
    pos = input_api.dart_throw(n_target, L, min_dist, seed)
    types = np.random.default_rng(seed).choice(3, size=n_target, p=[0.5, 0.3, 0.2]).astype(np.int32)
    return System(name=f"solid_{n_target}", pos=pos, box=np.full(3, L), types=types, charge=np.zeros(n_target),
                  mass=np.ones(n_target), eps=np.ones((3, 3)), sig=np.ones((3, 3)), cutoff=cutoff, skin=0.0,
                  meta=dict(seed=seed, density=density, min_dist=min_dist))


def disordered_solid_lattice(n_side=100, *, density=0.05, jitter=0.45, cutoff=5.0, seed=99) -> System:
    """A second solid of the same density and species mix: a simple-cubic lattice with a seeded uniform jitter per
    coordinate, which keeps every pair further apart than spacing - 2 * jitter (2.714 - 0.9 = 1.81 A at density 0.05).
    Used by tests that want a different neighbour-count distribution from disordered_solid()."""
    rng = np.random.default_rng(seed)
    n = n_side ** 3
    a = (1.0 / density) ** (1.0 / 3.0)
    g = np.arange(n_side, dtype=np.float64)
    pos = (np.stack(np.meshgrid(g, g, g, indexing="ij"), axis=-1).reshape(-1, 3) + 0.5) * a
    pos += rng.uniform(-jitter, jitter, pos.shape)
    types = rng.choice(3, size=n, p=[0.5, 0.3, 0.2]).astype(np.int32)
    return System(name=f"solid_lattice_{n}", pos=pos, box=np.full(3, n_side * a), types=types, charge=np.zeros(n),
                  mass=np.ones(n), eps=np.ones((3, 3)), sig=np.ones((3, 3)), cutoff=cutoff, skin=0.0,
                  meta=dict(seed=seed, density=density, jitter=jitter))


def brick_decompose(pos, box, dims, halo):
    """Host-side spatial decomposition used by tests and the benchmark set-up: for every brick of a dims grid over the
    periodic box, the indices of its owned atoms and (source index, image shift) of its ghost atoms - every periodic
    image of an atom that lies within `halo` of the brick on the split axes (edges and corners included)."""
    pos = np.asarray(pos, dtype=np.float64)
    box = np.asarray(box, dtype=np.float64)
    dims = np.asarray(dims, dtype=np.int64)
    wrapped = pos - box * np.floor(pos / box)
    cell = np.minimum((wrapped / box * dims).astype(np.int64), dims - 1)
    out = []
    for cx in range(dims[0]):
        for cy in range(dims[1]):
            for cz in range(dims[2]):
                c = np.array([cx, cy, cz])
                lo = box * c / dims
                hi = box * (c + 1) / dims
                owned = np.nonzero((cell == c).all(1))[0]
                src_all, img_all = [], []
                ranges = [(-1, 0, 1) if dims[a] > 1 else (0,) for a in range(3)]
                for sx in ranges[0]:
                    for sy in ranges[1]:
                        for sz in ranges[2]:
                            s = np.array([sx, sy, sz])
                            q = wrapped + s * box
                            inside = np.ones(len(pos), dtype=bool)
                            brick = np.ones(len(pos), dtype=bool)
                            for a in range(3):
                                if dims[a] == 1:
                                    continue
                                inside &= (q[:, a] >= lo[a] - halo) & (q[:, a] < hi[a] + halo)
                                brick &= (q[:, a] >= lo[a]) & (q[:, a] < hi[a])
                            if sx == 0 and sy == 0 and sz == 0:
                                inside &= ~brick
                            idx = np.nonzero(inside)[0]
                            src_all.append(idx)
                            img_all.append(np.tile(s, (len(idx), 1)))
                src = np.concatenate(src_all)
                img = np.concatenate(img_all)
                key = np.lexsort((img[:, 2], img[:, 1], img[:, 0], src))
                out.append(dict(coords=c, lo=lo, hi=hi, owned=owned, ghost_src=src[key], ghost_image=img[key]))
    return out
