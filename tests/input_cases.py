"""Input-file cases shared by the input-layer tests and the generator of their golden fixture: small seeded systems written
in the reference's formats, and the call into the reference's own Topology reader (test infrastructure)."""
import ctypes
import os

import numpy as np

from deepscalemd_b200 import input_files
from deepscalemd_b200 import synthetic as syn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_TOPOLOGY = os.path.join(ROOT, "oracle", "_ref", "libdsmd_ref_topology.so")


def topology_cases(folder):
    """name -> dict(topology_file, parameter_file or None, coordinate_file, box, n)."""
    cases = {}
    # 1. legacy .top, one type (argon)
    s = syn.fcc_lj(3, seed=4)
    sub = os.path.join(folder, "argon")
    _, scale = input_files.argon_files(sub, s)
    cases["legacy_argon"] = dict(topology_file=os.path.join(sub, "argon.top"), parameter_file=None,
                                 coordinate_file=os.path.join(sub, "argon.xyz"), box=scale["box"], n=s.n)
    # 2. legacy .top, three types named out of alphabetical order (ids follow first appearance among the atoms),
    #    comments, blank lines, CRLF line ends and a bonded section
    rng = np.random.default_rng(9)
    n = 60
    names = ["Zn", "C", "Ar"]
    rows = {"Ar": (39.948, 0.0, 3.405, 0.238), "C": (12.011, -0.1, 3.4, 0.086), "Zn": (65.38, 0.2, 2.46, 0.124)}
    atom_types = [names[k] for k in rng.integers(0, 3, n)]
    sub = os.path.join(folder, "mixed")
    os.makedirs(sub, exist_ok=True)
    box = np.array([20.0, 22.0, 24.0])
    pos = rng.uniform(0, 1, (n, 3)) * box
    input_files.write_xyz(os.path.join(sub, "mixed.xyz"), pos, atom_types)
    with open(os.path.join(sub, "mixed.top"), "w", newline="") as f:
        f.write("# a comment\r\n; another\r\n\r\n[ AtomTypes ]\r\n")
        for name, (m, q, sg, ep) in rows.items():
            f.write(f"  {name}\t{m} {q} {sg} {ep}   extra tokens ignored\r\n")
        f.write("short row\r\n[ atoms ]\r\n")
        for i, name in enumerate(atom_types):
            f.write(f"{i + 1} {name}\r\n")
        f.write("[ bondtypes ]\r\nC C 300.0 1.5\r\n[ bonds ]\r\n1 2 C-C\r\n")
    cases["legacy_mixed"] = dict(topology_file=os.path.join(sub, "mixed.top"), parameter_file=None,
                                 coordinate_file=os.path.join(sub, "mixed.xyz"), box=box, n=n)
    # 3. dsMD_input: binary mixture with an explicit pair table
    ka = syn.kob_andersen(256, seed=5)
    sub = os.path.join(folder, "ka")
    sig = np.asarray(ka.sig) * 3.405
    eps = np.asarray(ka.eps) * 0.238
    input_files.write_dsmd_input(sub, "ka", ka.pos * 3.405, ["Ar" if t == 0 else "Kr" for t in ka.types], ka.types,
                                 ["A", "B"], ka.mass * 39.948, ka.charge, sig, eps)
    cases["dsmd_binary"] = dict(topology_file=os.path.join(sub, "ka.dsMDtop"), parameter_file=os.path.join(sub, "ka.dsMDprm"),
                                coordinate_file=os.path.join(sub, "ka.xyz"), box=np.asarray(ka.box) * 3.405, n=ka.n,
                                manifest=os.path.join(sub, "manifest.yaml"))
    # 4. dsMD_input: rigid water (charges, exclusions, constraints)
    w = syn.water_box(3, seed=3)
    sub = os.path.join(folder, "water")
    elements = ["O" if t == 0 else "H" for t in w.types]
    constraints = []
    for m in range(w.n // 3):
        o, h1, h2 = 3 * m, 3 * m + 1, 3 * m + 2
        constraints += [(o, h1, 1.0), (o, h2, 1.0), (h1, h2, 1.6329931618554521)]
    input_files.write_dsmd_input(sub, "water", w.pos, elements, w.types, ["OW", "HW"], w.mass, w.charge, np.asarray(w.sig),
                                 np.asarray(w.eps), exclusions=w.exclusions, constraints=constraints)
    cases["dsmd_water"] = dict(topology_file=os.path.join(sub, "water.dsMDtop"),
                               parameter_file=os.path.join(sub, "water.dsMDprm"),
                               coordinate_file=os.path.join(sub, "water.xyz"), box=np.asarray(w.box), n=w.n,
                               manifest=os.path.join(sub, "manifest.yaml"))
    # 5. dsMD_input: flexible chains with every bonded section (each term with a parameter id of its own)
    c = syn.chain_fluid(3, 8, seed=5)
    sub = os.path.join(folder, "chains")
    input_files.write_dsmd_input(sub, "chains", c.pos, ["C"] * c.n, c.types, ["CH3", "CH2"], c.mass, c.charge, np.asarray(c.sig),
                                 np.asarray(c.eps), bonded=c.bonded)
    cases["dsmd_chains"] = dict(topology_file=os.path.join(sub, "chains.dsMDtop"),
                                parameter_file=os.path.join(sub, "chains.dsMDprm"),
                                coordinate_file=os.path.join(sub, "chains.xyz"), box=np.asarray(c.box), n=c.n,
                                manifest=os.path.join(sub, "manifest.yaml"))
    return cases


def reference_available():
    return os.path.exists(REF_TOPOLOGY)


def reference_topology(topology_file, parameter_file=None):
    """What the reference's Topology class parses from the files, or None when it refuses them."""
    L = ctypes.CDLL(REF_TOPOLOGY)
    L.dsmd_reftop_load.restype = ctypes.c_void_p
    h = L.dsmd_reftop_load(str(topology_file).encode(), (parameter_file or "").encode())
    if not h:
        return None
    h = ctypes.c_void_p(h)
    atoms, entries, excl, cons = ctypes.c_long(), ctypes.c_long(), ctypes.c_long(), ctypes.c_long()
    mn, mm = ctypes.c_int(), ctypes.c_int()
    L.dsmd_reftop_counts(h, ctypes.byref(atoms), ctypes.byref(entries), ctypes.byref(excl), ctypes.byref(cons),
                         ctypes.byref(mn), ctypes.byref(mm))
    n = atoms.value
    type_ = np.zeros(n, dtype=np.int32)
    mass, charge, sigma, eps = (np.zeros(n) for _ in range(4))
    dp = lambda a: a.ctypes.data_as(ctypes.POINTER(ctypes.c_double))
    ip = lambda a: a.ctypes.data_as(ctypes.POINTER(ctypes.c_int))
    L.dsmd_reftop_atoms(h, ip(type_), dp(mass), dp(charge), dp(sigma), dp(eps))
    ps, pe = np.zeros(max(entries.value, 1)), np.zeros(max(entries.value, 1))
    ex = np.zeros(max(2 * excl.value, 1), dtype=np.int32)
    ci, cj = np.zeros(max(cons.value, 1), dtype=np.int32), np.zeros(max(cons.value, 1), dtype=np.int32)
    cd = np.zeros(max(cons.value, 1))
    L.dsmd_reftop_pairs(h, dp(ps), dp(pe), ip(ex), ip(ci), ip(cj), dp(cd))
    counts = (ctypes.c_long * 5)()
    L.dsmd_reftop_bonded_counts(h, counts)
    nb, na, nt, nd, ns = (int(v) for v in counts)
    ib = lambda k: np.zeros(max(k, 1), dtype=np.int32)
    db = lambda k: np.zeros(max(k, 1))
    ba, bp, aa, ap, ta, tp, tn, sa, sp = ib(2 * nb), db(2 * nb), ib(3 * na), db(2 * na), ib(4 * nt), db(2 * nt), ib(nt), ib(2 * ns), db(4 * ns)
    L.dsmd_reftop_bonded(h, ip(ba), dp(bp), ip(aa), dp(ap), ip(ta), dp(tp), ip(tn), ip(sa), dp(sp))
    bonded = dict(counts=[nb, na, nt, nd, ns], bond_atoms=ba[:2 * nb].tolist(), bond_par=bp[:2 * nb].tolist(),
                  angle_atoms=aa[:3 * na].tolist(), angle_par=ap[:2 * na].tolist(), torsion_atoms=ta[:4 * nt].tolist(),
                  torsion_par=tp[:2 * nt].tolist(), torsion_n=tn[:nt].tolist(), special_atoms=sa[:2 * ns].tolist(),
                  special_par=sp[:4 * ns].tolist())
    L.dsmd_reftop_destroy(h)
    return dict(bonded=bonded, atoms=n, type=type_.tolist(), mass=mass.tolist(), charge=charge.tolist(), sigma=sigma.tolist(),
                epsilon=eps.tolist(), pair_sigma=ps[:entries.value].tolist(), pair_epsilon=pe[:entries.value].tolist(),
                exclusions=ex[:2 * excl.value].tolist(), constraint_i=ci[:cons.value].tolist(),
                constraint_j=cj[:cons.value].tolist(), constraint_d=cd[:cons.value].tolist(), mie=[mn.value, mm.value])
