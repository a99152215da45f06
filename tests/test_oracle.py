"""CPU tests of the oracle itself: the restatement against brute force, against the committed golden fixtures (outputs of
the reference's own CPU code) and, where the compiled reference is present, against that code directly."""
import hashlib
import os

import numpy as np
import pytest

from deepscalemd_b200 import synthetic as syn
from oracle import cpu_oracle as co

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden_cases():
    return {
        "lj_fcc_864": (lambda: syn.fcc_lj(6, seed=1)),
        "lj_fcc_4000_switch": (lambda: syn.fcc_lj(10, seed=2)),
        "kob_andersen_4096": (lambda: syn.kob_andersen(4096, seed=5)),
        "water_3993": (lambda: syn.water_box(11, seed=3)),
    }


def rms(a):
    return float(np.sqrt((np.asarray(a) ** 2).sum(-1).mean()))


def oracle_eval(s, switch, ewald_mode):
    x, y, z = (np.ascontiguousarray(s.pos[:, k]) for k in range(3))
    pairs = co.pairs(x, y, z, s.n, s.box, search=s.cutoff + s.skin)
    c6, c12 = co.lj_tables(s.eps, s.sig)
    alpha = co.ewald_alpha(s.cutoff) if s.coulomb else 0.0
    f, sc = co.forces(x, y, z, s.n, s.box, pairs, c6, c12, s.cutoff, charge=s.charge, types=s.types, switch=switch,
                      do_coulomb=s.coulomb, alpha=alpha, ewald_mode=ewald_mode, exclusions=s.exclusions)
    return pairs, f, sc


def test_pairs_match_brute_force():
    s = syn.fcc_lj(5, seed=11)
    R = s.cutoff + s.skin
    x, y, z = (np.ascontiguousarray(s.pos[:, k]) for k in range(3))
    got = co.canonical_pairs(co.pairs(x, y, z, s.n, s.box, search=R))
    want = co.canonical_pairs(co.brute_pairs(s.pos, s.box, R))
    assert np.array_equal(got, want)


def test_no_pair_sits_on_the_list_boundary():
    """The seeded inputs have no pair within 1e-9 (relative) of the list radius, so fp64 evaluation order cannot
    change the pair set."""
    s = syn.fcc_lj(6, seed=1)
    R = s.cutoff + s.skin
    d = s.pos[:, None, :] - s.pos[None, :, :]
    d -= s.box * np.round(d / s.box)
    r2 = (d * d).sum(-1)
    assert not np.any(np.abs(r2 / (R * R) - 1.0) < 1e-9)


@pytest.mark.parametrize("name", list(golden_cases()))
def test_restatement_matches_golden_reference_output(name):
    """Pins the oracle: pair set identical (checksum of the canonical list), forces/energy/virial equal to the
    reference CPU code's to fp64 round-off (the restatement uses the reference's own Ewald table arithmetic here)."""
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    s = golden_cases()[name]()
    pairs, f, sc = oracle_eval(s, float(g["switch"]), ewald_mode=0)
    assert len(pairs) == int(g["pairs_in_list"])
    assert sc["pairs_in_cutoff"] == int(g["pairs_in_cutoff"])
    sha = hashlib.sha256(co.canonical_pairs(pairs).astype(np.int64).tobytes()).hexdigest()
    assert sha == str(g["pair_sha256"])
    assert rms(f - g["forces"]) <= 1e-12 * rms(g["forces"])
    assert abs(sc["pe"] - float(g["pe_real"])) <= 1e-11 * abs(float(g["pe_real"]))
    assert abs(sc["virial"] - float(g["virial"])) <= 1e-11 * abs(float(g["virial"]))
    assert np.allclose(sc["virial_diag"], g["virial_diag"], rtol=1e-10)


def test_reference_table_distance_from_exact_erfc():
    """The reference CPU path interpolates erfc linearly in r^2 (spacing 0.04 A^2): its own forces sit about 2e-4
    (relative RMS) from the exact-erfc result. Documented here because it bounds how closely any accurate
    implementation can agree with that path on a charged system."""
    g = np.load(os.path.join(GOLDEN, "water_3993.npz"))
    s = golden_cases()["water_3993"]()
    _, f_exact, sc = oracle_eval(s, -1.0, ewald_mode=1)
    rel = rms(f_exact - g["forces"]) / rms(g["forces"])
    assert 1e-5 < rel < 1e-3
    assert abs(sc["pe"] - float(g["pe_real"])) < 1e-4 * abs(float(g["pe_real"]))


@pytest.mark.skipif(not co.ref_available(), reason="compiled reference (oracle/_ref) not present")
def test_restatement_matches_compiled_reference_with_ghosts():
    """Two-brick split along x emulated in one process: each brick's owned + ghost atoms go through the reference's
    list builder and force code and through the restatement; both must agree, and the bricks must add up to the
    undivided system."""
    s = syn.fcc_lj(8, seed=21)
    R = s.cutoff + s.skin
    halo = R
    whole_pairs, whole_f, whole_sc = oracle_eval(s, -1.0, 1)
    total_pe = 0.0
    f_sum = np.zeros_like(whole_f)
    for brick in syn.brick_decompose(s.pos, s.box, (2, 1, 1), halo):
        own, src, img = brick["owned"], brick["ghost_src"], brick["ghost_image"]
        wrapped = s.pos - s.box * np.floor(s.pos / s.box)
        pos = np.concatenate([wrapped[own], wrapped[src] + img * s.box])
        gid = np.concatenate([own, src]).astype(np.int32)
        x, y, z = (np.ascontiguousarray(pos[:, k]) for k in range(3))
        lo, hi = brick["lo"].copy(), brick["hi"].copy()
        ref = co.RefCase(x, y, z, len(own), s.box, s.cutoff, s.skin, lo=lo, hi=hi, gid=gid, n_global=s.n)
        ref.build_list()
        rp = co.canonical_pairs(ref.list_pairs())
        split = (1, 0, 0)
        op = co.pairs(x, y, z, len(own), s.box, split=split, search=R)
        assert np.array_equal(rp, co.canonical_pairs(op))
        f_ref, sc_ref = ref.compute()
        c6, c12 = co.lj_tables(s.eps, s.sig)
        f, sc = co.forces(x, y, z, len(own), s.box, op, c6, c12, s.cutoff, gid=gid, split=split)
        assert rms(f - f_ref) <= 1e-12 * rms(f_ref)
        assert abs(sc["pe"] - sc_ref["pe"]) <= 1e-11 * abs(sc_ref["pe"])
        total_pe += sc["pe"]
        f_sum[own] = f
        ref.close()
    assert abs(total_pe - whole_sc["pe"]) <= 1e-10 * abs(whole_sc["pe"])
    assert rms(f_sum - whole_f) <= 1e-12 * rms(whole_f)


def test_cubic_ewald_table_accuracy():
    """The float-bit indexed cubic table reproduces erfc(a r)/r and its force factor to ~1e-6 relative of the value at worst (float evaluation; the values near the cutoff are ~1e-6 themselves)."""
    from math import erfc, exp, pi, sqrt
    alpha = co.ewald_alpha(10.0)
    fc, ec = co.cubic_table(alpha, 100.0)
    assert fc.shape[0] == 256
    rng = np.random.default_rng(0)
    worst_e = worst_f = 0.0
    for r2 in rng.uniform(0.5, 100.0, 2000):
        r = sqrt(r2)
        e_true = erfc(alpha * r) / r
        f_true = (e_true + 2 * alpha / sqrt(pi) * exp(-alpha * alpha * r2)) / r2
        e_tab, f_tab = co.cubic_eval(ec, np.float32(r2)), co.cubic_eval(fc, np.float32(r2))
        r2f = float(np.float32(r2))
        rf = sqrt(r2f)
        e_t = erfc(alpha * rf) / rf
        f_t = (e_t + 2 * alpha / sqrt(pi) * exp(-alpha * alpha * r2f)) / r2f
        worst_e = max(worst_e, abs(e_tab - e_t) / e_t)
        worst_f = max(worst_f, abs(f_tab - f_t) / f_t)
    assert worst_e < 2e-6 and worst_f < 2e-6
    assert co.cubic_eval(ec, np.float32(0.3)) is None          # below the table


def test_edges_match_brute_force_and_images():
    rng = np.random.default_rng(3)
    n, L, cutoff = 400, 12.0, 2.5
    pos = rng.uniform(0, L, (n, 3))
    x, y, z = (np.ascontiguousarray(pos[:, k]) for k in range(3))
    idx, _ = co.edges(x, y, z, cutoff)
    bf = co.brute_edges(pos, cutoff)
    key = lambda e: e[:, np.lexsort((e[1], e[0]))]
    assert np.array_equal(key(idx), key(bf))
    # periodic images as shifts: every atom gets its images within the cutoff of the box; edges centred on real atoms
    box = np.full(3, L)
    im = co.images(x, y, z, box, np.zeros(3), -np.full(3, cutoff + 1e-8), box + cutoff + 1e-8, np.ones(3, dtype=np.int32))
    total = len(im["x"])
    assert total > n and np.all(im["owner"][:n] == np.arange(n))
    idx2, sh2 = co.edges(im["x"], im["y"], im["z"], cutoff, n_centers=n, owner=im["owner"], shift=im["shift"])
    # the same graph by minimum image
    d = pos[None, :, :] - pos[:, None, :]
    img = -np.round(d / L)
    d += img * L
    m = (d * d).sum(-1) < cutoff * cutoff
    np.fill_diagonal(m, False)
    i, j = np.nonzero(m)
    want = np.stack([i, j, *(img[i, j, k].astype(np.int64) for k in range(3))])
    got = np.stack([idx2[0], idx2[1], *(np.rint(sh2[:, k] / L).astype(np.int64) for k in range(3))])
    order = lambda e: e[:, np.lexsort(e[::-1])]
    assert np.array_equal(order(got), order(want))
    # vector reconstruction: pos[j] - pos[i] + shift is the found displacement
    w = pos - L * np.floor(pos / L)
    vec = w[idx2[1]] - w[idx2[0]] + sh2
    assert np.all((vec * vec).sum(1) < cutoff * cutoff)


def test_edge_pruning_rows():
    rng = np.random.default_rng(4)
    pos = rng.uniform(0, 8.0, (200, 3))
    x, y, z = (np.ascontiguousarray(pos[:, k]) for k in range(3))
    ok = (rng.uniform(size=200) < 0.5).astype(np.uint8)
    full, _ = co.edges(x, y, z, 2.0)
    for row in (0, 1):
        pruned, _ = co.edges(x, y, z, 2.0, receiver_ok=ok, row=row)
        keep = ok[full[row]] != 0
        assert np.array_equal(pruned, full[:, keep])


def test_ghost_selection_matches_independent_construction():
    s = syn.fcc_lj(6, seed=9)
    x, y, z = (np.ascontiguousarray(s.pos[:, k]) for k in range(3))
    halo = s.cutoff + s.skin
    for dims in ((2, 1, 1), (2, 2, 1), (2, 2, 2)):
        bricks = syn.brick_decompose(s.pos, s.box, dims, halo)
        owned_total = 0
        for b in bricks:
            src, img = co.ghosts(x, y, z, s.box, (1, 1, 1), dims, b["coords"], halo)
            assert np.array_equal(src, b["ghost_src"]) and np.array_equal(img, b["ghost_image"])
            owned_total += len(b["owned"])
        assert owned_total == s.n


def test_velocity_verlet_conserves_energy_on_oracle_forces():
    s = syn.fcc_lj(4, seed=5)
    pos = [np.ascontiguousarray(s.pos[:, k]) for k in range(3)]
    vel = [np.ascontiguousarray(s.vel[:, k]) for k in range(3)]
    c6, c12 = co.lj_tables(s.eps, s.sig)

    def force():
        p = co.pairs(*pos, s.n, s.box, search=s.cutoff)
        f, sc = co.forces(*pos, s.n, s.box, p, c6, c12, s.cutoff)
        return [np.ascontiguousarray(f[:, k]) for k in range(3)], sc["pe"]

    frc, pe = force()
    e0 = pe + 0.5 * sum((v * v).sum() for v in vel)
    dt = 0.002
    for _ in range(50):
        co.vv_half(True, dt, 1.0, pos, vel, frc, s.mass)
        frc, pe = force()
        co.vv_half(False, dt, 1.0, pos, vel, frc, s.mass)
    e1 = pe + 0.5 * sum((v * v).sum() for v in vel)
    # plain truncation at the cutoff makes the energy jump when pairs cross it: small but not round-off small
    assert abs(e1 - e0) / s.n < 5e-3


def test_pair_checksum_is_the_same_in_numpy_and_torch():
    """The full-size list checks compare a checksum computed in numpy (generator) with one computed in torch (device)."""
    import sys
    import torch
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    sys.path.insert(0, here)
    from pair_checksum import checksum_numpy, checksum_torch
    rng = np.random.default_rng(3)
    a = rng.integers(0, 4_000_000, 100_000)
    b = a + rng.integers(1, 4_000_000, 100_000)
    want = checksum_numpy(a, b)
    assert checksum_torch(torch.from_numpy(a), torch.from_numpy(b), chunk=30_000) == want
    perm = rng.permutation(len(a))
    assert checksum_numpy(a[perm], b[perm]) == want
    b2 = b.copy()
    b2[7] += 1
    assert checksum_numpy(a, b2) != want


def _water_constraints(w):
    """O-H1, O-H2, H1-H2 of every molecule at the lengths the generated (rigid) geometry has."""
    out = []
    for m in range(w.n // 3):
        o, h1, h2 = 3 * m, 3 * m + 1, 3 * m + 2
        for i, j in ((o, h1), (o, h2), (h1, h2)):
            r = w.pos[i] - w.pos[j]
            r -= w.box * np.round(r / w.box)
            out.append((i, j, float(np.sqrt(r @ r))))
    return out


@pytest.mark.skipif(not co.ref_available(), reason="oracle/_ref is not built")
def test_shake_and_rattle_match_the_reference_constraint_solver():
    """Rigid water after an unconstrained drift: the oracle's SHAKE / RATTLE and the reference's own ConstraintSolver
    (compiled in place) give the same positions, velocities and constraint virial; the constraints hold afterwards."""
    w = syn.water_box(4, seed=11)
    cons = _water_constraints(w)
    rng = np.random.default_rng(5)
    dt = 2.0
    vel0 = rng.normal(0.0, 0.004, (w.n, 3)) / np.sqrt(w.mass)[:, None] * 4.0
    pre = [np.ascontiguousarray(w.pos[:, k]) for k in range(3)]
    drifted = [p + dt * vel0[:, k] for k, p in enumerate(pre)]

    def copies():
        return [c.copy() for c in drifted], [np.ascontiguousarray(vel0[:, k]).copy() for k in range(3)]

    def violation(pos):
        P = np.stack(pos, axis=1)
        worst = 0.0
        for i, j, d in cons:
            r = P[i] - P[j]
            r -= w.box * np.round(r / w.box)
            worst = max(worst, abs(r @ r - d * d) / (d * d))
        return worst

    assert violation(pre) < 1e-12 and violation(drifted) > 1e-4
    pos_o, vel_o = copies()
    pos_r, vel_r = copies()
    assert co.shake(cons, pos_o, vel_o, w.mass, pre, w.box, dt)
    ok_ref, _ = co.ref_constrain("shake", cons, pos_r, vel_r, w.mass, w.box, dt, pre=pre)
    assert ok_ref
    for a, b in zip(pos_o + vel_o, pos_r + vel_r):
        assert np.abs(a - b).max() < 1e-13
    assert violation(pos_o) < 1e-8
    momentum = sum((w.mass * v).sum() for v in vel_o), sum((w.mass * vel0[:, k]).sum() for k in range(3))
    assert abs(momentum[0] - momentum[1]) < 1e-12
    # the velocity part
    ok, virial = co.rattle(cons, pos_o, vel_o, w.mass, w.box, dt, 4.184e-4)
    ok_ref, virial_ref = co.ref_constrain("rattle", cons, pos_r, vel_r, w.mass, w.box, dt)
    assert ok and ok_ref
    for a, b in zip(vel_o, vel_r):
        assert np.abs(a - b).max() < 1e-13
    assert np.allclose(virial, virial_ref, rtol=1e-11, atol=0.0) and np.abs(virial).min() > 0.0
    P, V = np.stack(pos_o, axis=1), np.stack(vel_o, axis=1)
    for i, j, _ in cons:
        r = P[i] - P[j]
        r -= w.box * np.round(r / w.box)
        assert abs(r @ (V[i] - V[j])) < 1e-8
    # a solver that cannot converge says so
    pos_x, vel_x = copies()
    assert not co.shake(cons, pos_x, vel_x, w.mass, pre, w.box, dt, max_iterations=1)


def test_image_force_fold_and_virial_restatement():
    """The oracle's fold of image forces (src/MLIPStep.cu:108-124) against an independent numpy scatter-add, and its
    r.F sums (src/MLIPStep.cu:126-148) against numpy."""
    rng = np.random.default_rng(11)
    n, L = 500, 12.0
    pos = rng.uniform(0, L, (n, 3))
    box = np.full(3, L)
    img = co.images(pos[:, 0], pos[:, 1], pos[:, 2], box, np.zeros(3), -np.full(3, 3.0), box + 3.0, (1, 1, 1))
    n_all = len(img["x"])
    f = rng.normal(size=(n_all, 3))
    target = rng.normal(size=(n, 3))
    want = target + f[:n]
    np.add.at(want, img["owner"][n:], f[n:])
    got = co.fold_image_forces(f, n, img["owner"], target)
    assert np.allclose(got, want, rtol=0, atol=1e-12)
    assert np.array_equal(co.fold_image_forces(f, n, img["owner"], target, with_images=False), target + f[:n])
    part = co.fold_image_forces(f, n, img["owner"], target, n_out=100)
    assert np.array_equal(part[100:], target[100:]) and np.array_equal(part[:100], got[:100])
    all_pos = np.stack([img["x"], img["y"], img["z"]], axis=1)
    v = co.virial_from_forces(all_pos, f)
    assert np.allclose(v[1:], (all_pos * f).sum(0), rtol=1e-12) and np.isclose(v[0], (all_pos * f).sum(), rtol=1e-12)


@pytest.mark.skipif(not co.ref_available(), reason="oracle/_ref is not built")
def test_bonded_terms_match_the_reference_routines():
    """Bonds, angles, periodic and harmonic torsions (dihedrals and impropers) and scaled special pairs of the restatement
    against the reference's own compute_bond_forces / compute_angle_forces / compute_torsion_forces /
    compute_special_pair_forces (compiled in place) on flexible chains wrapped into a periodic box; then the ownership
    rule: with only part of the atoms owned, owned atoms keep their forces and the energies of the two halves add up."""
    s = syn.chain_fluid(4, 8, seed=11)
    t = co.BondedTerms(**s.bonded)
    assert len(t.bonds) == 64 * 7 and len(t.angles) == 64 * 6 and len(t.torsions) == 64 * 5 + 160 and t.n_dihedrals == 320
    f, sc = co.bonded(s.pos, s.n, s.box, t, charge=s.charge)
    ref = co.RefCase(s.pos[:, 0], s.pos[:, 1], s.pos[:, 2], s.n, s.box, s.cutoff, s.skin, charge=s.charge, types=s.types,
                     eps=s.eps, sig=s.sig)
    fr, rsc = ref.bonded(t)
    ref.close()
    scale = np.sqrt((fr * fr).sum(1).mean())
    assert scale > 1.0
    assert np.abs(f - fr).max() <= 1e-11 * scale
    assert abs(sc["pe"] - rsc["pe"]) <= 1e-12 * abs(rsc["pe"])
    assert abs(sc["virial"] - rsc["virial"]) <= 1e-11 * abs(rsc["virial"])
    assert np.abs(sc["virial_diag"] - rsc["virial_diag"]).max() <= 1e-11 * np.abs(rsc["virial_diag"]).max()
    assert np.abs(f.sum(0)).max() <= 1e-9 * scale                      # Newton's third law over all terms
    # every kind of term contributes
    for part in (dict(bonds=s.bonded["bonds"], bond_k=s.bonded["bond_k"], bond_r0=s.bonded["bond_r0"]),
                 dict(angles=s.bonded["angles"], angle_k=s.bonded["angle_k"], angle_theta0=s.bonded["angle_theta0"]),
                 dict(torsions=s.bonded["torsions"], torsion_k=s.bonded["torsion_k"], torsion_phi0=s.bonded["torsion_phi0"],
                      torsion_n=s.bonded["torsion_n"]),
                 dict(specials=s.bonded["specials"], special_sigma=s.bonded["special_sigma"],
                      special_epsilon=s.bonded["special_epsilon"], special_lj_scale=s.bonded["special_lj_scale"],
                      special_coulomb_scale=s.bonded["special_coulomb_scale"])):
        fp, _ = co.bonded(s.pos, s.n, s.box, co.BondedTerms(**part), charge=s.charge)
        assert np.sqrt((fp * fp).sum(1).mean()) > 1e-2
    # ownership: the first 300 atoms owned (chains are cut), then the others owned (atoms reordered so that they come first)
    n_a = 300
    fa, sa = co.bonded(s.pos, n_a, s.box, t, charge=s.charge, gid=np.arange(s.n))
    order = np.concatenate([np.arange(n_a, s.n), np.arange(n_a)])
    inverse = np.argsort(order)
    moved = {k: (inverse[v] if k in ("bonds", "angles", "torsions", "specials") else v) for k, v in s.bonded.items()}
    fb, sb = co.bonded(s.pos[order], s.n - n_a, s.box, co.BondedTerms(**moved), charge=s.charge[order], gid=order)
    assert np.abs(fa - f[:n_a]).max() <= 1e-12 * scale and np.abs(fb - f[n_a:]).max() <= 1e-12 * scale
    assert abs(sa["pe"] + sb["pe"] - sc["pe"]) <= 1e-12 * abs(sc["pe"])
    assert np.abs(sa["virial_diag"] + sb["virial_diag"] - sc["virial_diag"]).max() <= 1e-10 * np.abs(sc["virial_diag"]).max()


@pytest.mark.parametrize("kind", ["all", "bonds", "angles", "torsions", "specials"])
def test_bonded_restatement_matches_the_golden_reference_output(kind):
    """The same check against the committed output of the reference's routines (tests/golden/make_bonded_golden.py), which
    needs no compiled reference: all kinds of term together and each alone."""
    import os
    sys_path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "chains_bonded_512.npz")
    g = np.load(sys_path)
    s = syn.chain_fluid(4, 8, seed=11)
    keys = dict(all=None, bonds=("bonds", "bond_k", "bond_r0"), angles=("angles", "angle_k", "angle_theta0"),
                torsions=("torsions", "torsion_k", "torsion_phi0", "torsion_n", "n_dihedrals"),
                specials=("specials", "special_sigma", "special_epsilon", "special_lj_scale", "special_coulomb_scale"))[kind]
    terms = co.BondedTerms(**(s.bonded if keys is None else {k: s.bonded[k] for k in keys}))
    f, sc = co.bonded(s.pos, s.n, s.box, terms, charge=s.charge)
    want_f, want = g[f"f_{kind}"], g[f"scalars_{kind}"]
    scale = np.sqrt((want_f * want_f).sum(1).mean())
    assert scale > 1e-2 and np.abs(f - want_f).max() <= 1e-11 * max(scale, 1.0)
    got = np.array([sc["pe"], sc["virial"], *sc["virial_diag"]])
    assert np.abs(got - want).max() <= 1e-11 * np.abs(want).max()
