// Bonded terms and scaled special (1-4) pairs: harmonic bonds, harmonic angles, periodic and harmonic torsions (proper
// dihedrals and impropers share one form), and 12-6 Lennard-Jones + plain Coulomb pairs with per-pair scale factors.
// Included by dsmd_core.cu.
//
// What the reference does in compute_bond_forces_kernel / compute_angle_forces_kernel / compute_dihedral_forces_kernel /
// compute_improper_forces_kernel / compute_special_pair_forces_kernel (src/force_calculator_cuda.cu:2703-3170; the same
// formulas on the host in src/force_calculator_cpu.cpp:2437-2895): one thread per term, minimum image per displacement,
// and, on several ranks, redundant evaluation - a term is worked out wherever one of its atoms is owned, forces go to
// owned atoms only (no force lands on a ghost, so no reverse exchange), energy and virial are counted on the rank that
// owns the atom with the lowest global id.
//
// Where this differs: the reference adds the forces with atomics, whose order changes from run to run. Here a term
// writes its per-atom contributions into its own slots of a scratch array and a second kernel, one thread per owned
// atom, adds up the slots that belong to the atom in a fixed order (a table by global id, built once when the terms
// are set): forces stay bitwise reproducible, as those of the pair kernel are.
//
// Atoms are re-sorted by cell at every list build, so terms name their atoms by global id and go through a
// gid -> slot map (owned slot before ghost slot, lowest ghost slot among images) refreshed after every build.
#pragma once

namespace {

struct BondedTable {
    int n_bonds, n_angles, n_torsions, n_specials;
    const int* bond_atoms;        // [2 * n_bonds] global ids
    const double* bond_par;       // [2 * n_bonds] k, r0
    const int* angle_atoms;       // [3 * n_angles], the middle one is the vertex
    const double* angle_par;      // [2 * n_angles] k, theta0 (radians)
    const int* torsion_atoms;     // [4 * n_torsions]
    const double* torsion_par;    // [2 * n_torsions] k, phi0 (radians)
    const int* torsion_n;         // multiplicity; 0: harmonic in the wrapped angle difference
    const int* special_atoms;     // [2 * n_specials]
    const double* special_par;    // [4 * n_specials] sigma, epsilon, LJ scale, Coulomb scale
    const int* slot_of_gid;       // [n_global], kNoSlot: not on this rank
    int n_global;
    int n_owned;
    double box[3];
    int periodic[3];
};

constexpr int kNoSlot = 0x7F7F7F7F;   // what a byte-wise fill of the map with 0x7F leaves: beyond any slot
constexpr double kCoulombConstant = 332.0636;   // kcal/mol A / e^2, the reference's constant

__global__ void k_bonded_slot_map(int n_total, const int* __restrict__ gid, int n_global, int* __restrict__ slot_of) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= n_total) return;
    const int g = gid[s];
    if (g >= 0 && g < n_global) atomicMin(&slot_of[g], s);
}

__device__ __forceinline__ void bonded_image(double d[3], const BondedTable& t) {
#pragma unroll
    for (int a = 0; a < 3; ++a)
        if (t.periodic[a]) d[a] -= t.box[a] * rint(d[a] / t.box[a]);
}

// Slots of the COUNT atoms of a term. Returns false when the term is not this rank's business (no atom owned); sets
// *missing when an owned atom's partner is not on this rank at all (halo narrower than the term is long).
template <int COUNT>
__device__ __forceinline__ bool term_slots(const BondedTable& t, const int* atoms, int (&slot)[COUNT], bool& owner,
                                           unsigned* missing) {
    bool any_owned = false, all_here = true;
    int lowest_gid = 0x7FFFFFFF, lowest_slot = kNoSlot;
#pragma unroll
    for (int k = 0; k < COUNT; ++k) {
        const int g = atoms[k];
        slot[k] = (g >= 0 && g < t.n_global) ? t.slot_of_gid[g] : kNoSlot;
        if (slot[k] == kNoSlot) all_here = false;
        else if (slot[k] < t.n_owned) any_owned = true;
        if (g < lowest_gid) { lowest_gid = g; lowest_slot = slot[k]; }
    }
    if (!any_owned) return false;
    if (!all_here) { atomicAdd(missing, 1u); return false; }
    owner = lowest_slot < t.n_owned;
    return true;
}

// One thread per term, the four kinds one after the other in the index space. contrib holds three doubles per (term,
// atom of the term): bonds, then angles, torsions and specials; a term that is skipped writes zeros.
// partials: {PE, W, Wxx, Wyy, Wzz} per block.
__global__ void k_bonded_terms(BondedTable t, const double* __restrict__ x, const double* __restrict__ y,
                               const double* __restrict__ z, const double* __restrict__ charge,
                               double* __restrict__ contrib, double* __restrict__ partials, unsigned* __restrict__ missing) {
    const long long id = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    double sums[5] = {0.0, 0.0, 0.0, 0.0, 0.0};
    const long long first_angle = t.n_bonds, first_torsion = first_angle + t.n_angles;
    const long long first_special = first_torsion + t.n_torsions, end = first_special + t.n_specials;
    if (id < first_angle) {
        const int b = static_cast<int>(id);
        double* out = contrib + 6ll * b;
        double f[3] = {0.0, 0.0, 0.0};
        int slot[2];
        bool owner = false;
        if (term_slots<2>(t, t.bond_atoms + 2 * b, slot, owner, missing)) {
            double d[3] = {x[slot[0]] - x[slot[1]], y[slot[0]] - y[slot[1]], z[slot[0]] - z[slot[1]]};
            bonded_image(d, t);
            const double r = sqrt(d[0] * d[0] + d[1] * d[1] + d[2] * d[2]);
            if (r >= 1e-10) {
                const double k = t.bond_par[2 * b], dr = r - t.bond_par[2 * b + 1];
                const double fm = -k * dr / r;
                for (int c = 0; c < 3; ++c) f[c] = fm * d[c];
                if (owner) {
                    sums[0] = 0.5 * k * dr * dr;
                    sums[1] = fm * (d[0] * d[0] + d[1] * d[1] + d[2] * d[2]);
                    for (int c = 0; c < 3; ++c) sums[2 + c] = fm * d[c] * d[c];
                }
            }
        }
        for (int c = 0; c < 3; ++c) { out[c] = f[c]; out[3 + c] = -f[c]; }
    } else if (id < first_torsion) {
        const int a = static_cast<int>(id - first_angle);
        double* out = contrib + 6ll * t.n_bonds + 9ll * a;
        double fi[3] = {0.0, 0.0, 0.0}, fk[3] = {0.0, 0.0, 0.0};
        int slot[3];
        bool owner = false;
        if (term_slots<3>(t, t.angle_atoms + 3 * a, slot, owner, missing)) {
            double u[3] = {x[slot[0]] - x[slot[1]], y[slot[0]] - y[slot[1]], z[slot[0]] - z[slot[1]]};
            double v[3] = {x[slot[2]] - x[slot[1]], y[slot[2]] - y[slot[1]], z[slot[2]] - z[slot[1]]};
            bonded_image(u, t);
            bonded_image(v, t);
            const double ru = sqrt(u[0] * u[0] + u[1] * u[1] + u[2] * u[2]);
            const double rv = sqrt(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]);
            if (ru >= 1e-10 && rv >= 1e-10) {
                double cosine = (u[0] * v[0] + u[1] * v[1] + u[2] * v[2]) / (ru * rv);
                cosine = fmin(1.0, fmax(-1.0, cosine));
                const double k = t.angle_par[2 * a], dtheta = acos(cosine) - t.angle_par[2 * a + 1];
                if (owner) sums[0] = 0.5 * k * dtheta * dtheta;
                const double sine = sqrt(1.0 - cosine * cosine);
                if (fabs(dtheta) >= 1e-10 && sine >= 1e-10) {
                    const double fc = k * dtheta / sine;
                    for (int c = 0; c < 3; ++c) {
                        fi[c] = fc * (v[c] / (ru * rv) - u[c] * cosine / (ru * ru));
                        fk[c] = fc * (u[c] / (ru * rv) - v[c] * cosine / (rv * rv));
                    }
                    if (owner)
                        for (int c = 0; c < 3; ++c) sums[2 + c] = u[c] * fi[c] + v[c] * fk[c];
                }
            }
        }
        for (int c = 0; c < 3; ++c) { out[c] = fi[c]; out[3 + c] = -(fi[c] + fk[c]); out[6 + c] = fk[c]; }
    } else if (id < first_special) {
        const int q = static_cast<int>(id - first_torsion);
        double* out = contrib + 6ll * t.n_bonds + 9ll * t.n_angles + 12ll * q;
        double fi[3] = {0.0, 0.0, 0.0}, fj[3] = {0.0, 0.0, 0.0}, fk[3] = {0.0, 0.0, 0.0}, fl[3] = {0.0, 0.0, 0.0};
        int slot[4];
        bool owner = false;
        if (term_slots<4>(t, t.torsion_atoms + 4 * q, slot, owner, missing)) {
            double ij[3] = {x[slot[0]] - x[slot[1]], y[slot[0]] - y[slot[1]], z[slot[0]] - z[slot[1]]};
            double jk[3] = {x[slot[1]] - x[slot[2]], y[slot[1]] - y[slot[2]], z[slot[1]] - z[slot[2]]};
            double kl[3] = {x[slot[2]] - x[slot[3]], y[slot[2]] - y[slot[3]], z[slot[2]] - z[slot[3]]};
            bonded_image(ij, t);
            bonded_image(jk, t);
            bonded_image(kl, t);
            const double n1[3] = {ij[1] * jk[2] - ij[2] * jk[1], ij[2] * jk[0] - ij[0] * jk[2], ij[0] * jk[1] - ij[1] * jk[0]};
            const double n2[3] = {jk[1] * kl[2] - jk[2] * kl[1], jk[2] * kl[0] - jk[0] * kl[2], jk[0] * kl[1] - jk[1] * kl[0]};
            const double n1sq = n1[0] * n1[0] + n1[1] * n1[1] + n1[2] * n1[2];
            const double n2sq = n2[0] * n2[0] + n2[1] * n2[1] + n2[2] * n2[2];
            const double jksq = jk[0] * jk[0] + jk[1] * jk[1] + jk[2] * jk[2];
            if (n1sq >= 1e-20 && n2sq >= 1e-20 && jksq >= 1e-20) {
                const double jkm = sqrt(jksq);
                const double cosine = n1[0] * n2[0] + n1[1] * n2[1] + n1[2] * n2[2];
                const double sine = (n1[1] * n2[2] - n1[2] * n2[1]) * jk[0] + (n1[2] * n2[0] - n1[0] * n2[2]) * jk[1] +
                                    (n1[0] * n2[1] - n1[1] * n2[0]) * jk[2];
                const double phi = atan2(sine, cosine * jkm);
                const double k = t.torsion_par[2 * q], phi0 = t.torsion_par[2 * q + 1];
                const int mult = t.torsion_n[q];
                double slope;
                if (mult == 0) {
                    const double dphi = remainder(phi - phi0, 6.283185307179586476925286766559);
                    if (owner) sums[0] = k * dphi * dphi;
                    slope = 2.0 * k * dphi;
                } else {
                    const double dphi = mult * phi - phi0;
                    if (owner) sums[0] = k * (1.0 + cos(dphi));
                    slope = -k * mult * sin(dphi);
                }
                const double si = -slope * jkm / n1sq, sl = slope * jkm / n2sq;
                const double pp = -(ij[0] * jk[0] + ij[1] * jk[1] + ij[2] * jk[2]) / jksq;
                const double qq = -(kl[0] * jk[0] + kl[1] * jk[1] + kl[2] * jk[2]) / jksq;
                for (int c = 0; c < 3; ++c) {
                    fi[c] = si * n1[c];
                    fl[c] = sl * n2[c];
                    fj[c] = (pp - 1.0) * fi[c] - qq * fl[c];
                    fk[c] = -pp * fi[c] + (qq - 1.0) * fl[c];
                }
                if (owner)
                    for (int c = 0; c < 3; ++c) sums[2 + c] = ij[c] * fi[c] - jk[c] * fk[c] - (jk[c] + kl[c]) * fl[c];
            }
        }
        for (int c = 0; c < 3; ++c) { out[c] = fi[c]; out[3 + c] = fj[c]; out[6 + c] = fk[c]; out[9 + c] = fl[c]; }
    } else if (id < end) {
        const int p = static_cast<int>(id - first_special);
        double* out = contrib + 6ll * t.n_bonds + 9ll * t.n_angles + 12ll * t.n_torsions + 6ll * p;
        double f[3] = {0.0, 0.0, 0.0};
        int slot[2];
        bool owner = false;
        if (term_slots<2>(t, t.special_atoms + 2 * p, slot, owner, missing)) {
            double d[3] = {x[slot[0]] - x[slot[1]], y[slot[0]] - y[slot[1]], z[slot[0]] - z[slot[1]]};
            bonded_image(d, t);
            const double r2 = d[0] * d[0] + d[1] * d[1] + d[2] * d[2];
            if (r2 >= 1e-10) {
                const double* par = t.special_par + 4 * p;
                double fm = 0.0, u = 0.0;
                if (par[1] != 0.0) {
                    const double r2inv = 1.0 / r2, sig2 = par[0] * par[0];
                    const double att = sig2 * sig2 * sig2 * r2inv * r2inv * r2inv, rep = att * att;
                    fm += 4.0 * par[1] * r2inv * (12.0 * rep - 6.0 * att) * par[2];
                    u += 4.0 * par[1] * (rep - att) * par[2];
                }
                const double qi = charge[slot[0]], qj = charge[slot[1]];
                if (qi != 0.0 && qj != 0.0) {
                    const double r = sqrt(r2);
                    const double qq = kCoulombConstant * qi * qj * par[3];
                    fm += qq / (r2 * r);
                    u += qq / r;
                }
                if (owner) sums[0] = u;
                if (fm != 0.0) {
                    for (int c = 0; c < 3; ++c) f[c] = fm * d[c];
                    if (owner) {
                        sums[1] = r2 * fm;
                        for (int c = 0; c < 3; ++c) sums[2 + c] = fm * d[c] * d[c];
                    }
                }
            }
        }
        for (int c = 0; c < 3; ++c) { out[c] = f[c]; out[3 + c] = -f[c]; }
    }
    block_sum_to_partials<5>(sums, partials);
}

// One thread per owned atom: adds up, in table order, the contributions of the terms the atom takes part in.
// entries_of[g] .. entries_of[g + 1]: places in `entry` (indices of 3-double groups in contrib) for global id g.
__global__ void k_bonded_gather(int n_owned, const int* __restrict__ gid, int n_global,
                                const long long* __restrict__ entries_of, const int* __restrict__ entry,
                                const double* __restrict__ contrib, double* __restrict__ fx, double* __restrict__ fy,
                                double* __restrict__ fz) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= n_owned) return;
    const int g = gid[s];
    if (g < 0 || g >= n_global) return;
    const long long first = entries_of[g], last = entries_of[g + 1];
    if (last == first) return;
    double ax = 0.0, ay = 0.0, az = 0.0;
    for (long long e = first; e < last; ++e) {
        const double* c = contrib + 3ll * entry[e];
        ax += c[0]; ay += c[1]; az += c[2];
    }
    fx[s] += ax; fy[s] += ay; fz[s] += az;
}

}  // namespace
