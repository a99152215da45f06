// Test infrastructure, not product code.
//
// C entry points around the reference's own CPU implementation of the short-range nonbonded path:
// SpatialVerletList::build (src/neighbor_list_cpu.cpp:220) and ForceCalculatorCPU::compute_forces
// (src/force_calculator_cpu.cpp:749 -> compute_tiled_nonbonded :1915). The reference sources are compiled
// where they lie (see the Makefile beside this file); this translation unit only supplies what a one-rank,
// real-space-only build needs around them: the few MDSystem / Topology / ForceManager members the two
// sources call but which live in files that need MPI, dsDecompX or FFTW, and an inert reciprocal-space
// engine. Nothing here is linked into the shipped library.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>
#include <iostream>
#include <chrono>
#include <limits>
#include <stdexcept>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "reference_members.hpp"
#include "constraint_solver.h"

// ---- the C entry points ----------------------------------------------------------------------------

namespace {

struct RefCase {
    MDSystem system;
    std::unique_ptr<SpatialVerletList> list;
    std::unique_ptr<ForceCalculatorCPU> calc;
    double cutoff = 0.0, skin = 0.0;
    size_t n_local = 0;
};

}  // namespace

extern "C" {

void* dsmd_ref_create() {
    auto* c = new RefCase();
    c->system.topology = std::make_unique<Topology>();
    c->system.force_manager = std::make_unique<ForceManager>();
    return c;
}

void dsmd_ref_destroy(void* h) { delete static_cast<RefCase*>(h); }

int dsmd_ref_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// 1 = scalar, 4 = AVX2, 8 = AVX-512: which of the reference's fp64 tile kernels this build runs.
int dsmd_ref_simd_width() {
#if defined(__AVX512F__)
    return 8;
#elif defined(__AVX2__) || defined(__AVX__)
    return 4;
#else
    return 1;
#endif
}

// lo == hi on an axis means "the whole box length on that axis" (no subdomain), as SimulationBox treats it.
void dsmd_ref_set_box(void* h, const double L[3], const int periodic[3], const double lo[3], const double hi[3]) {
    SimulationBox& b = static_cast<RefCase*>(h)->system.box;
    b.lx = L[0]; b.ly = L[1]; b.lz = L[2];
    b.xlo = lo[0]; b.xhi = hi[0];
    b.ylo = lo[1]; b.yhi = hi[1];
    b.zlo = lo[2]; b.zhi = hi[2];
    b.periodic_x = periodic[0] != 0; b.periodic_y = periodic[1] != 0; b.periodic_z = periodic[2] != 0;
    b.update_box_length();
}

void dsmd_ref_set_particles(void* h, long n_total, long n_local, const double* x, const double* y, const double* z,
                            const double* charge, const int* type, const int* gid) {
    auto* c = static_cast<RefCase*>(h);
    ParticleData& p = c->system.particles;
    p.reset_counts(static_cast<size_t>(n_local), static_cast<size_t>(n_total - n_local));
    p.resize(static_cast<size_t>(n_total));
    p.reset_counts(static_cast<size_t>(n_local), static_cast<size_t>(n_total - n_local));
    for (long i = 0; i < n_total; ++i) {
        p.x[i] = x[i]; p.y[i] = y[i]; p.z[i] = z[i];
        p.charge[i] = charge ? charge[i] : 0.0;
        p.type[i] = type ? type[i] : 0;
        p.global_id[i] = gid ? gid[i] : static_cast<int>(i);
        p.mass[i] = 1.0;
    }
    c->n_local = static_cast<size_t>(n_local);
}

// New positions for the atoms already set (same order); everything else is kept.
void dsmd_ref_update_positions(void* h, const double* x, const double* y, const double* z) {
    ParticleData& p = static_cast<RefCase*>(h)->system.particles;
    for (size_t i = 0; i < p.num_particles; ++i) { p.x[i] = x[i]; p.y[i] = y[i]; p.z[i] = z[i]; }
}

// SpatialVerletList::needs_rebuild (src/neighbor_list_cpu.cpp:205-218): largest owned displacement since the last build
// above (skin / 2)^2.
int dsmd_ref_needs_rebuild(void* h) {
    auto* c = static_cast<RefCase*>(h);
    if (!c->list) return 1;
    return c->list->needs_rebuild(c->system.particles, c->system.box, c->n_local) ? 1 : 0;
}

// eps / sig: full symmetric [ntypes x ntypes] matrices (what ForceFieldParams::epsilon_mixed / sigma_mixed hold
// after mixing or after an explicit [pair_parameters] table). switch_distance <= 0: plain truncation.
void dsmd_ref_set_force_field(void* h, int ntypes, const double* eps, const double* sig, double switch_distance) {
    ForceFieldParams& ff = static_cast<RefCase*>(h)->system.ff_params;
    ff.num_atom_types = ntypes;
    ff.epsilon.assign(ntypes, 0.0);
    ff.sigma.assign(ntypes, 0.0);
    ff.epsilon_mixed.assign(ntypes, std::vector<Real>(ntypes));
    ff.sigma_mixed.assign(ntypes, std::vector<Real>(ntypes));
    for (int i = 0; i < ntypes; ++i) {
        ff.epsilon[i] = eps[i * ntypes + i];
        ff.sigma[i] = sig[i * ntypes + i];
        for (int j = 0; j < ntypes; ++j) {
            ff.epsilon_mixed[i][j] = eps[i * ntypes + j];
            ff.sigma_mixed[i][j] = sig[i * ntypes + j];
        }
    }
    ff.explicit_pair_parameters = true;
    ff.lj_switch_distance = switch_distance;
}

// Exclusions by global id; n_atoms_global = the number of atoms of the whole system.
void dsmd_ref_set_exclusions(void* h, int n_atoms_global, long n_pairs, const int* a, const int* b) {
    Topology& t = *static_cast<RefCase*>(h)->system.topology;
    t.atom_name_ids.assign(static_cast<size_t>(n_atoms_global), 0);
    t.exclusion_keys.clear();
    for (long k = 0; k < n_pairs; ++k) {
        const std::uint64_t lo = static_cast<std::uint64_t>(std::min(a[k], b[k]));
        const std::uint64_t hi = static_cast<std::uint64_t>(std::max(a[k], b[k]));
        t.exclusion_keys.push_back((lo << 32) | hi);
    }
    std::sort(t.exclusion_keys.begin(), t.exclusion_keys.end());
    t.exclusion_keys.erase(std::unique(t.exclusion_keys.begin(), t.exclusion_keys.end()), t.exclusion_keys.end());
}

void dsmd_ref_set_cutoff(void* h, double cutoff, double skin) {
    auto* c = static_cast<RefCase*>(h);
    c->cutoff = cutoff;
    c->skin = skin;
    c->system.set_physical_cutoff(cutoff);
    c->system.set_verlet_skin(skin);
}

// Builds the reference list ("tiled" layout, the CPU default). Returns the number of tile pairs.
long dsmd_ref_build_list(void* h) {
    auto* c = static_cast<RefCase*>(h);
    if (c->system.topology->atom_name_ids.empty()) {
        int max_gid = -1;
        for (int g : c->system.particles.global_id) max_gid = std::max(max_gid, g);
        c->system.topology->atom_name_ids.assign(static_cast<size_t>(max_gid + 1), 0);
    }
    c->list = std::make_unique<SpatialVerletList>(c->cutoff, c->skin);
    c->list->set_nonbonded_kernel("tiled");
    c->list->build(c->system.particles, c->system.box, c->n_local);
    c->system.set_neighbor_list(c->list.get());
    c->calc.reset();   // caches keyed on the list are rebuilt
    return c->list->num_tile_pairs();
}

unsigned long long dsmd_ref_pairs_inside_list(void* h) { return static_cast<RefCase*>(h)->list->pairs_inside_rc_plus_skin(); }
unsigned long long dsmd_ref_pairs_inside_cutoff(void* h) { return static_cast<RefCase*>(h)->list->pairs_inside_rc(); }

// Expands the tile-pair Verlet masks into atom pairs (i = atom of the home tile, always owned; j = atom of the other
// tile), in particle-array indices. Returns the pair count; writes at most `capacity` pairs.
long dsmd_ref_list_pairs(void* h, int* out_i, int* out_j, long capacity) {
    auto* c = static_cast<RefCase*>(h);
    const SpatialVerletList& l = *c->list;
    const int* atoms = l.get_tile_atoms();
    const int* off = l.get_tile_pair_offsets();
    const int* other = l.get_tile_pair_other();
    const std::uint64_t* mask = l.get_tile_pair_verlet_mask();
    long count = 0;
    for (int T = 0; T < l.num_tiles(); ++T) {
        for (int e = off[T]; e < off[T + 1]; ++e) {
            const std::uint64_t m = mask[e];
            if (!m) continue;
            const int O = other[e];
            for (int slot = 0; slot < kCpuTileSize; ++slot) {
                for (int lane = 0; lane < kCpuTileSize; ++lane) {
                    if (!((m >> (slot * kCpuTileSize + lane)) & 1u)) continue;
                    if (count < capacity) {
                        out_i[count] = atoms[static_cast<size_t>(T) * kCpuTileSize + lane];
                        out_j[count] = atoms[static_cast<size_t>(O) * kCpuTileSize + slot];
                    }
                    ++count;
                }
            }
        }
    }
    return count;
}

// One ForceCalculatorCPU::compute_forces call on the current list.
// out_scalars = {PE, virial, Wxx, Wyy, Wzz, alpha, self}. The reference folds the Ewald self energy
// -k alpha / sqrt(pi) sum q^2 into the potential energy when it closes the (here inert) reciprocal-space step
// (src/force_calculator_cpu.cpp:2422-2428); `self` is that term, so PE - self is the real-space sum alone.
// Forces are written for the n_local owned atoms.
int dsmd_ref_compute_forces(void* h, int do_lj, int do_coulomb, int tensor, int mixed_precision,
                            double* fx, double* fy, double* fz, double* out_scalars) {
    auto* c = static_cast<RefCase*>(h);
    try {
        if (!c->calc) {
            c->calc = std::make_unique<ForceCalculatorCPU>();
            c->calc->set_nonbonded_kernel("tiled");
            c->calc->set_mixed_precision(mixed_precision != 0);
            c->calc->set_virial_tensor_enabled(tensor != 0);
        }
        ForceManager::ForceConfig& cfg = c->system.force_manager->config;
        cfg.enable_bonds = cfg.enable_angles = cfg.enable_dihedrals = false;
        cfg.enable_lennard_jones = do_lj != 0;
        cfg.enable_coulomb = do_coulomb != 0;
        c->calc->compute_forces(c->system);
        const ParticleData& p = c->system.particles;
        for (size_t i = 0; i < c->n_local; ++i) { fx[i] = p.fx[i]; fy[i] = p.fy[i]; fz[i] = p.fz[i]; }
        out_scalars[0] = c->calc->get_potential_energy();
        out_scalars[1] = c->calc->get_virial();
        Real d[3];
        c->calc->get_virial_diag(d);
        out_scalars[2] = d[0]; out_scalars[3] = d[1]; out_scalars[4] = d[2];
        out_scalars[5] = c->calc->ewald_alpha_;
        double sum_q2 = 0.0;
        if (do_coulomb) for (size_t i = 0; i < c->n_local; ++i) sum_q2 += p.charge[i] * p.charge[i];
        out_scalars[6] = -332.0636 * c->calc->ewald_alpha_ / 1.7724538509055159 * sum_q2;
    } catch (const std::exception& e) {
        std::cerr << "dsmd_ref_compute_forces: " << e.what() << std::endl;
        return 1;
    }
    return 0;
}

// The reference's CPU constraint solver (src/constraint_solver.cpp) on a system given as plain arrays: positions and
// velocities are updated in place. which = 0: ConstraintSolver::apply_shake (pre = positions before the drift);
// which = 1: apply_rattle (virial_out receives the diagonal of the constraint virial). Returns 1 when it converged.
int dsmd_ref_constrain(int which, long n, long n_local, double* x, double* y, double* z, double* vx, double* vy, double* vz,
                       const double* mass, const int* gid, const double L[3], const int periodic[3], long n_constraints,
                       const long* atom1, const long* atom2, const double* distance, double dt, const double* pre_x,
                       const double* pre_y, const double* pre_z, int max_iterations, double tolerance, double virial_out[3]) {
    MDSystem system;
    SimulationBox& b = system.box;
    b.lx = L[0]; b.ly = L[1]; b.lz = L[2];
    b.xlo = b.ylo = b.zlo = 0.0;
    b.xhi = L[0]; b.yhi = L[1]; b.zhi = L[2];
    b.periodic_x = periodic[0] != 0; b.periodic_y = periodic[1] != 0; b.periodic_z = periodic[2] != 0;
    b.update_box_length();
    ParticleData& p = system.particles;
    p.reset_counts(static_cast<size_t>(n_local), static_cast<size_t>(n - n_local));
    p.resize(static_cast<size_t>(n));
    p.reset_counts(static_cast<size_t>(n_local), static_cast<size_t>(n - n_local));
    for (long i = 0; i < n; ++i) {
        p.x[i] = x[i]; p.y[i] = y[i]; p.z[i] = z[i];
        p.vx[i] = vx[i]; p.vy[i] = vy[i]; p.vz[i] = vz[i];
        p.mass[i] = mass[i];
        p.global_id[i] = gid ? gid[i] : static_cast<int>(i);
    }
    for (long k = 0; k < n_constraints; ++k)
        system.local_constraints_.push_back({static_cast<size_t>(atom1[k]), static_cast<size_t>(atom2[k]), distance[k]});
    ConstraintSolver solver(max_iterations, tolerance, tolerance);
    bool ok = false;
    if (which == 0) {
        std::vector<Real> px(pre_x, pre_x + n), py(pre_y, pre_y + n), pz(pre_z, pre_z + n);
        ok = solver.apply_shake(system, dt, px, py, pz);
    } else {
        ok = solver.apply_rattle(system, dt);
        if (virial_out) solver.get_virial_diag(virial_out);
    }
    for (long i = 0; i < n; ++i) {
        x[i] = p.x[i]; y[i] = p.y[i]; z[i] = p.z[i];
        vx[i] = p.vx[i]; vy[i] = p.vy[i]; vz[i] = p.vz[i];
    }
    return ok ? 1 : 0;
}

// The reference's bonded terms and scaled special pairs on the particles and box of this case (one rank: every atom is
// owned): ForceCalculatorCPU::compute_bond_forces, compute_angle_forces, compute_torsion_forces (dihedrals and impropers
// share it) and compute_special_pair_forces (src/force_calculator_cpu.cpp:2437-2895), called one after the other on
// cleared force arrays. Every term carries its own parameters (a type per term). Torsions: the first n_dihedrals entries
// go in as dihedrals, the rest as impropers. special_sigma / special_epsilon < 0: the mixing tables of the force field.
// out_scalars = {PE, virial, Wxx, Wyy, Wzz}.
int dsmd_ref_bonded(void* h, long n_bonds, const long* bond_atoms, const double* bond_k, const double* bond_r0,
                    long n_angles, const long* angle_atoms, const double* angle_k, const double* angle_theta0,
                    long n_torsions, long n_dihedrals, const long* torsion_atoms, const double* torsion_k,
                    const double* torsion_phi0, const int* torsion_n,
                    long n_specials, const long* special_atoms, const double* special_sigma, const double* special_epsilon,
                    const double* special_lj_scale, const double* special_coulomb_scale, int do_lj, int do_coulomb,
                    double* fx, double* fy, double* fz, double* out_scalars) {
    auto* c = static_cast<RefCase*>(h);
    try {
        if (!c->calc) c->calc = std::make_unique<ForceCalculatorCPU>();
        c->calc->set_virial_tensor_enabled(true);
        MDSystem& sys = c->system;
        g_ref_bond_types.clear(); g_ref_angle_types.clear(); g_ref_dihedral_types.clear();
        sys.local_bonds_.clear(); sys.local_angles_.clear(); sys.local_dihedrals_.clear(); sys.local_impropers_.clear();
        sys.local_special_pairs_.clear();
        for (long b = 0; b < n_bonds; ++b) {
            g_ref_bond_types.push_back(BondType{"b", bond_k[b], bond_r0[b]});
            sys.local_bonds_.push_back({static_cast<size_t>(bond_atoms[2 * b]), static_cast<size_t>(bond_atoms[2 * b + 1]),
                                        static_cast<int>(b), bond_k[b], bond_r0[b]});
        }
        for (long a = 0; a < n_angles; ++a) {
            g_ref_angle_types.push_back(AngleType{"a", angle_k[a], angle_theta0[a]});
            sys.local_angles_.push_back({static_cast<size_t>(angle_atoms[3 * a]), static_cast<size_t>(angle_atoms[3 * a + 1]),
                                         static_cast<size_t>(angle_atoms[3 * a + 2]), static_cast<int>(a), angle_k[a],
                                         angle_theta0[a]});
        }
        for (long t = 0; t < n_torsions; ++t) {
            g_ref_dihedral_types.push_back(DihedralType{"d", torsion_k[t], torsion_phi0[t], torsion_n[t]});
            MDSystem::LocalDihedral d{static_cast<size_t>(torsion_atoms[4 * t]), static_cast<size_t>(torsion_atoms[4 * t + 1]),
                                      static_cast<size_t>(torsion_atoms[4 * t + 2]), static_cast<size_t>(torsion_atoms[4 * t + 3]),
                                      static_cast<int>(t), torsion_k[t], torsion_phi0[t], torsion_n[t]};
            (t < n_dihedrals ? sys.local_dihedrals_ : sys.local_impropers_).push_back(d);
        }
        for (long s = 0; s < n_specials; ++s)
            sys.local_special_pairs_.push_back({static_cast<size_t>(special_atoms[2 * s]), static_cast<size_t>(special_atoms[2 * s + 1]),
                                                special_lj_scale[s], special_coulomb_scale[s], special_sigma[s],
                                                special_epsilon[s]});
        ForceManager::ForceConfig& cfg = sys.force_manager->config;
        cfg.enable_lennard_jones = do_lj != 0;
        cfg.enable_coulomb = do_coulomb != 0;
        ParticleData& p = sys.particles;
        std::fill(p.fx.begin(), p.fx.end(), 0.0);
        std::fill(p.fy.begin(), p.fy.end(), 0.0);
        std::fill(p.fz.begin(), p.fz.end(), 0.0);
        c->calc->last_potential_energy = 0.0;
        c->calc->last_virial = 0.0;
        for (int a = 0; a < 3; ++a) c->calc->last_virial_diag[a] = 0.0;
        c->calc->compute_bond_forces(sys);
        c->calc->compute_angle_forces(sys);
        c->calc->compute_dihedral_forces(sys);
        c->calc->compute_improper_forces(sys);
        c->calc->compute_special_pair_forces(sys);
        for (size_t i = 0; i < c->n_local; ++i) { fx[i] = p.fx[i]; fy[i] = p.fy[i]; fz[i] = p.fz[i]; }
        out_scalars[0] = c->calc->last_potential_energy;
        out_scalars[1] = c->calc->last_virial;
        for (int a = 0; a < 3; ++a) out_scalars[2 + a] = c->calc->last_virial_diag[a];
        sys.local_bonds_.clear(); sys.local_angles_.clear(); sys.local_dihedrals_.clear(); sys.local_impropers_.clear();
        sys.local_special_pairs_.clear();
    } catch (const std::exception& e) {
        std::cerr << "dsmd_ref_bonded: " << e.what() << std::endl;
        return 1;
    }
    return 0;
}

}  // extern "C"
