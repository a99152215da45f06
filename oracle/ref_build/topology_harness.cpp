// Test infrastructure: drives the REFERENCE's own Topology reader (src/topology.cpp, compiled where it lies) on a
// topology / parameter file and returns what it parsed, so that the input layer of this repository can be compared with
// it. Never part of the product.
#include <cstdint>
#include <cstring>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

#include "topology.h"

namespace {

struct Loaded {
    Topology topology;
    bool ok = false;
    std::vector<int> type;
    std::vector<double> mass, charge, sigma, epsilon, pair_sigma, pair_epsilon, constraint_d;
    std::vector<int> exclusion_pairs, constraint_i, constraint_j;
    // bonded terms with the parameters the reader resolved for each of them
    std::vector<int> bond_atoms, angle_atoms, torsion_atoms, torsion_n, special_atoms;
    std::vector<double> bond_par, angle_par, torsion_par, special_par;
    long n_dihedrals = 0;
};

// The reference prints progress to std::cout / std::cerr: keep the test output clean.
struct Quiet {
    std::streambuf* out;
    std::streambuf* err;
    std::ostringstream sink;
    Quiet() : out(std::cout.rdbuf(sink.rdbuf())), err(std::cerr.rdbuf(sink.rdbuf())) {}
    ~Quiet() { std::cout.rdbuf(out); std::cerr.rdbuf(err); }
};

void collect(Loaded& l) {
    const Topology& t = l.topology;
    const int n = t.get_num_atoms();
    for (int i = 0; i < n; ++i) {
        l.type.push_back(t.get_atom_type_id(i));
        l.mass.push_back(t.get_atom_mass(i));
        l.charge.push_back(t.get_atom_charge(i));
        l.sigma.push_back(t.get_atom_sigma(i));
        l.epsilon.push_back(t.get_atom_epsilon(i));
    }
    for (const auto& row : t.get_pair_sigma()) l.pair_sigma.insert(l.pair_sigma.end(), row.begin(), row.end());
    for (const auto& row : t.get_pair_epsilon()) l.pair_epsilon.insert(l.pair_epsilon.end(), row.begin(), row.end());
    for (const std::uint64_t key : t.get_exclusion_keys()) {
        l.exclusion_pairs.push_back(static_cast<int>(key >> 32));
        l.exclusion_pairs.push_back(static_cast<int>(key & 0xffffffffu));
    }
    for (const Constraint& c : t.get_constraints()) {
        l.constraint_i.push_back(c.atom1);
        l.constraint_j.push_back(c.atom2);
        l.constraint_d.push_back(c.distance);
    }
    for (const Bond& b : t.get_bonds()) {
        const BondType& p = t.get_bond_type(b.type);
        l.bond_atoms.insert(l.bond_atoms.end(), {b.atom1, b.atom2});
        l.bond_par.insert(l.bond_par.end(), {p.k, p.r0});
    }
    for (const Angle& a : t.get_angles()) {
        const AngleType& p = t.get_angle_type(a.type);
        l.angle_atoms.insert(l.angle_atoms.end(), {a.atom1, a.atom2, a.atom3});
        l.angle_par.insert(l.angle_par.end(), {p.k, p.theta0});
    }
    auto torsion = [&](const Dihedral& d) {
        const DihedralType& p = t.get_dihedral_type(d.type);
        l.torsion_atoms.insert(l.torsion_atoms.end(), {d.atom1, d.atom2, d.atom3, d.atom4});
        l.torsion_par.insert(l.torsion_par.end(), {p.k, p.phi0});
        l.torsion_n.push_back(p.n);
    };
    for (const Dihedral& d : t.get_dihedrals()) torsion(d);
    l.n_dihedrals = static_cast<long>(t.get_dihedrals().size());
    for (const Dihedral& d : t.get_impropers()) torsion(d);
    for (const SpecialPair& p : t.get_special_pairs()) {
        // sigma / epsilon below zero: the force routines look the pair matrix of the two atom types up
        // (src/force_calculator_cpu.cpp:2820-2821); the same is done here
        const int ti = t.get_atom_type_id(p.atom1), tj = t.get_atom_type_id(p.atom2);
        const double sigma = p.sigma >= 0.0 ? p.sigma : t.get_pair_sigma()[ti][tj];
        const double epsilon = p.epsilon >= 0.0 ? p.epsilon : t.get_pair_epsilon()[ti][tj];
        l.special_atoms.insert(l.special_atoms.end(), {p.atom1, p.atom2});
        l.special_par.insert(l.special_par.end(), {sigma, epsilon, p.lj_scale, p.coulomb_scale});
    }
}

}  // namespace

extern "C" {

// parameter_file empty: legacy .top. Returns null when the reference's reader refuses the files.
void* dsmd_reftop_load(const char* topology_file, const char* parameter_file) {
    auto* l = new Loaded();
    try {
        Quiet quiet;
        const std::string prm = parameter_file ? parameter_file : "";
        l->ok = prm.empty() ? l->topology.load_topology(topology_file, 0) : l->topology.load_canonical(topology_file, prm, 0);
        if (l->ok) collect(*l);
    } catch (const std::exception&) {
        l->ok = false;
    }
    if (!l->ok) {
        delete l;
        return nullptr;
    }
    return l;
}

void dsmd_reftop_destroy(void* h) { delete static_cast<Loaded*>(h); }

void dsmd_reftop_counts(void* h, long* atoms, long* pair_matrix_entries, long* exclusions, long* constraints, int* mie_n,
                        int* mie_m) {
    auto* l = static_cast<Loaded*>(h);
    *atoms = static_cast<long>(l->type.size());
    *pair_matrix_entries = static_cast<long>(l->pair_sigma.size());
    *exclusions = static_cast<long>(l->exclusion_pairs.size() / 2);
    *constraints = static_cast<long>(l->constraint_i.size());
    *mie_n = l->topology.get_mie_repulsive_exponent();
    *mie_m = l->topology.get_mie_attractive_exponent();
}

void dsmd_reftop_atoms(void* h, int* type, double* mass, double* charge, double* sigma, double* epsilon) {
    auto* l = static_cast<Loaded*>(h);
    const size_t n = l->type.size();
    std::memcpy(type, l->type.data(), n * sizeof(int));
    std::memcpy(mass, l->mass.data(), n * sizeof(double));
    std::memcpy(charge, l->charge.data(), n * sizeof(double));
    std::memcpy(sigma, l->sigma.data(), n * sizeof(double));
    std::memcpy(epsilon, l->epsilon.data(), n * sizeof(double));
}

void dsmd_reftop_pairs(void* h, double* pair_sigma, double* pair_epsilon, int* exclusion_pairs, int* constraint_i,
                       int* constraint_j, double* constraint_d) {
    auto* l = static_cast<Loaded*>(h);
    std::memcpy(pair_sigma, l->pair_sigma.data(), l->pair_sigma.size() * sizeof(double));
    std::memcpy(pair_epsilon, l->pair_epsilon.data(), l->pair_epsilon.size() * sizeof(double));
    std::memcpy(exclusion_pairs, l->exclusion_pairs.data(), l->exclusion_pairs.size() * sizeof(int));
    std::memcpy(constraint_i, l->constraint_i.data(), l->constraint_i.size() * sizeof(int));
    std::memcpy(constraint_j, l->constraint_j.data(), l->constraint_j.size() * sizeof(int));
    std::memcpy(constraint_d, l->constraint_d.data(), l->constraint_d.size() * sizeof(double));
}

// counts = {bonds, angles, torsions (dihedrals, then impropers), dihedrals, special pairs}
void dsmd_reftop_bonded_counts(void* h, long counts[5]) {
    auto* l = static_cast<Loaded*>(h);
    counts[0] = static_cast<long>(l->bond_atoms.size() / 2);
    counts[1] = static_cast<long>(l->angle_atoms.size() / 3);
    counts[2] = static_cast<long>(l->torsion_n.size());
    counts[3] = l->n_dihedrals;
    counts[4] = static_cast<long>(l->special_atoms.size() / 2);
}

// atoms: 2, 3, 4, 2 ids per term; parameters: (k, r0), (k, theta0), (k, phi0), (sigma, epsilon, LJ scale, Coulomb scale).
void dsmd_reftop_bonded(void* h, int* bond_atoms, double* bond_par, int* angle_atoms, double* angle_par, int* torsion_atoms,
                        double* torsion_par, int* torsion_n, int* special_atoms, double* special_par) {
    auto* l = static_cast<Loaded*>(h);
    auto copy_i = [](int* dst, const std::vector<int>& v) { if (!v.empty()) std::memcpy(dst, v.data(), v.size() * sizeof(int)); };
    auto copy_d = [](double* dst, const std::vector<double>& v) { if (!v.empty()) std::memcpy(dst, v.data(), v.size() * sizeof(double)); };
    copy_i(bond_atoms, l->bond_atoms); copy_d(bond_par, l->bond_par);
    copy_i(angle_atoms, l->angle_atoms); copy_d(angle_par, l->angle_par);
    copy_i(torsion_atoms, l->torsion_atoms); copy_d(torsion_par, l->torsion_par); copy_i(torsion_n, l->torsion_n);
    copy_i(special_atoms, l->special_atoms); copy_d(special_par, l->special_par);
}

}  // extern "C"

// The reference's real-space Ewald table builder (include/ewald_real_table.h:41-105), header-only: force and energy cubic
// coefficients of every interval, interleaved as the device table is laid out ({force cubic, energy cubic} per interval).
#include "ewald_real_table.h"

extern "C" int dsmd_ref_ewald_table(double alpha, double cutoff_sq, float* out, int capacity_intervals) {
    const int intervals = ewald_real_table_intervals(cutoff_sq);
    if (!out || capacity_intervals < intervals) return intervals;
    std::vector<float> force, energy;
    ewald_real_table_build(alpha, intervals, force, energy);
    for (int i = 0; i < intervals; ++i)
        for (int k = 0; k < 4; ++k) {
            out[8 * i + k] = force[4 * static_cast<size_t>(i) + k];
            out[8 * i + 4 + k] = energy[4 * static_cast<size_t>(i) + k];
        }
    return intervals;
}

