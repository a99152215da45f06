// The particle system of a run as the input files describe it: coordinates (XYZ), atom types / masses / charges and the
// pair-parameter matrix from a legacy .top file or a dsMD_input pair (.dsMDtop + .dsMDprm), exclusions and constraints.
// Formats and rules follow the reference's readers (src/md_system.cpp:562-671, src/topology.cpp:335-881,
// src/md_system.cpp:730-766). The bonded terms of a dsMD_input pair are kept with their parameters resolved per term; those
// of a legacy .top file are counted only.
#pragma once

#include <cstdint>
#include <string>
#include <utility>
#include <vector>

namespace dsmd::host {

struct Constraint {
    int i, j;
    double distance;
};

// Bonded terms with the parameters of every term written out (angles in radians), in the form dsmd_set_bonded takes.
// Torsions: the proper dihedrals first, the impropers behind them; multiplicity 0 marks the harmonic form.
struct BondedInput {
    std::vector<int32_t> bond_atoms, angle_atoms, torsion_atoms, torsion_n, special_atoms;
    std::vector<double> bond_k, bond_r0, angle_k, angle_theta0, torsion_k, torsion_phi0;
    std::vector<double> special_sigma, special_epsilon, special_lj_scale, special_coulomb_scale;
    bool empty() const { return bond_k.empty() && angle_k.empty() && torsion_k.empty() && special_sigma.empty(); }
};

struct SystemInput {
    int64_t n = 0;
    std::vector<double> x, y, z, vx, vy, vz, mass, charge;
    std::vector<int> type;                 // type id per atom
    std::vector<std::string> element;      // first column of the coordinate file
    int ntypes = 0;
    std::vector<std::string> type_name;    // by type id
    std::vector<double> epsilon, sigma;    // [ntypes * ntypes], symmetric
    bool explicit_pairs = false;           // matrix given by the parameter file (else Lorentz-Berthelot)
    int mie_n = 12, mie_m = 6;
    std::vector<std::pair<int, int>> exclusions;   // (smaller id, larger id), sorted, unique
    std::vector<Constraint> constraints;
    int64_t n_bonds = 0, n_angles = 0, n_dihedrals = 0, n_impropers = 0, n_special_pairs = 0;
    BondedInput bonded;                    // filled by apply_dsmd_input; a legacy topology leaves it empty
    double shift[3] = {0.0, 0.0, 0.0};     // what recentring added to every coordinate
};

// Coordinates: line 1 the atom count, line 2 skipped, then "element x y z"; lines that do not parse are skipped; the
// atoms are moved so that their mean position sits at the box centre. Masses 1, charges 0, types 0 until a topology
// is applied.
void read_xyz(const std::string& path, const double box[3], SystemInput& out);

// Legacy .top ([atomtypes] name mass charge sigma epsilon; [atoms] id(1-based) type; bonded sections counted): type ids
// in order of first appearance among the atoms, Lorentz-Berthelot matrix, no exclusions.
void apply_legacy_topology(const std::string& path, SystemInput& system);

// dsMD_input: parameter file ([meta] [nonbonded] [atom_types] [pair_parameters] ...) and topology file ([meta] [atoms]
// [exclusions] [constraints] [bonds] [angles] [dihedrals] ...). Exclusions = listed pairs + bond ends + angle ends +
// dihedral ends, deduplicated.
void apply_dsmd_input(const std::string& topology_path, const std::string& parameter_path, SystemInput& system);

}  // namespace dsmd::host
