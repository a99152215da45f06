// Test infrastructure, not product code.
//
// Shared by the harness translation units under oracle/ref_build: includes the reference's interface headers with their
// private state opened up (the harnesses fill MDSystem / Topology / ForceManager directly) and defines the few members
// of reference classes whose own source files need MPI, dsDecompX or FFTW and are therefore not part of these builds.
// Include it in exactly one translation unit per library.
#pragma once

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

// The harness fills the private state of MDSystem / Topology / ForceManager directly.
#define private public
#define protected public
#include "md_system.h"
#include "force_calculator_cpu.h"
#include "neighbor_list.h"
#include "topology.h"
#include "force_manager.h"
#include "pme_rank_split.h"
#include "pme_reciprocal_engine.h"
#include "mpi_utils.h"
#undef private
#undef protected

// ---- members of reference classes whose own source files are not part of this build ----------------

MDSystem::MDSystem() : physical_cutoff(0.0), rank(0), size(1) {}
MDSystem::~MDSystem() = default;
void MDSystem::initialize() {}
void MDSystem::finalize() {}

Topology::Topology() : rank(0) {}
Topology::~Topology() = default;
// Bonded parameters by type id: the harness keeps them in plain tables (one entry per term is enough for a check); the
// reference's own tables are string-keyed maps filled by its file reader.
inline std::vector<BondType> g_ref_bond_types;
inline std::vector<AngleType> g_ref_angle_types;
inline std::vector<DihedralType> g_ref_dihedral_types;
int Topology::get_atom_type_id(int atom_id) const { return atom_type_ids.at(static_cast<size_t>(atom_id)); }
const BondType& Topology::get_bond_type(int id) const { return g_ref_bond_types.at(static_cast<size_t>(id)); }
const AngleType& Topology::get_angle_type(int id) const { return g_ref_angle_types.at(static_cast<size_t>(id)); }
const DihedralType& Topology::get_dihedral_type(int id) const { return g_ref_dihedral_types.at(static_cast<size_t>(id)); }

ForceManager::ForceManager() : backend_type("cpu") {}

PmePpSplit& PmePpSplit::instance() {
    static PmePpSplit split;
    return split;
}

bool is_rank_zero() { return false; }   // false: keeps the reference's progress messages off stdout

// Reciprocal space is outside the path under test: the engine only has to hand out the Ewald splitting
// parameter, found as the reference does (bisection of erfc(alpha rc) = 1e-5 on [1e-4, 10/rc], 100 halvings:
// src/pme_reciprocal_engine.cpp:17-24).
PmeReciprocalEngine::~PmeReciprocalEngine() = default;
void PmeReciprocalEngine::ensure_initialized(Real cutoff, const SimulationBox&) {
    if (initialized_) return;
    Real lo = 1e-4, hi = 10.0 / cutoff;
    for (int it = 0; it < 100; ++it) {
        const Real mid = 0.5 * (lo + hi);
        if (std::erfc(mid * cutoff) > 1e-5) lo = mid; else hi = mid;
    }
    ewald_alpha_ = 0.5 * (lo + hi);
    initialized_ = true;
}
void PmeReciprocalEngine::free_resources() { initialized_ = false; }
void PmeReciprocalEngine::ensure_green_cached(const SimulationBox&) {}
void PmeReciprocalEngine::spread_charges(const ParticleData&, size_t, const SimulationBox&) {}
size_t PmeReciprocalEngine::real_grid_size() const { return 0; }
size_t PmeReciprocalEngine::num_k() const { return 0; }
Real PmeReciprocalEngine::solve(Real& virial_out) { virial_out = 0.0; return 0.0; }
Real PmeReciprocalEngine::solve(Real& virial_out, Real d[3]) { virial_out = 0.0; d[0] = d[1] = d[2] = 0.0; return 0.0; }
void PmeReciprocalEngine::set_virial_tensor_enabled(bool enabled) { virial_tensor_enabled_ = enabled; }
void PmeReciprocalEngine::interpolate_forces(ParticleData&, size_t, const SimulationBox&) {}

