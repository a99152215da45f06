// C ABI of the host-side input layer (include/dsmd_input.h).
#include "dsmd_input.h"

#include <cstring>
#include <exception>
#include <stdexcept>
#include <string>
#include <vector>

#include "dynamics.hpp"
#include "../ewald_table.hpp"
#include "brick_plan.hpp"
#include "dart_throw.hpp"
#include "deadline.hpp"
#include "restart_file.hpp"
#include "run_config.hpp"
#include "system_input.hpp"

using namespace dsmd::host;

struct dsmd_input_config {
    RunConfig config;
    std::string json;
};

struct dsmd_input_system {
    SystemInput s;
    std::vector<int32_t> type32, exclusion_pairs, constraint_i, constraint_j;
    std::vector<double> constraint_d;
    void refresh() {
        type32.assign(s.type.begin(), s.type.end());
        exclusion_pairs.clear();
        for (const auto& e : s.exclusions) {
            exclusion_pairs.push_back(e.first);
            exclusion_pairs.push_back(e.second);
        }
        constraint_i.clear(); constraint_j.clear(); constraint_d.clear();
        for (const auto& c : s.constraints) {
            constraint_i.push_back(c.i);
            constraint_j.push_back(c.j);
            constraint_d.push_back(c.distance);
        }
    }
};

namespace {

thread_local std::string g_error;

int failed(int code, const std::string& what) {
    g_error = what;
    return code;
}

template <class F>
int guarded(F&& body) {
    try {
        return body();
    } catch (const std::exception& e) {
        return failed(DSMD_INPUT_ERR_FORMAT, e.what());
    } catch (...) {
        return failed(DSMD_INPUT_ERR_FORMAT, "unknown failure");
    }
}

void load_into(SystemInput& s, const std::string& coordinates, const std::string& topology, const std::string& parameters,
               const double box[3]) {
    read_xyz(coordinates, box, s);
    if (!parameters.empty()) apply_dsmd_input(topology, parameters, s);
    else if (!topology.empty()) apply_legacy_topology(topology, s);
}

}  // namespace

extern "C" {

const char* dsmd_input_last_error(void) { return g_error.c_str(); }

int dsmd_input_config_read(const char* path, dsmd_input_config** out) {
    if (!path || !out) return failed(DSMD_INPUT_ERR_INVALID, "null argument");
    *out = nullptr;
    return guarded([&]() {
        auto* c = new dsmd_input_config();
        try {
            c->config = read_run_config(path);
            c->json = c->config.to_json();
        } catch (...) {
            delete c;
            throw;
        }
        *out = c;
        return DSMD_INPUT_OK;
    });
}

void dsmd_input_config_destroy(dsmd_input_config* config) { delete config; }

int dsmd_input_config_json(const dsmd_input_config* config, const char** json) {
    if (!config || !json) return failed(DSMD_INPUT_ERR_INVALID, "null argument");
    *json = config->json.c_str();
    return DSMD_INPUT_OK;
}

int dsmd_input_system_load(const dsmd_input_config* config, dsmd_input_system** out) {
    if (!config || !out) return failed(DSMD_INPUT_ERR_INVALID, "null argument");
    const RunConfig& c = config->config;
    return dsmd_input_system_load_files(c.coordinate_file.c_str(), c.topology_file.c_str(), c.parameter_file.c_str(), c.box, out);
}

int dsmd_input_system_load_files(const char* coordinate_file, const char* topology_file, const char* parameter_file,
                                 const double box[3], dsmd_input_system** out) {
    if (!coordinate_file || !box || !out) return failed(DSMD_INPUT_ERR_INVALID, "null argument");
    *out = nullptr;
    return guarded([&]() {
        auto* sys = new dsmd_input_system();
        try {
            load_into(sys->s, coordinate_file, topology_file ? topology_file : "", parameter_file ? parameter_file : "", box);
            sys->refresh();
        } catch (...) {
            delete sys;
            throw;
        }
        *out = sys;
        return DSMD_INPUT_OK;
    });
}

void dsmd_input_system_destroy(dsmd_input_system* system) { delete system; }

int dsmd_input_system_counts(const dsmd_input_system* system, int64_t* atoms, int32_t* types, int64_t* exclusions,
                             int64_t* constraints, int32_t* explicit_pairs) {
    if (!system) return failed(DSMD_INPUT_ERR_INVALID, "null argument");
    if (atoms) *atoms = system->s.n;
    if (types) *types = system->s.ntypes;
    if (exclusions) *exclusions = static_cast<int64_t>(system->s.exclusions.size());
    if (constraints) *constraints = static_cast<int64_t>(system->s.constraints.size());
    if (explicit_pairs) *explicit_pairs = system->s.explicit_pairs ? 1 : 0;
    return DSMD_INPUT_OK;
}

int dsmd_input_system_real(const dsmd_input_system* system, int field, const double** data) {
    if (!system || !data) return failed(DSMD_INPUT_ERR_INVALID, "null argument");
    const SystemInput& s = system->s;
    const std::vector<double>* fields[8] = {&s.x, &s.y, &s.z, &s.vx, &s.vy, &s.vz, &s.mass, &s.charge};
    if (field < 0 || field >= 8) return failed(DSMD_INPUT_ERR_INVALID, "field out of range");
    *data = fields[field]->data();
    return DSMD_INPUT_OK;
}

int dsmd_input_system_types(const dsmd_input_system* system, const int32_t** type) {
    if (!system || !type) return failed(DSMD_INPUT_ERR_INVALID, "null argument");
    *type = system->type32.data();
    return DSMD_INPUT_OK;
}

int dsmd_input_system_pair_table(const dsmd_input_system* system, const double** epsilon, const double** sigma,
                                 int32_t* mie_n, int32_t* mie_m) {
    if (!system) return failed(DSMD_INPUT_ERR_INVALID, "null argument");
    if (epsilon) *epsilon = system->s.epsilon.data();
    if (sigma) *sigma = system->s.sigma.data();
    if (mie_n) *mie_n = system->s.mie_n;
    if (mie_m) *mie_m = system->s.mie_m;
    return DSMD_INPUT_OK;
}

int dsmd_input_system_exclusions(const dsmd_input_system* system, const int32_t** pairs) {
    if (!system || !pairs) return failed(DSMD_INPUT_ERR_INVALID, "null argument");
    *pairs = system->exclusion_pairs.data();
    return DSMD_INPUT_OK;
}

int dsmd_input_system_constraints(const dsmd_input_system* system, const int32_t** i, const int32_t** j,
                                  const double** distance) {
    if (!system) return failed(DSMD_INPUT_ERR_INVALID, "null argument");
    if (i) *i = system->constraint_i.data();
    if (j) *j = system->constraint_j.data();
    if (distance) *distance = system->constraint_d.data();
    return DSMD_INPUT_OK;
}

int dsmd_input_system_bonded(const dsmd_input_system* system, int64_t counts[5], const int32_t** atoms[4],
                             const double** parameters[10], const int32_t** torsion_multiplicity) {
    if (!system || !counts) return failed(DSMD_INPUT_ERR_INVALID, "null argument");
    const BondedInput& b = system->s.bonded;
    counts[0] = static_cast<int64_t>(b.bond_k.size());
    counts[1] = static_cast<int64_t>(b.angle_k.size());
    counts[2] = static_cast<int64_t>(b.torsion_k.size());
    counts[3] = b.torsion_k.empty() ? 0 : system->s.n_dihedrals;
    counts[4] = static_cast<int64_t>(b.special_sigma.size());
    if (atoms) {
        const std::vector<int32_t>* a[4] = {&b.bond_atoms, &b.angle_atoms, &b.torsion_atoms, &b.special_atoms};
        for (int k = 0; k < 4; ++k)
            if (atoms[k]) *atoms[k] = a[k]->data();
    }
    if (parameters) {
        const std::vector<double>* p[10] = {&b.bond_k, &b.bond_r0, &b.angle_k, &b.angle_theta0, &b.torsion_k, &b.torsion_phi0,
                                            &b.special_sigma, &b.special_epsilon, &b.special_lj_scale, &b.special_coulomb_scale};
        for (int k = 0; k < 10; ++k)
            if (parameters[k]) *parameters[k] = p[k]->data();
    }
    if (torsion_multiplicity) *torsion_multiplicity = b.torsion_n.data();
    return DSMD_INPUT_OK;
}

int dsmd_input_system_velocities(dsmd_input_system* system, double temperature, uint64_t seed) {
    if (!system) return failed(DSMD_INPUT_ERR_INVALID, "null argument");
    if (!(temperature >= 0.0)) return failed(DSMD_INPUT_ERR_INVALID, "temperature must not be negative");
    maxwell_boltzmann(system->s.mass, temperature, seed, system->s.vx, system->s.vy, system->s.vz);
    return DSMD_INPUT_OK;
}

int dsmd_input_restart_read(const char* path, dsmd_input_system* system, int64_t* step, double box[3], double* timestep,
                            char thermostat_name[64], double* xi) {
    if (!path || !system) return failed(DSMD_INPUT_ERR_INVALID, "null argument");
    return guarded([&]() {
        const RestartState r = read_restart(path);
        SystemInput& s = system->s;
        if (static_cast<int64_t>(r.x.size()) != s.n)
            throw std::runtime_error("restart file " + std::string(path) + " has " + std::to_string(r.x.size()) +
                                     " atoms, the coordinate file has " + std::to_string(s.n));
        s.x = r.x; s.y = r.y; s.z = r.z;
        s.vx = r.vx; s.vy = r.vy; s.vz = r.vz;
        if (step) *step = r.step;
        if (box) for (int a = 0; a < 3; ++a) box[a] = r.box[a];
        if (timestep) *timestep = r.timestep;
        if (thermostat_name) {
            std::strncpy(thermostat_name, r.thermostat.c_str(), 63);
            thermostat_name[63] = '\0';
        }
        if (xi) *xi = (r.thermostat == "nose_hoover" && r.thermostat_state.size() == 1) ? r.thermostat_state[0] : 0.0;
        return DSMD_INPUT_OK;
    });
}

int dsmd_input_restart_write(const char* path, int64_t step, double timestep, const double box[3], const int32_t periodic[3],
                             const char* thermostat_name, const double* thermostat_state, int32_t n_thermostat_state,
                             int64_t atoms, const double* x, const double* y, const double* z, const double* vx,
                             const double* vy, const double* vz) {
    if (!path || !box || !periodic || atoms <= 0 || !x || !y || !z || !vx || !vy || !vz || n_thermostat_state < 0 ||
        (n_thermostat_state > 0 && !thermostat_state))
        return failed(DSMD_INPUT_ERR_INVALID, "null or bad argument");
    return guarded([&]() {
        RestartState r;
        r.step = step;
        r.timestep = timestep;
        for (int a = 0; a < 3; ++a) { r.box[a] = box[a]; r.periodic[a] = periodic[a]; }
        r.thermostat = thermostat_name ? thermostat_name : "none";
        r.thermostat_state.assign(thermostat_state, thermostat_state + n_thermostat_state);
        const size_t n = static_cast<size_t>(atoms);
        r.x.assign(x, x + n); r.y.assign(y, y + n); r.z.assign(z, z + n);
        r.vx.assign(vx, vx + n); r.vy.assign(vy, vy + n); r.vz.assign(vz, vz + n);
        if (!write_restart(path, r)) throw std::runtime_error(std::string("could not write ") + path);
        return DSMD_INPUT_OK;
    });
}

int dsmd_input_nose_hoover_scale(double kinetic_kcal, int64_t atoms, double target_temperature, double tau, double dt,
                                 double dof_fraction, double* xi, double* scale) {
    if (!xi || !scale) return failed(DSMD_INPUT_ERR_INVALID, "null argument");
    *scale = nose_hoover_scale(kinetic_kcal, atoms, target_temperature, tau, dt, *xi, dof_fraction);
    return DSMD_INPUT_OK;
}

// ---- host logic of the multi-GPU domain code, callable without a GPU (CPU tests) ------------------------------------------

int dsmd_host_brick_plan(const int32_t dims[3], int32_t rank, int32_t* n_dirs, int32_t dir_dest[26], int32_t* n_peers,
                         int32_t peers[26], int32_t from_count[26]) {
    if (!dims || !n_dirs || !n_peers || dims[0] < 1 || dims[1] < 1 || dims[2] < 1) return failed(DSMD_INPUT_ERR_INVALID, "null argument");
    const int world = dims[0] * dims[1] * dims[2];
    if (rank < 0 || rank >= world) return failed(DSMD_INPUT_ERR_INVALID, "rank outside the grid");
    const int d[3] = {dims[0], dims[1], dims[2]};
    std::vector<dsmd::host::RankDirs> all(world);
    for (int r = 0; r < world; ++r) all[r] = dsmd::host::dirs_of(d, r);
    const dsmd::host::PeerPlan plan = dsmd::host::peer_plan(all, rank);
    *n_dirs = all[rank].n;
    *n_peers = plan.n_peers;
    for (int k = 0; k < all[rank].n && dir_dest; ++k) dir_dest[k] = all[rank].dest[k];
    for (int p = 0; p < plan.n_peers; ++p) {
        if (peers) peers[p] = plan.peer[p];
        if (from_count) from_count[p] = plan.from_last[p] - plan.from_first[p];
    }
    return DSMD_INPUT_OK;
}

int dsmd_host_counts_verdict(const int32_t dims[3], const int32_t* counts, int64_t scratch_capacity, int32_t* code,
                             int32_t* about_rank, int32_t messages[64]) {
    if (!dims || !counts || !code) return failed(DSMD_INPUT_ERR_INVALID, "null argument");
    const int world = dims[0] * dims[1] * dims[2];
    const int d[3] = {dims[0], dims[1], dims[2]};
    std::vector<dsmd::host::RankDirs> all(world);
    for (int r = 0; r < world; ++r) all[r] = dsmd::host::dirs_of(d, r);
    const dsmd::host::CountsVerdict v = dsmd::host::counts_verdict(all, counts, scratch_capacity, "atoms");
    *code = v.code;
    if (about_rank) *about_rank = v.rank;
    g_error = v.text;
    if (messages) {   // messages each rank posts for these counts: one per neighbour rank and way with anything in it
        for (int r = 0; r < world && r < 64; ++r) {
            const dsmd::host::PeerPlan plan = dsmd::host::peer_plan(all, r);
            int send_to[dsmd::host::kMaxDirs], recv_from[dsmd::host::kMaxDirs];
            long long ns = 0, nr = 0;
            dsmd::host::per_peer_counts(plan, counts, r, send_to, recv_from, ns, nr);
            int m = 0;
            for (int p = 0; p < plan.n_peers; ++p) m += (send_to[p] > 0) + (recv_from[p] > 0);
            messages[r] = m;
        }
    }
    return DSMD_INPUT_OK;
}

int dsmd_host_ewald_table(double alpha, double cutoff_sq, float* out, int32_t capacity_intervals) {
    const int intervals = dsmd::ewald_intervals(cutoff_sq);
    if (!out || capacity_intervals < intervals) return intervals;
    const std::vector<float> coef = dsmd::ewald_build_table(alpha, intervals);
    std::copy(coef.begin(), coef.end(), out);
    return intervals;
}

int dsmd_host_dart_throw(int64_t n, double box, double min_dist, uint64_t seed, double* xyz, int64_t* draws) {
    return guarded([&]() {
        const int64_t used = dart_throw(n, box, min_dist, seed, xyz);
        if (draws) *draws = used;
        return 0;
    });
}

int dsmd_host_wait_probe(double limit_s, int64_t ready_after_polls, int64_t fail_after_polls) {
    int64_t polls = 0;
    const dsmd::host::WaitResult r = dsmd::host::poll_until(
        [&]() {
            ++polls;
            if (fail_after_polls >= 0 && polls > fail_after_polls) return -1;
            if (ready_after_polls >= 0 && polls > ready_after_polls) return 1;
            return 0;
        },
        limit_s);
    return r == dsmd::host::WaitResult::kReady ? 0 : (r == dsmd::host::WaitResult::kTimedOut ? 7 : 2);
}

}  // extern "C"
