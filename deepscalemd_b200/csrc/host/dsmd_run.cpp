// dsmd_b200_run: runs an MD job described by the reference's input files (run description in its YAML subset, XYZ
// coordinates, legacy .top or dsMD_input topology + parameters, optional DSMDRST1 restart file) on the B200 short-range
// nonbonded path, through the C ABI of dsmd_b200.h only. Covers what that path covers: Lennard-Jones (plain cutoff or
// CHARMM switch) and real-space Ewald with exclusions, velocity Verlet, no thermostat or Nose-Hoover, one GPU.
// Anything else the run description asks for is reported and refused, never silently dropped.
//
//   dsmd_b200_run run.yaml [--device N] [--check-input]
//
// --check-input parses every input file, prints the resolved configuration and the system summary as JSON and exits
// without touching the GPU.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iomanip>
#include <iostream>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "dsmd_b200.h"
#include "dynamics.hpp"
#include "restart_file.hpp"
#include "run_config.hpp"
#include "system_input.hpp"
#include "text_util.hpp"

using namespace dsmd::host;

namespace {

struct Options {
    std::string config_file;
    int device = 0;
    bool check_only = false;
};

void ok(dsmd_ctx* ctx, int rc, const char* what) {
    if (rc != DSMD_OK) throw std::runtime_error(std::string(what) + ": " + (ctx ? dsmd_last_error(ctx) : "failed"));
}

// What the device path cannot run for this system, beyond what the run description alone shows.
std::vector<std::string> refusals(const RunConfig& c, const SystemInput& s) {
    std::vector<std::string> out = c.unsupported();
    if (s.mie_n != 12 || s.mie_m != 6) out.push_back("Mie exponents other than (12, 6)");
    // the bonded terms of a dsMD_input system run on the device; a legacy topology's are only counted by the reader
    if (c.enable_bonded() && (s.n_bonds || s.n_angles || s.n_dihedrals || s.n_impropers || s.n_special_pairs) && s.bonded.empty())
        out.push_back("bonded terms of a legacy topology file (switch them off with force_calculation.type: lj[, PME], or "
                      "give the system as a dsMD_input folder)");
    const bool charged = std::any_of(s.charge.begin(), s.charge.end(), [](double q) { return q != 0.0; });
    if (c.enable_coulomb && charged && c.text("real_space_only") != "true")
        out.push_back("electrostatics of a charged system: reciprocal-space PME stays on the reference's path "
                      "(real_space_only: true runs the real-space part alone)");
    for (int a = 0; a < 3; ++a)
        if (!(c.box[a] > 0.0)) out.push_back("box_x / box_y / box_z must be given and positive");
    return out;
}

std::string summary_json(const RunConfig& c, const SystemInput& s, const std::vector<std::string>& refused) {
    std::ostringstream o;
    o << "{\"config\": " << c.to_json() << ", \"system\": {\"atoms\": " << s.n << ", \"types\": " << s.ntypes
      << ", \"explicit_pairs\": " << (s.explicit_pairs ? "true" : "false") << ", \"exclusions\": " << s.exclusions.size()
      << ", \"constraints\": " << s.constraints.size() << ", \"bonds\": " << s.n_bonds << ", \"total_mass\": "
      << std::setprecision(17) << [&] { double m = 0.0; for (double v : s.mass) m += v; return m; }()
      << ", \"total_charge\": " << [&] { double q = 0.0; for (double v : s.charge) q += v; return q; }() << "}, \"refused\": [";
    for (size_t k = 0; k < refused.size(); ++k) {
        std::string text = refused[k];
        for (char& ch : text) if (ch == '"') ch = '\'';
        o << (k ? ", " : "") << "\"" << text << "\"";
    }
    o << "]}";
    return o.str();
}

// The fields of output_info, in the order given, as the reference prints them ("Step: 10, T: 85.1, KE: ...").
struct Metrics {
    double temperature = 0.0, ke = 0.0, pe = 0.0;
};

std::string status_line(const std::string& output_info, long long step, const Metrics& m) {
    std::ostringstream line;
    line << std::fixed << std::setprecision(6);
    std::vector<std::string> fields = comma_list(output_info);
    if (fields.empty()) fields = {"STEP", "T", "KE"};
    for (std::string f : fields) {
        f = uppered(f);
        if (f == "STEP") line << "Step: " << step;
        else if (f == "T") line << ", T: " << m.temperature;
        else if (f == "KE") line << ", KE: " << m.ke;
        else if (f == "PE") line << ", PE: " << m.pe;
        else if (f == "ETOTAL") line << ", Etot: " << m.ke + m.pe;
    }
    return line.str();
}

class Run {
public:
    Run(const RunConfig& c, SystemInput& s, int device, const double box[3]) : c_(c), s_(s) {
        for (int a = 0; a < 3; ++a) box_[a] = box[a];
        ok(nullptr, dsmd_create(device, s.n + 1024, &ctx_), "dsmd_create");
        const int periodic[3] = {c.periodic[0] ? 1 : 0, c.periodic[1] ? 1 : 0, c.periodic[2] ? 1 : 0};
        const double zero[3] = {0.0, 0.0, 0.0};
        ok(ctx_, dsmd_set_box(ctx_, box_, periodic, zero, zero, 0.0), "dsmd_set_box");
    }
    ~Run() {
        if (ctx_) dsmd_destroy(ctx_);
    }
    Run(const Run&) = delete;
    Run& operator=(const Run&) = delete;

    void upload() {
        std::vector<double> eps = s_.epsilon, sig = s_.sigma;
        if (!c_.enable_lennard_jones) std::fill(eps.begin(), eps.end(), 0.0);
        ok(ctx_, dsmd_set_pair_params(ctx_, s_.ntypes, eps.data(), sig.data(), c_.cutoff_distance, c_.verlet_skin,
                                      c_.lj_switch_distance),
           "dsmd_set_pair_params");
        const bool charged = std::any_of(s_.charge.begin(), s_.charge.end(), [](double q) { return q != 0.0; });
        ok(ctx_, dsmd_set_coulomb(ctx_, c_.enable_coulomb && charged ? 1 : 0, 0.0), "dsmd_set_coulomb");
        if (!s_.exclusions.empty()) {
            std::vector<int32_t> a, b;
            for (const auto& e : s_.exclusions) {
                a.push_back(e.first);
                b.push_back(e.second);
            }
            ok(ctx_, dsmd_set_exclusions(ctx_, s_.n, static_cast<int64_t>(a.size()), a.data(), b.data()), "dsmd_set_exclusions");
        }
        if (!s_.constraints.empty()) {   // rigid groups: SHAKE / RATTLE inside the library's integration halves
            std::vector<int32_t> a, b;
            std::vector<double> d;
            for (const auto& k : s_.constraints) {
                a.push_back(k.i);
                b.push_back(k.j);
                d.push_back(k.distance);
            }
            ok(ctx_, dsmd_set_constraints(ctx_, s_.n, static_cast<int64_t>(a.size()), a.data(), b.data(), d.data(), 0.0, 0),
               "dsmd_set_constraints");
        }
        if (!s_.bonded.empty()) {
            const BondedInput& b = s_.bonded;
            // each kind follows its own switch (force_calculation.type / enable_bonds / enable_angles / enable_dihedrals:
            // src/force_manager.cpp:88-160); impropers go with the dihedrals (src/force_calculator_cpu.cpp:798-803)
            const int64_t n_bonds = c_.enable_bonds ? static_cast<int64_t>(b.bond_k.size()) : 0;
            const int64_t n_angles = c_.enable_angles ? static_cast<int64_t>(b.angle_k.size()) : 0;
            const int64_t n_torsions = c_.enable_dihedrals ? static_cast<int64_t>(b.torsion_k.size()) : 0;
            const int64_t n_specials = (c_.enable_lennard_jones || c_.enable_coulomb) ? static_cast<int64_t>(b.special_sigma.size()) : 0;
            // special pairs follow the nonbonded switches: no Lennard-Jones -> epsilon 0, no Coulomb -> scale 0
            std::vector<double> eps14 = b.special_epsilon, coul14 = b.special_coulomb_scale;
            if (!c_.enable_lennard_jones) std::fill(eps14.begin(), eps14.end(), 0.0);
            if (!c_.enable_coulomb) std::fill(coul14.begin(), coul14.end(), 0.0);
            ok(ctx_, dsmd_set_bonded(ctx_, s_.n, n_bonds, b.bond_atoms.data(), b.bond_k.data(), b.bond_r0.data(), n_angles,
                                     b.angle_atoms.data(), b.angle_k.data(), b.angle_theta0.data(), n_torsions,
                                     b.torsion_atoms.data(), b.torsion_k.data(), b.torsion_phi0.data(), b.torsion_n.data(),
                                     n_specials, b.special_atoms.data(), b.special_sigma.data(), eps14.data(),
                                     b.special_lj_scale.data(), coul14.data()),
               "dsmd_set_bonded");
            bonded_ = n_bonds + n_angles + n_torsions + n_specials > 0;
        }
        std::vector<int32_t> type(s_.type.begin(), s_.type.end());
        ok(ctx_, dsmd_upload(ctx_, s_.n, s_.n, s_.x.data(), s_.y.data(), s_.z.data(), s_.vx.data(), s_.vy.data(), s_.vz.data(),
                             s_.mass.data(), s_.charge.data(), type.data(), nullptr, nullptr),
           "dsmd_upload");
        // where every atom of a type carries the same charge (water models, ions, united-atom chains with typed charges)
        // the pair kernel reads the charges from a table by type
        if (c_.enable_coulomb && charged) {
            std::vector<double> by_type(static_cast<size_t>(s_.ntypes), 0.0);
            std::vector<char> seen(by_type.size(), 0);
            bool function_of_type = true;
            for (size_t i = 0; i < s_.type.size() && function_of_type; ++i) {
                const size_t t = static_cast<size_t>(s_.type[i]);
                if (!seen[t]) { seen[t] = 1; by_type[t] = s_.charge[i]; }
                else if (by_type[t] != s_.charge[i]) function_of_type = false;
            }
            if (function_of_type) ok(ctx_, dsmd_set_type_charges(ctx_, s_.ntypes, by_type.data()), "dsmd_set_type_charges");
        }
    }

    void build_list() {
        ok(ctx_, dsmd_build_neighbor_list(ctx_, nullptr), "dsmd_build_neighbor_list");
        ++builds_;
    }

    void forces(bool want_energy) {
        ok(ctx_, dsmd_compute_forces(ctx_, DSMD_PHASE_FULL, want_energy ? 1 : 0, nullptr), "dsmd_compute_forces");
        if (bonded_) ok(ctx_, dsmd_compute_bonded(ctx_, nullptr), "dsmd_compute_bonded");
        if (want_energy) {
            double out[6];
            ok(ctx_, dsmd_read_scalars(ctx_, out, nullptr), "dsmd_read_scalars");
            pe_ = out[0];
            if (bonded_) {
                double terms[5];
                ok(ctx_, dsmd_read_bonded_scalars(ctx_, terms, nullptr), "dsmd_read_bonded_scalars");
                pe_ += terms[0];
            }
        }
    }

    double kinetic_kcal() {
        double raw = 0.0;
        ok(ctx_, dsmd_kinetic_energy(ctx_, &raw, nullptr), "dsmd_kinetic_energy");
        return raw * kMvv2e;
    }

    // One step in the reference's order (MDSimulation::single_step): first half + drift, list rebuild when due (every
    // neighbor_list_update_freq steps by the step counter, or when an atom has moved hi_frac of the skin:
    // src/md_simulation.cpp:1161-1163, 1211-1261), forces, second half, thermostat. `completed` = the step counter
    // before this step.
    void step(long long completed, bool want_energy) {
        ok(ctx_, dsmd_integrate(ctx_, 1, c_.timestep, kForceToAccel, nullptr), "dsmd_integrate");
        bool rebuild = completed > 0 && completed % c_.neighbor_list_update_freq == 0;
        if (!rebuild) {
            double d2 = 0.0;
            ok(ctx_, dsmd_max_displacement_sq(ctx_, &d2, nullptr), "dsmd_max_displacement_sq");
            const double limit = c_.neighbor_rebuild_hi_frac * c_.verlet_skin;
            rebuild = d2 > limit * limit;
        }
        if (rebuild) build_list();
        forces(want_energy);
        ok(ctx_, dsmd_integrate(ctx_, 2, c_.timestep, kForceToAccel, nullptr), "dsmd_integrate");
        if (nose_hoover_) {
            const double scale = nose_hoover_scale(kinetic_kcal(), s_.n, c_.target_temperature, c_.tau_t, c_.timestep, xi_, 1.0);
            ok(ctx_, dsmd_scale_velocities(ctx_, scale, nullptr), "dsmd_scale_velocities");
        }
    }

    // Steps without thermostat, output or restart in between: the library's own loop (displacement read back one step
    // late, as the reference does on several ranks).
    void plain_steps(long long n) {
        int64_t rebuilds = 0;
        double worst = 0.0;
        const long long every = std::min<long long>(c_.neighbor_list_update_freq, 1 << 30);
        ok(ctx_, dsmd_run_nve(ctx_, n, c_.timestep, kForceToAccel, c_.neighbor_rebuild_hi_frac, static_cast<int>(every), 1,
                              &rebuilds, &worst, nullptr),
           "dsmd_run_nve");
        builds_ += rebuilds;
    }

    Metrics metrics() {
        Metrics m;
        m.ke = kinetic_kcal();
        m.pe = pe_;
        m.temperature = temperature_of(m.ke, s_.n, static_cast<int64_t>(s_.constraints.size()));
        return m;
    }

    // Positions and velocities back in global atom id order.
    void download(RestartState& r) {
        const size_t n = static_cast<size_t>(s_.n);
        std::vector<int32_t> gid(n);
        ok(ctx_, dsmd_download(ctx_, DSMD_GLOBAL_ID, s_.n, gid.data(), nullptr), "dsmd_download");
        std::vector<double> buffer(n);
        std::vector<double>* targets[6] = {&r.x, &r.y, &r.z, &r.vx, &r.vy, &r.vz};
        const int fields[6] = {DSMD_X, DSMD_Y, DSMD_Z, DSMD_VX, DSMD_VY, DSMD_VZ};
        for (int f = 0; f < 6; ++f) {
            ok(ctx_, dsmd_download(ctx_, fields[f], s_.n, buffer.data(), nullptr), "dsmd_download");
            targets[f]->assign(n, 0.0);
            for (size_t k = 0; k < n; ++k) (*targets[f])[static_cast<size_t>(gid[k])] = buffer[k];
        }
    }

    // One frame "<output_prefix>_<step>.xyz" in the reference's layout (MDSimulation::write_xyz_trajectory,
    // src/md_simulation.cpp:3819-3863): atom count, a comment line with step, time and energies, then element and
    // position (and velocity, force when asked for) of every atom in coordinate-file order, six decimals.
    void write_xyz_frame(long long step, const Metrics& m) {
        const size_t n = static_cast<size_t>(s_.n);
        std::vector<int32_t> gid(n);
        ok(ctx_, dsmd_download(ctx_, DSMD_GLOBAL_ID, s_.n, gid.data(), nullptr), "dsmd_download");
        std::vector<int> fields = {DSMD_X, DSMD_Y, DSMD_Z};
        if (c_.trajectory_include_velocities) fields.insert(fields.end(), {DSMD_VX, DSMD_VY, DSMD_VZ});
        if (c_.trajectory_include_forces) fields.insert(fields.end(), {DSMD_FX, DSMD_FY, DSMD_FZ});
        std::vector<std::vector<double>> columns(fields.size(), std::vector<double>(n));
        std::vector<double> buffer(n);
        for (size_t f = 0; f < fields.size(); ++f) {
            ok(ctx_, dsmd_download(ctx_, fields[f], s_.n, buffer.data(), nullptr), "dsmd_download");
            for (size_t k = 0; k < n; ++k) columns[f][static_cast<size_t>(gid[k])] = buffer[k];
        }
        const std::string name = c_.output_prefix + "_" + std::to_string(step) + ".xyz";
        std::ofstream out(name);
        if (!out.is_open()) {
            std::cerr << "[trajectory] cannot write to " << name << std::endl;
            return;
        }
        out << n << "\n";
        out << "Step " << step << " Time " << std::fixed << std::setprecision(3) << static_cast<double>(step) * c_.timestep << " fs"
            << " KE=" << std::setprecision(6) << m.ke << " PE=" << m.pe << " Total=" << (m.ke + m.pe) << "\n";
        for (size_t i = 0; i < n; ++i) {
            out << s_.element[i];
            for (size_t f = 0; f < fields.size(); ++f) out << " " << columns[f][i];
            out << "\n";
        }
    }

    void write_restart_file(long long step) {
        RestartState r;
        r.step = step;
        r.timestep = c_.timestep;
        for (int a = 0; a < 3; ++a) {
            r.box[a] = box_[a];
            r.periodic[a] = c_.periodic[a] ? 1 : 0;
        }
        r.thermostat = nose_hoover_ ? "nose_hoover" : "none";
        if (nose_hoover_) r.thermostat_state = {xi_};
        download(r);
        if (write_restart(c_.restart_output, r)) std::cout << "[restart] wrote " << c_.restart_output << " at step " << step << std::endl;
        else std::cerr << "[restart] failed to write " << c_.restart_output << " at step " << step << std::endl;
    }

    bool nose_hoover_ = false;
    bool bonded_ = false;
    double xi_ = 0.0;
    long long builds_ = 0;
    double box_[3] = {0.0, 0.0, 0.0};

private:
    const RunConfig& c_;
    SystemInput& s_;
    dsmd_ctx* ctx_ = nullptr;
    double pe_ = 0.0;
};

int run(const Options& opt) {
    const RunConfig c = read_run_config(opt.config_file);
    SystemInput s;
    read_xyz(c.coordinate_file, c.box, s);
    if (!c.parameter_file.empty()) apply_dsmd_input(c.topology_file, c.parameter_file, s);
    else if (!c.topology_file.empty()) apply_legacy_topology(c.topology_file, s);
    else throw std::runtime_error("topology_file is required: it supplies the atom types, masses and charges");

    double box[3] = {c.box[0], c.box[1], c.box[2]};
    long long start_step = 0;
    double xi = 0.0;
    bool restarted = false;
    if (!c.restart_file.empty()) {
        const RestartState r = read_restart(c.restart_file);
        if (static_cast<int64_t>(r.x.size()) != s.n)
            throw std::runtime_error("restart file " + c.restart_file + " has " + std::to_string(r.x.size()) +
                                     " atoms, the coordinate file " + c.coordinate_file + " has " + std::to_string(s.n));
        s.x = r.x; s.y = r.y; s.z = r.z;
        s.vx = r.vx; s.vy = r.vy; s.vz = r.vz;
        for (int a = 0; a < 3; ++a) box[a] = r.box[a];     // the box of the restart file wins over the YAML's
        start_step = r.step;
        if (r.thermostat == "nose_hoover" && r.thermostat_state.size() == 1) xi = r.thermostat_state[0];
        restarted = true;
    } else {
        maxwell_boltzmann(s.mass, c.target_temperature, static_cast<uint64_t>(c.velocity_seed), s.vx, s.vy, s.vz);
    }

    const auto refused = refusals(c, s);
    if (opt.check_only) {
        std::cout << summary_json(c, s, refused) << std::endl;
        return refused.empty() ? 0 : 3;
    }
    if (!refused.empty()) {
        std::cerr << "dsmd_b200_run: this run description asks for what the B200 nonbonded path does not cover:\n";
        for (const auto& r : refused) std::cerr << "  - " << r << "\n";
        return 3;
    }

    std::cout << "dsmd_b200_run: " << s.n << " atoms, " << s.ntypes << " types, box " << box[0] << " x " << box[1] << " x "
              << box[2] << " A, cutoff " << c.cutoff_distance << " A, skin " << c.verlet_skin << " A, dt " << c.timestep
              << " fs, " << c.total_steps << " steps from step " << start_step << ", thermostat " << trimmed(c.thermostat)
              << (restarted ? ", restarted" : "") << std::endl;

    Run md(c, s, opt.device, box);
    md.nose_hoover_ = trimmed(c.thermostat) == "nose_hoover";
    md.xi_ = xi;
    md.upload();
    md.build_list();
    md.forces(true);

    auto output_due = [&](long long step) { return c.output_freq > 0 && step % c.output_freq == 0; };
    auto trajectory_due = [&](long long step) { return c.trajectory_output_freq > 0 && step % c.trajectory_output_freq == 0; };
    auto restart_due = [&](long long step) {
        return c.restart_output_freq > 0 && (step % c.restart_output_freq == 0 || step == start_step + c.total_steps);
    };
    if (output_due(start_step)) std::cout << status_line(c.output_info, start_step, md.metrics()) << std::endl;
    if (trajectory_due(start_step)) md.write_xyz_frame(start_step, md.metrics());

    const auto t0 = std::chrono::steady_clock::now();
    const long long last = start_step + c.total_steps;
    long long step = start_step;   // steps completed (absolute)
    while (step < last) {
        // steps up to the one before the next output / restart step run without interruption when nothing is applied
        // between steps
        if (!md.nose_hoover_) {
            long long next_event = last;
            for (long long k = step + 1; k <= last; ++k)
                if (output_due(k) || restart_due(k) || trajectory_due(k)) { next_event = k; break; }
            const long long plain = next_event - 1 - step;
            if (plain > 0) {
                md.plain_steps(plain);
                step += plain;
            }
        }
        const long long next = step + 1;
        md.step(step, output_due(next) || trajectory_due(next));
        step = next;
        if (output_due(step)) std::cout << status_line(c.output_info, step, md.metrics()) << std::endl;
        if (trajectory_due(step)) md.write_xyz_frame(step, md.metrics());
        if (restart_due(step)) md.write_restart_file(step);
    }
    const double seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    const double per_step = seconds / static_cast<double>(c.total_steps);
    std::cout << "\nNeighbor list builds = " << md.builds_ << "\n";
    std::cout << "Performance: " << std::fixed << std::setprecision(3) << static_cast<double>(s.n) * c.total_steps / seconds / 1e6
              << " Matom-step/s, " << per_step * 1e3 << " ms/step, " << (c.timestep * 1e-6) * (86400.0 / per_step)
              << " ns/day (md_loop only, dt=" << c.timestep << " fs)\n" << std::endl;
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    Options opt;
    for (int k = 1; k < argc; ++k) {
        const std::string a = argv[k];
        if (a == "--check-input") opt.check_only = true;
        else if (a == "--device" && k + 1 < argc) opt.device = std::atoi(argv[++k]);
        else if (!a.empty() && a[0] != '-' && opt.config_file.empty()) opt.config_file = a;
        else {
            std::cerr << "usage: dsmd_b200_run run.yaml [--device N] [--check-input]" << std::endl;
            return 2;
        }
    }
    if (opt.config_file.empty()) {
        std::cerr << "usage: dsmd_b200_run run.yaml [--device N] [--check-input]" << std::endl;
        return 2;
    }
    try {
        return run(opt);
    } catch (const std::exception& e) {
        std::cerr << "dsmd_b200_run: " << e.what() << std::endl;
        return 1;
    }
}
