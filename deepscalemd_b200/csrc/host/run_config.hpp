// The run description of an MD job: the reference's YAML subset (one "key: value" per line, a few sections), read by a
// line-based reader with the reference's rules (docs/03_Input_Reference.md:24-48, src/md_simulation.cpp:2753-3100).
// Only the keys that the short-range nonbonded path and its MD driver use are interpreted; every other key of the
// reference's grammar is kept as text, so that a driver can tell "not supported here" from "misspelled".
#pragma once

#include <map>
#include <string>
#include <vector>

namespace dsmd::host {

struct RunConfig {
    // input files (resolved: an input_system manifest fills the ones that the YAML leaves out)
    std::string coordinate_file, topology_file, parameter_file, input_system;
    // box
    double box[3] = {0.0, 0.0, 0.0};
    bool periodic[3] = {false, false, false};
    // dynamics
    double target_temperature = 0.0;   // K
    double timestep = 0.0;             // fs
    long long total_steps = 0;
    std::string integrator = "verlet";           // the reference's initial value; unknown names mean velocity Verlet
    std::string thermostat = "none";
    double tau_t = 100.0;                        // fs
    std::string barostat = "none";
    // pair interactions and list
    double cutoff_distance = 12.0;               // A
    double lj_switch_distance = -1.0;            // off
    double verlet_skin = 2.0;                    // A
    long long neighbor_list_update_freq = 10;
    double neighbor_rebuild_hi_frac = 0.5, neighbor_rebuild_lo_frac = 0.4;
    // force_calculation section
    std::string force_mode = "builtin", force_type, force_precision = "double", nonbonded_kernel = "tiled";
    bool enable_lennard_jones = true, enable_coulomb = true;
    bool enable_bonds = true, enable_angles = true, enable_dihedrals = true;   // dihedrals: impropers with them
    bool enable_bonded() const { return enable_bonds || enable_angles || enable_dihedrals; }
    // output and restart
    std::string output_prefix = "md_output", output_info = "STEP, T, KE";
    long long output_freq = 10, energy_output_freq = 10, trajectory_output_freq = 100;
    std::string trajectory_format = "xyz";       // comma list; "both" = xyz,dump
    bool trajectory_include_velocities = false, trajectory_include_forces = false;
    std::string restart_file, restart_output;
    long long restart_output_freq = 0;
    // keys this implementation adds (the reference ignores unknown keys): seed of the initial velocities
    long long velocity_seed = 12345;

    // every "section.key" (top level: "key") that was read, as text, in file order
    std::vector<std::pair<std::string, std::string>> entries;

    bool has(const std::string& key) const;
    const std::string& text(const std::string& key) const;   // "" when absent

    // Which of the requested features the B200 path does not cover (empty = runnable): anything but the built-in LJ /
    // real-space Ewald terms with velocity Verlet and no thermostat or Nose-Hoover.
    std::vector<std::string> unsupported() const;

    std::string to_json() const;
};

// Throws std::runtime_error with the reference's messages ("Cannot open config file: ...", "Missing required
// configuration parameters: ...").
RunConfig read_run_config(const std::string& path);

// manifest.yaml of a dsMD_input folder: flat "key: value" lines; schema_version must be 1 and format dsMD_input
// (src/md_simulation.cpp:280-303).
std::map<std::string, std::string> read_manifest(const std::string& path);

}  // namespace dsmd::host
