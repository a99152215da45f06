#include "run_config.hpp"

#include <filesystem>
#include <fstream>
#include <set>
#include <sstream>

#include "text_util.hpp"

namespace dsmd::host {

namespace {

const std::string kEmpty;

// The sections of the grammar; a key inside one is stored as "section.key" ("advanced.decomposition.key" for the one
// nested sub-section).
const std::set<std::string> kSections = {"force_calculation", "minimize", "advanced", "mlip_config", "mace_config",
                                         "mlip_elements"};

std::string json_escape(const std::string& s) {
    std::string out;
    for (char c : s) {
        if (c == '"' || c == '\\') { out += '\\'; out += c; }
        else if (c == '\n') out += "\\n";
        else if (c == '\t') out += "\\t";
        else if (static_cast<unsigned char>(c) < 0x20) out += ' ';
        else out += c;
    }
    return out;
}

std::string json_number(double v) {
    std::ostringstream s;
    s.precision(17);
    s << v;
    return s.str();
}

// One physical line -> (indent, key, value, header?) following the reference's reader: everything from '#' on is dropped,
// a line without ':' is skipped, the value loses one pair of enclosing double quotes.
struct Line {
    size_t indent = 0;
    std::string key, value;
    bool blank = true, header = false;
};

Line split_line(std::string raw) {
    Line out;
    const size_t hash = raw.find('#');
    if (hash != std::string::npos) raw.erase(hash);
    if (raw.empty()) return out;
    size_t indent = raw.find_first_not_of(" \t");
    if (indent == std::string::npos) return out;
    out.indent = indent;
    const std::string body = trimmed(raw, " \t");
    if (body.empty()) return out;
    const size_t colon = body.find(':');
    if (colon == std::string::npos) return out;
    out.blank = false;
    out.key = trimmed(body.substr(0, colon));
    std::string value = trimmed(body.substr(colon + 1));
    out.header = value.empty();
    if (value.size() >= 2 && value.front() == '"' && value.back() == '"') value = trimmed(value.substr(1, value.size() - 2));
    out.value = value;
    return out;
}

}  // namespace

bool RunConfig::has(const std::string& key) const {
    for (const auto& e : entries)
        if (e.first == key) return true;
    return false;
}

const std::string& RunConfig::text(const std::string& key) const {
    const std::string* found = &kEmpty;
    for (const auto& e : entries)
        if (e.first == key) found = &e.second;   // the last occurrence wins, as in a sequential reader
    return *found;
}

std::map<std::string, std::string> read_manifest(const std::string& path) {
    std::ifstream file(path);
    if (!file) throw std::runtime_error("input system manifest " + path + " cannot be opened");
    std::map<std::string, std::string> values;
    std::string line;
    while (std::getline(file, line)) {
        const size_t hash = line.find('#');
        if (hash != std::string::npos) line.erase(hash);
        const size_t colon = line.find(':');
        if (colon == std::string::npos) continue;
        const std::string key = trimmed(line.substr(0, colon));
        std::string value = trimmed(line.substr(colon + 1));
        if (value.size() >= 2 && ((value.front() == '"' && value.back() == '"') || (value.front() == '\'' && value.back() == '\'')))
            value = value.substr(1, value.size() - 2);
        if (!key.empty() && !value.empty()) values[key] = value;
    }
    if (values["schema_version"] != "1") throw std::runtime_error("input system manifest " + path + ": schema_version must be 1");
    if (values["format"] != "dsMD_input") throw std::runtime_error("input system manifest " + path + ": format must be dsMD_input");
    return values;
}

RunConfig read_run_config(const std::string& path) {
    std::ifstream file(path);
    if (!file.is_open()) throw std::runtime_error("run description " + path + " cannot be opened");
    RunConfig c;
    bool have_coordinates = false, have_temperature = false, have_timestep = false, have_steps = false;
    std::string section, subsection;
    size_t subsection_indent = 0;
    std::string raw;
    while (std::getline(file, raw)) {
        const Line line = split_line(raw);
        if (line.blank) continue;
        const bool indented = line.indent > 0;
        if (line.header && !indented) {           // "name:" at the left margin opens a section
            section = line.key;
            subsection.clear();
            subsection_indent = 0;
            continue;
        }
        if (line.header && indented && section == "advanced") {   // the one nested level: advanced.<name>:
            subsection = line.key;
            subsection_indent = line.indent;
            continue;
        }
        // (an indented "key:" with nothing behind the colon elsewhere is a key with an empty value)
        if (!indented) {                          // an unindented key closes the open section
            section.clear();
            subsection.clear();
            subsection_indent = 0;
        }
        const std::string& key = line.key;
        const std::string& value = line.value;
        // a section name outside the grammar captures nothing: its keys are read as top-level keys
        const bool in_section = kSections.count(section) != 0;
        std::string full = key;
        if (in_section) {
            full = section + "." + key;
            if (section == "advanced" && !subsection.empty() && line.indent > subsection_indent)
                full = section + "." + subsection + "." + key;
        }
        c.entries.emplace_back(full, value);

        if (section == "force_calculation") {
            if (key == "mode" || key == "force_calculation_mode") c.force_mode = trimmed(value);
            else if (key == "type" || key == "force_calculation_type") c.force_type = value;
            else if (key == "precision") c.force_precision = trimmed(value);
            else if (key == "nonbonded_kernel") c.nonbonded_kernel = trimmed(value);
            continue;
        }
        if (in_section) continue;                 // the other sections: kept as text only

        if (key == "input_system") c.input_system = value;
        else if (key == "coordinate_file") { c.coordinate_file = value; have_coordinates = true; }
        else if (key == "topology_file") c.topology_file = value;
        else if (key == "parameter_file") c.parameter_file = value;
        else if (key == "target_temperature") { c.target_temperature = number_of(key, value); have_temperature = true; }
        else if (key == "timestep") { c.timestep = number_of(key, value); have_timestep = true; }
        else if (key == "total_steps") { c.total_steps = integer_of(key, value); have_steps = true; }
        else if (key == "output_prefix") c.output_prefix = value;
        else if (key == "restart_file") c.restart_file = trimmed(value);
        else if (key == "restart_output") c.restart_output = trimmed(value);
        else if (key == "restart_output_freq") c.restart_output_freq = integer_of(key, value);
        else if (key == "trajectory_output_freq") c.trajectory_output_freq = integer_of(key, value);
        else if (key == "trajectory_format") c.trajectory_format = value;
        else if (key == "trajectory_include_velocities") c.trajectory_include_velocities = value == "true";
        else if (key == "trajectory_include_forces") c.trajectory_include_forces = value == "true";
        else if (key == "energy_output_freq") c.energy_output_freq = integer_of(key, value);
        else if (key == "output_freq") c.output_freq = integer_of(key, value);
        else if (key == "output_info") c.output_info = value;
        else if (key == "cutoff_distance" || key == "cutoff") c.cutoff_distance = number_of(key, value);
        else if (key == "lj_switch_distance" || key == "switchdist") c.lj_switch_distance = number_of(key, value);
        else if (key == "neighbor_list_update_freq") c.neighbor_list_update_freq = integer_of(key, value);
        else if (key == "verlet_skin") c.verlet_skin = number_of(key, value);
        else if (key == "neighbor_rebuild_hi_frac") c.neighbor_rebuild_hi_frac = number_of(key, value);
        else if (key == "neighbor_rebuild_lo_frac") c.neighbor_rebuild_lo_frac = number_of(key, value);
        else if (key == "integrator") c.integrator = value;
        else if (key == "thermostat") c.thermostat = value;
        else if (key == "tau_t" || key == "thermostat_damping") c.tau_t = number_of(key, value);
        else if (key == "barostat") c.barostat = value;
        else if (key == "box_x") c.box[0] = number_of(key, value);
        else if (key == "box_y") c.box[1] = number_of(key, value);
        else if (key == "box_z") c.box[2] = number_of(key, value);
        else if (key == "periodic_x") c.periodic[0] = value == "true";   // only the exact text "true"
        else if (key == "periodic_y") c.periodic[1] = value == "true";
        else if (key == "periodic_z") c.periodic[2] = value == "true";
        else if (key == "velocity_seed") c.velocity_seed = integer_of(key, value);
    }

    if (!c.input_system.empty()) {
        const auto manifest = read_manifest(c.input_system);
        const std::filesystem::path base = std::filesystem::absolute(std::filesystem::path(c.input_system)).parent_path();
        auto resolve = [&](const char* key) -> std::string {
            const auto it = manifest.find(key);
            if (it == manifest.end()) return std::string();
            const std::filesystem::path p(it->second);
            return (p.is_absolute() ? p : base / p).lexically_normal().string();
        };
        if (c.coordinate_file.empty()) c.coordinate_file = resolve("coordinate_file");
        if (c.topology_file.empty()) c.topology_file = resolve("topology_file");
        if (c.parameter_file.empty()) c.parameter_file = resolve("parameter_file");
        have_coordinates = !c.coordinate_file.empty();
    }

    std::vector<std::string> missing;
    if (!have_coordinates) missing.push_back("coordinate_file");
    if (!c.input_system.empty() && c.topology_file.empty()) missing.push_back("topology_file");
    if (!c.input_system.empty() && c.parameter_file.empty()) missing.push_back("parameter_file");
    if (!have_temperature) missing.push_back("target_temperature");
    if (!have_timestep) missing.push_back("timestep");
    if (!have_steps) missing.push_back("total_steps");
    if (!missing.empty()) {
        std::string message = "the run description lacks required keys: ";
        for (size_t k = 0; k < missing.size(); ++k) message += (k ? ", " : "") + missing[k];
        throw std::runtime_error(message);
    }

    // force_calculation.mode: a comma list of builtin / mlip
    const auto modes = comma_list(c.force_mode);
    if (modes.empty())
        throw std::runtime_error("force_calculation.mode '" + c.force_mode + "' names no force provider (builtin, mlip, or both separated by a comma)");
    for (const auto& m : modes)
        if (m != "builtin" && m != "mlip")
            throw std::runtime_error("force_calculation.mode: '" + m + "' is not a force provider (builtin and mlip are)");

    // which built-in terms: a "type" list switches every term it does not name off; without it the enable_* keys apply
    // (only the exact text "true" switches a term on), default all on (src/force_manager.cpp:88-160)
    const auto types = comma_list(c.force_type);
    if (!types.empty()) {
        c.enable_lennard_jones = c.enable_coulomb = c.enable_bonds = c.enable_angles = c.enable_dihedrals = false;
        for (std::string t : types) {
            t = trimmed(t, " \t\r\n\"");
            if (t == "lj" || t == "lennard_jones" || t == "LJ") c.enable_lennard_jones = true;
            else if (t == "coulomb" || t == "PME" || t == "electrostatic") c.enable_coulomb = true;
            else if (t == "bonds" || t == "bond") c.enable_bonds = true;
            else if (t == "angles" || t == "angle") c.enable_angles = true;
            else if (t == "dihedrals" || t == "dihedral") c.enable_dihedrals = true;
        }
    } else {
        if (c.has("force_calculation.enable_lennard_jones"))
            c.enable_lennard_jones = c.text("force_calculation.enable_lennard_jones") == "true";
        if (c.has("force_calculation.enable_coulomb")) c.enable_coulomb = c.text("force_calculation.enable_coulomb") == "true";
        if (c.has("force_calculation.enable_bonds")) c.enable_bonds = c.text("force_calculation.enable_bonds") == "true";
        if (c.has("force_calculation.enable_angles")) c.enable_angles = c.text("force_calculation.enable_angles") == "true";
        if (c.has("force_calculation.enable_dihedrals")) c.enable_dihedrals = c.text("force_calculation.enable_dihedrals") == "true";
    }

    {
        std::string formats = trimmed(c.trajectory_format) == "both" ? "xyz,dump" : c.trajectory_format;
        for (const auto& f : comma_list(formats))
            if (f != "xyz" && f != "dump" && f != "dcd" && f != "bp" && f != "h5md")
                throw std::runtime_error("trajectory_format: '" + f + "' is not a trajectory format (xyz, dump, dcd, bp, h5md; 'both' = xyz,dump)");
    }
    if (c.total_steps <= 0) throw std::runtime_error("total_steps must be positive");
    if (c.target_temperature < 0.0) throw std::runtime_error("target_temperature must not be negative");
    if (c.neighbor_list_update_freq <= 0) throw std::runtime_error("neighbor_list_update_freq must be positive");
    if (c.lj_switch_distance >= 0.0 && !(c.lj_switch_distance > 0.0 && c.lj_switch_distance < c.cutoff_distance))
        throw std::runtime_error("lj_switch_distance must be positive and smaller than cutoff_distance");
    if (c.restart_output.empty()) c.restart_output = c.output_prefix + ".restart";
    return c;
}

std::vector<std::string> RunConfig::unsupported() const {
    std::vector<std::string> out;
    for (const auto& m : comma_list(force_mode))
        if (m == "mlip") out.push_back("force_calculation.mode: mlip (the model runners are outside the nonbonded path)");
    const std::string integ = lowered(trimmed(integrator));
    if (integ == "leap_frog" || integ == "leapfrog") out.push_back("integrator: " + integ + " (velocity Verlet only)");
    if (integ == "r_respa") out.push_back("integrator: r_respa");
    const std::string thermo = trimmed(thermostat);
    if (thermo == "langevin" || thermo == "andersen") out.push_back("thermostat: " + thermo + " (none or nose_hoover)");
    if (trajectory_output_freq > 0) {
        const std::string formats = trimmed(trajectory_format) == "both" ? "xyz,dump" : trajectory_format;
        for (const auto& f : comma_list(formats))
            if (f != "xyz") out.push_back("trajectory_format: " + f + " (xyz frames only)");
    }
    const std::string baro = trimmed(barostat);
    if (baro == "berendsen" || baro == "parrinello_rahman" || baro == "andersen") out.push_back("barostat: " + baro);
    return out;
}

std::string RunConfig::to_json() const {
    std::ostringstream s;
    auto str = [&](const char* k, const std::string& v) { s << "\"" << k << "\": \"" << json_escape(v) << "\", "; };
    auto num = [&](const char* k, double v) { s << "\"" << k << "\": " << json_number(v) << ", "; };
    auto integer = [&](const char* k, long long v) { s << "\"" << k << "\": " << v << ", "; };
    auto boolean = [&](const char* k, bool v) { s << "\"" << k << "\": " << (v ? "true" : "false") << ", "; };
    s << "{";
    str("coordinate_file", coordinate_file); str("topology_file", topology_file); str("parameter_file", parameter_file);
    str("input_system", input_system);
    s << "\"box\": [" << json_number(box[0]) << ", " << json_number(box[1]) << ", " << json_number(box[2]) << "], ";
    s << "\"periodic\": [" << (periodic[0] ? "true" : "false") << ", " << (periodic[1] ? "true" : "false") << ", "
      << (periodic[2] ? "true" : "false") << "], ";
    num("target_temperature", target_temperature); num("timestep", timestep); integer("total_steps", total_steps);
    str("integrator", integrator); str("thermostat", thermostat); num("tau_t", tau_t); str("barostat", barostat);
    num("cutoff_distance", cutoff_distance); num("lj_switch_distance", lj_switch_distance); num("verlet_skin", verlet_skin);
    integer("neighbor_list_update_freq", neighbor_list_update_freq);
    num("neighbor_rebuild_hi_frac", neighbor_rebuild_hi_frac); num("neighbor_rebuild_lo_frac", neighbor_rebuild_lo_frac);
    str("force_mode", force_mode); str("force_type", force_type); str("force_precision", force_precision);
    str("nonbonded_kernel", nonbonded_kernel);
    boolean("enable_lennard_jones", enable_lennard_jones); boolean("enable_coulomb", enable_coulomb);
    boolean("enable_bonded", enable_bonded());
    boolean("enable_bonds", enable_bonds);
    boolean("enable_angles", enable_angles);
    boolean("enable_dihedrals", enable_dihedrals);
    str("output_prefix", output_prefix); str("output_info", output_info); integer("output_freq", output_freq);
    integer("energy_output_freq", energy_output_freq); integer("trajectory_output_freq", trajectory_output_freq);
    str("trajectory_format", trajectory_format); boolean("trajectory_include_velocities", trajectory_include_velocities);
    boolean("trajectory_include_forces", trajectory_include_forces);
    str("restart_file", restart_file); str("restart_output", restart_output);
    integer("restart_output_freq", restart_output_freq); integer("velocity_seed", velocity_seed);
    s << "\"unsupported\": [";
    const auto u = unsupported();
    for (size_t k = 0; k < u.size(); ++k) s << (k ? ", " : "") << "\"" << json_escape(u[k]) << "\"";
    s << "], \"entries\": [";
    for (size_t k = 0; k < entries.size(); ++k)
        s << (k ? ", " : "") << "[\"" << json_escape(entries[k].first) << "\", \"" << json_escape(entries[k].second) << "\"]";
    s << "]}";
    return s.str();
}

}  // namespace dsmd::host
