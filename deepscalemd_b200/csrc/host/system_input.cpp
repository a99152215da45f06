#include "system_input.hpp"

#include <algorithm>
#include <cmath>
#include <fstream>
#include <limits>
#include <map>
#include <sstream>
#include <stdexcept>

#include "text_util.hpp"

namespace dsmd::host {

namespace {

// A data line of the bracketed formats: the text behind the first ';' or '#' is a comment.
std::vector<std::string> data_tokens(std::string line) {
    const size_t cut = line.find_first_of(";#");
    if (cut != std::string::npos) line.erase(cut);
    return words(line);
}

// "[ name ]" -> lower-case name; false when the line is not a section header.
bool section_header(const std::string& cleaned, std::string& name) {
    if (cleaned.size() < 2 || cleaned.front() != '[' || cleaned.back() != ']') return false;
    name = lowered(trimmed(cleaned.substr(1, cleaned.size() - 2), " \t"));
    return true;
}

std::pair<int, int> ordered(int a, int b) { return {std::min(a, b), std::max(a, b)}; }

int to_int(const std::string& s) { return std::stoi(s); }
double to_real(const std::string& s) { return std::stod(s); }

void require_atom_count(const SystemInput& s, size_t topology_atoms, const std::string& path) {
    if (static_cast<size_t>(s.n) != topology_atoms)
        throw std::runtime_error("topology " + path + " describes " + std::to_string(topology_atoms) +
                                 " atoms, the coordinate file has " + std::to_string(s.n));
}

}  // namespace

void read_xyz(const std::string& raw_path, const double box[3], SystemInput& out) {
    const std::string path = clean_file_name(raw_path);
    std::ifstream file(path);
    if (!file.is_open()) throw std::runtime_error("coordinate file " + path + " cannot be opened");
    std::string line;
    std::getline(file, line);
    long long declared = 0;
    try {
        declared = std::stoll(line);
    } catch (const std::exception&) {
        throw std::runtime_error("coordinate file " + path + ": the first line must be the atom count");
    }
    if (declared <= 0 || declared >= (1ll << 30)) throw std::runtime_error("coordinate file " + path + ": bad atom count");
    std::getline(file, line);   // comment line
    const size_t n = static_cast<size_t>(declared);
    out = SystemInput();
    out.n = declared;
    out.x.resize(n); out.y.resize(n); out.z.resize(n);
    out.vx.assign(n, 0.0); out.vy.assign(n, 0.0); out.vz.assign(n, 0.0);
    out.mass.assign(n, 1.0); out.charge.assign(n, 0.0);
    out.type.assign(n, 0);
    out.element.assign(n, std::string());
    size_t read = 0;
    while (read < n && std::getline(file, line)) {
        std::istringstream in(line);
        std::string element;
        double px, py, pz;
        if (in >> element >> px >> py >> pz) {
            out.element[read] = element;
            out.x[read] = px; out.y[read] = py; out.z[read] = pz;
            ++read;
        }
    }
    if (read != n)
        throw std::runtime_error("coordinate file " + path + ": line 1 announces " + std::to_string(n) + " atoms, " + std::to_string(read) +
                                 " usable 'element x y z' lines follow");
    // recentre: mean position -> box centre (plain sums in file order, as the reference adds them)
    double mean[3] = {0.0, 0.0, 0.0};
    for (size_t i = 0; i < n; ++i) { mean[0] += out.x[i]; mean[1] += out.y[i]; mean[2] += out.z[i]; }
    for (double& m : mean) m /= static_cast<double>(n);
    for (int a = 0; a < 3; ++a) out.shift[a] = box[a] / 2.0 - mean[a];
    for (size_t i = 0; i < n; ++i) { out.x[i] += out.shift[0]; out.y[i] += out.shift[1]; out.z[i] += out.shift[2]; }
    out.ntypes = 1;
    out.type_name = {""};
    out.epsilon = {0.0};
    out.sigma = {0.0};
}

void apply_legacy_topology(const std::string& raw_path, SystemInput& s) {
    const std::string path = clean_file_name(raw_path);
    std::ifstream file(path);
    if (!file.is_open()) throw std::runtime_error("topology file " + path + " cannot be opened");
    struct TypeRow { double mass, charge, sigma, epsilon; };
    std::map<std::string, TypeRow> rows;
    std::vector<std::string> atom_type_name;   // by 0-based atom id; "" = never named
    std::string line, section;
    while (std::getline(file, line)) {
        if (!line.empty() && line.back() == '\r') line.pop_back();
        if (line.empty() || line[0] == '#' || line[0] == ';') continue;   // comment marks count in column 1 only
        const std::string cleaned = trimmed(line, " \t");
        if (cleaned.empty()) continue;
        if (section_header(cleaned, section)) continue;
        const auto t = words(cleaned);
        if (t.empty()) continue;
        if (section == "atomtypes") {
            if (t.size() >= 5) rows[t[0]] = TypeRow{to_real(t[1]), to_real(t[2]), to_real(t[3]), to_real(t[4])};
        } else if (section == "atoms") {
            if (t.size() >= 2) {
                const int id = to_int(t[0]) - 1;
                if (id < 0) throw std::runtime_error("topology " + path + ": atom ids start at 1");
                if (static_cast<size_t>(id) >= atom_type_name.size()) atom_type_name.resize(static_cast<size_t>(id) + 1);
                atom_type_name[static_cast<size_t>(id)] = t[1];
            }
        } else if (section == "bonds") {
            if (t.size() >= 3) ++s.n_bonds;
        } else if (section == "angles") {
            if (t.size() >= 4) ++s.n_angles;
        } else if (section == "dihedrals") {
            if (t.size() >= 5) ++s.n_dihedrals;
        }
    }
    require_atom_count(s, atom_type_name.size(), path);
    // type ids: order of first appearance among the atoms
    std::map<std::string, int> id_of;
    s.type_name.clear();
    std::vector<TypeRow> by_id;
    for (size_t i = 0; i < atom_type_name.size(); ++i) {
        const std::string& name = atom_type_name[i];
        auto found = id_of.find(name);
        if (found == id_of.end()) {
            const auto row = rows.find(name);
            if (row == rows.end()) throw std::runtime_error("topology " + path + ": [ atoms ] uses type '" + name + "', which [ atomtypes ] does not define");
            found = id_of.emplace(name, static_cast<int>(id_of.size())).first;
            s.type_name.push_back(name);
            by_id.push_back(row->second);
        }
        s.type[i] = found->second;
        s.mass[i] = by_id[static_cast<size_t>(found->second)].mass;
        s.charge[i] = by_id[static_cast<size_t>(found->second)].charge;
    }
    s.ntypes = static_cast<int>(by_id.size());
    s.epsilon.assign(static_cast<size_t>(s.ntypes) * s.ntypes, 0.0);
    s.sigma.assign(s.epsilon.size(), 0.0);
    for (int a = 0; a < s.ntypes; ++a)
        for (int b = 0; b < s.ntypes; ++b) {   // Lorentz-Berthelot (include/md_types.h:122-136)
            s.epsilon[static_cast<size_t>(a) * s.ntypes + b] = std::sqrt(by_id[a].epsilon * by_id[b].epsilon);
            s.sigma[static_cast<size_t>(a) * s.ntypes + b] = 0.5 * (by_id[a].sigma + by_id[b].sigma);
        }
    s.explicit_pairs = false;
    s.mie_n = 12;
    s.mie_m = 6;
    s.exclusions.clear();
    s.constraints.clear();
}

void apply_dsmd_input(const std::string& raw_topology, const std::string& raw_parameters, SystemInput& s) {
    const std::string topology_path = clean_file_name(raw_topology), parameter_path = clean_file_name(raw_parameters);
    const double nan = std::numeric_limits<double>::quiet_NaN();

    // ---- parameter file ------------------------------------------------------------------------------------------------
    std::ifstream parameters(parameter_path);
    if (!parameters) throw std::runtime_error("parameter file " + parameter_path + " cannot be opened");
    std::map<int, std::string> type_names;
    struct PairRow { int i, j; double sigma, epsilon; };
    std::vector<PairRow> pair_rows;
    struct Harmonic { double k, at; };
    struct Periodic { double k, phase; int n; };
    std::map<std::string, Harmonic> bond_ids, angle_ids;
    std::map<std::string, Periodic> torsion_ids, improper_ids;
    std::map<int, std::pair<double, double>> special_ids;   // sigma, epsilon
    // degrees to radians as the reference writes it, (value * pi) / 180: the same roundings, the same bits
    auto radians = [](double degrees) { return degrees * 3.14159265358979323846 / 180.0; };
    bool mie_seen = false;
    std::string line, section;
    size_t line_number = 0;
    while (std::getline(parameters, line)) {
        ++line_number;
        const std::string cleaned = trimmed(line);
        if (cleaned.empty() || cleaned[0] == ';' || cleaned[0] == '#') continue;
        if (section_header(cleaned, section)) continue;
        const auto t = data_tokens(line);
        if (t.empty()) continue;
        auto fail = [&](const std::string& what) {
            throw std::runtime_error(parameter_path + ":" + std::to_string(line_number) + ": " + what);
        };
        if (section == "meta") {
            if (t.size() < 2) fail("a [meta] line is 'key value'");
            if (t[0] == "schema_version" && t[1] != "1") fail("schema_version " + t[1] + " is not understood (this reader knows version 1)");
            if (t[0] == "length_unit" && t[1] != "angstrom") fail("lengths must be given in angstrom (length_unit)");
            if (t[0] == "energy_unit" && t[1] != "kcal_per_mol") fail("energies must be given in kcal_per_mol (energy_unit)");
            if (t[0] == "charge_unit" && t[1] != "elementary_charge") fail("charges must be given in elementary_charge (charge_unit)");
        } else if (section == "nonbonded") {
            if (t[0] == "component") {
                bool mie = false;
                int n = -1, m = -1;
                for (const auto& w : t) {
                    if (w == "mie") mie = true;
                    if (w.rfind("n=", 0) == 0) n = to_int(w.substr(2));
                    if (w.rfind("m=", 0) == 0) m = to_int(w.substr(2));
                }
                if (mie) {
                    if (mie_seen) fail("a second Mie component: one pair potential per system");
                    if (!((n == 12 && m == 6) || (n == 9 && m == 6))) fail("Mie exponents n=" + std::to_string(n) + " m=" + std::to_string(m) + ": only 12-6 and 9-6 exist here");
                    s.mie_n = n;
                    s.mie_m = m;
                    mie_seen = true;
                }
            }
        } else if (section == "atom_types") {
            if (t.size() < 2) fail("an [atom_types] line is 'id name'");
            const int id = to_int(t[0]);
            if (id < 0 || !type_names.emplace(id, t[1]).second) fail("atom type id " + t[0] + " is negative or given twice");
        } else if (section == "pair_parameters") {
            if (t.size() < 5) fail("a [pair_parameters] line has five fields: component, two type ids, sigma, epsilon");
            pair_rows.push_back({to_int(t[1]), to_int(t[2]), to_real(t[3]), to_real(t[4])});
        } else if (section == "bond_parameters") {
            if (t.size() < 4 || t[1] != "harmonic") fail("bond parameters must read 'id harmonic k r0'");
            const double k = to_real(t[2]), r0 = to_real(t[3]);
            if (!std::isfinite(k) || !std::isfinite(r0) || k < 0.0 || r0 <= 0.0) fail("a bond needs a finite k >= 0 and a finite r0 > 0");
            if (!bond_ids.emplace(t[0], Harmonic{k, r0}).second) fail("bond parameter id " + t[0] + " is given twice");
        } else if (section == "angle_parameters") {
            if (t.size() < 4 || t[1] != "harmonic") fail("angle parameters must read 'id harmonic k theta0' (degrees)");
            const double k = to_real(t[2]), theta = radians(to_real(t[3]));
            if (!std::isfinite(k) || !std::isfinite(theta) || k < 0.0) fail("an angle needs a finite k >= 0 and a finite theta0");
            if (!angle_ids.emplace(t[0], Harmonic{k, theta}).second) fail("angle parameter id " + t[0] + " is given twice");
        } else if (section == "torsion_parameters") {
            if (t.size() < 5 || t[1] != "periodic") fail("torsion parameters must read 'id periodic k phase multiplicity' (phase in degrees)");
            const double k = to_real(t[2]), phase = radians(to_real(t[3]));
            const int multiplicity = to_int(t[4]);
            if (!std::isfinite(k) || !std::isfinite(phase) || multiplicity <= 0) fail("a torsion needs finite k and phase and a multiplicity > 0");
            if (!torsion_ids.emplace(t[0], Periodic{k, phase, multiplicity}).second) fail("torsion parameter id " + t[0] + " is given twice");
        } else if (section == "improper_parameters") {
            if (t.size() < 4 || (t[1] != "periodic" && t[1] != "harmonic"))
                fail("improper parameters must read 'id periodic k phase multiplicity' or 'id harmonic k phi0' (degrees)");
            const double k = to_real(t[2]), phase = radians(to_real(t[3]));
            const int multiplicity = t[1] == "harmonic" ? 0 : (t.size() >= 5 ? to_int(t[4]) : -1);
            if (!std::isfinite(k) || !std::isfinite(phase) || k < 0.0 || (t[1] == "periodic" && multiplicity <= 0))
                fail("an improper needs a finite k >= 0, a finite phase and, in the periodic form, a multiplicity > 0");
            if (!improper_ids.emplace(t[0], Periodic{k, phase, multiplicity}).second) fail("improper parameter id " + t[0] + " is given twice");
        } else if (section == "special_pair_parameters") {
            if (t.size() < 3) fail("a [special_pair_parameters] line is 'id sigma epsilon'");
            const int id = to_int(t[0]);
            const double sigma = to_real(t[1]), epsilon = to_real(t[2]);
            if (id < 0 || !std::isfinite(sigma) || !std::isfinite(epsilon) || sigma < 0.0 || epsilon < 0.0 ||
                !special_ids.emplace(id, std::make_pair(sigma, epsilon)).second)
                fail("a special pair parameter needs an id >= 0 given once and finite sigma, epsilon >= 0");
        } else {
            fail("unknown parameter section [" + section + "]");
        }
    }
    if (!mie_seen) throw std::runtime_error("parameter file " + parameter_path + ": [nonbonded] names no Mie component");
    if (type_names.empty()) throw std::runtime_error("parameter file " + parameter_path + ": the [atom_types] section is missing or empty");
    const int nt = type_names.rbegin()->first + 1;
    if (static_cast<int>(type_names.size()) != nt) throw std::runtime_error("parameter file " + parameter_path + ": atom type ids must run 0, 1, 2, ... without gaps");
    std::vector<double> sig(static_cast<size_t>(nt) * nt, nan), eps(sig.size(), nan);
    for (const PairRow& r : pair_rows) {
        if (r.i < 0 || r.j < 0 || r.i >= nt || r.j >= nt) throw std::runtime_error("[pair_parameters] names the type pair " + std::to_string(r.i) + "," + std::to_string(r.j) + ": invalid atom type ID");
        if (!std::isfinite(r.sigma) || !std::isfinite(r.epsilon) || r.sigma < 0.0 || r.epsilon < 0.0)
            throw std::runtime_error("[pair_parameters] " + std::to_string(r.i) + "," + std::to_string(r.j) + ": sigma and epsilon must be finite numbers >= 0");
        const size_t ab = static_cast<size_t>(r.i) * nt + r.j, ba = static_cast<size_t>(r.j) * nt + r.i;
        if (std::isfinite(sig[ab]) || std::isfinite(eps[ab]))
            throw std::runtime_error("[pair_parameters] gives the type pair " + std::to_string(r.i) + "," + std::to_string(r.j) + " twice");
        sig[ab] = sig[ba] = r.sigma;
        eps[ab] = eps[ba] = r.epsilon;
    }
    for (int a = 0; a < nt; ++a)
        for (int b = 0; b < nt; ++b)
            if (!std::isfinite(sig[static_cast<size_t>(a) * nt + b]) || !std::isfinite(eps[static_cast<size_t>(a) * nt + b]))
                throw std::runtime_error("[pair_parameters] has no line for the type pair " + std::to_string(a) + "," + std::to_string(b) +
                                         " (every pair of types needs one)");

    // ---- topology file -------------------------------------------------------------------------------------------------
    std::ifstream topology(topology_path);
    if (!topology) throw std::runtime_error("topology file " + topology_path + " cannot be opened");
    section.clear();
    line_number = 0;
    long long expected_atoms = -1;
    std::vector<int> type;
    std::vector<double> mass, charge;
    std::vector<std::pair<int, int>> listed, bond_ends, angle_ends, dihedral_ends, improper_atoms, special;
    std::vector<std::string> bond_par, angle_par, dihedral_par, improper_par;
    struct SpecialRow { int param; double lj_scale, coulomb_scale; };
    std::vector<SpecialRow> special_rows;
    std::vector<Constraint> constraints;
    struct Quad { int a, b, c, d; };
    std::vector<Quad> angles3, dihedrals4, impropers4;
    while (std::getline(topology, line)) {
        ++line_number;
        const std::string cleaned = trimmed(line);
        if (cleaned.empty() || cleaned[0] == ';' || cleaned[0] == '#') continue;
        if (section_header(cleaned, section)) continue;
        const auto t = data_tokens(line);
        if (t.empty()) continue;
        auto fail = [&](const std::string& what) {
            throw std::runtime_error(topology_path + ":" + std::to_string(line_number) + ": " + what);
        };
        if (section == "meta") {
            if (t.size() < 2) fail("a [meta] line is 'key value'");
            if (t[0] == "schema_version" && t[1] != "1") fail("schema_version " + t[1] + " is not understood (this reader knows version 1)");
            if (t[0] == "atom_count") {
                expected_atoms = std::stoll(t[1]);
                if (expected_atoms <= 0) fail("atom_count " + t[1] + ": must be at least 1");
            }
        } else if (section == "atoms") {
            if (t.size() < 5) fail("an [atoms] line starts with five fields: id, element, type id, mass, charge");
            if (to_int(t[0]) != static_cast<int>(type.size())) fail("atom ids must run 0, 1, 2, ... in file order (expected " + std::to_string(type.size()) + ")");
            const int type_id = to_int(t[2]);
            if (type_names.find(type_id) == type_names.end()) fail("type id " + t[2] + " is not in the parameter file's [atom_types]");
            const double m = to_real(t[3]), q = to_real(t[4]);
            if (!std::isfinite(m) || m <= 0.0 || !std::isfinite(q))
                fail("mass must be a finite number > 0 and charge a finite number");
            type.push_back(type_id);
            mass.push_back(m);
            charge.push_back(q);
        } else if (section == "bonds") {
            if (t.size() < 3) fail("a [bonds] line is two atom ids and a bond parameter id");
            if (!bond_ids.count(t[2])) fail("bond parameter id " + t[2] + " is not defined in the parameter file");
            bond_ends.push_back({to_int(t[0]), to_int(t[1])});
            bond_par.push_back(t[2]);
        } else if (section == "angles") {
            if (t.size() < 4) fail("an [angles] line is three atom ids and an angle parameter id");
            if (!angle_ids.count(t[3])) fail("angle parameter id " + t[3] + " is not defined in the parameter file");
            angles3.push_back({to_int(t[0]), to_int(t[1]), to_int(t[2]), 0});
            angle_par.push_back(t[3]);
        } else if (section == "dihedrals") {
            if (t.size() < 5) fail("a [dihedrals] line is four atom ids and a torsion parameter id");
            if (!torsion_ids.count(t[4])) fail("torsion parameter id " + t[4] + " is not defined in the parameter file");
            dihedrals4.push_back({to_int(t[0]), to_int(t[1]), to_int(t[2]), to_int(t[3])});
            dihedral_par.push_back(t[4]);
        } else if (section == "exclusions") {
            if (t.size() < 2) fail("an [exclusions] line is two atom ids");
            listed.push_back({to_int(t[0]), to_int(t[1])});
        } else if (section == "impropers") {
            if (t.size() < 5) fail("an [impropers] line is four atom ids and an improper parameter id");
            if (!improper_ids.count(t[4])) fail("improper parameter id " + t[4] + " is not defined in the parameter file");
            impropers4.push_back({to_int(t[0]), to_int(t[1]), to_int(t[2]), to_int(t[3])});
            improper_par.push_back(t[4]);
        } else if (section == "special_pairs") {
            if (t.size() < 5) fail("a [special_pairs] line is two atom ids, a pair parameter id and the LJ and Coulomb scale factors");
            special.push_back({to_int(t[0]), to_int(t[1])});
            special_rows.push_back({to_int(t[2]), to_real(t[3]), to_real(t[4])});
        } else if (section == "constraints") {
            if (t.size() < 3) fail("a [constraints] line is two atom ids and a distance");
            constraints.push_back({to_int(t[0]), to_int(t[1]), to_real(t[2])});
        } else if (section == "virtual_sites") {
            fail("section [" + section + "] is part of the file format, but nothing here can simulate it");
        } else {
            fail("unknown topology section [" + section + "]");
        }
    }
    if (type.empty()) throw std::runtime_error("topology file " + topology_path + ": the [atoms] section is missing or empty");
    if (expected_atoms < 0) throw std::runtime_error("topology file " + topology_path + ": [meta] must state atom_count");
    if (expected_atoms != static_cast<long long>(type.size()))
        throw std::runtime_error("topology file " + topology_path + ": atom_count is " + std::to_string(expected_atoms) + " but [atoms] contains " +
                                 std::to_string(type.size()) + " lines");
    const int n_atoms = static_cast<int>(type.size());
    auto check = [&](int id, const char* kind) {
        if (id < 0 || id >= n_atoms) throw std::runtime_error("a [" + std::string(kind) + "] line names atom " + std::to_string(id) + ", which does not exist");
    };
    for (const auto& b : bond_ends) { check(b.first, "bonds"); check(b.second, "bonds"); }
    for (const auto& a : angles3) { check(a.a, "angles"); check(a.b, "angles"); check(a.c, "angles"); }
    for (const auto& d : dihedrals4) { check(d.a, "dihedrals"); check(d.b, "dihedrals"); check(d.c, "dihedrals"); check(d.d, "dihedrals"); }
    for (const auto& d : impropers4) { check(d.a, "impropers"); check(d.b, "impropers"); check(d.c, "impropers"); check(d.d, "impropers"); }
    for (const auto& p : special) { check(p.first, "special_pairs"); check(p.second, "special_pairs"); }
    for (const auto& c : constraints) {
        check(c.i, "constraints"); check(c.j, "constraints");
        if (!std::isfinite(c.distance) || c.distance <= 0.0) throw std::runtime_error("a [constraints] distance must be a finite number > 0");
    }
    for (const auto& e : listed) { check(e.first, "exclusions"); check(e.second, "exclusions"); }

    std::vector<std::pair<int, int>> exclusions;
    for (const auto& e : listed) exclusions.push_back(ordered(e.first, e.second));
    for (const auto& b : bond_ends) exclusions.push_back(ordered(b.first, b.second));
    for (const auto& a : angles3) exclusions.push_back(ordered(a.a, a.c));
    for (const auto& d : dihedrals4) exclusions.push_back(ordered(d.a, d.d));
    std::sort(exclusions.begin(), exclusions.end());
    exclusions.erase(std::unique(exclusions.begin(), exclusions.end()), exclusions.end());
    for (const auto& p : special)
        if (!std::binary_search(exclusions.begin(), exclusions.end(), ordered(p.first, p.second)))
            throw std::runtime_error("[special_pairs] " + std::to_string(p.first) + "-" + std::to_string(p.second) +
                                     ": the pair must be excluded from the normal pair sum as well ([exclusions] or a bonded term)");

    require_atom_count(s, type.size(), topology_path);
    s.type = type;
    s.mass = mass;
    s.charge = charge;
    s.ntypes = nt;
    s.type_name.clear();
    for (const auto& kv : type_names) s.type_name.push_back(kv.second);
    s.epsilon = eps;
    s.sigma = sig;
    s.explicit_pairs = true;
    s.exclusions = exclusions;
    s.constraints = constraints;
    s.n_bonds = static_cast<int64_t>(bond_ends.size());
    s.n_angles = static_cast<int64_t>(angles3.size());
    s.n_dihedrals = static_cast<int64_t>(dihedrals4.size());
    s.n_impropers = static_cast<int64_t>(impropers4.size());
    s.n_special_pairs = static_cast<int64_t>(special.size());

    // every term with its own parameters, as the device library takes them
    BondedInput& b = s.bonded;
    b = BondedInput();
    for (size_t k = 0; k < bond_ends.size(); ++k) {
        b.bond_atoms.push_back(bond_ends[k].first); b.bond_atoms.push_back(bond_ends[k].second);
        const Harmonic& h = bond_ids.at(bond_par[k]);
        b.bond_k.push_back(h.k); b.bond_r0.push_back(h.at);
    }
    for (size_t k = 0; k < angles3.size(); ++k) {
        b.angle_atoms.push_back(angles3[k].a); b.angle_atoms.push_back(angles3[k].b); b.angle_atoms.push_back(angles3[k].c);
        const Harmonic& h = angle_ids.at(angle_par[k]);
        b.angle_k.push_back(h.k); b.angle_theta0.push_back(h.at);
    }
    auto torsion = [&](const Quad& q, const Periodic& par) {
        b.torsion_atoms.push_back(q.a); b.torsion_atoms.push_back(q.b); b.torsion_atoms.push_back(q.c); b.torsion_atoms.push_back(q.d);
        b.torsion_k.push_back(par.k); b.torsion_phi0.push_back(par.phase); b.torsion_n.push_back(par.n);
    };
    for (size_t k = 0; k < dihedrals4.size(); ++k) torsion(dihedrals4[k], torsion_ids.at(dihedral_par[k]));
    for (size_t k = 0; k < impropers4.size(); ++k) torsion(impropers4[k], improper_ids.at(improper_par[k]));
    for (size_t k = 0; k < special.size(); ++k) {
        b.special_atoms.push_back(special[k].first); b.special_atoms.push_back(special[k].second);
        // a pair whose parameter id is not listed takes the pair matrix of its two atom types (the reference hands the
        // kernel -1 for such a pair and looks the matrix up there: src/force_calculator_cpu.cpp:2820-2821)
        const auto par = special_ids.find(special_rows[k].param);
        const size_t ab = static_cast<size_t>(type[special[k].first]) * nt + type[special[k].second];
        b.special_sigma.push_back(par != special_ids.end() ? par->second.first : sig[ab]);
        b.special_epsilon.push_back(par != special_ids.end() ? par->second.second : eps[ab]);
        b.special_lj_scale.push_back(special_rows[k].lj_scale);
        b.special_coulomb_scale.push_back(special_rows[k].coulomb_scale);
    }
}

}  // namespace dsmd::host
