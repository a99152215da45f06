#include "restart_file.hpp"

#include <cstring>
#include <filesystem>
#include <fstream>
#include <limits>
#include <stdexcept>

namespace dsmd::host {

namespace {

const char kBegin[8] = {'D', 'S', 'M', 'D', 'R', 'S', 'T', '1'};
const char kEnd[8] = {'D', 'S', 'M', 'D', 'E', 'N', 'D', '1'};

struct Reader {
    std::ifstream in;
    std::string path;
    template <class T>
    T value() {
        T v{};
        in.read(reinterpret_cast<char*>(&v), sizeof(T));
        if (!in) throw std::runtime_error("restart file " + path + " ends early (truncated or not a dsMD restart file)");
        return v;
    }
    std::string text() {
        const int32_t length = value<int32_t>();
        if (length < 0 || length > 4096) throw std::runtime_error("restart file " + path + " is damaged (bad string length)");
        std::string s(static_cast<size_t>(length), '\0');
        if (length > 0) in.read(&s[0], length);
        if (!in) throw std::runtime_error("restart file " + path + " ends early");
        return s;
    }
    std::vector<double> reals() {
        const int32_t count = value<int32_t>();
        if (count < 0 || count > 1024) throw std::runtime_error("restart file " + path + " is damaged (bad state length)");
        std::vector<double> v(static_cast<size_t>(count));
        for (double& x : v) x = value<double>();
        return v;
    }
    void array(std::vector<double>& v) {
        in.read(reinterpret_cast<char*>(v.data()), static_cast<std::streamsize>(v.size() * sizeof(double)));
        if (!in) throw std::runtime_error("restart file " + path + " ends early (truncated)");
    }
};

template <class T>
void put(std::ofstream& out, const T& v) {
    out.write(reinterpret_cast<const char*>(&v), sizeof(T));
}

void put_text(std::ofstream& out, const std::string& s) {
    put<int32_t>(out, static_cast<int32_t>(s.size()));
    out.write(s.data(), static_cast<std::streamsize>(s.size()));
}

void put_reals(std::ofstream& out, const std::vector<double>& v) {
    put<int32_t>(out, static_cast<int32_t>(v.size()));
    for (double x : v) put<double>(out, x);
}

}  // namespace

RestartState read_restart(const std::string& path) {
    Reader r;
    r.path = path;
    r.in.open(path, std::ios::binary);
    if (!r.in.is_open()) throw std::runtime_error("cannot open restart file " + path);
    char magic[8];
    r.in.read(magic, 8);
    if (!r.in || std::memcmp(magic, kBegin, 8) != 0) throw std::runtime_error(path + " is not a dsMD restart file (DSMDRST1)");
    RestartState s;
    s.step = r.value<int64_t>();
    const int64_t atoms = r.value<int64_t>();
    s.timestep = r.value<double>();
    for (double& b : s.box) b = r.value<double>();
    for (int32_t& p : s.periodic) p = r.value<int32_t>();
    s.thermostat = r.text();
    s.thermostat_state = r.reals();
    s.barostat = r.text();
    s.barostat_state = r.reals();
    if (atoms <= 0 || atoms >= (1ll << 30)) throw std::runtime_error("restart file " + path + " has an invalid atom count");
    if (s.step < 0 || s.step > static_cast<int64_t>(std::numeric_limits<int>::max()))
        throw std::runtime_error("restart file " + path + " has an invalid step " + std::to_string(s.step));
    if (!(s.box[0] > 0.0 && s.box[1] > 0.0 && s.box[2] > 0.0)) throw std::runtime_error("restart file " + path + " has an invalid box");
    for (std::vector<double>* a : {&s.x, &s.y, &s.z, &s.vx, &s.vy, &s.vz}) {
        a->resize(static_cast<size_t>(atoms));
        r.array(*a);
    }
    char end[8];
    r.in.read(end, 8);
    if (!r.in || std::memcmp(end, kEnd, 8) != 0) throw std::runtime_error("restart file " + path + " is truncated (no end marker)");
    return s;
}

bool write_restart(const std::string& path, const RestartState& s) {
    const std::string temporary = path + ".tmp";
    bool ok = false;
    {
        std::ofstream out(temporary, std::ios::binary | std::ios::trunc);
        if (out.is_open()) {
            out.write(kBegin, 8);
            put<int64_t>(out, s.step);
            put<int64_t>(out, static_cast<int64_t>(s.x.size()));
            put<double>(out, s.timestep);
            for (double b : s.box) put<double>(out, b);
            for (int32_t p : s.periodic) put<int32_t>(out, p ? 1 : 0);
            put_text(out, s.thermostat);
            put_reals(out, s.thermostat_state);
            put_text(out, s.barostat);
            put_reals(out, s.barostat_state);
            for (const std::vector<double>* a : {&s.x, &s.y, &s.z, &s.vx, &s.vy, &s.vz})
                out.write(reinterpret_cast<const char*>(a->data()), static_cast<std::streamsize>(a->size() * sizeof(double)));
            out.write(kEnd, 8);
            out.flush();
            ok = static_cast<bool>(out);
        }
    }
    std::error_code ec;
    if (ok) std::filesystem::rename(temporary, path, ec);
    return ok && !ec;
}

}  // namespace dsmd::host
