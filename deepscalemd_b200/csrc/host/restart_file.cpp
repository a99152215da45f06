#include "restart_file.hpp"

#include <cstdio>
#include <cstring>
#include <filesystem>
#include <limits>
#include <stdexcept>

namespace dsmd::host {

namespace {

constexpr char kHead[] = "DSMDRST1";
constexpr char kTail[] = "DSMDEND1";
constexpr size_t kTag = 8;
constexpr int32_t kLongestName = 4096;    // thermostat / barostat names
constexpr int32_t kMostStateValues = 1024;

// The file is small next to device memory traffic (48 bytes per atom): it is read whole, then taken apart from a byte
// image with a moving offset, and written the same way in reverse.
class ByteImage {
public:
    ByteImage(std::vector<unsigned char> bytes, std::string name) : bytes_(std::move(bytes)), name_(std::move(name)) {}

    void take(void* into, size_t count, const char* what) {
        if (count > bytes_.size() - at_) {
            throw std::runtime_error("restart file " + name_ + ": truncated inside " + what + " (" + std::to_string(bytes_.size()) +
                                     " bytes on disk)");
        }
        std::memcpy(into, bytes_.data() + at_, count);
        at_ += count;
    }
    template <class T>
    T scalar(const char* what) {
        T v;
        take(&v, sizeof(T), what);
        return v;
    }
    std::string name_field(const char* what) {
        const int32_t length = scalar<int32_t>(what);
        if (length < 0 || length > kLongestName) throw std::runtime_error(bad_length(what, length));
        std::string s(static_cast<size_t>(length), ' ');
        take(s.data(), s.size(), what);
        return s;
    }
    std::vector<double> state_field(const char* what) {
        const int32_t count = scalar<int32_t>(what);
        if (count < 0 || count > kMostStateValues) throw std::runtime_error(bad_length(what, count));
        std::vector<double> v(static_cast<size_t>(count));
        take(v.data(), v.size() * sizeof(double), what);
        return v;
    }
    bool tag_is(const char* tag) {
        if (kTag > bytes_.size() - at_) return false;
        const bool same = std::memcmp(bytes_.data() + at_, tag, kTag) == 0;
        at_ += kTag;
        return same;
    }

private:
    std::string bad_length(const char* what, int32_t got) const {
        return "restart file " + name_ + ": the length stored for " + what + " (" + std::to_string(got) + ") is not plausible";
    }
    std::vector<unsigned char> bytes_;
    std::string name_;
    size_t at_ = 0;
};

std::vector<unsigned char> slurp(const std::string& path) {
    std::FILE* f = std::fopen(path.c_str(), "rb");
    if (!f) throw std::runtime_error("cannot open restart file " + path);
    std::vector<unsigned char> bytes;
    unsigned char chunk[1 << 16];
    size_t got;
    while ((got = std::fread(chunk, 1, sizeof(chunk), f)) > 0) bytes.insert(bytes.end(), chunk, chunk + got);
    std::fclose(f);
    return bytes;
}

void append(std::vector<unsigned char>& image, const void* from, size_t count) {
    const unsigned char* p = static_cast<const unsigned char*>(from);
    image.insert(image.end(), p, p + count);
}

template <class T>
void append_scalar(std::vector<unsigned char>& image, T v) {
    append(image, &v, sizeof(T));
}

}  // namespace

RestartState read_restart(const std::string& path) {
    ByteImage file(slurp(path), path);
    if (!file.tag_is(kHead)) throw std::runtime_error(path + " is not a dsMD restart file (no DSMDRST1 tag)");
    RestartState s;
    s.step = file.scalar<int64_t>("the step number");
    const int64_t atoms = file.scalar<int64_t>("the atom count");
    s.timestep = file.scalar<double>("the time step");
    file.take(s.box, sizeof(s.box), "the box");
    file.take(s.periodic, sizeof(s.periodic), "the periodic flags");
    s.thermostat = file.name_field("the thermostat name");
    s.thermostat_state = file.state_field("the thermostat state");
    s.barostat = file.name_field("the barostat name");
    s.barostat_state = file.state_field("the barostat state");
    if (atoms <= 0 || atoms >= (1ll << 30)) throw std::runtime_error("restart file " + path + ": atom count " + std::to_string(atoms) + " out of range");
    if (s.step < 0 || s.step > static_cast<int64_t>(std::numeric_limits<int>::max()))
        throw std::runtime_error("restart file " + path + ": step " + std::to_string(s.step) + " out of range");
    if (!(s.box[0] > 0.0 && s.box[1] > 0.0 && s.box[2] > 0.0)) throw std::runtime_error("restart file " + path + ": box lengths must be positive");
    std::vector<double>* arrays[6] = {&s.x, &s.y, &s.z, &s.vx, &s.vy, &s.vz};
    const char* names[6] = {"x", "y", "z", "vx", "vy", "vz"};
    for (int k = 0; k < 6; ++k) {
        arrays[k]->resize(static_cast<size_t>(atoms));
        file.take(arrays[k]->data(), arrays[k]->size() * sizeof(double), names[k]);
    }
    if (!file.tag_is(kTail)) throw std::runtime_error("restart file " + path + ": truncated (the closing DSMDEND1 tag is missing)");
    return s;
}

bool write_restart(const std::string& path, const RestartState& s) {
    std::vector<unsigned char> image;
    image.reserve(128 + s.thermostat.size() + s.barostat.size() + 8 * (s.thermostat_state.size() + s.barostat_state.size()) +
                  48 * s.x.size());
    append(image, kHead, kTag);
    append_scalar<int64_t>(image, s.step);
    append_scalar<int64_t>(image, static_cast<int64_t>(s.x.size()));
    append_scalar<double>(image, s.timestep);
    append(image, s.box, sizeof(s.box));
    for (int32_t flag : s.periodic) append_scalar<int32_t>(image, flag ? 1 : 0);
    const std::string* names[2] = {&s.thermostat, &s.barostat};
    const std::vector<double>* states[2] = {&s.thermostat_state, &s.barostat_state};
    for (int k = 0; k < 2; ++k) {
        append_scalar<int32_t>(image, static_cast<int32_t>(names[k]->size()));
        append(image, names[k]->data(), names[k]->size());
        append_scalar<int32_t>(image, static_cast<int32_t>(states[k]->size()));
        append(image, states[k]->data(), states[k]->size() * sizeof(double));
    }
    for (const std::vector<double>* a : {&s.x, &s.y, &s.z, &s.vx, &s.vy, &s.vz}) append(image, a->data(), a->size() * sizeof(double));
    append(image, kTail, kTag);

    const std::string scratch = path + ".tmp";
    std::FILE* f = std::fopen(scratch.c_str(), "wb");
    if (!f) return false;
    const bool written = std::fwrite(image.data(), 1, image.size(), f) == image.size();
    const bool closed = std::fclose(f) == 0;
    if (!written || !closed) return false;
    std::error_code ec;
    std::filesystem::rename(scratch, path, ec);
    return !ec;
}

}  // namespace dsmd::host
