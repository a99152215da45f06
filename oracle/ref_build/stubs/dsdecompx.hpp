// Minimal stand-in for the un-vendored dsDecompX 1.0 header: test infrastructure only.
// Only what the reference's CPU neighbour-list and force sources touch: the particle container
// (owned atoms first, then ghosts) and two opaque types named in md_system.h.
#ifndef DSMD_ORACLE_STUB_DSDECOMPX_HPP
#define DSMD_ORACLE_STUB_DSDECOMPX_HPP
#include <cstddef>
#include <vector>

namespace dsdecompx {

struct ParticleInfo {
    std::vector<double> x, y, z, vx, vy, vz, fx, fy, fz, mass, charge;
    std::vector<int> type, global_id;
    size_t num_particles = 0;
    size_t owned_ = 0, ghost_ = 0;

    size_t size() const { return num_particles; }
    size_t owned_count() const { return owned_; }
    size_t ghost_count() const { return ghost_; }
    void reset_counts(size_t owned, size_t ghosts) { owned_ = owned; ghost_ = ghosts; }
    void resize(size_t n) {
        for (auto* v : {&x, &y, &z, &vx, &vy, &vz, &fx, &fy, &fz, &mass, &charge}) v->resize(n, 0.0);
        type.resize(n, 0);
        global_id.resize(n, 0);
        num_particles = n;
        if (owned_ + ghost_ != n) { owned_ = n; ghost_ = 0; }
    }
};

struct HaloResult {
    size_t ghost_count = 0;
    bool plan_reused = false, layout_changed = false, storage_reallocated = false;
};

class Decomp {
public:
    bool mpi_takes_device_pointers() const { return false; }
};

}  // namespace dsdecompx
#endif
