// Seeded random sequential placement: points drawn uniformly in a periodic cube, each kept only if it lies at least
// min_dist from every point kept before it ("dart throwing" over a cell grid). The generator of the disordered-solid
// input of the radius-graph build; the counter-based random stream makes the positions the same on every machine.
#pragma once

#include <cmath>
#include <cstdint>
#include <stdexcept>
#include <vector>

namespace dsmd::host {

struct SplitMix64 {
    uint64_t state;
    uint64_t next() {
        uint64_t z = (state += 0x9E3779B97F4A7C15ull);
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    }
    double uniform() { return double(next() >> 11) * 0x1.0p-53; }      // [0, 1)
};

// Writes n points (x, y, z interleaved) and returns the number of draws it took. Cells are at most min_dist / sqrt(3)
// wide, so a cell holds one point at most and the grid is a plain index array.
inline int64_t dart_throw(int64_t n, double box, double min_dist, uint64_t seed, double* xyz) {
    if (n < 0 || !(box > 0.0) || !(min_dist >= 0.0)) throw std::invalid_argument("dart_throw: bad arguments");
    SplitMix64 rng{seed};
    if (min_dist == 0.0) {
        for (int64_t k = 0; k < 3 * n; ++k) xyz[k] = rng.uniform() * box;
        return n;
    }
    const int64_t nc = int64_t(std::ceil(box * std::sqrt(3.0) / min_dist));
    const double edge = box / double(nc);
    const int64_t reach = int64_t(std::ceil(min_dist / edge));
    if (nc < 2 * reach + 1) throw std::invalid_argument("dart_throw: the box is too small for this minimum distance");
    if (nc * nc * nc > (int64_t(1) << 31)) throw std::invalid_argument("dart_throw: too many grid cells");
    std::vector<int32_t> grid(size_t(nc * nc * nc), -1);
    const double d2 = min_dist * min_dist, half = 0.5 * box;
    const int64_t draw_limit = 200 * n + 1000;
    int64_t draws = 0;
    for (int64_t i = 0; i < n;) {
        if (++draws > draw_limit) throw std::runtime_error("dart_throw: the requested density cannot be reached");
        const double x = rng.uniform() * box, y = rng.uniform() * box, z = rng.uniform() * box;
        int64_t cx = int64_t(x / edge), cy = int64_t(y / edge), cz = int64_t(z / edge);
        cx = cx < nc ? cx : nc - 1; cy = cy < nc ? cy : nc - 1; cz = cz < nc ? cz : nc - 1;
        bool free_spot = grid[size_t((cz * nc + cy) * nc + cx)] < 0;
        for (int64_t dz = -reach; dz <= reach && free_spot; ++dz) {
            const int64_t gz = (cz + dz + nc) % nc;
            for (int64_t dy = -reach; dy <= reach && free_spot; ++dy) {
                const int64_t gy = (cy + dy + nc) % nc;
                for (int64_t dx = -reach; dx <= reach; ++dx) {
                    const int64_t gx = (cx + dx + nc) % nc;
                    const int32_t j = grid[size_t((gz * nc + gy) * nc + gx)];
                    if (j < 0) continue;
                    double ex = std::fabs(x - xyz[3 * j]), ey = std::fabs(y - xyz[3 * j + 1]), ez = std::fabs(z - xyz[3 * j + 2]);
                    if (ex > half) ex = box - ex;
                    if (ey > half) ey = box - ey;
                    if (ez > half) ez = box - ez;
                    if (ex * ex + ey * ey + ez * ez < d2) { free_spot = false; break; }
                }
            }
        }
        if (!free_spot) continue;
        xyz[3 * i] = x; xyz[3 * i + 1] = y; xyz[3 * i + 2] = z;
        grid[size_t((cz * nc + cy) * nc + cx)] = int32_t(i);
        ++i;
    }
    return draws;
}

}  // namespace dsmd::host
