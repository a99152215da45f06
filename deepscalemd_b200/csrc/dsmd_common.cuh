// Shared device/host definitions of the short-range nonbonded path (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace dsmd {

// ---------------------------------------------------------------------------------------------------------------------
// Fixed-point coordinates.
//
// Every atom's position is held, besides the caller-visible doubles, as three 32-bit integers. On an axis that wraps
// (periodic and not split between ranks) one box length is exactly 2^32 units, so the signed 32-bit difference of two
// coordinates IS the minimum-image displacement: no image search, no shift codes, no wrap bookkeeping, and the same
// relative precision (2^-24 after the int->float conversion of the difference) at every place in the box. On an axis
// that does not wrap (split between ranks: ghosts arrive image-shifted; or not periodic) the range
// [lo - halo, hi + halo) maps onto [0, 2^31), so differences never wrap.
// ---------------------------------------------------------------------------------------------------------------------
struct Grid {
    double org[3];      // coordinate of fixed-point 0
    double inv_len[3];  // 1 / (length mapped onto the integer range)
    double box[3];      // periodic box lengths (fp64 boundary re-check)
    float scale[3];     // length of one fixed-point unit
    int wrap[3];        // 1: 2^32 units = one period; 0: 2^31 units = the mapped range
    int nc[3];          // cells per axis
    int ncells;
    int stencil;        // cells searched in each direction (1 or 2)
    float r2_list;      // (cutoff + skin)^2
    float band;         // |r2 - r2_list| below this is decided in fp64
    double r2_list_d;
    float cellw[3];     // cell width per axis (length units); the x cells are finer than the y and z cells
    float r_pad;        // list radius plus a rounding margin: the reach used to prune cell rows
    float x_reach;      // widest half window along x (stencil * width of an unrefined cell, a hair less)
    float band_search;  // the band of the list search (fp32 coordinates relative to the grid origin, image shifts added)
};

struct Status {
    unsigned int need_stride;      // largest neighbour count seen (list rows that overflowed)
    unsigned int out_of_domain;    // atoms outside the mapped range or NaN
    unsigned int rechecked;        // pair tests decided in fp64
    unsigned int timeout;
    unsigned long long max_disp2;  // bits of the largest squared displacement (double, non-negative)
    unsigned long long entries;    // directed list entries
    unsigned long long interior;   // of which the partner is owned
    unsigned long long select_count;
    unsigned int dropped;          // owned atoms found outside the brick by a sort that removes them
    unsigned int constraint_failed;   // constraint clusters whose SHAKE / RATTLE sweeps did not converge
    unsigned int boundary_atoms;      // owned atoms with a ghost partner in their list row (the boundary pass runs over them)
    unsigned int reserved;
};

__host__ __device__ inline unsigned int cell_of(unsigned int fixed, int wrap, int nc) {
#ifdef __CUDA_ARCH__
    return __umulhi(wrap ? fixed : (fixed << 1), static_cast<unsigned int>(nc));
#else
    const unsigned long long v = wrap ? fixed : (static_cast<unsigned long long>(fixed) << 1) & 0xFFFFFFFFull;
    return static_cast<unsigned int>((v * static_cast<unsigned long long>(nc)) >> 32);
#endif
}

#ifdef __CUDACC__
__device__ __forceinline__ unsigned int to_fixed(double v, int axis, const Grid& g, unsigned int& bad) {
    double u = (v - g.org[axis]) * g.inv_len[axis];
    if (!(u == u) || fabs(u) > 1.0e9) {   // NaN, or so far away that it is garbage
        bad = 1u;
        return 0u;
    }
    if (g.wrap[axis]) {
        u -= floor(u);
        if (u >= 1.0) u = 0.0;
        return static_cast<unsigned int>(u * 4294967296.0);
    }
    if (!(u >= 0.0 && u < 1.0)) {
        bad = 1u;
        u = fmin(fmax(u, 0.0), 0.9999999999);
    }
    return static_cast<unsigned int>(u * 2147483648.0);
}

__device__ __forceinline__ float fixed_delta(unsigned int a, unsigned int b, float scale) {
    return static_cast<float>(static_cast<int>(a - b)) * scale;
}

// The x cells of the cell row (cy + dy, cz + dz) that can hold a partner of the atom `pi` (home cell cx, cy, cz): the
// row is skipped when its distance from the atom in the y-z plane already exceeds the list radius; otherwise the
// x window is the chord of the list sphere at that distance, never wider than the stencil, rounded outwards to whole
// x cells (which is why the grid is finer along x: a row is a contiguous run of slots whatever the x cell width, and
// narrow x cells waste less of it). One range [a0, b0], or two when the window crosses the periodic boundary
// ([a1, b1] is empty otherwise).
struct RowWindow {
    int a0, b0, a1, b1;
};

__device__ __forceinline__ bool row_window(const Grid& g, const int4& pi, int cy, int cz, int dy, int dz,
                                           RowWindow& w) {
    const unsigned ux = static_cast<unsigned>(pi.x), uy = static_cast<unsigned>(pi.y), uz = static_cast<unsigned>(pi.z);
    // position inside the home cell, in units of the cell width (0 .. 1)
    const float ty = __uint2float_rn(g.wrap[1] ? uy : uy << 1) * (static_cast<float>(g.nc[1]) * 2.3283064e-10f);
    const float tz = __uint2float_rn(g.wrap[2] ? uz : uz << 1) * (static_cast<float>(g.nc[2]) * 2.3283064e-10f);
    // relative to the integer home cell (the float product may round across a cell boundary: clamp, never re-floor)
    const float fy = fminf(fmaxf(ty - static_cast<float>(cy), 0.f), 1.f);
    const float fz = fminf(fmaxf(tz - static_cast<float>(cz), 0.f), 1.f);
    float gy = dy > 0 ? (static_cast<float>(dy) - fy) : (dy < 0 ? (fy - static_cast<float>(dy + 1)) : 0.f);
    float gz = dz > 0 ? (static_cast<float>(dz) - fz) : (dz < 0 ? (fz - static_cast<float>(dz + 1)) : 0.f);
    gy = fmaxf(gy - 1e-4f, 0.f) * g.cellw[1];   // 1e-4 of a cell: rounding of the in-cell position
    gz = fmaxf(gz - 1e-4f, 0.f) * g.cellw[2];
    const float d2 = gy * gy + gz * gz;
    const float reach2 = g.r_pad * g.r_pad;
    if (d2 >= reach2) return false;
    float hw = sqrtf(reach2 - d2);
    hw = fminf(hw, g.x_reach);
    const unsigned hw_fixed = static_cast<unsigned>(hw / g.scale[0]) + 1u;
    w.a1 = 0;
    w.b1 = -1;
    if (g.wrap[0]) {
        const int c_lo = static_cast<int>(cell_of(ux - hw_fixed, 1, g.nc[0]));
        const int c_hi = static_cast<int>(cell_of(ux + hw_fixed, 1, g.nc[0]));
        if (c_lo <= c_hi) {
            w.a0 = c_lo;
            w.b0 = c_hi;
        } else {
            w.a0 = 0;
            w.b0 = c_hi;
            w.a1 = c_lo;
            w.b1 = g.nc[0] - 1;
        }
    } else {
        const long long lo = static_cast<long long>(ux) - hw_fixed, hi = static_cast<long long>(ux) + hw_fixed;
        w.a0 = static_cast<int>(cell_of(static_cast<unsigned>(lo < 0 ? 0 : lo), 0, g.nc[0]));
        w.b0 = static_cast<int>(cell_of(static_cast<unsigned>(hi > 2147483647ll ? 2147483647ll : hi), 0, g.nc[0]));
    }
    return true;
}

#endif

}  // namespace dsmd
