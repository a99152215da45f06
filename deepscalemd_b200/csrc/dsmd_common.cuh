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
#endif

}  // namespace dsmd
