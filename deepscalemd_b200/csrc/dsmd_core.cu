// The short-range nonbonded path on one B200 (sm_100a): cell binning and sort, Verlet list build with skin,
// LJ + real-space Ewald pair kernel, displacement check, velocity-Verlet halves, ghost pack/unpack, and the C ABI
// declared in include/dsmd_b200.h.
//
// Data layout in HBM (all arrays indexed by "slot"; owned atoms occupy [0, n_owned), ghosts [n_owned, n_total); both
// segments are sorted by cell, x fastest, at every list build):
//   x y z vx vy vz fx fy fz mass charge   double[capacity] each, two sets (the sort gathers from one into the other)
//   type gid                               int32[capacity], two sets
//   pq                                     int4[capacity]: fixed-point x, y, z and the type in w (what the kernels read)
//   qf                                     float[capacity]: charge (read only with Coulomb on)
//   xref yref zref                         double[capacity]: owned positions at the last build (displacement check)
//   cell_start                             int32[2 * cells + 1]: first slot of every cell, owned cells then ghost cells
//   nbr                                    uint32[ceil(n_owned / 32) * stride * 32]: 32-atom slices, entry k of the 32
//                                          atoms of a slice is one 128-byte line; bit 31 = excluded pair
//   deg, deg_int                           int32[n_owned]: entries per atom; of which the partner is owned (come first)
//
// No tensor cores: the path is a gather over a sparse geometric neighbourhood, not a dense contraction.

#include <cub/cub.cuh>
#include <thrust/iterator/counting_iterator.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/dsmd_b200.h"
#include "dsmd_common.cuh"
#include "ewald_table.hpp"

using dsmd::Grid;
using dsmd::Status;

namespace {

constexpr int kThreads = 256;
constexpr int kPairThreads = 128;
constexpr int kBuildThreads = 64;   // k_build_list: 64, 128, 256 threads per block measured 2.62, 2.67, 2.86 ms (4 M atoms)
constexpr int kXRefine = 4;    // x cells per cell width of the y and z axes (tighter row windows in the list build)
constexpr unsigned kExclBit = 0x80000000u;
constexpr unsigned kIndexMask = 0x3FFFFFFFu;
constexpr int kNumReal = 11;   // x y z vx vy vz fx fy fz mass charge
constexpr double kCoulomb = 332.0636;

inline unsigned blocks_for(int64_t n, int threads) { return static_cast<unsigned>((n + threads - 1) / threads); }

// ---------------------------------------------------------------------------------------------------------------------
// kernels: binning, sort support, reorder
// ---------------------------------------------------------------------------------------------------------------------

struct RealArrays {
    double* p[kNumReal];
};

// This rank's brick on the axes that are split between ranks (drop != 0: atoms outside it are to be removed).
struct Brick {
    double lo[3], hi[3];
    int split[3];
    int drop;
};

__global__ void k_cell_keys(Grid g, Brick brick, int first, int n_owned, int n_total, const double* __restrict__ x,
                            const double* __restrict__ y, const double* __restrict__ z, unsigned* __restrict__ key,
                            int* __restrict__ val, Status* st) {
    const int s = first + blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= n_total) return;
    const double p[3] = {x[s], y[s], z[s]};
    unsigned bad = 0;
    const unsigned fx = dsmd::to_fixed(p[0], 0, g, bad);
    const unsigned fy = dsmd::to_fixed(p[1], 1, g, bad);
    const unsigned fz = dsmd::to_fixed(p[2], 2, g, bad);
    if (bad) atomicAdd(&st->out_of_domain, 1u);
    const unsigned cx = dsmd::cell_of(fx, g.wrap[0], g.nc[0]);
    const unsigned cy = dsmd::cell_of(fy, g.wrap[1], g.nc[1]);
    const unsigned cz = dsmd::cell_of(fz, g.wrap[2], g.nc[2]);
    unsigned c = (cz * g.nc[1] + cy) * g.nc[0] + cx;
    if (s >= n_owned) c += g.ncells;
    if (brick.drop) {   // an atom that left the brick (the same comparisons as the migration's classifier) sorts last
        bool outside = false;
        for (int a = 0; a < 3; ++a)
            if (brick.split[a] && (p[a] < brick.lo[a] || p[a] >= brick.hi[a])) outside = true;
        if (outside) {
            c = 2u * static_cast<unsigned>(g.ncells);
            atomicAdd(&st->dropped, 1u);
        }
    }
    key[s - first] = c;
    val[s - first] = s;
}

// Gathers every particle array into sorted order, writes the fixed-point layout, the displacement reference, the
// ghost slot map and the cell start table (a thread whose key differs from its predecessor's owns the cells between).
__global__ void k_reorder(Grid g, int first, int n_owned, int n_total, const unsigned* __restrict__ key,
                          const int* __restrict__ val, RealArrays src, RealArrays dst, const int* __restrict__ type_src,
                          const int* __restrict__ gid_src, int* __restrict__ type_dst, int* __restrict__ gid_dst,
                          int4* __restrict__ pq, float4* __restrict__ pf, float* __restrict__ qf, double* __restrict__ xref,
                          double* __restrict__ yref, double* __restrict__ zref, int* __restrict__ cell_start,
                          int* __restrict__ ghost_slot) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    const int s = first + t;
    if (s >= n_total) return;
    const int from = val[t];
    double r[kNumReal];
#pragma unroll
    for (int f = 0; f < kNumReal; ++f) r[f] = src.p[f][from];
#pragma unroll
    for (int f = 0; f < kNumReal; ++f) dst.p[f][s] = r[f];
    const int ty = type_src[from];
    type_dst[s] = ty;
    gid_dst[s] = gid_src[from];
    unsigned bad = 0;
    int4 p;
    p.x = static_cast<int>(dsmd::to_fixed(r[0], 0, g, bad));
    p.y = static_cast<int>(dsmd::to_fixed(r[1], 1, g, bad));
    p.z = static_cast<int>(dsmd::to_fixed(r[2], 2, g, bad));
    p.w = ty;
    pq[s] = p;
    // the list search's copy: single-precision offsets from the grid origin (the value of the fixed-point coordinate);
    // the fourth word carries the global id, so that the exclusion test of a hit needs no second gather
    pf[s] = make_float4(__uint2float_rn(static_cast<unsigned>(p.x)) * g.scale[0],
                        __uint2float_rn(static_cast<unsigned>(p.y)) * g.scale[1],
                        __uint2float_rn(static_cast<unsigned>(p.z)) * g.scale[2], __int_as_float(gid_src[from]));
    qf[s] = static_cast<float>(r[10]);
    if (s < n_owned) {
        xref[s] = r[0];
        yref[s] = r[1];
        zref[s] = r[2];
    } else {
        ghost_slot[from - n_owned] = s;
    }
    // Cell starts. Keys of the sorted range [first, n_total) are key[0 .. n_total - first). When only the owned atoms
    // are sorted (first == 0, n_total == n_owned) the ghost half of the table is filled by the later full build.
    const int k_here = static_cast<int>(key[t]);
    if (k_here >= 2 * g.ncells) return;   // an atom being removed: behind every cell
    const int k_prev = t == 0 ? (first == 0 ? -1 : g.ncells - 1) : static_cast<int>(key[t - 1]);
    for (int c = k_prev + 1; c <= k_here; ++c) cell_start[c] = s;
}

// Cells behind the last occupied one (and, when only owned atoms were sorted, the whole ghost half) start at the end.
__global__ void k_cell_tail(const unsigned* __restrict__ key, int n_sorted, int n_total, int table_size,
                            int* __restrict__ cell_start) {
    const int c = static_cast<int>(key[n_sorted - 1]) + 1 + blockIdx.x * blockDim.x + threadIdx.x;
    if (c < table_size) cell_start[c] = n_total;
}

// ---------------------------------------------------------------------------------------------------------------------
// kernel: Verlet list build
// ---------------------------------------------------------------------------------------------------------------------

// A ghost-only sort gathers the ghosts into the other buffer set; this brings them back, so that the owned atoms
// (already in place) need not be copied across: one thread per ghost, all per-atom arrays.
__global__ void k_copy_back(int first, int count, RealArrays from, RealArrays to, const int* __restrict__ type_from,
                            const int* __restrict__ gid_from, int* __restrict__ type_to, int* __restrict__ gid_to) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= count) return;
    const int s = first + t;
#pragma unroll
    for (int f = 0; f < kNumReal; ++f) to.p[f][s] = from.p[f][s];
    type_to[s] = type_from[s];
    gid_to[s] = gid_from[s];
}

// First slot of every z layer of (owned) cells, and the end: what lets a caller cut the sorted atoms into slabs.
__global__ void k_layer_starts(const int* __restrict__ cell_start, int cells_per_layer, int layers, int* __restrict__ out) {
    const int l = blockIdx.x * blockDim.x + threadIdx.x;
    if (l <= layers) out[l] = cell_start[static_cast<size_t>(l) * cells_per_layer];
}

// Where the ghosts of a cell row sit: lo_end = one past the last x cell of the row's lower half that holds a ghost (0:
// none), hi_begin = the first x cell of its upper half that holds one (nc[0]: none). One warp per (y, z) row.
__global__ void k_ghost_row_extent(Grid g, const int* __restrict__ ghost_cell_start, int* __restrict__ lo_end,
                                   int* __restrict__ hi_begin) {
    const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= g.nc[1] * g.nc[2]) return;
    const int* cells = ghost_cell_start + static_cast<size_t>(row) * g.nc[0];
    const int half = g.nc[0] >> 1;
    int lo = 0, hi = g.nc[0];
    for (int c = lane; c < g.nc[0]; c += 32) {
        if (cells[c + 1] > cells[c]) {
            if (c < half) lo = max(lo, c + 1);
            else hi = min(hi, c);
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        lo = max(lo, __shfl_down_sync(0xffffffffu, lo, o));
        hi = min(hi, __shfl_down_sync(0xffffffffu, hi, o));
    }
    if (lane == 0) { lo_end[row] = lo; hi_begin[row] = hi; }
}

// The same over the rows a centre of row (yc, zc) searches (stencil reach in y and z, wrapping where the axis does): an
// owned atom whose x window stays inside [near_lo, near_hi) of its row cannot have a ghost partner and skips the ghost
// pass of the list build altogether.
__global__ void k_ghost_rows_near(Grid g, const int* __restrict__ lo_end, const int* __restrict__ hi_begin,
                                  int* __restrict__ near_lo, int* __restrict__ near_hi) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= g.nc[1] * g.nc[2]) return;
    const int yc0 = row % g.nc[1], zc0 = row / g.nc[1];
    int lo = 0, hi = g.nc[0];
    for (int dz = -g.stencil; dz <= g.stencil; ++dz) {
        int zc = zc0 + dz;
        if (g.wrap[2]) zc = (zc + g.nc[2]) % g.nc[2];
        else if (zc < 0 || zc >= g.nc[2]) continue;
        for (int dy = -g.stencil; dy <= g.stencil; ++dy) {
            int yc = yc0 + dy;
            if (g.wrap[1]) yc = (yc + g.nc[1]) % g.nc[1];
            else if (yc < 0 || yc >= g.nc[1]) continue;
            lo = max(lo, lo_end[zc * g.nc[1] + yc]);
            hi = min(hi, hi_begin[zc * g.nc[1] + yc]);
        }
    }
    near_lo[row] = lo;
    near_hi[row] = hi;
}

struct ExclusionTable {
    const int* offsets;    // [n_global + 1] by global id, or null
    const int* partners;   // sorted per atom
    int n_global;          // ids at or beyond this have no exclusions
};

__device__ __forceinline__ bool within_list_fp64(const Grid& g, const double* __restrict__ x,
                                                 const double* __restrict__ y, const double* __restrict__ z, int i,
                                                 int j) {
    double dx = x[i] - x[j], dy = y[i] - y[j], dz = z[i] - z[j];
    if (g.wrap[0]) dx -= g.box[0] * rint(dx / g.box[0]);
    if (g.wrap[1]) dy -= g.box[1] * rint(dy / g.box[1]);
    if (g.wrap[2]) dz -= g.box[2] * rint(dz / g.box[2]);
    // No FMA contraction: the sum must round as the plain fp64 expression dx*dx + dy*dy + dz*dz does.
    const double r2 = __dadd_rn(__dadd_rn(__dmul_rn(dx, dx), __dmul_rn(dy, dy)), __dmul_rn(dz, dz));
    return r2 < g.r2_list_d;
}

// One thread per owned atom. The cell rows of the stencil are contiguous runs of slots (cells are sorted x fastest), so
// a row costs two table reads and a linear scan. The candidate test runs in fp32 on `pf`, a copy of the positions as
// single-precision offsets from the grid origin written at the sort; the periodic image of a cell row (or of the piece
// of a row window that lies across the box boundary) is one shift of the CENTRE's coordinate per row, so a candidate
// costs three subtractions, no integer arithmetic and no conversion. Results inside the rounding band around the list
// radius are re-decided in fp64 on the caller's double positions, which makes list membership identical to an fp64
// search. Owned partners are scanned first, then ghosts, so the first deg_int entries of a row are the interior part.
// 16 resident blocks of 64 threads: the 64-register budget that gives is worth more than the registers (measured: 2.76 ms
// against 4.24 ms per build at 4 M atoms with 110 registers and 8 blocks).
// EXCL: launched for systems with an exclusion table; keeps the first four partners of an atom in registers. The other
// instantiation is launched for systems without one and keeps the plain table walk (never taken there): written this way
// because removing the exclusion code from it altogether made the compiler spill more in the search loop (2.76 ms
// against 2.67 ms per build at 4 M atoms).
template <bool EXCL>
__global__ void __launch_bounds__(kBuildThreads, 16)
k_build_list(Grid g, int n_owned, int n_total, const int4* __restrict__ pq, const float4* __restrict__ pf,
             const double* __restrict__ x, const double* __restrict__ y, const double* __restrict__ z,
             const int* __restrict__ gid, ExclusionTable excl, const int* __restrict__ cell_start,
             const int* __restrict__ ghost_near_lo, const int* __restrict__ ghost_near_hi,
             unsigned* __restrict__ nbr, int stride, int* __restrict__ deg, int* __restrict__ deg_int,
             int* __restrict__ boundary_list, Status* st) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const bool active = i < n_owned;   // lanes past the end stay for the warp sums at the bottom
    const int4 pi = active ? pq[i] : make_int4(0, 0, 0, 0);
    const float4 fi = active ? pf[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    const int cx = static_cast<int>(dsmd::cell_of(static_cast<unsigned>(pi.x), g.wrap[0], g.nc[0]));
    const int cy = static_cast<int>(dsmd::cell_of(static_cast<unsigned>(pi.y), g.wrap[1], g.nc[1]));
    const int cz = static_cast<int>(dsmd::cell_of(static_cast<unsigned>(pi.z), g.wrap[2], g.nc[2]));
    const int S = g.stencil;
    const size_t base = (static_cast<size_t>(i >> 5) * stride) * 32 + (i & 31);
    int ex_begin = 0, ex_end = 0;
    // the first four exclusion partners (rigid water has two) are kept in registers: a hit is compared with them without
    // touching memory; atoms with more partners walk the rest of their table row
    constexpr int kNoPartner = static_cast<int>(0x80000000u);   // no atom carries this id
    int ex0 = kNoPartner, ex1 = kNoPartner, ex2 = kNoPartner, ex3 = kNoPartner;
    if (active && excl.offsets) {
        const int gi = gid[i];
        if (gi >= 0 && gi < excl.n_global) {
            ex_begin = excl.offsets[gi];
            ex_end = excl.offsets[gi + 1];
            if (EXCL) {
                if (ex_end > ex_begin) ex0 = excl.partners[ex_begin];
                if (ex_end > ex_begin + 1) ex1 = excl.partners[ex_begin + 1];
                if (ex_end > ex_begin + 2) ex2 = excl.partners[ex_begin + 2];
                if (ex_end > ex_begin + 3) ex3 = excl.partners[ex_begin + 3];
            }
        }
    }
    const float hi_band = g.r2_list + g.band_search;
    const float in_band = g.r2_list - g.band_search;
    // every hit of an atom with exclusions takes the slow path, which looks the partner up in the exclusion table
    const float lo_band = ex_end > ex_begin ? -1.0f : in_band;
    const float box_x = static_cast<float>(g.box[0]), box_y = static_cast<float>(g.box[1]), box_z = static_cast<float>(g.box[2]);
    unsigned* dst = nbr + base;   // next entry of this atom's row (entries of a row are 32 words apart)
    unsigned* const dst_end = dst + static_cast<size_t>(stride) * 32;
    int interior = 0;
    unsigned rechecked = 0;
    // the ghost pass only for atoms whose x window reaches an x cell with ghosts in one of the rows they search (on an
    // axis that wraps the window may come round the box: any ghost in those rows counts)
    int n_seg = active ? 1 : 0;
    if (active && n_total > n_owned) {
        const int row_yz = cz * g.nc[1] + cy;
        const int near_lo = ghost_near_lo[row_yz], near_hi = ghost_near_hi[row_yz];
        const int reach_cells = static_cast<int>(g.x_reach / g.cellw[0]) + 2;
        if (g.wrap[0] ? (near_lo > 0 || near_hi < g.nc[0]) : (cx - reach_cells < near_lo || cx + reach_cells >= near_hi))
            n_seg = 2;
    }
    // The x window of a cell row is the chord of the list sphere at the row's distance from the atom in the y-z plane
    // (dsmd::row_window spells the rule out): the distance has one term per axis, each a function of the cell offset and
    // of the atom's place inside its home cell, so the z term is worked out per layer and the y term per row.
    const unsigned ux = static_cast<unsigned>(pi.x), uy = static_cast<unsigned>(pi.y), uz = static_cast<unsigned>(pi.z);
    const float ty = __uint2float_rn(g.wrap[1] ? uy : uy << 1) * (static_cast<float>(g.nc[1]) * 2.3283064e-10f);
    const float tz = __uint2float_rn(g.wrap[2] ? uz : uz << 1) * (static_cast<float>(g.nc[2]) * 2.3283064e-10f);
    const float in_y = fminf(fmaxf(ty - static_cast<float>(cy), 0.f), 1.f);   // place inside the home cell, 0 .. 1
    const float in_z = fminf(fmaxf(tz - static_cast<float>(cz), 0.f), 1.f);
    const float reach2 = g.r_pad * g.r_pad;
    const float units_per_length = 1.0f / g.scale[0];
    for (int seg = 0; seg < n_seg; ++seg) {
        for (int dz = -S; dz <= S; ++dz) {
            int zc = cz + dz;
            float zi = fi.z;   // the centre as the atoms of this cell row see it
            if (g.wrap[2]) { if (zc < 0) { zc += g.nc[2]; zi += box_z; } else if (zc >= g.nc[2]) { zc -= g.nc[2]; zi -= box_z; } }
            else if (zc < 0 || zc >= g.nc[2]) continue;
            float gz = dz > 0 ? (static_cast<float>(dz) - in_z) : (dz < 0 ? (in_z - static_cast<float>(dz + 1)) : 0.f);
            gz = fmaxf(gz - 1e-4f, 0.f) * g.cellw[2];   // 1e-4 of a cell: rounding of the in-cell position
            const float room2 = reach2 - gz * gz;
            if (room2 <= 0.f) continue;
            for (int dy = -S; dy <= S; ++dy) {
                int yc = cy + dy;
                float yi = fi.y;
                if (g.wrap[1]) { if (yc < 0) { yc += g.nc[1]; yi += box_y; } else if (yc >= g.nc[1]) { yc -= g.nc[1]; yi -= box_y; } }
                else if (yc < 0 || yc >= g.nc[1]) continue;
                float gy = dy > 0 ? (static_cast<float>(dy) - in_y) : (dy < 0 ? (in_y - static_cast<float>(dy + 1)) : 0.f);
                gy = fmaxf(gy - 1e-4f, 0.f) * g.cellw[1];
                const float chord2 = room2 - gy * gy;
                if (chord2 <= 0.f) continue;
                // half window: the chord, never wider than the stencil, rounded outwards to whole x cells (r_pad carries
                // 1e-4 of slack, far more than the approximate square root gives away)
                const float hw = fminf(chord2 * rsqrtf(chord2), g.x_reach);
                const unsigned hw_fixed = static_cast<unsigned>(hw * units_per_length) + 2u;
                const int row = seg * g.ncells + (zc * g.nc[1] + yc) * g.nc[0];
                dsmd::RowWindow win;
                win.a1 = 0;
                win.b1 = -1;
                if (g.wrap[0]) {
                    const int c_lo = static_cast<int>(dsmd::cell_of(ux - hw_fixed, 1, g.nc[0]));
                    const int c_hi = static_cast<int>(dsmd::cell_of(ux + hw_fixed, 1, g.nc[0]));
                    if (c_lo <= c_hi) { win.a0 = c_lo; win.b0 = c_hi; }
                    else { win.a0 = 0; win.b0 = c_hi; win.a1 = c_lo; win.b1 = g.nc[0] - 1; }
                } else {
                    const long long lo = static_cast<long long>(ux) - hw_fixed, hi = static_cast<long long>(ux) + hw_fixed;
                    win.a0 = static_cast<int>(dsmd::cell_of(static_cast<unsigned>(lo < 0 ? 0 : lo), 0, g.nc[0]));
                    win.b0 = static_cast<int>(dsmd::cell_of(static_cast<unsigned>(hi > 2147483647ll ? 2147483647ll : hi), 0, g.nc[0]));
                }
                const bool two = win.b1 >= win.a1;   // the x window crosses the periodic boundary: [0, b0] and [a1, nc - 1]
                for (int part = 0; part < 2; ++part) {
                    const int a = part == 0 ? win.a0 : win.a1, b = part == 0 ? win.b0 : win.b1;
                    if (b < a) continue;
                    // the piece the centre's own cell is not in holds images one box length away
                    float xi = fi.x;
                    if (two) {
                        const bool centre_low = cx <= win.b0;
                        if (part == 0 && !centre_low) xi -= box_x;
                        if (part == 1 && centre_low) xi += box_x;
                    }
                    const int s_begin = cell_start[row + a], s_end = cell_start[row + b + 1];
                    for (int s = s_begin; s < s_end; ++s) {
                        const float4 c = __ldg(&pf[s]);
                        const float dx = c.x - xi, ddy = c.y - yi, ddz = c.z - zi;
                        const float r2 = dx * dx + ddy * ddy + ddz * ddz;
                        if (r2 < hi_band && s != i) {
                            unsigned entry = static_cast<unsigned>(s);
                            if (r2 >= lo_band) {   // inside the rounding band, or an atom with exclusions: the slow, exact way
                                if (r2 >= in_band) {
                                    ++rechecked;
                                    if (!within_list_fp64(g, x, y, z, i, s)) continue;
                                }
                                if (ex_end > ex_begin) {
                                    const int gj = __float_as_int(c.w);
                                    if (EXCL && (gj == ex0 || gj == ex1 || gj == ex2 || gj == ex3)) entry |= kExclBit;   // an unused register never matches
                                    for (int e = ex_begin + (EXCL ? 4 : 0); e < ex_end; ++e)
                                        if (excl.partners[e] == gj) entry |= kExclBit;
                                }
                            }
                            if (dst < dst_end) *dst = entry;
                            dst += 32;
                        }
                    }
                }
            }
        }
        if (seg == 0) interior = static_cast<int>((dst - (nbr + base)) >> 5);
    }
    const int count = static_cast<int>((dst - (nbr + base)) >> 5);
    if (active) {
        deg[i] = min(count, stride);
        deg_int[i] = min(interior, stride);
        if (count > stride) atomicMax(&st->need_stride, static_cast<unsigned>(count));
    }
    // atoms with a ghost partner, collected for the boundary pass of the pair kernel (one atomic per warp; the order of
    // the collection does not matter: every atom's sum is its own thread's)
    {
        const bool has_ghost_partner = active && count > interior;
        const unsigned ballot = __ballot_sync(0xffffffffu, has_ghost_partner);
        if (ballot) {
            const int lane = threadIdx.x & 31;
            unsigned first = 0;
            if (lane == 0) first = atomicAdd(&st->boundary_atoms, static_cast<unsigned>(__popc(ballot)));
            first = __shfl_sync(0xffffffffu, first, 0);
            if (has_ghost_partner) boundary_list[first + __popc(ballot & ((1u << lane) - 1u))] = i;
        }
    }
    // statistics: one atomic per warp
    unsigned long long c64 = count, i64 = interior;
    unsigned rc = rechecked;
    for (int o = 16; o > 0; o >>= 1) {
        c64 += __shfl_down_sync(0xffffffffu, c64, o);
        i64 += __shfl_down_sync(0xffffffffu, i64, o);
        rc += __shfl_down_sync(0xffffffffu, rc, o);
    }
    if ((threadIdx.x & 31) == 0) {
        atomicAdd(&st->entries, c64);
        atomicAdd(&st->interior, i64);
        if (rc) atomicAdd(&st->rechecked, rc);
    }
}

__global__ void k_list_export(int n_owned, const unsigned* __restrict__ nbr, int stride, const int* __restrict__ deg,
                              const unsigned long long* __restrict__ offsets, int* out_i, int* out_j,
                              unsigned char* out_flags, long long capacity) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_owned) return;
    const size_t base = (static_cast<size_t>(i >> 5) * stride) * 32 + (i & 31);
    unsigned long long o = offsets[i];
    for (int k = 0; k < deg[i]; ++k, ++o) {
        if (static_cast<long long>(o) >= capacity) return;
        const unsigned e = nbr[base + static_cast<size_t>(k) * 32];
        out_i[o] = i;
        out_j[o] = static_cast<int>(e & kIndexMask);
        if (out_flags) out_flags[o] = (e & kExclBit) ? 1 : 0;
    }
}

__global__ void k_deg_to_u64(int n, const int* deg, unsigned long long* out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = static_cast<unsigned long long>(deg[i]);
}

// ---------------------------------------------------------------------------------------------------------------------
// kernels: per-step pack, displacement, integration
// ---------------------------------------------------------------------------------------------------------------------

__device__ __forceinline__ void block_max_to_status(double v, Status* st) {
    for (int o = 16; o > 0; o >>= 1) v = fmax(v, __shfl_down_sync(0xffffffffu, v, o));
    __shared__ double warp_max[32];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) warp_max[w] = v;
    __syncthreads();
    if (w == 0) {
        v = lane < (blockDim.x >> 5) ? warp_max[lane] : 0.0;
        for (int o = 16; o > 0; o >>= 1) v = fmax(v, __shfl_down_sync(0xffffffffu, v, o));
        if (lane == 0 && v > 0.0) atomicMax(&st->max_disp2, static_cast<unsigned long long>(__double_as_longlong(v)));
    }
}

// INTEGRATE: kick and drift before the pack (v += kick_c f / m, x += dt v): the first velocity-Verlet half with
// kick_c = dt/2 (times the force-to-acceleration factor), or, with kick_c = dt, the second half of the previous step and
// the first half of this one in one pass (both use the same forces).
template <bool INTEGRATE>
__global__ void k_pack(Grid g, int first, int count, int n_owned, double* __restrict__ x, double* __restrict__ y,
                       double* __restrict__ z, double* __restrict__ vx, double* __restrict__ vy,
                       double* __restrict__ vz, const double* __restrict__ fx, const double* __restrict__ fy,
                       const double* __restrict__ fz, const double* __restrict__ mass, const int* __restrict__ type,
                       const double* __restrict__ xref, const double* __restrict__ yref,
                       const double* __restrict__ zref, int4* __restrict__ pq, double dt, double kick_c,
                       Status* st) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    const int s = first + t;
    double d2 = 0.0;
    if (t < count) {
        double px = x[s], py = y[s], pz = z[s];
        if (INTEGRATE) {
            const double a = kick_c / mass[s];
            const double ux = vx[s] + a * fx[s], uy = vy[s] + a * fy[s], uz = vz[s] + a * fz[s];
            vx[s] = ux; vy[s] = uy; vz[s] = uz;
            px += dt * ux; py += dt * uy; pz += dt * uz;
            x[s] = px; y[s] = py; z[s] = pz;
        }
        unsigned bad = 0;
        int4 p;
        p.x = static_cast<int>(dsmd::to_fixed(px, 0, g, bad));
        p.y = static_cast<int>(dsmd::to_fixed(py, 1, g, bad));
        p.z = static_cast<int>(dsmd::to_fixed(pz, 2, g, bad));
        p.w = type[s];
        pq[s] = p;
        if (bad) atomicAdd(&st->out_of_domain, 1u);
        if (s < n_owned) {
            const double ddx = px - xref[s], ddy = py - yref[s], ddz = pz - zref[s];
            d2 = ddx * ddx + ddy * ddy + ddz * ddz;
            // a position that is no number must not vanish in the block maximum (fmax drops NaN): it forces a rebuild,
            // and the rebuild reports the atom
            if (!(d2 == d2)) d2 = __longlong_as_double(0x7FF0000000000000ll);
        }
    }
    block_max_to_status(d2, st);
}

__global__ void k_vv2(int n, double half_dt_c, double* __restrict__ vx, double* __restrict__ vy,
                      double* __restrict__ vz, const double* __restrict__ fx, const double* __restrict__ fy,
                      const double* __restrict__ fz, const double* __restrict__ mass) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= n) return;
    const double a = half_dt_c / mass[s];
    vx[s] += a * fx[s];
    vy[s] += a * fy[s];
    vz[s] += a * fz[s];
}

// Thermostat step of the velocity-scaling kind (the reference's nose_hoover_thermostat_kernel,
// src/thermostat_kernels.cu:68-76): v *= factor.
__global__ void k_scale_velocities(int n, double factor, double* __restrict__ vx, double* __restrict__ vy,
                                   double* __restrict__ vz) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= n) return;
    vx[s] *= factor;
    vy[s] *= factor;
    vz[s] *= factor;
}

// Deterministic two-level sums: per-block partials, then one block adds them in a fixed order.
template <int NV>
__device__ __forceinline__ void block_sum_to_partials(double (&v)[NV], double* partials) {
    __shared__ double sh[32][NV];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
    for (int k = 0; k < NV; ++k)
        for (int o = 16; o > 0; o >>= 1) v[k] += __shfl_down_sync(0xffffffffu, v[k], o);
    if (lane == 0)
        for (int k = 0; k < NV; ++k) sh[w][k] = v[k];
    __syncthreads();
    if (threadIdx.x == 0) {
        const int nw = blockDim.x >> 5;
        for (int k = 0; k < NV; ++k) {
            double sum = 0.0;
            for (int q = 0; q < nw; ++q) sum += sh[q][k];
            partials[static_cast<size_t>(blockIdx.x) * NV + k] = sum;
        }
    }
}

template <int NV>
__global__ void k_reduce_partials(const double* __restrict__ partials, int n_blocks, double* __restrict__ out,
                                  int accumulate) {
    __shared__ double sh[kThreads];
    for (int k = 0; k < NV; ++k) {
        double sum = 0.0;
        for (int b = threadIdx.x; b < n_blocks; b += blockDim.x) sum += partials[static_cast<size_t>(b) * NV + k];
        sh[threadIdx.x] = sum;
        __syncthreads();
        for (int o = blockDim.x / 2; o > 0; o >>= 1) {
            if (threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
            __syncthreads();
        }
        if (threadIdx.x == 0) out[k] = accumulate ? out[k] + sh[0] : sh[0];
        __syncthreads();
    }
}

__global__ void k_kinetic(int n, const double* __restrict__ vx, const double* __restrict__ vy,
                          const double* __restrict__ vz, const double* __restrict__ mass, double* partials) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    double v[1] = {0.0};
    if (s < n) v[0] = 0.5 * mass[s] * (vx[s] * vx[s] + vy[s] * vy[s] + vz[s] * vz[s]);
    block_sum_to_partials<1>(v, partials);
}

}  // namespace

#include "dsmd_constraints.cuh"
#include "dsmd_bonded.cuh"

namespace {

// ---------------------------------------------------------------------------------------------------------------------
// kernel: LJ + real-space Ewald over the list
// ---------------------------------------------------------------------------------------------------------------------

struct PairParams {
    float scale[3];
    float rc2;
    float rs2, inv_denom;        // CHARMM switch on r^2 (rs2 < 0: off)
    float kq;                    // Coulomb constant
    float alpha, two_alpha_sqrtpi;
    int ntypes;
    int ewald_intervals;
    const float2* c6c12;         // [ntypes * ntypes]
    const float4* ewald;         // [2 * intervals]: force cubic, energy cubic
    const float* type_charge;    // [ntypes] when every atom's charge is that of its type (dsmd_set_type_charges), else null
};

// 1 / v: the hardware approximation (1 ulp) for the force-only kernels, one Newton step more (full single precision)
// where energy and virial sums are taken.
template <bool REFINE>
__device__ __forceinline__ float fast_rcp(float v) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return REFINE ? r * (2.0f - v * r) : r;
}

// One pair of the list, evaluated from atom i's side: adds to the force (and energy / virial) accumulators.
template <bool COULOMB, bool ENERGY, bool MULTI, bool SWITCH>
struct PairAccumulator {
    float ax = 0.f, ay = 0.f, az = 0.f;
    float e_sum = 0.f, w_sum = 0.f, wx = 0.f, wy = 0.f, wz = 0.f, n_in = 0.f;

    __device__ __forceinline__ void add(const PairParams& p, const int4& pi, const int4& pj, float qi, float qj,
                                        bool excluded, const float2* s_c6c12, const float4* s_ewald, float2 single,
                                        int trow) {
        const float dx = dsmd::fixed_delta(pi.x, pj.x, p.scale[0]);
        const float dy = dsmd::fixed_delta(pi.y, pj.y, p.scale[1]);
        const float dz = dsmd::fixed_delta(pi.z, pj.z, p.scale[2]);
        const float r2 = dx * dx + dy * dy + dz * dz;
        if (r2 < p.rc2 && r2 >= 1e-10f) {
            float fmag = 0.f, epair = 0.f;
            const float r2inv = fast_rcp<ENERGY>(r2);
            if (!excluded) {
                const float2 c = MULTI ? s_c6c12[trow + pj.w] : single;
                const float r6 = r2inv * r2inv * r2inv;
                const float t = c.y * r6;
                float f = (r2inv * r6) * (12.f * t - 6.f * c.x);
                float u = (ENERGY || SWITCH) ? r6 * (t - c.x) : 0.f;
                if (SWITCH) {
                    if (r2 > p.rs2) {
                        const float a = p.rc2 - r2, b = p.rc2 + 2.f * r2 - 3.f * p.rs2;
                        const float sw = a * a * b * p.inv_denom;
                        f = sw * f + 12.f * u * a * (r2 - p.rs2) * p.inv_denom;
                        u *= sw;
                    }
                }
                fmag = f;
                if (ENERGY) epair = u;
            }
            if (COULOMB) {
                const float qq = qi * qj;
                const unsigned shifted = __float_as_uint(r2) - dsmd::kEwaldBaseBits;
                const unsigned idx = shifted >> dsmd::kEwaldIndexShift;
                float ff, ef = 0.f;
                if (idx < static_cast<unsigned>(p.ewald_intervals)) {
                    const float t = __uint_as_float(0x3F800000u | ((shifted << dsmd::kEwaldBits) & 0x007FFFFFu)) - 1.0f;
                    const float4 cf = s_ewald[2 * idx];
                    ff = ((cf.w * t + cf.z) * t + cf.y) * t + cf.x;
                    if (ENERGY) {
                        const float4 ce = s_ewald[2 * idx + 1];
                        ef = ((ce.w * t + ce.z) * t + ce.y) * t + ce.x;
                    }
                } else {   // below the table (r^2 < 0.5): analytic
                    const float r = sqrtf(r2), ar = p.alpha * r;
                    const float ec = erfcf(ar) / r;
                    ff = (ec + p.two_alpha_sqrtpi * __expf(-ar * ar)) * r2inv;
                    ef = ec;
                }
                if (excluded) {   // the pair's 1/r is not part of the Ewald sum: erfc -> -erf
                    const float rinv = rsqrtf(r2);
                    ff -= rinv * r2inv;
                    ef -= rinv;
                }
                fmag += qq * ff;
                if (ENERGY) epair += qq * ef;
            }
            ax += fmag * dx;
            ay += fmag * dy;
            az += fmag * dz;
            if (ENERGY) {
                e_sum += epair;
                w_sum += fmag * r2;
                wx += fmag * dx * dx;
                wy += fmag * dy * dy;
                wz += fmag * dz * dz;
                n_in += 1.f;
            }
        }
    }
};

// One thread per owned atom, 32 atoms of a slice per warp: entry k of the slice is one coalesced 128-byte read (streamed
// past L2 with an evict-first hint, so that the positions stay resident there), the partner's int4 comes through the
// read-only path. The loop runs four entries at a time with the next four entries and the current four positions in
// flight before any arithmetic starts; rows are padded to the loop's stride with the atom's own index, which the
// r^2 >= 1e-10 test discards. Every listed pair is evaluated from the side of each of its owned atoms (full list), so
// forces need no scatter and no atomics, and the summation order is fixed (bitwise reproducible). Energy and virial
// take half of every directed entry; an owned-ghost pair is then counted half on each rank, as the reference's list
// kernel does (src/force_calculator_cuda.cu:1784-1789).
template <bool COULOMB, bool ENERGY, bool MULTI, bool SWITCH, bool EXCL, bool QTYPE>
__global__ void __launch_bounds__(kPairThreads)
k_pair(PairParams p, int n_owned, const int4* __restrict__ pq, const float* __restrict__ qf,
       const unsigned* __restrict__ nbr, int stride, const int* __restrict__ deg, const int* __restrict__ deg_int,
       int phase, const int* __restrict__ atom_list, int first, int n_threads, double* __restrict__ fx,
       double* __restrict__ fy, double* __restrict__ fz, double* __restrict__ partials) {
    extern __shared__ float4 smem[];
    float2* s_c6c12 = reinterpret_cast<float2*>(smem);
    float4* s_ewald = smem + (MULTI ? (p.ntypes * p.ntypes + 1) / 2 : 0);
    // charges by type: the partner's charge comes out of a small table in shared memory (its type arrives with its
    // position) instead of a second gather from global memory
    constexpr bool by_type = COULOMB && QTYPE;   // QTYPE: launched when dsmd_set_type_charges gave a table
    float* s_type_charge = reinterpret_cast<float*>(s_ewald + (COULOMB ? 2 * p.ewald_intervals : 0));
    if (MULTI)
        for (int k = threadIdx.x; k < p.ntypes * p.ntypes; k += blockDim.x) s_c6c12[k] = p.c6c12[k];
    if (COULOMB)
        for (int k = threadIdx.x; k < 2 * p.ewald_intervals; k += blockDim.x) s_ewald[k] = p.ewald[k];
    if (by_type)
        for (int k = threadIdx.x; k < p.ntypes; k += blockDim.x) s_type_charge[k] = p.type_charge[k];
    if (MULTI || COULOMB) __syncthreads();

    // atom_list (boundary pass): the atoms that have a ghost partner, a small part of a brick; null: the owned atoms
    // first .. first + n_threads
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    const int i = t < n_threads ? (atom_list ? atom_list[t] : first + t) : n_owned;
    PairAccumulator<COULOMB, ENERGY, MULTI, SWITCH> acc;
    if (i < n_owned) {
        const int4 pi = pq[i];
        const float qi = COULOMB ? p.kq * (by_type ? s_type_charge[pi.w] : qf[i]) : 0.f;
        const float2 single = MULTI ? make_float2(0.f, 0.f) : p.c6c12[0];
        const int trow = MULTI ? pi.w * p.ntypes : 0;
        const int k_begin = phase == DSMD_PHASE_BOUNDARY ? deg_int[i] : 0;
        const int k_end = phase == DSMD_PHASE_INTERIOR ? deg_int[i] : deg[i];
        const unsigned* row = nbr + (static_cast<size_t>(i >> 5) * stride) * 32 + (i & 31);
        const unsigned self = static_cast<unsigned>(i);
        constexpr int U = 4;
        unsigned e[U], e_next[U];
#pragma unroll
        for (int u = 0; u < U; ++u) e_next[u] = (k_begin + u < k_end) ? __ldcs(row + static_cast<size_t>(k_begin + u) * 32) : self;
        for (int k = k_begin; k < k_end; k += U) {
            int4 pj[U];
            float qj[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                e[u] = e_next[u];
                pj[u] = __ldg(&pq[EXCL ? (e[u] & kIndexMask) : e[u]]);
                if (COULOMB && !by_type) qj[u] = __ldg(&qf[EXCL ? (e[u] & kIndexMask) : e[u]]);
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
                e_next[u] = (k + U + u < k_end) ? __ldcs(row + static_cast<size_t>(k + U + u) * 32) : self;
#pragma unroll
            for (int u = 0; u < U; ++u)
                acc.add(p, pi, pj[u], qi, COULOMB ? (by_type ? s_type_charge[pj[u].w] : qj[u]) : 0.f,
                        EXCL && (e[u] & kExclBit) != 0u, s_c6c12, s_ewald, single, trow);
        }
        if (phase == DSMD_PHASE_BOUNDARY) {
            if (k_end > k_begin) {   // most atoms of a brick have no ghost partner: leave their forces alone
                fx[i] += static_cast<double>(acc.ax);
                fy[i] += static_cast<double>(acc.ay);
                fz[i] += static_cast<double>(acc.az);
            }
        } else {
            fx[i] = static_cast<double>(acc.ax);
            fy[i] = static_cast<double>(acc.ay);
            fz[i] = static_cast<double>(acc.az);
        }
    }
    if (ENERGY) {
        double v[6] = {0.5 * static_cast<double>(acc.e_sum), 0.5 * static_cast<double>(acc.w_sum),
                       0.5 * static_cast<double>(acc.wx),    0.5 * static_cast<double>(acc.wy),
                       0.5 * static_cast<double>(acc.wz),    0.5 * static_cast<double>(acc.n_in)};
        block_sum_to_partials<6>(v, partials);
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// kernels: ghosts
// ---------------------------------------------------------------------------------------------------------------------

__global__ void k_halo_pack(int count, const int* __restrict__ index, const signed char* __restrict__ image,
                            const double* __restrict__ x, const double* __restrict__ y, const double* __restrict__ z,
                            double bx, double by, double bz, double* __restrict__ out) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= count) return;
    const int s = index[k];
    double sx = 0.0, sy = 0.0, sz = 0.0;
    if (image) {
        sx = image[3 * k] * bx;
        sy = image[3 * k + 1] * by;
        sz = image[3 * k + 2] * bz;
    }
    out[3 * k] = x[s] + sx;
    out[3 * k + 1] = y[s] + sy;
    out[3 * k + 2] = z[s] + sz;
}

__global__ void k_halo_unpack(Grid g, int first_ghost, int count, const double* __restrict__ in,
                              const int* __restrict__ ghost_slot, double* __restrict__ x, double* __restrict__ y,
                              double* __restrict__ z, const int* __restrict__ type, int4* __restrict__ pq, Status* st) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= count) return;
    const int s = ghost_slot[first_ghost + k];
    const double px = in[3 * k], py = in[3 * k + 1], pz = in[3 * k + 2];
    x[s] = px; y[s] = py; z[s] = pz;
    unsigned bad = 0;
    int4 p;
    p.x = static_cast<int>(dsmd::to_fixed(px, 0, g, bad));
    p.y = static_cast<int>(dsmd::to_fixed(py, 1, g, bad));
    p.z = static_cast<int>(dsmd::to_fixed(pz, 2, g, bad));
    p.w = type[s];
    pq[s] = p;
    if (bad) atomicAdd(&st->out_of_domain, 1u);
}

__global__ void k_halo_flag(int n_owned, const double* __restrict__ x, const double* __restrict__ y,
                            const double* __restrict__ z, double lx, double ly, double lz, double hx, double hy,
                            double hz, unsigned char* __restrict__ flag) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= n_owned) return;
    const double px = x[s], py = y[s], pz = z[s];
    flag[s] = (px >= lx && px < hx && py >= ly && py < hy && pz >= lz && pz < hz) ? 1 : 0;
}

__global__ void k_halo_pack_records(int count, const int* __restrict__ index, RealArrays a,
                                    const int* __restrict__ type, const int* __restrict__ gid, double sx, double sy,
                                    double sz, double* __restrict__ real_out, int* __restrict__ int_out) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= count) return;
    const int s = index[k];
    double* o = real_out + 8 * static_cast<size_t>(k);
    o[0] = a.p[0][s] + sx; o[1] = a.p[1][s] + sy; o[2] = a.p[2][s] + sz;
    o[3] = a.p[3][s]; o[4] = a.p[4][s]; o[5] = a.p[5][s];
    o[6] = a.p[9][s]; o[7] = a.p[10][s];
    int_out[2 * k] = type[s];
    int_out[2 * k + 1] = gid[s];
}

__global__ void k_halo_append_records(int count, int first_slot, const double* __restrict__ real_in,
                                      const int* __restrict__ int_in, RealArrays a, int* __restrict__ type,
                                      int* __restrict__ gid) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= count) return;
    const int s = first_slot + k;
    const double* r = real_in + 8 * static_cast<size_t>(k);
    a.p[0][s] = r[0]; a.p[1][s] = r[1]; a.p[2][s] = r[2];
    a.p[3][s] = r[3]; a.p[4][s] = r[4]; a.p[5][s] = r[5];
    a.p[6][s] = 0.0; a.p[7][s] = 0.0; a.p[8][s] = 0.0;
    a.p[9][s] = r[6]; a.p[10][s] = r[7];
    type[s] = int_in[2 * k];
    gid[s] = int_in[2 * k + 1];
}

// Full records as one run of nine doubles per atom: x y z vx vy vz mass charge and the two int32 words (type, gid) in the
// ninth - one message per peer carries every field.
__global__ void k_halo_append_packed(int count, int first_slot, const double* __restrict__ rec, RealArrays a,
                                     int* __restrict__ type, int* __restrict__ gid) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= count) return;
    const int s = first_slot + k;
    const double* r = rec + 9 * static_cast<size_t>(k);
    a.p[0][s] = r[0]; a.p[1][s] = r[1]; a.p[2][s] = r[2];
    a.p[3][s] = r[3]; a.p[4][s] = r[4]; a.p[5][s] = r[5];
    a.p[6][s] = 0.0; a.p[7][s] = 0.0; a.p[8][s] = 0.0;
    a.p[9][s] = r[6]; a.p[10][s] = r[7];
    const long long words = __double_as_longlong(r[8]);
    type[s] = static_cast<int>(words & 0xFFFFFFFFll);
    gid[s] = static_cast<int>(words >> 32);
}

// Dependent-FMA-free throughput probe: 8 independent fp32 FMA chains per thread. The benchmark times it to get the
// fp32 CUDA-core peak of the device it runs on (the denominator of the pair kernel's compute roofline).
__global__ void __launch_bounds__(256) k_fma_probe(int iters, float seed, float* out) {
    float a0 = seed + threadIdx.x, a1 = a0 + 1.f, a2 = a0 + 2.f, a3 = a0 + 3.f, a4 = a0 + 4.f, a5 = a0 + 5.f,
          a6 = a0 + 6.f, a7 = a0 + 7.f;
    const float m = 0.999f, c = 0.001f;
#pragma unroll 4
    for (int k = 0; k < iters; ++k) {
        a0 = a0 * m + c; a1 = a1 * m + c; a2 = a2 * m + c; a3 = a3 * m + c;
        a4 = a4 * m + c; a5 = a5 * m + c; a6 = a6 * m + c; a7 = a7 * m + c;
    }
    const float sum = a0 + a1 + a2 + a3 + a4 + a5 + a6 + a7;
    if (sum == 12345.678f) out[0] = sum;   // never true: keeps the chains alive
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------------------
// the context
// ---------------------------------------------------------------------------------------------------------------------

struct dsmd_ctx {
    int device = 0;
    int64_t capacity = 0;
    int64_t n_owned = 0, n_total = 0;
    std::string error;
    int64_t launches = 0;

    // box
    double box[3] = {0, 0, 0}, lo[3] = {0, 0, 0}, hi[3] = {0, 0, 0}, halo = 0.0;
    int periodic[3] = {1, 1, 1};
    bool box_set = false;
    // parameters
    int ntypes = 0;
    double cutoff = 0.0, skin = 0.0, switch_distance = -1.0;
    bool params_set = false;
    bool coulomb = false;
    double alpha = 0.0;
    int ewald_intervals = 0;
    Grid grid{};
    bool grid_valid = false;

    // device storage
    double* real[2][kNumReal] = {};
    int* type[2] = {};
    int* gid[2] = {};
    int cur = 0;
    int4* pq = nullptr;
    float4* pf = nullptr;          // positions as fp32 offsets from the grid origin, as of the last sort (list search)
    float* qf = nullptr;
    double* ref[3] = {};
    unsigned* key[2] = {};
    int* val[2] = {};
    int* ghost_slot = nullptr;
    // the host-buffer force call as a pipeline (dsmd_forces_host): first slot of every z layer of cells as of the last
    // build, two copy streams, one event pair per piece
    int* d_layer_start = nullptr;
    int* h_layer_start = nullptr;     // pinned, [nc_z + 1]
    int layer_capacity = 0;
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    cudaEvent_t piece_up[16] = {}, piece_done[16] = {}, pipe_begin = nullptr, pipe_end = nullptr;
    int* boundary_list = nullptr;     // [capacity] owned atoms with a ghost partner, as the last list build found them
    int64_t n_boundary = 0;
    float* type_charge = nullptr;     // [ntypes] charges by type (dsmd_set_type_charges), or null: per-atom charges
    int* cell_start = nullptr;
    int64_t cell_capacity = 0;
    int* ghost_rows = nullptr;        // [4 * rows]: lo_end, hi_begin per (y, z) row, then the same over the rows searched
    int64_t ghost_rows_capacity = 0;
    unsigned* nbr = nullptr;
    size_t nbr_capacity = 0;   // entries
    int stride = 0;
    int* deg = nullptr;
    int* deg_int = nullptr;
    void* cub_temp = nullptr;
    size_t cub_temp_bytes = 0;
    float2* c6c12 = nullptr;
    float4* ewald = nullptr;
    int* excl_off = nullptr;
    int* excl_partner = nullptr;
    int64_t excl_n_global = 0;
    double* partials = nullptr;
    int64_t partial_blocks = 0;
    double* scalars = nullptr;      // 6 force scalars + 1 kinetic
    Status* status = nullptr;
    Status* h_status = nullptr;     // pinned
    double* h_scalars = nullptr;    // pinned
    unsigned long long* h_disp[2] = {};   // pinned, lagged displacement read-back
    long long disp_epoch[2] = {-1, -1};   // list build each read-back slot was measured under
    int disp_pending = -1;                // slot queued by the previous lagged query
    long long build_epoch = 0;            // bumped by every list build (new reference positions)
    cudaEvent_t disp_event[2] = {};
    unsigned char* flag = nullptr;
    unsigned long long* offsets64 = nullptr;
    bool list_valid = false;
    // distance constraints (dsmd_constraints.cuh)
    // bonded terms (dsmd_set_bonded)
    struct Bonded {
        int64_t n_global = 0, n_bonds = 0, n_angles = 0, n_torsions = 0, n_specials = 0, n_entries = 0, blocks = 0;
        int *bond_atoms = nullptr, *angle_atoms = nullptr, *torsion_atoms = nullptr, *torsion_n = nullptr, *special_atoms = nullptr;
        double *bond_par = nullptr, *angle_par = nullptr, *torsion_par = nullptr, *special_par = nullptr;
        int* slot_of_gid = nullptr;          // [n_global]
        long long* entries_of = nullptr;     // [n_global + 1]
        int* entry = nullptr;                // [n_entries]
        double* contrib = nullptr;           // [3 * n_entries]
        double* partials = nullptr;          // [5 * blocks]
        double* scalars = nullptr;           // device: PE, W, Wxx, Wyy, Wzz
        unsigned* missing = nullptr;         // device: terms with an owned atom and a partner that is not on this rank
        double* h_scalars = nullptr;         // pinned: 5 scalars + the missing count
        int64_t map_epoch = -1;              // list build the gid -> slot map belongs to
        int64_t terms() const { return n_bonds + n_angles + n_torsions + n_specials; }
    } bonded;
    int n_clusters = 0;
    int64_t cons_n_global = 0;
    int* cl_gid = nullptr;
    unsigned char* cl_a = nullptr;
    unsigned char* cl_b = nullptr;
    double* cl_d2 = nullptr;
    int* slot_of_gid = nullptr;
    bool slot_map_valid = false;
    double* pre[3] = {};
    double cons_tolerance = 1e-8;
    int cons_max_iterations = 500;
    bool owned_sorted_only = false;
    int64_t expect_dropped = 0;    // atoms the last owned-only sort was told to remove (checked with the build status)
    int64_t stat_entries = 0, stat_interior = 0;
    int stat_rechecked = 0;
};

namespace {

#define DSMD_CUDA(ctx, call)                                                                       \
    do {                                                                                           \
        cudaError_t err_ = (call);                                                                 \
        if (err_ != cudaSuccess) {                                                                 \
            (ctx)->error = std::string(#call) + ": " + cudaGetErrorString(err_);                   \
            return DSMD_ERR_CUDA;                                                                  \
        }                                                                                          \
    } while (0)

#define DSMD_LAUNCHED(ctx)                                                                         \
    do {                                                                                           \
        ++(ctx)->launches;                                                                         \
        cudaError_t err_ = cudaGetLastError();                                                     \
        if (err_ != cudaSuccess) {                                                                 \
            (ctx)->error = std::string("kernel launch: ") + cudaGetErrorString(err_);              \
            return DSMD_ERR_CUDA;                                                                  \
        }                                                                                          \
    } while (0)

void free_bonded(dsmd_ctx* c) {
    dsmd_ctx::Bonded& b = c->bonded;
    cudaFree(b.bond_atoms); cudaFree(b.angle_atoms); cudaFree(b.torsion_atoms); cudaFree(b.torsion_n); cudaFree(b.special_atoms);
    cudaFree(b.bond_par); cudaFree(b.angle_par); cudaFree(b.torsion_par); cudaFree(b.special_par);
    cudaFree(b.slot_of_gid); cudaFree(b.entries_of); cudaFree(b.entry); cudaFree(b.contrib); cudaFree(b.partials);
    cudaFree(b.scalars); cudaFree(b.missing);
    if (b.h_scalars) cudaFreeHost(b.h_scalars);
    b = dsmd_ctx::Bonded();
}

int fail(dsmd_ctx* ctx, int code, const std::string& what) {
    ctx->error = what;
    return code;
}

RealArrays arrays_of(dsmd_ctx* c, int set) {
    RealArrays a;
    for (int f = 0; f < kNumReal; ++f) a.p[f] = c->real[set][f];
    return a;
}

// Chooses the fixed-point mapping and the cell grid for the current box, cutoff and skin.
int make_grid(dsmd_ctx* c) {
    if (!c->box_set || !c->params_set) return fail(c, DSMD_ERR_STATE, "box and pair parameters must be set first");
    Grid& g = c->grid;
    const double R = c->cutoff + c->skin;
    double max_scale = 0.0;
    bool split[3];
    for (int a = 0; a < 3; ++a) {
        const bool has_sub = c->hi[a] > c->lo[a];
        split[a] = has_sub && (c->hi[a] - c->lo[a]) < c->box[a] - 1e-6;
        g.box[a] = c->box[a];
        if (c->periodic[a] && !split[a]) {
            g.wrap[a] = 1;
            g.org[a] = 0.0;
            g.inv_len[a] = 1.0 / c->box[a];
            g.scale[a] = static_cast<float>(c->box[a] / 4294967296.0);
            max_scale = std::max(max_scale, c->box[a] / 4294967296.0);
        } else {
            const double lo = (has_sub ? c->lo[a] : 0.0) - c->halo;
            const double hi = (has_sub ? c->hi[a] : c->box[a]) + c->halo;
            g.wrap[a] = 0;
            g.org[a] = lo;
            g.inv_len[a] = 1.0 / (hi - lo);
            g.scale[a] = static_cast<float>((hi - lo) / 2147483648.0);
            max_scale = std::max(max_scale, (hi - lo) / 2147483648.0);
        }
    }
    // Cells at least R / stencil wide (a hair more, so that fixed-point rounding cannot push a partner one cell too far).
    int stencil = 2;
    int x_refine = kXRefine;
    if (const char* e = std::getenv("DSMD_XREFINE")) x_refine = std::max(1, std::min(8, std::atoi(e)));
    for (int attempt = 0; attempt < 2; ++attempt) {
        bool ok = true;
        for (int a = 0; a < 3; ++a) {
            const double len = 1.0 / g.inv_len[a];
            const double width = R / stencil * (1.0 + 1e-6);
            int nc = static_cast<int>(std::floor(len / width));
            nc = std::max(1, std::min(nc, 1024));
            if (g.wrap[a] && nc < 2 * stencil + 1) ok = false;
            g.nc[a] = nc;
        }
        if (ok) { g.stencil = stencil; break; }
        if (stencil == 1) {
            return fail(c, DSMD_ERR_BOX_TOO_SMALL,
                        "a periodic axis is shorter than three cells of width cutoff + skin");
        }
        stencil = 1;
    }
    // Rows of cells along x are contiguous runs of slots, searched through a window that is rounded outwards to whole
    // cells: finer x cells (kXRefine per unrefined cell) make the windows tighter at no cost per row.
    g.x_reach = static_cast<float>(g.stencil * (1.0 / (g.inv_len[0] * g.nc[0])) * 0.9999999);
    {
        int refine = x_refine;
        while (refine > 1 && (static_cast<int64_t>(g.nc[0]) * refine > 4096 ||
                              2 * static_cast<int64_t>(g.nc[0]) * refine * g.nc[1] * g.nc[2] + 1 > (1ll << 26)))
            refine >>= 1;
        g.nc[0] *= refine;
    }
    const int64_t ncells = static_cast<int64_t>(g.nc[0]) * g.nc[1] * g.nc[2];
    if (2 * ncells + 1 > (1ll << 30)) return fail(c, DSMD_ERR_INVALID, "cell grid too large");
    g.ncells = static_cast<int>(ncells);
    g.r2_list = static_cast<float>(R * R);
    g.r2_list_d = R * R;
    g.band = static_cast<float>(8.0 * R * max_scale + 16.0 * R * R * 5.9604645e-8);
    double max_len = 0.0;
    for (int a = 0; a < 3; ++a) {
        g.cellw[a] = static_cast<float>(1.0 / (g.inv_len[a] * g.nc[a]));
        max_len = std::max(max_len, 1.0 / g.inv_len[a]);
    }
    g.r_pad = static_cast<float>(R * (1.0 + 1e-4) + 8.0 * max_len * 1.2e-7);
    // Rounding band of the fp32 search: a coordinate is an offset of up to max_len from the grid origin, the centre's may
    // carry one more box length (image shift), so each carries a few ulp of 2 max_len; the squares and sums add a few
    // ulp of R^2; the fixed-point grid itself one unit per coordinate. Everything inside the band is re-decided in fp64.
    g.band_search = static_cast<float>(1.1920929e-7 * (24.0 * R * max_len + 16.0 * R * R) + 8.0 * R * max_scale);
    c->grid_valid = true;
    return DSMD_OK;
}

int ensure_cells(dsmd_ctx* c) {
    const int64_t need = 2ll * c->grid.ncells + 1;
    if (need > c->cell_capacity) {
        if (c->cell_start) cudaFree(c->cell_start);
        c->cell_start = nullptr;
        DSMD_CUDA(c, cudaMalloc(&c->cell_start, sizeof(int) * need));
        c->cell_capacity = need;
    }
    return DSMD_OK;
}

int ensure_list(dsmd_ctx* c, int stride) {
    const size_t slices = static_cast<size_t>((c->n_owned + 31) / 32);
    const size_t need = slices * static_cast<size_t>(stride) * 32;
    if (need > c->nbr_capacity) {
        // with headroom: the owned count of a brick changes by a few atoms at every migration, and a reallocation of this
        // (large) buffer synchronises the device
        const size_t grown = need + need / 8 + 4096;
        if (c->nbr) cudaFree(c->nbr);
        c->nbr = nullptr;
        c->nbr_capacity = 0;
        DSMD_CUDA(c, cudaMalloc(&c->nbr, sizeof(unsigned) * grown));
        c->nbr_capacity = grown;
    }
    c->stride = stride;
    return DSMD_OK;
}

int ensure_partials(dsmd_ctx* c, int64_t blocks) {
    if (blocks > c->partial_blocks) {
        if (c->partials) cudaFree(c->partials);
        c->partials = nullptr;
        DSMD_CUDA(c, cudaMalloc(&c->partials, sizeof(double) * 6 * blocks));
        c->partial_blocks = blocks;
    }
    return DSMD_OK;
}

// Sorts slots [first, n_total) by cell and gathers everything into the other buffer set. n_removed > 0 (owned-only
// sorts): that many atoms lie outside the brick; they sort behind every cell and fall off the end.
int sort_range(dsmd_ctx* c, int64_t first, cudaStream_t s, int64_t n_removed = 0, const Brick* bounds = nullptr) {
    const int64_t n = c->n_total - first;
    const int from = c->cur, to = 1 - c->cur;
    if (n > 0) {
        Brick brick{};
        if (bounds) brick = *bounds;
        brick.drop = (bounds && n_removed > 0) ? 1 : 0;
        k_cell_keys<<<blocks_for(n, kThreads), kThreads, 0, s>>>(
            c->grid, brick, static_cast<int>(first), static_cast<int>(c->n_owned), static_cast<int>(c->n_total),
            c->real[from][0], c->real[from][1], c->real[from][2], c->key[0], c->val[0], c->status);
        DSMD_LAUNCHED(c);
        int bits = 1;
        while ((1ll << bits) < 2ll * c->grid.ncells + 1) ++bits;
        size_t need = 0;
        cub::DeviceRadixSort::SortPairs(nullptr, need, c->key[0], c->key[1], c->val[0], c->val[1], static_cast<int>(n), 0,
                                        bits, s);
        if (need > c->cub_temp_bytes) {
            if (c->cub_temp) cudaFree(c->cub_temp);
            c->cub_temp = nullptr;
            DSMD_CUDA(c, cudaMalloc(&c->cub_temp, need + need / 4));
            c->cub_temp_bytes = need + need / 4;
        }
        DSMD_CUDA(c, cub::DeviceRadixSort::SortPairs(c->cub_temp, need, c->key[0], c->key[1], c->val[0], c->val[1],
                                                     static_cast<int>(n), 0, bits, s));
        k_reorder<<<blocks_for(n, kThreads), kThreads, 0, s>>>(
            c->grid, static_cast<int>(first), static_cast<int>(c->n_owned), static_cast<int>(c->n_total), c->key[1],
            c->val[1], arrays_of(c, from), arrays_of(c, to), c->type[from], c->gid[from], c->type[to], c->gid[to], c->pq,
            c->pf, c->qf, c->ref[0], c->ref[1], c->ref[2], c->cell_start, c->ghost_slot);
        DSMD_LAUNCHED(c);
        const int table = 2 * c->grid.ncells + 1;
        const int64_t kept = n - n_removed;
        if (kept > 0) {
            k_cell_tail<<<blocks_for(table, kThreads), kThreads, 0, s>>>(c->key[1], static_cast<int>(kept),
                                                                      static_cast<int>(c->n_total - n_removed), table,
                                                                      c->cell_start);
            DSMD_LAUNCHED(c);
        }
    }
    if (first > 0) {
        // a ghost-only sort: the owned atoms are in place in the current set, the sorted ghosts come back to it (far
        // fewer bytes than carrying the owned atoms across, and one launch instead of thirteen copies)
        if (n > 0) {
            k_copy_back<<<blocks_for(n, kThreads), kThreads, 0, s>>>(static_cast<int>(first), static_cast<int>(n),
                                                                    arrays_of(c, to), arrays_of(c, from), c->type[to],
                                                                    c->gid[to], c->type[from], c->gid[from]);
            DSMD_LAUNCHED(c);
        }
    } else {
        c->cur = to;
    }
    c->slot_map_valid = false;
    return DSMD_OK;
}

int read_status(dsmd_ctx* c, cudaStream_t s) {
    DSMD_CUDA(c, cudaMemcpyAsync(c->h_status, c->status, sizeof(Status), cudaMemcpyDeviceToHost, s));
    DSMD_CUDA(c, cudaStreamSynchronize(s));
    return DSMD_OK;
}

template <bool COULOMB, bool ENERGY, bool MULTI>
void launch_pair(dsmd_ctx* c, const PairParams& p, int phase, bool sw, cudaStream_t s, int first, int n_threads) {
    const int* atom_list = phase == DSMD_PHASE_BOUNDARY ? c->boundary_list : nullptr;
    const unsigned blocks = blocks_for(n_threads, kPairThreads);
    size_t smem = 0;
    if (MULTI) smem += sizeof(float4) * ((p.ntypes * p.ntypes + 1) / 2);
    if (COULOMB) smem += sizeof(float4) * 2 * p.ewald_intervals;
    if (COULOMB && p.type_charge) smem += sizeof(float4) * ((p.ntypes + 3) / 4);
    double* fx = c->real[c->cur][DSMD_FX];
    double* fy = c->real[c->cur][DSMD_FY];
    double* fz = c->real[c->cur][DSMD_FZ];
    const bool ex = c->excl_off != nullptr;
#define DSMD_PAIR_LAUNCH(SW, EX, QT)                                                                                  \
    k_pair<COULOMB, ENERGY, MULTI, SW, EX, QT><<<blocks, kPairThreads, smem, s>>>(                                      \
        p, static_cast<int>(c->n_owned), c->pq, c->qf, c->nbr, c->stride, c->deg, c->deg_int, phase, atom_list, first,  \
        n_threads, fx, fy, fz, c->partials)
    if (COULOMB && p.type_charge) {   // charges by type: only the kernels with Coulomb have this form
        if (sw) { if (ex) DSMD_PAIR_LAUNCH(true, true, COULOMB); else DSMD_PAIR_LAUNCH(true, false, COULOMB); }
        else    { if (ex) DSMD_PAIR_LAUNCH(false, true, COULOMB); else DSMD_PAIR_LAUNCH(false, false, COULOMB); }
    } else {
        if (sw) { if (ex) DSMD_PAIR_LAUNCH(true, true, false); else DSMD_PAIR_LAUNCH(true, false, false); }
        else    { if (ex) DSMD_PAIR_LAUNCH(false, true, false); else DSMD_PAIR_LAUNCH(false, false, false); }
    }
#undef DSMD_PAIR_LAUNCH
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------------------------------------

extern "C" {

int dsmd_create(int device, int64_t capacity, dsmd_ctx** out) {
    if (!out || capacity <= 0 || capacity >= (1ll << 30)) return DSMD_ERR_INVALID;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) return DSMD_ERR_CUDA;
    dsmd_ctx* c = new dsmd_ctx();
    c->device = device;
    c->capacity = capacity;
    *out = c;
    DSMD_CUDA(c, cudaSetDevice(device));
    for (int set = 0; set < 2; ++set) {
        for (int f = 0; f < kNumReal; ++f) {
            DSMD_CUDA(c, cudaMalloc(&c->real[set][f], sizeof(double) * capacity));
            DSMD_CUDA(c, cudaMemset(c->real[set][f], 0, sizeof(double) * capacity));
        }
        DSMD_CUDA(c, cudaMalloc(&c->type[set], sizeof(int) * capacity));
        DSMD_CUDA(c, cudaMalloc(&c->gid[set], sizeof(int) * capacity));
        DSMD_CUDA(c, cudaMalloc(&c->key[set], sizeof(unsigned) * capacity));
        DSMD_CUDA(c, cudaMalloc(&c->val[set], sizeof(int) * capacity));
    }
    DSMD_CUDA(c, cudaMalloc(&c->pq, sizeof(int4) * capacity));
    DSMD_CUDA(c, cudaMalloc(&c->pf, sizeof(float4) * capacity));
    DSMD_CUDA(c, cudaMalloc(&c->qf, sizeof(float) * capacity));
    for (int a = 0; a < 3; ++a) DSMD_CUDA(c, cudaMalloc(&c->ref[a], sizeof(double) * capacity));
    DSMD_CUDA(c, cudaMalloc(&c->ghost_slot, sizeof(int) * capacity));
    DSMD_CUDA(c, cudaMalloc(&c->deg, sizeof(int) * capacity));
    DSMD_CUDA(c, cudaMalloc(&c->deg_int, sizeof(int) * capacity));
    DSMD_CUDA(c, cudaMalloc(&c->boundary_list, sizeof(int) * capacity));
    DSMD_CUDA(c, cudaMalloc(&c->flag, capacity));
    DSMD_CUDA(c, cudaMalloc(&c->offsets64, sizeof(unsigned long long) * capacity));
    DSMD_CUDA(c, cudaMalloc(&c->scalars, sizeof(double) * 8));
    DSMD_CUDA(c, cudaMemset(c->scalars, 0, sizeof(double) * 8));
    DSMD_CUDA(c, cudaMalloc(&c->status, sizeof(Status)));
    DSMD_CUDA(c, cudaMemset(c->status, 0, sizeof(Status)));
    DSMD_CUDA(c, cudaMallocHost(&c->h_status, sizeof(Status)));
    DSMD_CUDA(c, cudaMallocHost(&c->h_scalars, sizeof(double) * 8));
    for (int k = 0; k < 2; ++k) {
        DSMD_CUDA(c, cudaMallocHost(&c->h_disp[k], sizeof(unsigned long long)));
        *c->h_disp[k] = 0ull;
        DSMD_CUDA(c, cudaEventCreateWithFlags(&c->disp_event[k], cudaEventDisableTiming));
    }
    return DSMD_OK;
}

void dsmd_destroy(dsmd_ctx* c) {
    if (!c) return;
    cudaSetDevice(c->device);
    for (int set = 0; set < 2; ++set) {
        for (int f = 0; f < kNumReal; ++f) cudaFree(c->real[set][f]);
        cudaFree(c->type[set]); cudaFree(c->gid[set]); cudaFree(c->key[set]); cudaFree(c->val[set]);
    }
    cudaFree(c->pq); cudaFree(c->pf); cudaFree(c->qf); cudaFree(c->type_charge);
    for (int a = 0; a < 3; ++a) cudaFree(c->ref[a]);
    cudaFree(c->ghost_slot); cudaFree(c->cell_start); cudaFree(c->ghost_rows); cudaFree(c->nbr); cudaFree(c->deg); cudaFree(c->deg_int);
    cudaFree(c->boundary_list);
    cudaFree(c->cub_temp); cudaFree(c->c6c12); cudaFree(c->ewald); cudaFree(c->excl_off); cudaFree(c->excl_partner);
    cudaFree(c->partials); cudaFree(c->scalars); cudaFree(c->status); cudaFree(c->flag); cudaFree(c->offsets64);
    cudaFree(c->cl_gid); cudaFree(c->cl_a); cudaFree(c->cl_b); cudaFree(c->cl_d2); cudaFree(c->slot_of_gid);
    free_bonded(c);
    cudaFree(c->d_layer_start);
    if (c->h_layer_start) cudaFreeHost(c->h_layer_start);
    if (c->copy_in) cudaStreamDestroy(c->copy_in);
    if (c->copy_out) cudaStreamDestroy(c->copy_out);
    for (int k = 0; k < 16; ++k) {
        if (c->piece_up[k]) cudaEventDestroy(c->piece_up[k]);
        if (c->piece_done[k]) cudaEventDestroy(c->piece_done[k]);
    }
    if (c->pipe_begin) cudaEventDestroy(c->pipe_begin);
    if (c->pipe_end) cudaEventDestroy(c->pipe_end);
    for (int a = 0; a < 3; ++a) cudaFree(c->pre[a]);
    cudaFreeHost(c->h_status); cudaFreeHost(c->h_scalars);
    for (int k = 0; k < 2; ++k) {
        cudaFreeHost(c->h_disp[k]);
        if (c->disp_event[k]) cudaEventDestroy(c->disp_event[k]);
    }
    delete c;
}

const char* dsmd_last_error(const dsmd_ctx* c) { return c ? c->error.c_str() : "null context"; }

int64_t dsmd_launch_count(const dsmd_ctx* c) { return c ? c->launches : 0; }

int dsmd_set_box(dsmd_ctx* c, const double box[3], const int periodic[3], const double lo[3], const double hi[3],
                 double halo) {
    if (!c || !box || !periodic) return DSMD_ERR_INVALID;
    for (int a = 0; a < 3; ++a) {
        if (!(box[a] > 0.0) || !std::isfinite(box[a])) return fail(c, DSMD_ERR_INVALID, "box lengths must be positive");
        c->box[a] = box[a];
        c->periodic[a] = periodic[a] != 0;
        c->lo[a] = lo ? lo[a] : 0.0;
        c->hi[a] = hi ? hi[a] : 0.0;
    }
    c->halo = halo > 0.0 ? halo : 0.0;
    c->box_set = true;
    c->grid_valid = false;
    c->list_valid = false;
    return DSMD_OK;
}

int dsmd_set_pair_params(dsmd_ctx* c, int ntypes, const double* eps, const double* sig, double cutoff, double skin,
                         double switch_distance) {
    if (!c || ntypes <= 0 || ntypes > 64 || !eps || !sig) return DSMD_ERR_INVALID;
    if (!(cutoff > 0.0) || skin < 0.0) return fail(c, DSMD_ERR_INVALID, "cutoff must be positive, skin non-negative");
    if (switch_distance >= cutoff) return fail(c, DSMD_ERR_INVALID, "switch distance must be below the cutoff");
    DSMD_CUDA(c, cudaSetDevice(c->device));
    std::vector<float2> table(static_cast<size_t>(ntypes) * ntypes);
    for (int k = 0; k < ntypes * ntypes; ++k) {
        const double s2 = sig[k] * sig[k], s6 = s2 * s2 * s2;
        const double c6 = 4.0 * eps[k] * s6;
        table[k] = make_float2(static_cast<float>(c6), static_cast<float>(c6 * s6));
    }
    if (c->c6c12) cudaFree(c->c6c12);
    c->c6c12 = nullptr;
    DSMD_CUDA(c, cudaMalloc(&c->c6c12, sizeof(float2) * table.size()));
    DSMD_CUDA(c, cudaMemcpy(c->c6c12, table.data(), sizeof(float2) * table.size(), cudaMemcpyHostToDevice));
    c->ntypes = ntypes;
    c->cutoff = cutoff;
    c->skin = skin;
    c->switch_distance = switch_distance;
    c->params_set = true;
    c->grid_valid = false;
    c->list_valid = false;
    if (c->coulomb) return dsmd_set_coulomb(c, 1, c->alpha);
    return DSMD_OK;
}

int dsmd_set_coulomb(dsmd_ctx* c, int enabled, double alpha) {
    if (!c) return DSMD_ERR_INVALID;
    c->coulomb = enabled != 0;
    if (!c->coulomb) return DSMD_OK;
    if (!c->params_set) return fail(c, DSMD_ERR_STATE, "set the pair parameters (cutoff) before Coulomb");
    DSMD_CUDA(c, cudaSetDevice(c->device));
    c->alpha = alpha > 0.0 ? alpha : dsmd::ewald_alpha_for(c->cutoff);
    c->ewald_intervals = dsmd::ewald_intervals(c->cutoff * c->cutoff);
    const std::vector<float> coef = dsmd::ewald_build_table(c->alpha, c->ewald_intervals);
    if (c->ewald) cudaFree(c->ewald);
    c->ewald = nullptr;
    DSMD_CUDA(c, cudaMalloc(&c->ewald, sizeof(float) * coef.size()));
    DSMD_CUDA(c, cudaMemcpy(c->ewald, coef.data(), sizeof(float) * coef.size(), cudaMemcpyHostToDevice));
    return DSMD_OK;
}

int dsmd_get_ewald_alpha(const dsmd_ctx* c, double* alpha) {
    if (!c || !alpha) return DSMD_ERR_INVALID;
    *alpha = c->alpha;
    return DSMD_OK;
}

int dsmd_set_exclusions(dsmd_ctx* c, int64_t n_global, int64_t n_pairs, const int32_t* a, const int32_t* b) {
    if (!c || n_global < 0 || n_pairs < 0 || (n_pairs > 0 && (!a || !b))) return DSMD_ERR_INVALID;
    DSMD_CUDA(c, cudaSetDevice(c->device));
    if (c->excl_off) cudaFree(c->excl_off);
    if (c->excl_partner) cudaFree(c->excl_partner);
    c->excl_off = c->excl_partner = nullptr;
    c->excl_n_global = 0;
    c->list_valid = false;
    if (n_pairs == 0) return DSMD_OK;
    std::vector<std::pair<int, int>> directed;
    directed.reserve(2 * n_pairs);
    for (int64_t k = 0; k < n_pairs; ++k) {
        if (a[k] < 0 || b[k] < 0 || a[k] >= n_global || b[k] >= n_global || a[k] == b[k])
            return fail(c, DSMD_ERR_INVALID, "exclusion pair out of range");
        directed.emplace_back(a[k], b[k]);
        directed.emplace_back(b[k], a[k]);
    }
    std::sort(directed.begin(), directed.end());
    directed.erase(std::unique(directed.begin(), directed.end()), directed.end());
    std::vector<int> off(n_global + 1, 0), partner(directed.size());
    for (const auto& d : directed) ++off[d.first + 1];
    for (int64_t g = 0; g < n_global; ++g) off[g + 1] += off[g];
    for (size_t k = 0; k < directed.size(); ++k) partner[k] = directed[k].second;
    DSMD_CUDA(c, cudaMalloc(&c->excl_off, sizeof(int) * off.size()));
    DSMD_CUDA(c, cudaMalloc(&c->excl_partner, sizeof(int) * std::max<size_t>(partner.size(), 1)));
    DSMD_CUDA(c, cudaMemcpy(c->excl_off, off.data(), sizeof(int) * off.size(), cudaMemcpyHostToDevice));
    DSMD_CUDA(c, cudaMemcpy(c->excl_partner, partner.data(), sizeof(int) * partner.size(), cudaMemcpyHostToDevice));
    c->excl_n_global = n_global;
    return DSMD_OK;
}

int dsmd_upload(dsmd_ctx* c, int64_t n_owned, int64_t n_total, const double* x, const double* y, const double* z,
                const double* vx, const double* vy, const double* vz, const double* mass, const double* charge,
                const int32_t* type, const int32_t* gid, void* stream) {
    if (!c || n_owned < 0 || n_total < n_owned || !x || !y || !z) return DSMD_ERR_INVALID;
    if (n_total > c->capacity) return fail(c, DSMD_ERR_CAPACITY, "more atoms than the context's capacity");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    DSMD_CUDA(c, cudaSetDevice(c->device));
    const double* src[kNumReal] = {x, y, z, vx, vy, vz, nullptr, nullptr, nullptr, mass, charge};
    for (int f = 0; f < kNumReal; ++f) {
        double* dst = c->real[c->cur][f];
        if (src[f]) {
            DSMD_CUDA(c, cudaMemcpyAsync(dst, src[f], sizeof(double) * n_total, cudaMemcpyHostToDevice, s));
        } else if (f == DSMD_MASS) {
            std::vector<double> ones(n_total, 1.0);
            DSMD_CUDA(c, cudaMemcpyAsync(dst, ones.data(), sizeof(double) * n_total, cudaMemcpyHostToDevice, s));
            DSMD_CUDA(c, cudaStreamSynchronize(s));
        } else {
            DSMD_CUDA(c, cudaMemsetAsync(dst, 0, sizeof(double) * n_total, s));
        }
    }
    if (type) {
        DSMD_CUDA(c, cudaMemcpyAsync(c->type[c->cur], type, sizeof(int) * n_total, cudaMemcpyHostToDevice, s));
    } else {
        DSMD_CUDA(c, cudaMemsetAsync(c->type[c->cur], 0, sizeof(int) * n_total, s));
    }
    if (gid) {
        DSMD_CUDA(c, cudaMemcpyAsync(c->gid[c->cur], gid, sizeof(int) * n_total, cudaMemcpyHostToDevice, s));
    } else {
        std::vector<int> iota(n_total);
        for (int64_t k = 0; k < n_total; ++k) iota[k] = static_cast<int>(k);
        DSMD_CUDA(c, cudaMemcpyAsync(c->gid[c->cur], iota.data(), sizeof(int) * n_total, cudaMemcpyHostToDevice, s));
        DSMD_CUDA(c, cudaStreamSynchronize(s));
    }
    c->n_owned = n_owned;
    c->n_total = n_total;
    c->list_valid = false;
    c->slot_map_valid = false;
    return DSMD_OK;
}

int dsmd_upload_positions(dsmd_ctx* c, const double* x, const double* y, const double* z, void* stream) {
    if (!c || !x || !y || !z) return DSMD_ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const double* src[3] = {x, y, z};
    for (int a = 0; a < 3; ++a)
        DSMD_CUDA(c, cudaMemcpyAsync(c->real[c->cur][a], src[a], sizeof(double) * c->n_total, cudaMemcpyHostToDevice, s));
    return DSMD_OK;
}

int dsmd_download(dsmd_ctx* c, int field, int64_t n, void* host_out, void* stream) {
    if (!c || field < 0 || field >= DSMD_FIELD_COUNT || n < 0 || n > c->capacity || !host_out) return DSMD_ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const void* src = field < kNumReal ? static_cast<const void*>(c->real[c->cur][field])
                                       : (field == DSMD_TYPE ? static_cast<const void*>(c->type[c->cur])
                                                             : static_cast<const void*>(c->gid[c->cur]));
    const size_t bytes = (field < kNumReal ? sizeof(double) : sizeof(int)) * static_cast<size_t>(n);
    DSMD_CUDA(c, cudaMemcpyAsync(host_out, src, bytes, cudaMemcpyDeviceToHost, s));
    DSMD_CUDA(c, cudaStreamSynchronize(s));
    return DSMD_OK;
}

int dsmd_device_pointer(dsmd_ctx* c, int field, void** out) {
    if (!c || field < 0 || field >= DSMD_FIELD_COUNT || !out) return DSMD_ERR_INVALID;
    *out = field < kNumReal ? static_cast<void*>(c->real[c->cur][field])
                            : (field == DSMD_TYPE ? static_cast<void*>(c->type[c->cur])
                                                  : static_cast<void*>(c->gid[c->cur]));
    return DSMD_OK;
}

int dsmd_counts(const dsmd_ctx* c, int64_t* n_owned, int64_t* n_total) {
    if (!c) return DSMD_ERR_INVALID;
    if (n_owned) *n_owned = c->n_owned;
    if (n_total) *n_total = c->n_total;
    return DSMD_OK;
}

int dsmd_set_counts(dsmd_ctx* c, int64_t n_owned, int64_t n_total) {
    if (!c || n_owned < 0 || n_total < n_owned) return DSMD_ERR_INVALID;
    if (n_total > c->capacity) return fail(c, DSMD_ERR_CAPACITY, "more atoms than the context's capacity");
    c->n_owned = n_owned;
    c->n_total = n_total;
    c->list_valid = false;
    return DSMD_OK;
}

static int sort_owned_impl(dsmd_ctx* c, const Brick* bounds, int64_t n_outside, bool check_now, cudaStream_t s) {
    DSMD_CUDA(c, cudaSetDevice(c->device));
    if (n_outside < 0 || n_outside >= c->n_owned) return fail(c, DSMD_ERR_INVALID, "sort: bad count of atoms to remove");
    if (!c->grid_valid) { const int rc = make_grid(c); if (rc) return rc; }
    { const int rc = ensure_cells(c); if (rc) return rc; }
    DSMD_CUDA(c, cudaMemsetAsync(c->status, 0, sizeof(Status), s));
    const int64_t keep_total = c->n_total;
    c->n_total = c->n_owned;   // sort the owned segment alone
    const int rc = sort_range(c, 0, s, n_outside, bounds);
    c->n_total = keep_total;
    if (rc) return rc;
    c->n_owned -= n_outside;
    c->n_total = c->n_owned;   // ghosts (if any were present) are dropped: the caller appends the new ones
    c->list_valid = false;
    c->owned_sorted_only = true;
    c->expect_dropped = n_outside;
    if (!check_now) return DSMD_OK;   // the status words stay and are read with the list build's
    { const int rc2 = read_status(c, s); if (rc2) return rc2; }
    if (c->h_status->out_of_domain)
        return fail(c, DSMD_ERR_OUT_OF_DOMAIN, "an atom lies outside the subdomain + halo, or has a NaN position");
    if (c->h_status->dropped != static_cast<unsigned>(n_outside))
        return fail(c, DSMD_ERR_STATE, "sort: the number of atoms outside the brick differs from the caller's count");
    return DSMD_OK;
}

int dsmd_sort_owned(dsmd_ctx* c, void* stream) {
    if (!c) return DSMD_ERR_INVALID;
    return sort_owned_impl(c, nullptr, 0, true, static_cast<cudaStream_t>(stream));
}

int dsmd_sort_owned_in_brick(dsmd_ctx* c, const double lo[3], const double hi[3], const int split[3], int64_t n_outside,
                             void* stream) {
    if (!c || !lo || !hi || !split) return DSMD_ERR_INVALID;
    Brick bounds{};
    for (int a = 0; a < 3; ++a) {
        bounds.lo[a] = lo[a];
        bounds.hi[a] = hi[a];
        bounds.split[a] = split[a] != 0;
    }
    return sort_owned_impl(c, &bounds, n_outside, false, static_cast<cudaStream_t>(stream));
}

int dsmd_build_neighbor_list(dsmd_ctx* c, void* stream) {
    if (!c) return DSMD_ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    DSMD_CUDA(c, cudaSetDevice(c->device));
    if (c->n_owned <= 0) return fail(c, DSMD_ERR_STATE, "no atoms uploaded");
    if (!c->grid_valid) { const int rc = make_grid(c); if (rc) return rc; }
    { const int rc = ensure_cells(c); if (rc) return rc; }
    // 1. bin + sort + reorder (everything, or only the ghosts when the owned segment was sorted just before: the
    //    status words of that sort are then still unread and are kept)
    const int64_t first = c->owned_sorted_only ? c->n_owned : 0;
    const int64_t expect_dropped = c->owned_sorted_only ? c->expect_dropped : 0;
    if (!c->owned_sorted_only) DSMD_CUDA(c, cudaMemsetAsync(c->status, 0, sizeof(Status), s));
    c->owned_sorted_only = false;
    c->expect_dropped = 0;
    if (first == 0 || c->n_total > first) { const int rc = sort_range(c, first, s); if (rc) return rc; }
    // 2. list rows
    if (c->stride == 0) {
        double volume = 1.0;
        for (int a = 0; a < 3; ++a) volume *= 1.0 / c->grid.inv_len[a];
        const double R = c->cutoff + c->skin;
        const double expect = static_cast<double>(c->n_total) / volume * 4.18879020479 * R * R * R;
        c->stride = std::max(32, static_cast<int>(expect * 1.3) + 24);
        c->stride = (c->stride + 3) & ~3;
    }
    const int64_t rows = static_cast<int64_t>(c->grid.nc[1]) * c->grid.nc[2];
    if (4 * rows > c->ghost_rows_capacity) {
        if (c->ghost_rows) cudaFree(c->ghost_rows);
        c->ghost_rows = nullptr;
        DSMD_CUDA(c, cudaMalloc(&c->ghost_rows, sizeof(int) * 4 * rows));
        c->ghost_rows_capacity = 4 * rows;
    }
    {   // slab boundaries for the pipelined host-buffer call; they arrive with the status read-back below
        const int layers = c->grid.nc[2];
        if (layers + 1 > c->layer_capacity) {
            cudaFree(c->d_layer_start);
            if (c->h_layer_start) cudaFreeHost(c->h_layer_start);
            c->d_layer_start = c->h_layer_start = nullptr;
            DSMD_CUDA(c, cudaMalloc(&c->d_layer_start, sizeof(int) * (layers + 1)));
            DSMD_CUDA(c, cudaMallocHost(&c->h_layer_start, sizeof(int) * (layers + 1)));
            c->layer_capacity = layers + 1;
        }
        k_layer_starts<<<blocks_for(layers + 1, kThreads), kThreads, 0, s>>>(c->cell_start, c->grid.nc[0] * c->grid.nc[1], layers,
                                                                           c->d_layer_start);
        DSMD_LAUNCHED(c);
        DSMD_CUDA(c, cudaMemcpyAsync(c->h_layer_start, c->d_layer_start, sizeof(int) * (layers + 1), cudaMemcpyDeviceToHost, s));
    }
    if (c->n_total > c->n_owned) {
        k_ghost_row_extent<<<blocks_for(rows * 32, kThreads), kThreads, 0, s>>>(c->grid, c->cell_start + c->grid.ncells,
                                                                               c->ghost_rows, c->ghost_rows + rows);
        DSMD_LAUNCHED(c);
        k_ghost_rows_near<<<blocks_for(rows, kThreads), kThreads, 0, s>>>(c->grid, c->ghost_rows, c->ghost_rows + rows,
                                                                         c->ghost_rows + 2 * rows, c->ghost_rows + 3 * rows);
        DSMD_LAUNCHED(c);
    }
    for (int attempt = 0; attempt < 4; ++attempt) {
        { const int rc = ensure_list(c, c->stride); if (rc) return rc; }
        ExclusionTable ex{c->excl_off, c->excl_partner, static_cast<int>(c->excl_n_global)};
        if (ex.offsets)
            k_build_list<true><<<blocks_for(c->n_owned, kBuildThreads), kBuildThreads, 0, s>>>(
                c->grid, static_cast<int>(c->n_owned), static_cast<int>(c->n_total), c->pq, c->pf, c->real[c->cur][0],
                c->real[c->cur][1], c->real[c->cur][2], c->gid[c->cur], ex, c->cell_start, c->ghost_rows + 2 * rows,
                c->ghost_rows + 3 * rows, c->nbr, c->stride, c->deg, c->deg_int, c->boundary_list, c->status);
        else
            k_build_list<false><<<blocks_for(c->n_owned, kBuildThreads), kBuildThreads, 0, s>>>(
                c->grid, static_cast<int>(c->n_owned), static_cast<int>(c->n_total), c->pq, c->pf, c->real[c->cur][0],
                c->real[c->cur][1], c->real[c->cur][2], c->gid[c->cur], ex, c->cell_start, c->ghost_rows + 2 * rows,
                c->ghost_rows + 3 * rows, c->nbr, c->stride, c->deg, c->deg_int, c->boundary_list, c->status);
        DSMD_LAUNCHED(c);
        { const int rc = read_status(c, s); if (rc) return rc; }
        if (c->h_status->out_of_domain)
            return fail(c, DSMD_ERR_OUT_OF_DOMAIN, "an atom lies outside the subdomain + halo, or has a NaN position");
        if (attempt == 0 && c->h_status->dropped != static_cast<unsigned>(expect_dropped))
            return fail(c, DSMD_ERR_STATE, "sort: the number of atoms outside the brick differs from the caller's count");
        if (c->h_status->need_stride <= static_cast<unsigned>(c->stride)) break;
        // a row overflowed: grow and build again
        c->stride = (static_cast<int>(c->h_status->need_stride * 1.1) + 8 + 3) & ~3;
        DSMD_CUDA(c, cudaMemsetAsync(c->status, 0, sizeof(Status), s));
        if (attempt == 3) return fail(c, DSMD_ERR_CAPACITY, "neighbour rows kept overflowing");
    }
    c->stat_entries = static_cast<int64_t>(c->h_status->entries);
    c->stat_interior = static_cast<int64_t>(c->h_status->interior);
    c->stat_rechecked = static_cast<int>(c->h_status->rechecked);
    c->n_boundary = static_cast<int64_t>(c->h_status->boundary_atoms);
    ++c->build_epoch;
    DSMD_CUDA(c, cudaMemsetAsync(c->status, 0, sizeof(Status), s));   // displacement word restarts at zero
    c->list_valid = true;
    return DSMD_OK;
}

int dsmd_ghost_slots(dsmd_ctx* c, const int32_t** out) {
    if (!c || !out) return DSMD_ERR_INVALID;
    *out = c->ghost_slot;
    return DSMD_OK;
}

int dsmd_list_stats(dsmd_ctx* c, int64_t* directed_entries, int64_t* interior_entries, int32_t* row_stride,
                    int32_t* cells, int32_t* rechecked) {
    if (!c) return DSMD_ERR_INVALID;
    if (!c->list_valid) return fail(c, DSMD_ERR_STATE, "no neighbour list");
    if (directed_entries) *directed_entries = c->stat_entries;
    if (interior_entries) *interior_entries = c->stat_interior;
    if (row_stride) *row_stride = c->stride;
    if (cells) *cells = c->grid.ncells;
    if (rechecked) *rechecked = c->stat_rechecked;
    return DSMD_OK;
}

int dsmd_list_export(dsmd_ctx* c, int32_t* d_i, int32_t* d_j, uint8_t* d_flags, int64_t capacity, int64_t* n_pairs,
                     void* stream) {
    if (!c || !n_pairs) return DSMD_ERR_INVALID;
    if (!c->list_valid) return fail(c, DSMD_ERR_STATE, "no neighbour list");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int n = static_cast<int>(c->n_owned);
    *n_pairs = c->stat_entries;
    if (!d_i || !d_j || capacity < c->stat_entries) return DSMD_OK;   // size query
    unsigned long long* scratch = nullptr;
    DSMD_CUDA(c, cudaMalloc(&scratch, sizeof(unsigned long long) * n));
    k_deg_to_u64<<<blocks_for(n, kThreads), kThreads, 0, s>>>(n, c->deg, scratch);
    DSMD_LAUNCHED(c);
    size_t need = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, need, scratch, c->offsets64, n, s);
    void* temp = nullptr;
    DSMD_CUDA(c, cudaMalloc(&temp, need));
    DSMD_CUDA(c, cub::DeviceScan::ExclusiveSum(temp, need, scratch, c->offsets64, n, s));
    k_list_export<<<blocks_for(n, kThreads), kThreads, 0, s>>>(n, c->nbr, c->stride, c->deg, c->offsets64, d_i, d_j,
                                                              d_flags, capacity);
    DSMD_LAUNCHED(c);
    DSMD_CUDA(c, cudaStreamSynchronize(s));
    cudaFree(temp);
    cudaFree(scratch);
    return DSMD_OK;
}

// kick: 0.5 for the first velocity-Verlet half, 1.0 for the merged second-and-first half.
static int pack_impl(dsmd_ctx* c, int64_t first, int64_t count, bool integrate, double dt, double f2a, cudaStream_t s,
                     double kick = 0.5) {
    if (count <= 0) return DSMD_OK;
    double** r = c->real[c->cur];
    if (integrate)
        k_pack<true><<<blocks_for(count, kThreads), kThreads, 0, s>>>(
            c->grid, static_cast<int>(first), static_cast<int>(count), static_cast<int>(c->n_owned), r[0], r[1], r[2],
            r[3], r[4], r[5], r[6], r[7], r[8], r[9], c->type[c->cur], c->ref[0], c->ref[1], c->ref[2], c->pq, dt,
            kick * dt * f2a, c->status);
    else
        k_pack<false><<<blocks_for(count, kThreads), kThreads, 0, s>>>(
            c->grid, static_cast<int>(first), static_cast<int>(count), static_cast<int>(c->n_owned), r[0], r[1], r[2],
            r[3], r[4], r[5], r[6], r[7], r[8], r[9], c->type[c->cur], c->ref[0], c->ref[1], c->ref[2], c->pq, 0.0, 0.0,
            c->status);
    DSMD_LAUNCHED(c);
    return DSMD_OK;
}

int dsmd_pack_positions(dsmd_ctx* c, int64_t first, int64_t count, void* stream) {
    if (!c || first < 0 || count < 0 || first + count > c->n_total) return DSMD_ERR_INVALID;
    if (!c->grid_valid) return fail(c, DSMD_ERR_STATE, "no neighbour list built yet");
    return pack_impl(c, first, count, false, 0.0, 0.0, static_cast<cudaStream_t>(stream));
}

int dsmd_max_displacement_sq(dsmd_ctx* c, double* out, void* stream) {
    if (!c || !out) return DSMD_ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    { const int rc = read_status(c, s); if (rc) return rc; }
    double v;
    const unsigned long long bits = c->h_status->max_disp2;
    std::memcpy(&v, &bits, sizeof(v));
    *out = v;
    if (c->h_status->out_of_domain)
        return fail(c, DSMD_ERR_OUT_OF_DOMAIN, "an atom left the subdomain + halo, or has a NaN position");
    return DSMD_OK;
}

int dsmd_max_displacement_sq_lagged(dsmd_ctx* c, double* out, void* stream) {
    if (!c || !out) return DSMD_ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    *out = -1.0;
    if (c->disp_pending >= 0) {
        const int slot = c->disp_pending;
        DSMD_CUDA(c, cudaEventSynchronize(c->disp_event[slot]));   // queued one call ago: long finished
        if (c->disp_epoch[slot] == c->build_epoch) {   // else it was measured against reference positions that are gone
            double v;
            const unsigned long long bits = *c->h_disp[slot];
            std::memcpy(&v, &bits, sizeof(v));
            *out = v;
        }
    }
    const int next = c->disp_pending == 0 ? 1 : 0;
    DSMD_CUDA(c, cudaMemcpyAsync(c->h_disp[next], &c->status->max_disp2, sizeof(unsigned long long), cudaMemcpyDeviceToHost, s));
    DSMD_CUDA(c, cudaEventRecord(c->disp_event[next], s));
    c->disp_epoch[next] = c->build_epoch;
    c->disp_pending = next;
    return DSMD_OK;
}

// The pair kernel over the owned atoms first .. first + count of a FULL or INTERIOR pass without energy (count < 0: all
// of them, any phase), or over the atoms with a ghost partner (BOUNDARY).
static int compute_forces_impl(dsmd_ctx* c, int phase, int want_energy, int64_t first, int64_t count, void* stream) {
    if (!c || phase < DSMD_PHASE_FULL || phase > DSMD_PHASE_BOUNDARY) return DSMD_ERR_INVALID;
    if (!c->list_valid) return fail(c, DSMD_ERR_STATE, "build the neighbour list before computing forces");
    const bool ranged = count >= 0;
    if (ranged && (phase == DSMD_PHASE_BOUNDARY || want_energy || first < 0 || first + count > c->n_owned))
        return fail(c, DSMD_ERR_INVALID, "a range of atoms is for FULL or INTERIOR passes without energy, inside the owned atoms");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    PairParams p{};
    for (int a = 0; a < 3; ++a) p.scale[a] = c->grid.scale[a];
    p.rc2 = static_cast<float>(c->cutoff * c->cutoff);
    const bool sw = c->switch_distance > 0.0;
    if (sw) {
        const double rs2 = c->switch_distance * c->switch_distance, d = c->cutoff * c->cutoff - rs2;
        p.rs2 = static_cast<float>(rs2);
        p.inv_denom = static_cast<float>(1.0 / (d * d * d));
    } else {
        p.rs2 = -1.f;
    }
    p.kq = static_cast<float>(kCoulomb);
    p.alpha = static_cast<float>(c->alpha);
    p.two_alpha_sqrtpi = static_cast<float>(2.0 * c->alpha / std::sqrt(3.14159265358979323846));
    p.ntypes = c->ntypes;
    p.ewald_intervals = c->ewald_intervals;
    p.c6c12 = c->c6c12;
    p.ewald = c->ewald;
    p.type_charge = c->coulomb ? c->type_charge : nullptr;
    const bool multi = c->ntypes > 1;
    // the boundary pass runs over the atoms the list build found a ghost partner for (none: nothing to launch)
    const int64_t pair_threads = phase == DSMD_PHASE_BOUNDARY ? c->n_boundary : (ranged ? count : c->n_owned);
    const int f0 = static_cast<int>(ranged ? first : 0), nt = static_cast<int>(pair_threads);
    const int64_t blocks = blocks_for(pair_threads, kPairThreads);
    if (want_energy) { const int rc = ensure_partials(c, std::max<int64_t>(blocks, 1)); if (rc) return rc; }
    const bool e = want_energy != 0;
    if (pair_threads == 0) {
        // nothing to add to the forces; the energy sums of a boundary pass stay as the interior pass left them
    } else if (c->coulomb) {
        if (e) { if (multi) launch_pair<true, true, true>(c, p, phase, sw, s, f0, nt); else launch_pair<true, true, false>(c, p, phase, sw, s, f0, nt); }
        else   { if (multi) launch_pair<true, false, true>(c, p, phase, sw, s, f0, nt); else launch_pair<true, false, false>(c, p, phase, sw, s, f0, nt); }
    } else {
        if (e) { if (multi) launch_pair<false, true, true>(c, p, phase, sw, s, f0, nt); else launch_pair<false, true, false>(c, p, phase, sw, s, f0, nt); }
        else   { if (multi) launch_pair<false, false, true>(c, p, phase, sw, s, f0, nt); else launch_pair<false, false, false>(c, p, phase, sw, s, f0, nt); }
    }
    if (pair_threads > 0) DSMD_LAUNCHED(c);
    if (e && (pair_threads > 0 || phase != DSMD_PHASE_BOUNDARY)) {
        k_reduce_partials<6><<<1, kThreads, 0, s>>>(c->partials, static_cast<int>(blocks), c->scalars,
                                                   phase == DSMD_PHASE_BOUNDARY ? 1 : 0);
        DSMD_LAUNCHED(c);
    }
    return DSMD_OK;
}

int dsmd_compute_forces(dsmd_ctx* c, int phase, int want_energy, void* stream) {
    return compute_forces_impl(c, phase, want_energy, 0, -1, stream);
}

int dsmd_read_scalars(dsmd_ctx* c, double out[6], void* stream) {
    if (!c || !out) return DSMD_ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    DSMD_CUDA(c, cudaMemcpyAsync(c->h_scalars, c->scalars, sizeof(double) * 6, cudaMemcpyDeviceToHost, s));
    DSMD_CUDA(c, cudaStreamSynchronize(s));
    for (int k = 0; k < 6; ++k) out[k] = c->h_scalars[k];
    return DSMD_OK;
}

namespace {

ClusterTable cluster_table(const dsmd_ctx* c) {
    ClusterTable t{};
    t.n_clusters = c->n_clusters;
    t.atom_gid = c->cl_gid;
    t.con_a = c->cl_a;
    t.con_b = c->cl_b;
    t.con_d2 = c->cl_d2;
    t.slot_of_gid = c->slot_of_gid;
    for (int a = 0; a < 3; ++a) {
        t.box[a] = c->box[a];
        t.periodic[a] = c->periodic[a];
    }
    return t;
}

int ensure_slot_map(dsmd_ctx* c, cudaStream_t s) {
    if (c->slot_map_valid) return DSMD_OK;
    k_slot_of_gid<<<blocks_for(c->n_owned, kThreads), kThreads, 0, s>>>(static_cast<int>(c->n_owned), c->gid[c->cur],
                                                                         static_cast<int>(c->cons_n_global), c->slot_of_gid);
    DSMD_LAUNCHED(c);
    c->slot_map_valid = true;
    return DSMD_OK;
}

// SHAKE after the drift of the first half step (positions before it are in c->pre), then the positions the kernels
// read are converted again.
int shake_impl(dsmd_ctx* c, double dt, cudaStream_t s) {
    { const int rc = ensure_slot_map(c, s); if (rc) return rc; }
    double** r = c->real[c->cur];
    k_shake<<<blocks_for(c->n_clusters, 128), 128, 0, s>>>(cluster_table(c), r[0], r[1], r[2], r[3], r[4], r[5], c->pre[0],
                                                            c->pre[1], c->pre[2], r[9], 1.0 / dt, c->cons_tolerance,
                                                            c->cons_max_iterations, &c->status->constraint_failed);
    DSMD_LAUNCHED(c);
    return DSMD_OK;
}

int rattle_impl(dsmd_ctx* c, double dt, double f2a, double* d_virial3, cudaStream_t s) {
    { const int rc = ensure_slot_map(c, s); if (rc) return rc; }
    double** r = c->real[c->cur];
    const unsigned blocks = blocks_for(c->n_clusters, 128);
    double* partials = nullptr;
    if (d_virial3) {
        { const int rc = ensure_partials(c, blocks); if (rc) return rc; }
        partials = c->partials;
    }
    k_rattle<<<blocks, 128, 0, s>>>(cluster_table(c), r[0], r[1], r[2], r[3], r[4], r[5], r[9], c->cons_tolerance,
                                    c->cons_max_iterations, -2.0 / (f2a * dt), partials, &c->status->constraint_failed);
    DSMD_LAUNCHED(c);
    if (d_virial3) {
        k_reduce_partials<3><<<1, kThreads, 0, s>>>(partials, static_cast<int>(blocks), d_virial3, 0);
        DSMD_LAUNCHED(c);
    }
    return DSMD_OK;
}

}  // namespace

int dsmd_set_constraints(dsmd_ctx* c, int64_t n_global, int64_t n_constraints, const int32_t* a, const int32_t* b,
                         const double* distance, double tolerance, int max_iterations) {
    if (!c || n_global < 0 || n_constraints < 0 || (n_constraints > 0 && (!a || !b || !distance))) return DSMD_ERR_INVALID;
    DSMD_CUDA(c, cudaSetDevice(c->device));
    cudaFree(c->cl_gid); cudaFree(c->cl_a); cudaFree(c->cl_b); cudaFree(c->cl_d2); cudaFree(c->slot_of_gid);
    c->cl_gid = c->slot_of_gid = nullptr;
    c->cl_a = c->cl_b = nullptr;
    c->cl_d2 = nullptr;
    c->n_clusters = 0;
    c->slot_map_valid = false;
    if (tolerance > 0.0) c->cons_tolerance = tolerance;
    if (max_iterations > 0) c->cons_max_iterations = max_iterations;
    if (n_constraints == 0) return DSMD_OK;
    // clusters = connected groups of constraints (union-find over the atoms), in the order of their first constraint;
    // inside a cluster the constraints keep their given order
    std::vector<int> parent(static_cast<size_t>(n_global));
    for (int64_t g = 0; g < n_global; ++g) parent[g] = static_cast<int>(g);
    auto find = [&](int v) {
        while (parent[v] != v) v = parent[v] = parent[parent[v]];
        return v;
    };
    for (int64_t k = 0; k < n_constraints; ++k) {
        if (a[k] < 0 || b[k] < 0 || a[k] >= n_global || b[k] >= n_global || a[k] == b[k] || !(distance[k] > 0.0))
            return fail(c, DSMD_ERR_INVALID, "constraint names an atom outside the system, or its distance is not positive");
        parent[find(a[k])] = find(b[k]);
    }
    std::vector<int> cluster_of(static_cast<size_t>(n_global), -1);
    std::vector<int> gids;
    std::vector<unsigned char> ca, cb;
    std::vector<double> d2;
    std::vector<int> n_atoms, n_cons;
    for (int64_t k = 0; k < n_constraints; ++k) {
        const int root = find(a[k]);
        int cl = cluster_of[root];
        if (cl < 0) {
            cl = cluster_of[root] = static_cast<int>(n_atoms.size());
            n_atoms.push_back(0);
            n_cons.push_back(0);
            gids.resize(gids.size() + kClusterAtoms, -1);
            ca.resize(ca.size() + kClusterCons, 255);
            cb.resize(cb.size() + kClusterCons, 255);
            d2.resize(d2.size() + kClusterCons, 1.0);
        }
        int local[2];
        const int ends[2] = {a[k], b[k]};
        for (int e = 0; e < 2; ++e) {
            local[e] = -1;
            for (int q = 0; q < n_atoms[cl]; ++q)
                if (gids[static_cast<size_t>(cl) * kClusterAtoms + q] == ends[e]) local[e] = q;
            if (local[e] < 0) {
                if (n_atoms[cl] == kClusterAtoms)
                    return fail(c, DSMD_ERR_CAPACITY, "a group of connected constraints has more than 4 atoms");
                local[e] = n_atoms[cl]++;
                gids[static_cast<size_t>(cl) * kClusterAtoms + local[e]] = ends[e];
            }
        }
        if (n_cons[cl] == kClusterCons) return fail(c, DSMD_ERR_CAPACITY, "a group of connected constraints has more than 6 constraints");
        const size_t at = static_cast<size_t>(cl) * kClusterCons + n_cons[cl]++;
        ca[at] = static_cast<unsigned char>(local[0]);
        cb[at] = static_cast<unsigned char>(local[1]);
        d2[at] = distance[k] * distance[k];
    }
    const size_t ncl = n_atoms.size();
    DSMD_CUDA(c, cudaMalloc(&c->cl_gid, sizeof(int) * gids.size()));
    DSMD_CUDA(c, cudaMalloc(&c->cl_a, ca.size()));
    DSMD_CUDA(c, cudaMalloc(&c->cl_b, cb.size()));
    DSMD_CUDA(c, cudaMalloc(&c->cl_d2, sizeof(double) * d2.size()));
    DSMD_CUDA(c, cudaMalloc(&c->slot_of_gid, sizeof(int) * static_cast<size_t>(n_global)));
    DSMD_CUDA(c, cudaMemcpy(c->cl_gid, gids.data(), sizeof(int) * gids.size(), cudaMemcpyHostToDevice));
    DSMD_CUDA(c, cudaMemcpy(c->cl_a, ca.data(), ca.size(), cudaMemcpyHostToDevice));
    DSMD_CUDA(c, cudaMemcpy(c->cl_b, cb.data(), cb.size(), cudaMemcpyHostToDevice));
    DSMD_CUDA(c, cudaMemcpy(c->cl_d2, d2.data(), sizeof(double) * d2.size(), cudaMemcpyHostToDevice));
    for (int ax = 0; ax < 3; ++ax)
        if (!c->pre[ax]) DSMD_CUDA(c, cudaMalloc(&c->pre[ax], sizeof(double) * c->capacity));
    c->n_clusters = static_cast<int>(ncl);
    c->cons_n_global = n_global;
    return DSMD_OK;
}

int dsmd_constraint_failures(dsmd_ctx* c, int64_t* failed, void* stream) {
    if (!c || !failed) return DSMD_ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    { const int rc = read_status(c, s); if (rc) return rc; }
    *failed = c->h_status->constraint_failed;
    return DSMD_OK;
}

int dsmd_rattle(dsmd_ctx* c, double dt, double f2a, double* d_virial_diag, void* stream) {
    if (!c || !(dt > 0.0)) return DSMD_ERR_INVALID;
    if (c->n_clusters == 0) return DSMD_OK;
    if (c->n_total != c->n_owned) return fail(c, DSMD_ERR_STATE, "constraints are solved on single-rank systems only");
    return rattle_impl(c, dt, f2a, d_virial_diag, static_cast<cudaStream_t>(stream));
}

int dsmd_integrate(dsmd_ctx* c, int half, double dt, double f2a, void* stream) {
    if (!c || half < 1 || half > 3) return DSMD_ERR_INVALID;
    if (!c->grid_valid) return fail(c, DSMD_ERR_STATE, "no neighbour list built yet");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool constrained = c->n_clusters > 0;
    if (constrained && c->n_total != c->n_owned)
        return fail(c, DSMD_ERR_STATE, "constraints are solved on single-rank systems only");
    if (half == 3) {
        if (constrained) return fail(c, DSMD_ERR_STATE, "the merged half steps are not available with constraints");
        return pack_impl(c, 0, c->n_owned, true, dt, f2a, s, 1.0);
    }
    if (half == 1) {
        if (!constrained) return pack_impl(c, 0, c->n_owned, true, dt, f2a, s);
        // constrained: keep the positions from before the drift, drift, SHAKE, then convert the corrected positions
        for (int a = 0; a < 3; ++a)
            DSMD_CUDA(c, cudaMemcpyAsync(c->pre[a], c->real[c->cur][a], sizeof(double) * c->n_owned, cudaMemcpyDeviceToDevice, s));
        { const int rc = pack_impl(c, 0, c->n_owned, true, dt, f2a, s); if (rc) return rc; }
        { const int rc = shake_impl(c, dt, s); if (rc) return rc; }
        return pack_impl(c, 0, c->n_owned, false, 0.0, 0.0, s);
    }
    double** r = c->real[c->cur];
    k_vv2<<<blocks_for(c->n_owned, kThreads), kThreads, 0, s>>>(static_cast<int>(c->n_owned), 0.5 * dt * f2a, r[3], r[4],
                                                               r[5], r[6], r[7], r[8], r[9]);
    DSMD_LAUNCHED(c);
    if (constrained) return rattle_impl(c, dt, f2a, nullptr, s);
    return DSMD_OK;
}

// ---- bonded terms ------------------------------------------------------------------------------------------------------


static int to_device_bytes(dsmd_ctx* c, void** dst, const void* src, size_t bytes) {
    *dst = nullptr;
    if (bytes == 0) return DSMD_OK;
    DSMD_CUDA(c, cudaMalloc(dst, bytes));
    DSMD_CUDA(c, cudaMemcpy(*dst, src, bytes, cudaMemcpyHostToDevice));
    return DSMD_OK;
}
#define DSMD_TO_DEVICE(c, dst, vec)                                                                                    \
    do {                                                                                                               \
        const int rc_ = to_device_bytes(c, reinterpret_cast<void**>(&(dst)), (vec).data(), sizeof((vec)[0]) * (vec).size()); \
        if (rc_) return rc_;                                                                                           \
    } while (0)

int dsmd_set_type_charges(dsmd_ctx* c, int ntypes, const double* charge_of_type) {
    if (!c) return DSMD_ERR_INVALID;
    DSMD_CUDA(c, cudaSetDevice(c->device));
    cudaFree(c->type_charge);
    c->type_charge = nullptr;
    if (!charge_of_type || ntypes <= 0) return DSMD_OK;
    if (!c->params_set || ntypes != c->ntypes)
        return fail(c, DSMD_ERR_INVALID, "dsmd_set_type_charges: the number of types differs from dsmd_set_pair_params'");
    // the atoms already on the device must agree with the table (those that arrive later are the caller's word)
    if (c->n_total > 0) {
        std::vector<double> q(static_cast<size_t>(c->n_total));
        std::vector<int> t(static_cast<size_t>(c->n_total));
        DSMD_CUDA(c, cudaMemcpy(q.data(), c->real[c->cur][10], sizeof(double) * q.size(), cudaMemcpyDeviceToHost));
        DSMD_CUDA(c, cudaMemcpy(t.data(), c->type[c->cur], sizeof(int) * t.size(), cudaMemcpyDeviceToHost));
        for (size_t k = 0; k < q.size(); ++k)
            if (t[k] < 0 || t[k] >= ntypes || q[k] != charge_of_type[t[k]])
                return fail(c, DSMD_ERR_INVALID, "dsmd_set_type_charges: an atom's charge is not the charge given for its type");
    }
    std::vector<float> table(static_cast<size_t>(ntypes));
    for (int k = 0; k < ntypes; ++k) table[static_cast<size_t>(k)] = static_cast<float>(charge_of_type[k]);
    DSMD_CUDA(c, cudaMalloc(&c->type_charge, sizeof(float) * table.size()));
    DSMD_CUDA(c, cudaMemcpy(c->type_charge, table.data(), sizeof(float) * table.size(), cudaMemcpyHostToDevice));
    return DSMD_OK;
}

int dsmd_set_bonded(dsmd_ctx* c, int64_t n_global, int64_t n_bonds, const int32_t* bond_atoms, const double* bond_k,
                    const double* bond_r0, int64_t n_angles, const int32_t* angle_atoms, const double* angle_k,
                    const double* angle_theta0, int64_t n_torsions, const int32_t* torsion_atoms, const double* torsion_k,
                    const double* torsion_phi0, const int32_t* torsion_n, int64_t n_specials, const int32_t* special_atoms,
                    const double* special_sigma, const double* special_epsilon, const double* special_lj_scale,
                    const double* special_coulomb_scale) {
    if (!c || n_global < 0 || n_bonds < 0 || n_angles < 0 || n_torsions < 0 || n_specials < 0) return DSMD_ERR_INVALID;
    if ((n_bonds > 0 && (!bond_atoms || !bond_k || !bond_r0)) || (n_angles > 0 && (!angle_atoms || !angle_k || !angle_theta0)) ||
        (n_torsions > 0 && (!torsion_atoms || !torsion_k || !torsion_phi0 || !torsion_n)) ||
        (n_specials > 0 && (!special_atoms || !special_sigma || !special_epsilon || !special_lj_scale || !special_coulomb_scale)))
        return DSMD_ERR_INVALID;
    DSMD_CUDA(c, cudaSetDevice(c->device));
    free_bonded(c);
    const int64_t terms = n_bonds + n_angles + n_torsions + n_specials;
    if (terms == 0) return DSMD_OK;
    if (n_global >= (1ll << 31) || terms >= (1ll << 29)) return fail(c, DSMD_ERR_INVALID, "too many atoms or bonded terms");
    // term tables, and for every global id the places (3-double groups of the scratch array) its forces are written to,
    // in the order bonds, angles, torsions, specials and, inside a kind, term by term: the order the forces are added in
    std::vector<int> ba(bond_atoms, bond_atoms + 2 * n_bonds), aa(angle_atoms, angle_atoms + 3 * n_angles),
        ta(torsion_atoms, torsion_atoms + 4 * n_torsions), tn(torsion_n, torsion_n + n_torsions),
        sa(special_atoms, special_atoms + 2 * n_specials);
    std::vector<double> bp(2 * n_bonds), ap(2 * n_angles), tp(2 * n_torsions), sp(4 * n_specials);
    for (int64_t k = 0; k < n_bonds; ++k) { bp[2 * k] = bond_k[k]; bp[2 * k + 1] = bond_r0[k]; }
    for (int64_t k = 0; k < n_angles; ++k) { ap[2 * k] = angle_k[k]; ap[2 * k + 1] = angle_theta0[k]; }
    for (int64_t k = 0; k < n_torsions; ++k) { tp[2 * k] = torsion_k[k]; tp[2 * k + 1] = torsion_phi0[k]; }
    for (int64_t k = 0; k < n_specials; ++k) {
        sp[4 * k] = special_sigma[k]; sp[4 * k + 1] = special_epsilon[k];
        sp[4 * k + 2] = special_lj_scale[k]; sp[4 * k + 3] = special_coulomb_scale[k];
    }
    const int64_t n_entries = 2 * n_bonds + 3 * n_angles + 4 * n_torsions + 2 * n_specials;
    std::vector<long long> entries_of(static_cast<size_t>(n_global) + 1, 0);
    const std::vector<int>* tables[4] = {&ba, &aa, &ta, &sa};
    for (const std::vector<int>* t : tables)
        for (int g : *t) {
            if (g < 0 || g >= n_global) return fail(c, DSMD_ERR_INVALID, "a bonded term names an atom id outside [0, n_global)");
            ++entries_of[static_cast<size_t>(g) + 1];
        }
    for (int64_t g = 0; g < n_global; ++g) entries_of[g + 1] += entries_of[g];
    std::vector<int> entry(static_cast<size_t>(n_entries));
    {
        std::vector<long long> next(entries_of.begin(), entries_of.end() - 1);
        int place = 0;
        for (const std::vector<int>* t : tables)
            for (int g : *t) entry[static_cast<size_t>(next[g]++)] = place++;
    }
    dsmd_ctx::Bonded& b = c->bonded;
    DSMD_TO_DEVICE(c, b.bond_atoms, ba);
    DSMD_TO_DEVICE(c, b.angle_atoms, aa);
    DSMD_TO_DEVICE(c, b.torsion_atoms, ta);
    DSMD_TO_DEVICE(c, b.torsion_n, tn);
    DSMD_TO_DEVICE(c, b.special_atoms, sa);
    DSMD_TO_DEVICE(c, b.bond_par, bp);
    DSMD_TO_DEVICE(c, b.angle_par, ap);
    DSMD_TO_DEVICE(c, b.torsion_par, tp);
    DSMD_TO_DEVICE(c, b.special_par, sp);
    DSMD_TO_DEVICE(c, b.entries_of, entries_of);
    DSMD_TO_DEVICE(c, b.entry, entry);
    b.blocks = blocks_for(terms, kThreads);
    DSMD_CUDA(c, cudaMalloc(&b.slot_of_gid, sizeof(int) * std::max<int64_t>(n_global, 1)));
    DSMD_CUDA(c, cudaMalloc(&b.contrib, sizeof(double) * 3 * n_entries));
    DSMD_CUDA(c, cudaMalloc(&b.partials, sizeof(double) * 5 * b.blocks));
    DSMD_CUDA(c, cudaMalloc(&b.scalars, sizeof(double) * 5));
    DSMD_CUDA(c, cudaMemset(b.scalars, 0, sizeof(double) * 5));
    DSMD_CUDA(c, cudaMalloc(&b.missing, sizeof(unsigned)));
    DSMD_CUDA(c, cudaMemset(b.missing, 0, sizeof(unsigned)));
    DSMD_CUDA(c, cudaMallocHost(&b.h_scalars, sizeof(double) * 6));
    b.n_global = n_global;
    b.n_bonds = n_bonds; b.n_angles = n_angles; b.n_torsions = n_torsions; b.n_specials = n_specials;
    b.n_entries = n_entries;
    b.map_epoch = -1;
    return DSMD_OK;
}

int dsmd_compute_bonded(dsmd_ctx* c, void* stream) {
    if (!c) return DSMD_ERR_INVALID;
    dsmd_ctx::Bonded& b = c->bonded;
    if (b.terms() == 0) return DSMD_OK;
    if (!c->list_valid) return fail(c, DSMD_ERR_STATE, "no neighbour list built yet (bonded terms find their atoms through the sorted arrays)");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (b.map_epoch != c->build_epoch) {   // the sort of a list build moved the atoms
        DSMD_CUDA(c, cudaMemsetAsync(b.slot_of_gid, 0x7F, sizeof(int) * b.n_global, s));   // 0x7F7F7F7F: beyond any slot
        k_bonded_slot_map<<<blocks_for(c->n_total, kThreads), kThreads, 0, s>>>(static_cast<int>(c->n_total), c->gid[c->cur],
                                                                               static_cast<int>(b.n_global), b.slot_of_gid);
        DSMD_LAUNCHED(c);
        b.map_epoch = c->build_epoch;
    }
    BondedTable t{};
    t.n_bonds = static_cast<int>(b.n_bonds); t.n_angles = static_cast<int>(b.n_angles);
    t.n_torsions = static_cast<int>(b.n_torsions); t.n_specials = static_cast<int>(b.n_specials);
    t.bond_atoms = b.bond_atoms; t.bond_par = b.bond_par; t.angle_atoms = b.angle_atoms; t.angle_par = b.angle_par;
    t.torsion_atoms = b.torsion_atoms; t.torsion_par = b.torsion_par; t.torsion_n = b.torsion_n;
    t.special_atoms = b.special_atoms; t.special_par = b.special_par;
    t.slot_of_gid = b.slot_of_gid;
    t.n_global = static_cast<int>(b.n_global);
    t.n_owned = static_cast<int>(c->n_owned);
    for (int a = 0; a < 3; ++a) { t.box[a] = c->box[a]; t.periodic[a] = c->periodic[a]; }
    double** r = c->real[c->cur];
    k_bonded_terms<<<static_cast<unsigned>(b.blocks), kThreads, 0, s>>>(t, r[0], r[1], r[2], r[10], b.contrib, b.partials, b.missing);
    DSMD_LAUNCHED(c);
    k_bonded_gather<<<blocks_for(c->n_owned, kThreads), kThreads, 0, s>>>(static_cast<int>(c->n_owned), c->gid[c->cur],
                                                                         static_cast<int>(b.n_global), b.entries_of, b.entry,
                                                                         b.contrib, r[6], r[7], r[8]);
    DSMD_LAUNCHED(c);
    k_reduce_partials<5><<<1, kThreads, 0, s>>>(b.partials, static_cast<int>(b.blocks), b.scalars, 0);
    DSMD_LAUNCHED(c);
    return DSMD_OK;
}

int dsmd_read_bonded_scalars(dsmd_ctx* c, double out[5], void* stream) {
    if (!c || !out) return DSMD_ERR_INVALID;
    dsmd_ctx::Bonded& b = c->bonded;
    for (int k = 0; k < 5; ++k) out[k] = 0.0;
    if (b.terms() == 0) return DSMD_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned* h_missing = reinterpret_cast<unsigned*>(b.h_scalars + 5);
    DSMD_CUDA(c, cudaMemcpyAsync(b.h_scalars, b.scalars, sizeof(double) * 5, cudaMemcpyDeviceToHost, s));
    DSMD_CUDA(c, cudaMemcpyAsync(h_missing, b.missing, sizeof(unsigned), cudaMemcpyDeviceToHost, s));
    DSMD_CUDA(c, cudaMemsetAsync(b.missing, 0, sizeof(unsigned), s));
    DSMD_CUDA(c, cudaStreamSynchronize(s));
    for (int k = 0; k < 5; ++k) out[k] = b.h_scalars[k];
    if (*h_missing)
        return fail(c, DSMD_ERR_STATE, std::to_string(*h_missing) + " bonded term(s) have an owned atom whose partner is not on "
                                       "this rank: the halo is narrower than the term is long");
    return DSMD_OK;
}

int dsmd_kinetic_energy(dsmd_ctx* c, double* out, void* stream) {
    if (!c || !out) return DSMD_ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t blocks = blocks_for(c->n_owned, kThreads);
    { const int rc = ensure_partials(c, blocks); if (rc) return rc; }
    double** r = c->real[c->cur];
    k_kinetic<<<static_cast<unsigned>(blocks), kThreads, 0, s>>>(static_cast<int>(c->n_owned), r[3], r[4], r[5], r[9],
                                                                 c->partials);
    DSMD_LAUNCHED(c);
    k_reduce_partials<1><<<1, kThreads, 0, s>>>(c->partials, static_cast<int>(blocks), c->scalars + 6, 0);
    DSMD_LAUNCHED(c);
    DSMD_CUDA(c, cudaMemcpyAsync(c->h_scalars + 6, c->scalars + 6, sizeof(double), cudaMemcpyDeviceToHost, s));
    DSMD_CUDA(c, cudaStreamSynchronize(s));
    *out = c->h_scalars[6];
    return DSMD_OK;
}

int dsmd_scale_velocities(dsmd_ctx* c, double factor, void* stream) {
    if (!c || !std::isfinite(factor)) return DSMD_ERR_INVALID;
    if (c->n_owned == 0) return DSMD_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    double** r = c->real[c->cur];
    k_scale_velocities<<<blocks_for(c->n_owned, kThreads), kThreads, 0, s>>>(static_cast<int>(c->n_owned), factor, r[3], r[4],
                                                                             r[5]);
    DSMD_LAUNCHED(c);
    return DSMD_OK;
}

int dsmd_run_nve(dsmd_ctx* c, int64_t n_steps, double dt, double f2a, double hi_frac, int every, int lagged,
                 int64_t* n_rebuilds, double* worst_disp_sq, void* stream) {
    if (!c || n_steps < 0) return DSMD_ERR_INVALID;
    if (c->n_total != c->n_owned) return fail(c, DSMD_ERR_STATE, "dsmd_run_nve handles single-rank systems only");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (!c->list_valid) {
        const int rc = dsmd_build_neighbor_list(c, s);
        if (rc) return rc;
        const int rc2 = dsmd_compute_forces(c, DSMD_PHASE_FULL, 0, s);
        if (rc2) return rc2;
        const int rc3 = dsmd_compute_bonded(c, s);
        if (rc3) return rc3;
    }
    const double limit2 = (hi_frac * c->skin) * (hi_frac * c->skin);
    int64_t rebuilds = 0;
    double worst = 0.0;
    int since_build = 0;
    double d_prev = 0.0, d_prev2 = 0.0;   // displacement (not squared) seen one and two steps ago (lagged mode)
    int pending = -1;                      // read-back slot in flight
    auto bits_to_double = [](unsigned long long b) { double v; std::memcpy(&v, &b, sizeof(v)); return v; };
    // Between two steps of this loop nobody reads the velocities, so the second half of one step and the first half of the
    // next (the same forces) are one pass over the atoms; with constraints RATTLE sits between them and they stay apart.
    const bool merge = c->n_clusters == 0;
    for (int64_t step = 0; step < n_steps; ++step) {
        { const int rc = dsmd_integrate(c, merge && step > 0 ? 3 : 1, dt, f2a, s); if (rc) return rc; }   // with SHAKE when constraints are set
        ++since_build;
        bool rebuild = every > 0 && since_build >= every;
        if (!lagged) {
            double d2 = 0.0;
            const int rc = dsmd_max_displacement_sq(c, &d2, s);
            if (rc) return rc;
            if (d2 > limit2) rebuild = true;
            if (!rebuild) worst = std::max(worst, d2);
        } else {
            // Read back what the previous step saw (its copy finished long ago), queue this step's copy, and decide on
            // the linear extrapolation of the last two values, as the reference does on several ranks
            // (src/md_simulation.cpp:1232-1245). The previous step's forces were evaluated under d_prev.
            if (pending >= 0) {
                DSMD_CUDA(c, cudaEventSynchronize(c->disp_event[pending]));
                d_prev2 = d_prev;
                d_prev = std::sqrt(bits_to_double(*c->h_disp[pending]));
                worst = std::max(worst, d_prev * d_prev);
            }
            const int slot = static_cast<int>(step & 1);
            DSMD_CUDA(c, cudaMemcpyAsync(c->h_disp[slot], &c->status->max_disp2, sizeof(unsigned long long),
                                         cudaMemcpyDeviceToHost, s));
            DSMD_CUDA(c, cudaEventRecord(c->disp_event[slot], s));
            pending = slot;
            const double predicted = d_prev + 1.5 * std::max(d_prev - d_prev2, 0.0);
            if (predicted * predicted > limit2) rebuild = true;
        }
        if (rebuild) {
            const int rc = dsmd_build_neighbor_list(c, s);
            if (rc) return rc;
            ++rebuilds;
            since_build = 0;
            d_prev = d_prev2 = 0.0;
            pending = -1;   // the copy queued above predates the new reference positions
        }
        { const int rc = dsmd_compute_forces(c, DSMD_PHASE_FULL, 0, s); if (rc) return rc; }
        { const int rc = dsmd_compute_bonded(c, s); if (rc) return rc; }
        if (!merge || step + 1 == n_steps) { const int rc = dsmd_integrate(c, 2, dt, f2a, s); if (rc) return rc; }
    }
    if (lagged && pending >= 0) {
        DSMD_CUDA(c, cudaEventSynchronize(c->disp_event[pending]));
        const double d = std::sqrt(bits_to_double(*c->h_disp[pending]));
        worst = std::max(worst, d * d);
    }
    DSMD_CUDA(c, cudaStreamSynchronize(s));
    if (n_rebuilds) *n_rebuilds = rebuilds;
    if (worst_disp_sq) *worst_disp_sq = worst;
    return DSMD_OK;
}

// The pipelined form of the host-buffer call, for a step without rebuild and without energy on a single-rank system:
// the sorted atoms are cut into slabs of z layers of cells; positions go up slab by slab on one copy stream (each slab is
// packed as it lands), the pair kernel of a slab starts once the slab and its two neighbours are on the device (a slab is
// at least twice the stencil thick, so a slab's partners lie in itself and the slabs next to it, the first and the last
// being neighbours through the periodic boundary), and its forces go down on a second copy stream while the later
// slabs are still coming up or being worked on: the two directions of the host link and the kernel run side by side.
// Returns DSMD_ERR_STATE when the system does not cut into at least four slabs (the caller falls back).
static int forces_host_pipelined(dsmd_ctx* c, const double* x, const double* y, const double* z, double* fx, double* fy,
                                 double* fz, cudaStream_t s) {
    const int layers = c->grid.nc[2];
    const int thick = 2 * c->grid.stencil;
    int pieces = std::min(8, layers / thick);
    if (pieces < 4 || !c->h_layer_start || c->n_total != c->n_owned) return DSMD_ERR_STATE;
    if (!c->copy_in) {
        DSMD_CUDA(c, cudaStreamCreateWithFlags(&c->copy_in, cudaStreamNonBlocking));
        DSMD_CUDA(c, cudaStreamCreateWithFlags(&c->copy_out, cudaStreamNonBlocking));
        for (int k = 0; k < 16; ++k) {
            DSMD_CUDA(c, cudaEventCreateWithFlags(&c->piece_up[k], cudaEventDisableTiming));
            DSMD_CUDA(c, cudaEventCreateWithFlags(&c->piece_done[k], cudaEventDisableTiming));
        }
        DSMD_CUDA(c, cudaEventCreateWithFlags(&c->pipe_begin, cudaEventDisableTiming));
        DSMD_CUDA(c, cudaEventCreateWithFlags(&c->pipe_end, cudaEventDisableTiming));
    }
    int64_t begin[17];
    for (int k = 0; k <= pieces; ++k) begin[k] = c->h_layer_start[static_cast<int64_t>(layers) * k / pieces];
    begin[0] = 0;
    begin[pieces] = c->n_owned;
    // everything queued on the caller's stream so far comes first
    DSMD_CUDA(c, cudaEventRecord(c->pipe_begin, s));
    DSMD_CUDA(c, cudaStreamWaitEvent(c->copy_in, c->pipe_begin, 0));
    DSMD_CUDA(c, cudaStreamWaitEvent(c->copy_out, c->pipe_begin, 0));
    const double* src[3] = {x, y, z};
    double* dst[3] = {fx, fy, fz};
    for (int k = 0; k < pieces; ++k) {
        const int64_t first = begin[k], count = begin[k + 1] - begin[k];
        for (int a = 0; a < 3 && count > 0; ++a)
            DSMD_CUDA(c, cudaMemcpyAsync(c->real[c->cur][a] + first, src[a] + first, sizeof(double) * count,
                                         cudaMemcpyHostToDevice, c->copy_in));
        { const int rc = pack_impl(c, first, count, false, 0.0, 0.0, c->copy_in); if (rc) return rc; }
        DSMD_CUDA(c, cudaEventRecord(c->piece_up[k], c->copy_in));
    }
    // slabs 1 .. pieces - 2 need only slabs that come up early; the last and the first (neighbours through the boundary)
    // close the round
    for (int turn = 0; turn < pieces; ++turn) {
        const int k = turn < pieces - 1 ? turn + 1 : 0;
        const int64_t first = begin[k], count = begin[k + 1] - begin[k];
        const int needs[3] = {(k + pieces - 1) % pieces, k, (k + 1) % pieces};
        for (int q = 0; q < 3; ++q) DSMD_CUDA(c, cudaStreamWaitEvent(s, c->piece_up[needs[q]], 0));
        if (count > 0) { const int rc = compute_forces_impl(c, DSMD_PHASE_FULL, 0, first, count, s); if (rc) return rc; }
        DSMD_CUDA(c, cudaEventRecord(c->piece_done[k], s));
        DSMD_CUDA(c, cudaStreamWaitEvent(c->copy_out, c->piece_done[k], 0));
        for (int a = 0; a < 3 && count > 0; ++a)
            DSMD_CUDA(c, cudaMemcpyAsync(dst[a] + first, c->real[c->cur][DSMD_FX + a] + first, sizeof(double) * count,
                                         cudaMemcpyDeviceToHost, c->copy_out));
    }
    DSMD_CUDA(c, cudaEventRecord(c->pipe_end, c->copy_out));
    DSMD_CUDA(c, cudaStreamWaitEvent(s, c->pipe_end, 0));
    DSMD_CUDA(c, cudaStreamSynchronize(s));
    return DSMD_OK;
}

int dsmd_forces_host(dsmd_ctx* c, const double* x, const double* y, const double* z, int rebuild, double* fx,
                     double* fy, double* fz, double* out6, void* stream) {
    if (!c || !x || !y || !z || !fx || !fy || !fz) return DSMD_ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (!rebuild && c->list_valid && !out6) {
        const int rc = forces_host_pipelined(c, x, y, z, fx, fy, fz, s);
        if (rc != DSMD_ERR_STATE) return rc;   // DSMD_ERR_STATE: too small to cut into slabs, the plain way below
    }
    { const int rc = dsmd_upload_positions(c, x, y, z, s); if (rc) return rc; }
    if (rebuild || !c->list_valid) {
        const int rc = dsmd_build_neighbor_list(c, s);
        if (rc) return rc;
    } else {
        const int rc = pack_impl(c, 0, c->n_total, false, 0.0, 0.0, s);
        if (rc) return rc;
    }
    { const int rc = dsmd_compute_forces(c, DSMD_PHASE_FULL, out6 ? 1 : 0, s); if (rc) return rc; }
    double* dst[3] = {fx, fy, fz};
    for (int a = 0; a < 3; ++a)
        DSMD_CUDA(c, cudaMemcpyAsync(dst[a], c->real[c->cur][DSMD_FX + a], sizeof(double) * c->n_owned,
                                     cudaMemcpyDeviceToHost, s));
    if (out6) return dsmd_read_scalars(c, out6, s);
    DSMD_CUDA(c, cudaStreamSynchronize(s));
    return DSMD_OK;
}

int dsmd_fma_probe(dsmd_ctx* c, int iters, double* flops, void* stream) {
    if (!c || iters <= 0 || !flops) return DSMD_ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int sms = 0;
    DSMD_CUDA(c, cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c->device));
    const int blocks = sms * 8;
    k_fma_probe<<<blocks, 256, 0, s>>>(iters, 1.0f, reinterpret_cast<float*>(c->flag));
    DSMD_LAUNCHED(c);
    *flops = static_cast<double>(blocks) * 256.0 * static_cast<double>(iters) * 8.0 * 2.0;
    return DSMD_OK;
}

// ---- ghosts ---------------------------------------------------------------------------------------------------------

int dsmd_halo_pack(dsmd_ctx* c, const int32_t* d_index, const int8_t* d_image, int64_t count, double* d_out,
                   void* stream) {
    if (!c || count < 0 || (count > 0 && (!d_index || !d_out))) return DSMD_ERR_INVALID;
    if (count == 0) return DSMD_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    double** r = c->real[c->cur];
    k_halo_pack<<<blocks_for(count, kThreads), kThreads, 0, s>>>(static_cast<int>(count), d_index,
                                                                reinterpret_cast<const signed char*>(d_image), r[0], r[1],
                                                                r[2], c->box[0], c->box[1], c->box[2], d_out);
    DSMD_LAUNCHED(c);
    return DSMD_OK;
}

int dsmd_displacement_word(dsmd_ctx* c, void** device_word) {
    if (!c || !device_word) return DSMD_ERR_INVALID;
    *device_word = &c->status->max_disp2;
    return DSMD_OK;
}

int dsmd_halo_unpack(dsmd_ctx* c, const double* d_in, int64_t first_ghost, int64_t count, void* stream) {
    if (!c || count < 0 || first_ghost < 0 || first_ghost + count > c->n_total - c->n_owned) return DSMD_ERR_INVALID;
    if (count == 0) return DSMD_OK;
    if (!c->list_valid) return fail(c, DSMD_ERR_STATE, "halo unpack needs the ghost slots of a built list");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    double** r = c->real[c->cur];
    k_halo_unpack<<<blocks_for(count, kThreads), kThreads, 0, s>>>(c->grid, static_cast<int>(first_ghost),
                                                                  static_cast<int>(count), d_in, c->ghost_slot, r[0],
                                                                  r[1], r[2], c->type[c->cur], c->pq, c->status);
    DSMD_LAUNCHED(c);
    return DSMD_OK;
}

int dsmd_halo_select(dsmd_ctx* c, const double lo[3], const double hi[3], int32_t* d_index, int64_t capacity,
                     int64_t* count, void* stream) {
    if (!c || !lo || !hi || !count) return DSMD_ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int n = static_cast<int>(c->n_owned);
    *count = 0;
    if (n == 0) return DSMD_OK;
    double** r = c->real[c->cur];
    k_halo_flag<<<blocks_for(n, kThreads), kThreads, 0, s>>>(n, r[0], r[1], r[2], lo[0], lo[1], lo[2], hi[0], hi[1],
                                                            hi[2], c->flag);
    DSMD_LAUNCHED(c);
    size_t need = 0;
    thrust::counting_iterator<int> iota(0);
    int* d_selected = c->val[0];   // scratch of capacity entries
    cub::DeviceSelect::Flagged(nullptr, need, iota, c->flag, d_selected, &c->status->select_count, n, s);
    if (need > c->cub_temp_bytes) {
        if (c->cub_temp) cudaFree(c->cub_temp);
        c->cub_temp = nullptr;
        DSMD_CUDA(c, cudaMalloc(&c->cub_temp, need));
        c->cub_temp_bytes = need;
    }
    DSMD_CUDA(c, cub::DeviceSelect::Flagged(c->cub_temp, need, iota, c->flag, d_selected, &c->status->select_count, n, s));
    unsigned long long selected = 0;
    DSMD_CUDA(c, cudaMemcpyAsync(&selected, &c->status->select_count, sizeof(selected), cudaMemcpyDeviceToHost, s));
    DSMD_CUDA(c, cudaStreamSynchronize(s));
    *count = static_cast<int64_t>(selected);
    if (d_index && static_cast<int64_t>(selected) <= capacity && selected > 0)
        DSMD_CUDA(c, cudaMemcpyAsync(d_index, d_selected, sizeof(int) * selected, cudaMemcpyDeviceToDevice, s));
    DSMD_CUDA(c, cudaStreamSynchronize(s));
    return DSMD_OK;
}

int dsmd_halo_pack_records(dsmd_ctx* c, const int32_t* d_index, int64_t count, const double shift[3],
                           double* d_real_out, int32_t* d_int_out, void* stream) {
    if (!c || count < 0 || (count > 0 && (!d_index || !d_real_out || !d_int_out))) return DSMD_ERR_INVALID;
    if (count == 0) return DSMD_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    k_halo_pack_records<<<blocks_for(count, kThreads), kThreads, 0, s>>>(
        static_cast<int>(count), d_index, arrays_of(c, c->cur), c->type[c->cur], c->gid[c->cur], shift ? shift[0] : 0.0,
        shift ? shift[1] : 0.0, shift ? shift[2] : 0.0, d_real_out, d_int_out);
    DSMD_LAUNCHED(c);
    return DSMD_OK;
}

int dsmd_halo_append_records(dsmd_ctx* c, const double* d_real_in, const int32_t* d_int_in, int64_t count,
                             void* stream) {
    if (!c || count < 0 || (count > 0 && (!d_real_in || !d_int_in))) return DSMD_ERR_INVALID;
    if (c->n_total + count > c->capacity) return fail(c, DSMD_ERR_CAPACITY, "ghosts exceed the context's capacity");
    if (count == 0) return DSMD_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    k_halo_append_records<<<blocks_for(count, kThreads), kThreads, 0, s>>>(
        static_cast<int>(count), static_cast<int>(c->n_total), d_real_in, d_int_in, arrays_of(c, c->cur),
        c->type[c->cur], c->gid[c->cur]);
    DSMD_LAUNCHED(c);
    c->n_total += count;
    c->list_valid = false;
    return DSMD_OK;
}

int dsmd_halo_append_packed(dsmd_ctx* c, const double* d_records, int64_t count, void* stream) {
    if (!c || count < 0 || (count > 0 && !d_records)) return DSMD_ERR_INVALID;
    if (c->n_total + count > c->capacity) return fail(c, DSMD_ERR_CAPACITY, "atoms exceed the context's capacity");
    if (count == 0) return DSMD_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    k_halo_append_packed<<<blocks_for(count, kThreads), kThreads, 0, s>>>(
        static_cast<int>(count), static_cast<int>(c->n_total), d_records, arrays_of(c, c->cur), c->type[c->cur],
        c->gid[c->cur]);
    DSMD_LAUNCHED(c);
    c->n_total += count;
    c->list_valid = false;
    return DSMD_OK;
}

int dsmd_capacity(const dsmd_ctx* c, int64_t* capacity) {
    if (!c || !capacity) return DSMD_ERR_INVALID;
    *capacity = c->capacity;
    return DSMD_OK;
}

}  // extern "C"
