// Radius-graph edge builder for the machine-learned-potential backends (sm_100a).
//
// Semantics of the reference's EdgeBuilder::build (include/EdgeBuilder.cuh:12-59, src/EdgeBuilder.cu:233-334): every
// ordered pair (i, j), i != j, |r_j - r_i| < cutoff over the atoms given, no minimum image; optional periodic-image
// description (centres restricted to the real atoms, neighbour replaced by the atom it copies, per-edge shift) and
// optional receiver pruning. Output int64 [2, E] + double [E, 3].
//
// What is done differently: the neighbourhood search runs ONCE (the reference searches twice, to count and to fill),
// on 32-bit fixed-point coordinates in fp32 with an fp64 re-decision inside the rounding band (so membership is that of
// an fp64 search), and leaves its hits in 32-atom slices; after one scan of the counts a warp-cooperative pass expands
// the slices into the interface arrays with fully coalesced stores, which is where the bytes are (40 B per edge).
// A second entry point emits the compact periodic form (int32 src/dst, int8 lattice shift, fp32 edge vector).

#include <cub/cub.cuh>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <string>

#include "../../include/dsmd_b200.h"
#include "dsmd_common.cuh"

using dsmd::Grid;

namespace {

constexpr int kThreads = 256;
constexpr int kSearchThreads = 128;

inline unsigned blocks_for(int64_t n, int threads) { return static_cast<unsigned>((n + threads - 1) / threads); }

struct EdgeStatus {
    long long edges;
    unsigned int out_of_bounds;
    unsigned int need_stride;
    unsigned int rechecked;
    unsigned int pad;
};

__global__ void k_edge_keys(Grid g, int n, const double* __restrict__ x, const double* __restrict__ y,
                            const double* __restrict__ z, unsigned* __restrict__ key, int* __restrict__ val,
                            EdgeStatus* st) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    unsigned bad = 0;
    const unsigned fx = dsmd::to_fixed(x[i], 0, g, bad);
    const unsigned fy = dsmd::to_fixed(y[i], 1, g, bad);
    const unsigned fz = dsmd::to_fixed(z[i], 2, g, bad);
    if (bad) atomicOr(&st->out_of_bounds, 1u);
    const unsigned cx = dsmd::cell_of(fx, g.wrap[0], g.nc[0]);
    const unsigned cy = dsmd::cell_of(fy, g.wrap[1], g.nc[1]);
    const unsigned cz = dsmd::cell_of(fz, g.wrap[2], g.nc[2]);
    key[i] = (cz * g.nc[1] + cy) * g.nc[0] + cx;
    val[i] = i;
}

// How many box lengths a coordinate lies from its wrapped place, consistent with to_fixed (which maps a coordinate that
// rounds up to the upper face onto the lower face of the next image).
__device__ __forceinline__ int wrap_count(double v, int axis, const Grid& g) {
    if (!g.wrap[axis]) return 0;
    const double u = (v - g.org[axis]) * g.inv_len[axis];
    if (!(u == u) || fabs(u) > 1.0e9) return 0;
    const double w = floor(u);
    return static_cast<int>(w) + (u - w >= 1.0 ? 1 : 0);
}

constexpr int kWrapBits = 10, kWrapBias = 1 << (kWrapBits - 1), kWrapMask = (1 << kWrapBits) - 1;

__device__ __forceinline__ int packed_wraps(int wx, int wy, int wz) {
    auto field = [](int w) { return min(max(w + kWrapBias, 0), kWrapMask); };
    return field(wx) | (field(wy) << kWrapBits) | (field(wz) << (2 * kWrapBits));
}

__device__ __forceinline__ int wrap_field(int packed, int axis) {
    return ((packed >> (axis * kWrapBits)) & kWrapMask) - kWrapBias;
}

// Sorted fixed-point atoms (w = the caller's atom index), their wrap counts (periodic form only) and cell starts.
__global__ void k_edge_gather(Grid g, int n, const unsigned* __restrict__ key, const int* __restrict__ val,
                              const double* __restrict__ x, const double* __restrict__ y, const double* __restrict__ z,
                              int4* __restrict__ pq, int* __restrict__ wraps, int* __restrict__ cell_start) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= n) return;
    const int a = val[s];
    unsigned bad = 0;
    const double px = x[a], py = y[a], pz = z[a];
    int4 p;
    p.x = static_cast<int>(dsmd::to_fixed(px, 0, g, bad));
    p.y = static_cast<int>(dsmd::to_fixed(py, 1, g, bad));
    p.z = static_cast<int>(dsmd::to_fixed(pz, 2, g, bad));
    p.w = a;
    pq[s] = p;
    if (wraps) wraps[s] = packed_wraps(wrap_count(px, 0, g), wrap_count(py, 1, g), wrap_count(pz, 2, g));
    const int k_here = static_cast<int>(key[s]);
    const int k_prev = s == 0 ? -1 : static_cast<int>(key[s - 1]);
    for (int c = k_prev + 1; c <= k_here; ++c) cell_start[c] = s;
}

// Cells behind the last occupied one start at the end of the atom array.
__global__ void k_edge_cell_tail(const unsigned* __restrict__ key, int n, int table_size, int* __restrict__ cell_start) {
    const int c = static_cast<int>(key[n - 1]) + 1 + blockIdx.x * blockDim.x + threadIdx.x;
    if (c < table_size) cell_start[c] = n;
}

struct SearchArgs {
    int n, n_centers, stride, row;
    const int4* pq;
    const double *x, *y, *z;
    const int* cell_start;
    const int* owner;
    const unsigned char* ok;
    unsigned* rows;
    int* counts;        // by sorted slot
    EdgeStatus* st;
};

template <bool PERIODIC>
__device__ __forceinline__ bool within_fp64(const Grid& g, const SearchArgs& a, int ai, int aj) {
    double dx = a.x[aj] - a.x[ai], dy = a.y[aj] - a.y[ai], dz = a.z[aj] - a.z[ai];
    if (PERIODIC) {
        dx -= g.box[0] * rint(dx / g.box[0]);
        dy -= g.box[1] * rint(dy / g.box[1]);
        dz -= g.box[2] * rint(dz / g.box[2]);
    }
    const double r2 = __dadd_rn(__dadd_rn(__dmul_rn(dx, dx), __dmul_rn(dy, dy)), __dmul_rn(dz, dz));
    return r2 < g.r2_list_d;
}

// One thread per sorted slot; hits go to the slot's column of its 32-atom slice: the neighbour's atom index, or, PERIODIC
// (all axes wrap), its sorted slot (the expansion reads the neighbour's position by slot).
template <bool PERIODIC>
__global__ void __launch_bounds__(kSearchThreads) k_edge_search(Grid g, SearchArgs a) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= a.n) return;
    const int4 pi = a.pq[p];
    const int centre = pi.w;
    int count = 0;
    const bool is_centre = centre < a.n_centers && !(a.ok && a.row == 0 && !a.ok[centre]);
    const size_t base = (static_cast<size_t>(p >> 5) * a.stride) * 32 + (p & 31);
    unsigned rechecked = 0;
    if (is_centre) {
        const bool check_nb = a.ok && a.row == 1;
            const int cy = static_cast<int>(dsmd::cell_of(static_cast<unsigned>(pi.y), g.wrap[1], g.nc[1]));
        const int cz = static_cast<int>(dsmd::cell_of(static_cast<unsigned>(pi.z), g.wrap[2], g.nc[2]));
        const int S = g.stencil;
        for (int dz = -S; dz <= S; ++dz) {
            int zc = cz + dz;
            if (g.wrap[2]) { if (zc < 0) zc += g.nc[2]; else if (zc >= g.nc[2]) zc -= g.nc[2]; }
            else if (zc < 0 || zc >= g.nc[2]) continue;
            for (int dy = -S; dy <= S; ++dy) {
                int yc = cy + dy;
                if (g.wrap[1]) { if (yc < 0) yc += g.nc[1]; else if (yc >= g.nc[1]) yc -= g.nc[1]; }
                else if (yc < 0 || yc >= g.nc[1]) continue;
                const int row = (zc * g.nc[1] + yc) * g.nc[0];
                dsmd::RowWindow win;
                if (!dsmd::row_window(g, pi, cy, cz, dy, dz, win)) continue;
                const int a0 = win.a0, b0 = win.b0, a1 = win.a1, b1 = win.b1;
                for (int part = 0; part < 2; ++part) {
                    const int lo = part == 0 ? a0 : a1, hi = part == 0 ? b0 : b1;
                    if (hi < lo) continue;
                    const int s_begin = a.cell_start[row + lo], s_end = a.cell_start[row + hi + 1];
                    for (int s = s_begin; s < s_end; ++s) {
                        const int4 pj = __ldg(&a.pq[s]);
                        const float fx = dsmd::fixed_delta(pj.x, pi.x, g.scale[0]);
                        const float fy = dsmd::fixed_delta(pj.y, pi.y, g.scale[1]);
                        const float fz = dsmd::fixed_delta(pj.z, pi.z, g.scale[2]);
                        const float r2 = fx * fx + fy * fy + fz * fz;
                        if (r2 >= g.r2_list + g.band || s == p) continue;
                        if (r2 >= g.r2_list - g.band) {
                            ++rechecked;
                            if (!within_fp64<PERIODIC>(g, a, centre, pj.w)) continue;
                        }
                        if (check_nb && !a.ok[a.owner ? a.owner[pj.w] : pj.w]) continue;
                        if (count < a.stride) a.rows[base + static_cast<size_t>(count) * 32] = static_cast<unsigned>(PERIODIC ? s : pj.w);
                        ++count;
                    }
                }
            }
        }
    }
    a.counts[p] = min(count, a.stride);
    if (count > a.stride) atomicMax(&a.st->need_stride, static_cast<unsigned>(count));
    if (rechecked) atomicAdd(&a.st->rechecked, rechecked);
}

__global__ void k_edge_total(int n, const long long* __restrict__ offsets, const int* __restrict__ counts,
                             EdgeStatus* st) {
    st->edges = offsets[n - 1] + counts[n - 1];
}

// Finds, for flat position t inside a warp's run of edges, the lane (centre) it belongs to: the last lane whose
// exclusive prefix is <= t.
__device__ __forceinline__ int owner_lane(int t, int my_prefix) {
    int lo = 0;
#pragma unroll
    for (int step = 16; step > 0; step >>= 1) {
        const int probe = lo + step;
        const int v = __shfl_sync(0xffffffffu, my_prefix, probe & 31);
        if (probe < 32 && v <= t) lo = probe;
    }
    return lo;
}

// Interface form. A warp takes 32 consecutive sorted slots and streams their edges out in flat order, so that the
// three output arrays are written with contiguous, coalesced stores.
__global__ void __launch_bounds__(kThreads) k_edge_fill(int n, long long n_edges, int stride, const int4* __restrict__ pq,
                            const unsigned* __restrict__ rows, const int* __restrict__ counts,
                            const long long* __restrict__ offsets, int n_centers, const int* __restrict__ owner,
                            const double* __restrict__ shift_x, const double* __restrict__ shift_y,
                            const double* __restrict__ shift_z, long long* __restrict__ edges,
                            double* __restrict__ shift) {
    // the three shift components of 32 edges are 96 consecutive doubles of the output: they pass through shared memory
    // so that the warp stores them as three unit-stride runs instead of three runs of stride 24 bytes
    __shared__ double stage[kThreads / 32][96];
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    double* mine = stage[threadIdx.x >> 5];
    const int p = warp * 32 + lane;
    if (warp * 32 >= n) return;
    const int cnt = p < n ? counts[p] : 0;
    const int centre = p < n ? pq[p].w : 0;
    int prefix = cnt;   // inclusive scan over the warp
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, prefix, o);
        if (lane >= o) prefix += v;
    }
    const int total = __shfl_sync(0xffffffffu, prefix, 31);
    prefix -= cnt;      // exclusive
    const long long out0 = offsets[warp * 32];
    const size_t slice = static_cast<size_t>(warp) * stride * 32;
    for (int t0 = 0; t0 < total; t0 += 32) {
        const int t = t0 + lane;
        const int c = owner_lane(min(t, total - 1), prefix);
        const int c_prefix = __shfl_sync(0xffffffffu, prefix, c);
        const int c_centre = __shfl_sync(0xffffffffu, centre, c);
        if (t < total) {
            const int k = t - c_prefix;
            const int nb = static_cast<int>(rows[slice + static_cast<size_t>(k) * 32 + c]);
            const long long o = out0 + t;
            // the first n_centers atoms are real: they stand for themselves and carry no shift (EdgeBuilder::Images'
            // contract), so only image atoms cost the four scattered reads
            const bool image = owner && nb >= n_centers;
            edges[o] = c_centre;
            edges[n_edges + o] = image ? owner[nb] : nb;
            if (shift) {
                mine[3 * lane] = image ? shift_x[nb] : 0.0;
                mine[3 * lane + 1] = image ? shift_y[nb] : 0.0;
                mine[3 * lane + 2] = image ? shift_z[nb] : 0.0;
            }
        }
        if (shift) {
            __syncwarp();
            const int filled = 3 * min(32, total - t0);
            double* out = shift + 3 * (out0 + t0);
            for (int q = lane; q < filled; q += 32) out[q] = mine[q];
            __syncwarp();
        }
    }
}

// Compact periodic form: as k_edge_fill, a warp takes 32 consecutive sorted slots and streams their edges out in flat
// order with contiguous stores (centres in cell order, the neighbours of a centre in the order of the search: the
// order of the interface form). Rows hold neighbour slots, so positions and wrap counts are read where they lie
// whatever the caller's atom numbering. Displacements come from the fixed-point coordinates (resolution box / 2^32);
// the lattice shift refers to the caller's coordinates: x[dst] + shift * box - x[src] = vec.
__global__ void __launch_bounds__(kThreads) k_edge_fill_compact(
    Grid g, int n, int stride, const int4* __restrict__ pq, const int* __restrict__ wraps,
    const unsigned* __restrict__ rows, const int* __restrict__ counts, const long long* __restrict__ offsets,
    int* __restrict__ src, int* __restrict__ dst, signed char* __restrict__ shift, float* __restrict__ vec) {
    // shift bytes and vector components of 32 edges are 96 consecutive bytes / floats of the output: staged in shared
    // memory and stored as unit-stride runs
    __shared__ float stage_vec[kThreads / 32][96];
    __shared__ signed char stage_shift[kThreads / 32][96];
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    float* my_vec = stage_vec[threadIdx.x >> 5];
    signed char* my_shift = stage_shift[threadIdx.x >> 5];
    const int p = warp * 32 + lane;
    if (warp * 32 >= n) return;
    int4 pi = make_int4(0, 0, 0, 0);
    int cnt = 0, wi = 0;
    if (p < n) {
        pi = pq[p];
        cnt = counts[p];
        wi = wraps[p];
    }
    const long long out0 = offsets[warp * 32];
    int prefix = cnt;
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, prefix, o);
        if (lane >= o) prefix += v;
    }
    const int total = __shfl_sync(0xffffffffu, prefix, 31);
    prefix -= cnt;
    const size_t slice = static_cast<size_t>(warp) * stride * 32;
    const double unit[3] = {g.box[0] / 4294967296.0, g.box[1] / 4294967296.0, g.box[2] / 4294967296.0};
    for (int t0 = 0; t0 < total; t0 += 32) {
        const int t = t0 + lane;
        const int c = owner_lane(min(t, total - 1), prefix);
        const int c_prefix = __shfl_sync(0xffffffffu, prefix, c);
        const int c_wraps = __shfl_sync(0xffffffffu, wi, c);
        const int ci[4] = {__shfl_sync(0xffffffffu, pi.x, c), __shfl_sync(0xffffffffu, pi.y, c),
                           __shfl_sync(0xffffffffu, pi.z, c), __shfl_sync(0xffffffffu, pi.w, c)};
        if (t < total) {
            const int k = t - c_prefix;
            const unsigned slot = rows[slice + static_cast<size_t>(k) * 32 + c];
            const int4 pj = __ldg(&pq[slot]);
            const int wj = __ldg(&wraps[slot]);
            const long long o = out0 + t;
            const int cj[3] = {pj.x, pj.y, pj.z};
#pragma unroll
            for (int a = 0; a < 3; ++a) {
                // the wrapped 32-bit difference is the minimum image; comparing it with the plain difference of the
                // wrapped coordinates tells which image of the neighbour that is
                const int nearest = static_cast<int>(static_cast<unsigned>(cj[a]) - static_cast<unsigned>(ci[a]));
                const long long plain = static_cast<long long>(static_cast<unsigned>(cj[a])) -
                                        static_cast<long long>(static_cast<unsigned>(ci[a]));
                const int image = static_cast<int>((static_cast<long long>(nearest) - plain) >> 32);
                my_shift[3 * lane + a] = static_cast<signed char>(image - (wrap_field(wj, a) - wrap_field(c_wraps, a)));
                my_vec[3 * lane + a] = static_cast<float>(static_cast<double>(nearest) * unit[a]);
            }
            src[o] = ci[3];
            dst[o] = pj.w;
        }
        __syncwarp();
        const int filled = 3 * min(32, total - t0);
        float* out_vec = vec + 3 * (out0 + t0);
        signed char* out_shift = shift + 3 * (out0 + t0);
        for (int q = lane; q < filled; q += 32) {
            out_vec[q] = my_vec[q];
            out_shift[q] = my_shift[q];
        }
        __syncwarp();
    }
}

// ---- periodic image atoms, their forces folded back, receiver marking (the work of MLIPStep::prepare / add_forces /
// virial around the edge build, src/MLIPStep.cu:214-432) ----------------------------------------------------------------
//
// Semantics (what parity depends on): on an axis with images, a position is first wrapped into [from, from + period);
// the image with lattice shift (sx, sy, sz) != 0, |s_a| <= reach[a], exists when p_a + s_a period_a lies inside
// [keep_lo, keep_hi] on every axis with images; the images of an atom are numbered in the order sx, sy, sz ascending and
// stored consecutively, atom after atom, behind the wrapped atoms.
//
// Along one axis the admissible shifts of an atom are a handful of values, found once and kept as a bit mask (bit
// s + reach). The images of an atom are then the product of three bit sets minus the origin, so their count is a product
// of population counts, and the k-th image is decoded from k by division - which lets the writing kernel run one thread
// per OUTPUT slot (unit-stride stores of every output array) instead of one thread per atom with scattered stores.
struct ImageLattice {
    double period[3], from[3], keep_lo[3], keep_hi[3];
    int reach[3];
};

constexpr int kMaskBits = 17;   // shifts -8 .. 8

__device__ __forceinline__ double image_coord(double p, int s, double period) {
    return __dadd_rn(p, __dmul_rn(static_cast<double>(s), period));   // no contraction: rounds as p + s * period
}

__device__ __forceinline__ double wrapped_coord(const ImageLattice& L, int a, double v) {
    return L.reach[a] > 0 ? v - L.period[a] * floor((v - L.from[a]) / L.period[a]) : v;
}

__device__ __forceinline__ unsigned axis_mask(const ImageLattice& L, int a, double p) {
    const int r = L.reach[a];
    if (r == 0) return 1u;
    unsigned m = 0;
    for (int s = -r; s <= r; ++s) {
        const double q = image_coord(p, s, L.period[a]);
        if (!(q < L.keep_lo[a] || q > L.keep_hi[a])) m |= 1u << (s + r);
    }
    return m;
}

__device__ __forceinline__ int nth_set_bit(unsigned mask, int n) {
    int b = 0;
    for (;; ++b)
        if ((mask >> b) & 1u) {
            if (n == 0) break;
            --n;
        }
    return b;
}

// Per atom: the three shift masks packed into one word, and how many images that makes.
__global__ void k_image_masks(ImageLattice L, int n, const double* __restrict__ x, const double* __restrict__ y,
                              const double* __restrict__ z, unsigned long long* __restrict__ masks,
                              long long* __restrict__ counts) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const unsigned mx = axis_mask(L, 0, wrapped_coord(L, 0, x[i]));
    const unsigned my = axis_mask(L, 1, wrapped_coord(L, 1, y[i]));
    const unsigned mz = axis_mask(L, 2, wrapped_coord(L, 2, z[i]));
    const bool self = ((mx >> L.reach[0]) & (my >> L.reach[1]) & (mz >> L.reach[2]) & 1u) != 0u;
    masks[i] = static_cast<unsigned long long>(mx) | (static_cast<unsigned long long>(my) << kMaskBits) |
               (static_cast<unsigned long long>(mz) << (2 * kMaskBits));
    counts[i] = static_cast<long long>(__popc(mx)) * __popc(my) * __popc(mz) - (self ? 1 : 0);
}

// One thread per output slot: slots [0, n) are the wrapped atoms, slot n + m is image number m of the whole system, which
// belongs to the last atom whose first image number is <= m.
__global__ void k_image_fill(ImageLattice L, int n, long long n_images, const double* __restrict__ x,
                             const double* __restrict__ y, const double* __restrict__ z, const int* __restrict__ type,
                             const unsigned long long* __restrict__ masks, const long long* __restrict__ first_image,
                             double* __restrict__ out_x, double* __restrict__ out_y, double* __restrict__ out_z,
                             int* __restrict__ out_type, int* __restrict__ out_owner, double* __restrict__ off_x,
                             double* __restrict__ off_y, double* __restrict__ off_z) {
    const long long t = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (t >= n + n_images) return;
    int owner;
    int s[3] = {0, 0, 0};
    if (t < n) {
        owner = static_cast<int>(t);
    } else {
        const long long m = t - n;
        int lo = 0, hi = n;   // first_image is non-decreasing; atoms without images repeat their successor's value
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (first_image[mid] <= m) lo = mid; else hi = mid;
        }
        owner = lo;
        const unsigned long long w = masks[owner];
        const unsigned field = (1u << kMaskBits) - 1u;
        const unsigned mx = static_cast<unsigned>(w) & field, my = static_cast<unsigned>(w >> kMaskBits) & field,
                       mz = static_cast<unsigned>(w >> (2 * kMaskBits)) & field;
        const int ny = __popc(my), nz = __popc(mz);
        int k = static_cast<int>(m - first_image[owner]);
        if ((mx >> L.reach[0]) & (my >> L.reach[1]) & (mz >> L.reach[2]) & 1u) {
            // the origin sits in the product too: images at or behind its rank move up by one
            const int rank = (__popc(mx & ((1u << L.reach[0]) - 1u)) * ny + __popc(my & ((1u << L.reach[1]) - 1u))) * nz +
                             __popc(mz & ((1u << L.reach[2]) - 1u));
            if (k >= rank) ++k;
        }
        s[0] = nth_set_bit(mx, k / (ny * nz)) - L.reach[0];
        s[1] = nth_set_bit(my, (k / nz) % ny) - L.reach[1];
        s[2] = nth_set_bit(mz, k % nz) - L.reach[2];
    }
    const double px = wrapped_coord(L, 0, x[owner]), py = wrapped_coord(L, 1, y[owner]), pz = wrapped_coord(L, 2, z[owner]);
    const double qx = s[0] ? image_coord(px, s[0], L.period[0]) : px;
    const double qy = s[1] ? image_coord(py, s[1], L.period[1]) : py;
    const double qz = s[2] ? image_coord(pz, s[2], L.period[2]) : pz;
    out_x[t] = qx; out_y[t] = qy; out_z[t] = qz;
    out_type[t] = type ? type[owner] : 0;
    out_owner[t] = owner;
    off_x[t] = qx - px; off_y[t] = qy - py; off_z[t] = qz - pz;
}

// target[i] += f[i] + the forces on the images of atom i, added in slot order (MLIPStep::add_forces,
// src/MLIPStep.cu:108-124, 373-381), for the first n_out of the n atoms. with_images == 0: the images were edge shifts,
// not atoms the model saw, and carry no force.
__global__ void k_image_fold(int n_out, int n, int with_images, const double* __restrict__ fx,
                             const double* __restrict__ fy, const double* __restrict__ fz,
                             const long long* __restrict__ first_image, const long long* __restrict__ counts,
                             double* __restrict__ tx, double* __restrict__ ty, double* __restrict__ tz) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_out) return;
    double sx = fx[i], sy = fy[i], sz = fz[i];
    if (with_images) {
        const long long begin = n + first_image[i], end = begin + counts[i];
        for (long long k = begin; k < end; ++k) {
            sx += fx[k];
            sy += fy[k];
            sz += fz[k];
        }
    }
    tx[i] += sx;
    ty[i] += sy;
    tz[i] += sz;
}

// Sum over atoms of r . F and of its three diagonal terms (MLIPStep::virial / virial_diag, src/MLIPStep.cu:126-148,
// 383-432): per-block sums in a fixed order, then one block adds the blocks' sums in a fixed order.
__global__ void k_virial_partials(long long n, const double* __restrict__ x, const double* __restrict__ y,
                                  const double* __restrict__ z, const double* __restrict__ fx,
                                  const double* __restrict__ fy, const double* __restrict__ fz,
                                  double* __restrict__ partials) {
    __shared__ double sh[kThreads / 32][3];
    double v[3] = {0.0, 0.0, 0.0};
    for (long long p = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; p < n;
         p += static_cast<long long>(gridDim.x) * blockDim.x) {
        v[0] += x[p] * fx[p];
        v[1] += y[p] * fy[p];
        v[2] += z[p] * fz[p];
    }
    for (int a = 0; a < 3; ++a)
        for (int o = 16; o > 0; o >>= 1) v[a] += __shfl_down_sync(0xffffffffu, v[a], o);
    if ((threadIdx.x & 31) == 0)
        for (int a = 0; a < 3; ++a) sh[threadIdx.x >> 5][a] = v[a];
    __syncthreads();
    if (threadIdx.x < 3) {
        double sum = 0.0;
        for (int w = 0; w < kThreads / 32; ++w) sum += sh[w][threadIdx.x];
        partials[3 * blockIdx.x + threadIdx.x] = sum;
    }
}

__global__ void k_virial_total(int n_blocks, const double* __restrict__ partials, double* __restrict__ out) {
    if (threadIdx.x < 3) {
        double sum = 0.0;
        for (int b = 0; b < n_blocks; ++b) sum += partials[3 * b + threadIdx.x];
        out[1 + threadIdx.x] = sum;
    }
    __syncthreads();
    if (threadIdx.x == 0) out[0] = out[1] + out[2] + out[3];
}

__global__ void k_mark_receivers(int n, const double* __restrict__ x, const double* __restrict__ y,
                                 const double* __restrict__ z, double lx, double ly, double lz, double hx, double hy,
                                 double hz, double reach2, unsigned char* __restrict__ ok) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const double dx = fmax(fmax(lx - x[i], x[i] - hx), 0.0);
    const double dy = fmax(fmax(ly - y[i], y[i] - hy), 0.0);
    const double dz = fmax(fmax(lz - z[i], z[i] - hz), 0.0);
    const double d2 = __dadd_rn(__dadd_rn(__dmul_rn(dx, dx), __dmul_rn(dy, dy)), __dmul_rn(dz, dz));
    ok[i] = d2 <= reach2 ? 1 : 0;   // a NaN position gives 0
}

template <class T>
bool grow(T*& ptr, size_t& capacity, size_t needed) {
    if (needed <= capacity) return true;
    const size_t grown = std::max(needed, capacity + capacity / 2);
    if (ptr) cudaFree(ptr);
    ptr = nullptr;
    capacity = 0;
    if (cudaMalloc(&ptr, grown * sizeof(T)) != cudaSuccess) return false;
    capacity = grown;
    return true;
}

}  // namespace

struct dsmd_edges {
    int device = 0;
    std::string error;
    unsigned* key[2] = {nullptr, nullptr};  size_t cap_key[2] = {0, 0};
    int* val[2] = {nullptr, nullptr};       size_t cap_val[2] = {0, 0};
    int4* pq = nullptr;                     size_t cap_pq = 0;
    int* wraps = nullptr;                   size_t cap_wraps = 0;     // per sorted slot, periodic form
    int* cell_start = nullptr;              size_t cap_cells = 0;
    unsigned* rows = nullptr;               size_t cap_rows = 0;
    int* counts = nullptr;                  size_t cap_counts = 0;
    long long* offsets = nullptr;           size_t cap_offsets = 0;
    unsigned char* temp = nullptr;          size_t cap_temp = 0;
    long long* edges = nullptr;             size_t cap_edges = 0;
    double* shift = nullptr;                size_t cap_shift = 0;
    int* c_src = nullptr;                   size_t cap_csrc = 0;
    int* c_dst = nullptr;                   size_t cap_cdst = 0;
    signed char* c_shift = nullptr;         size_t cap_cshift = 0;
    float* c_vec = nullptr;                 size_t cap_cvec = 0;
    // image atoms
    long long* img_counts = nullptr;        size_t cap_img_counts = 0;
    long long* img_offsets = nullptr;       size_t cap_img_offsets = 0;
    unsigned long long* img_masks = nullptr; size_t cap_img_masks = 0;
    int64_t n_img_src = 0;                  // atoms the last image build was given
    double* virial_partials = nullptr;      // [3 * kVirialBlocks] + 4 results
    double* h_virial = nullptr;             // pinned, 4 doubles
    double* ext[6] = {};                    size_t cap_ext[6] = {};     // x y z shift_x shift_y shift_z
    int* ext_type = nullptr;                size_t cap_ext_type = 0;
    int* ext_owner = nullptr;               size_t cap_ext_owner = 0;
    int64_t n_ext = 0;
    double* bounds = nullptr;               // 6 doubles for the device-side bounding box
    EdgeStatus* d_status = nullptr;
    EdgeStatus* h_status = nullptr;
    int stride = 0;
    int64_t n_edges = 0;
    bool have_shift = false;
    int64_t launches = 0;
};

namespace {

int efail(dsmd_edges* e, int code, const std::string& what) {
    e->error = what;
    return code;
}

#define EDGE_CUDA(e, call)                                                            \
    do {                                                                              \
        cudaError_t err_ = (call);                                                    \
        if (err_ != cudaSuccess) {                                                    \
            (e)->error = std::string(#call) + ": " + cudaGetErrorString(err_);        \
            return DSMD_ERR_CUDA;                                                     \
        }                                                                             \
    } while (0)

#define EDGE_ALLOC(e, ok)                                                             \
    do {                                                                              \
        if (!(ok)) return efail(e, DSMD_ERR_CUDA, "device allocation failed");        \
    } while (0)

// Grid over [lo, hi] (non-periodic) or [0, box) (periodic): cells at least cutoff / stencil wide, not more than about
// two cells per atom (a sparse box must not allocate a huge grid: src/EdgeBuilder.cu:50-61).
int edge_grid(dsmd_edges* e, Grid& g, const double lo[3], const double hi[3], bool periodic, double cutoff, int64_t n) {
    double max_scale = 0.0;
    double len[3];
    for (int a = 0; a < 3; ++a) {
        g.box[a] = periodic ? hi[a] : 0.0;
        if (periodic) {
            len[a] = hi[a];
            g.wrap[a] = 1;
            g.org[a] = 0.0;
            g.scale[a] = static_cast<float>(len[a] / 4294967296.0);
            max_scale = std::max(max_scale, len[a] / 4294967296.0);
        } else {
            // the upper face belongs to the box: stretch the mapped range by a hair so that hi maps below 1
            len[a] = std::max(hi[a] - lo[a], cutoff) * (1.0 + 1e-9);
            g.wrap[a] = 0;
            g.org[a] = lo[a];
            g.scale[a] = static_cast<float>(len[a] / 2147483648.0);
            max_scale = std::max(max_scale, len[a] / 2147483648.0);
        }
        g.inv_len[a] = 1.0 / len[a];
    }
    const long long max_cells = std::max<long long>(64, 2 * static_cast<long long>(n));
    // Half-width cells (25 cell rows around an atom) pay when a row holds a few atoms; in a sparse system the cost of
    // opening a row outweighs the tighter windows and 9 rows of full-width cells are faster (measured on 1,000,000
    // atoms at 0.05 / A^3, cutoff 5 A, 0.8 atoms per half-width cell: 0.79 ms against 0.89 ms per build).
    const double per_half_cell = static_cast<double>(n) / (len[0] * len[1] * len[2]) * (cutoff * cutoff * cutoff / 8.0);
    bool done = false;
    for (int stencil = per_half_cell >= 1.0 ? 2 : 1; stencil >= 1 && !done; --stencil) {
        double width = cutoff / stencil * (1.0 + 1e-6);
        for (int tries = 0; tries < 64; ++tries) {
            long long cells = 1;
            bool ok = true;
            for (int a = 0; a < 3; ++a) {
                int nc = std::max(1, static_cast<int>(std::floor(len[a] / width)));
                nc = std::min(nc, 1024);
                if (periodic && nc < 2 * stencil + 1) ok = false;
                g.nc[a] = nc;
                cells *= nc;
            }
            if (!ok) break;                       // box too small for this stencil: try the wider cells
            if (cells <= max_cells || stencil == 1) {
                if (cells > max_cells) { width *= 1.26; continue; }
                g.stencil = stencil;
                g.ncells = static_cast<int>(cells);
                done = true;
                break;
            }
            break;                                // too many half-width cells: fall back to full-width cells
        }
    }
    if (!done) return efail(e, DSMD_ERR_BOX_TOO_SMALL, "periodic box shorter than three cells of width cutoff");
    // finer cells along x: a cell row is a contiguous run of slots whatever the x cell width, and the search window
    // (rounded outwards to whole cells) is tighter
    g.x_reach = static_cast<float>(g.stencil * (len[0] / g.nc[0]) * 0.9999999);
    for (int refine = 4; refine > 1; refine >>= 1) {
        if (static_cast<long long>(g.nc[0]) * refine <= 4096 &&
            static_cast<long long>(g.ncells) * refine <= 4 * max_cells) {
            g.nc[0] *= refine;
            g.ncells *= refine;
            break;
        }
    }
    g.r2_list = static_cast<float>(cutoff * cutoff);
    g.r2_list_d = cutoff * cutoff;
    g.band = static_cast<float>(8.0 * cutoff * max_scale + 16.0 * cutoff * cutoff * 5.9604645e-8);
    double max_len = 0.0;
    for (int a = 0; a < 3; ++a) {
        g.cellw[a] = static_cast<float>(len[a] / g.nc[a]);
        max_len = std::max(max_len, len[a]);
    }
    g.r_pad = static_cast<float>(cutoff * (1.0 + 1e-4) + 8.0 * max_len * 1.2e-7);
    return DSMD_OK;
}

// bin, sort, gather, search (with row-overflow retry), scan; leaves the edge count in h_status.
template <bool PERIODIC>
int edge_search(dsmd_edges* e, const Grid& g, const double* d_x, const double* d_y, const double* d_z, int64_t n,
                int64_t n_centers, const int* d_owner, const unsigned char* d_ok, int row, double density_hint,
                cudaStream_t s) {
    const size_t un = static_cast<size_t>(n);
    for (int k = 0; k < 2; ++k) {
        EDGE_ALLOC(e, grow(e->key[k], e->cap_key[k], un));
        EDGE_ALLOC(e, grow(e->val[k], e->cap_val[k], un));
    }
    EDGE_ALLOC(e, grow(e->pq, e->cap_pq, un));
    if (PERIODIC) EDGE_ALLOC(e, grow(e->wraps, e->cap_wraps, un));
    EDGE_ALLOC(e, grow(e->cell_start, e->cap_cells, static_cast<size_t>(g.ncells) + 1));
    EDGE_ALLOC(e, grow(e->counts, e->cap_counts, un));
    EDGE_ALLOC(e, grow(e->offsets, e->cap_offsets, un));
    int bits = 1;
    while ((1ll << bits) < g.ncells) ++bits;
    size_t sort_bytes = 0, scan_bytes = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, sort_bytes, e->key[0], e->key[1], e->val[0], e->val[1], static_cast<int>(n),
                                    0, bits, s);
    cub::DeviceScan::ExclusiveSum(nullptr, scan_bytes, e->counts, e->offsets, static_cast<int>(n), s);
    EDGE_ALLOC(e, grow(e->temp, e->cap_temp, std::max(sort_bytes, scan_bytes)));

    EDGE_CUDA(e, cudaMemsetAsync(e->d_status, 0, sizeof(EdgeStatus), s));
    k_edge_keys<<<blocks_for(n, kThreads), kThreads, 0, s>>>(g, static_cast<int>(n), d_x, d_y, d_z, e->key[0], e->val[0],
                                                            e->d_status);
    EDGE_CUDA(e, cub::DeviceRadixSort::SortPairs(e->temp, sort_bytes, e->key[0], e->key[1], e->val[0], e->val[1],
                                                 static_cast<int>(n), 0, bits, s));
    k_edge_gather<<<blocks_for(n, kThreads), kThreads, 0, s>>>(g, static_cast<int>(n), e->key[1], e->val[1], d_x, d_y,
                                                              d_z, e->pq, PERIODIC ? e->wraps : nullptr, e->cell_start);
    k_edge_cell_tail<<<blocks_for(g.ncells + 1, kThreads), kThreads, 0, s>>>(e->key[1], static_cast<int>(n), g.ncells + 1,
                                                                           e->cell_start);
    e->launches += 3;
    if (e->stride == 0) {
        const double expect = density_hint * 4.18879020479 * g.r2_list_d * std::sqrt(g.r2_list_d);
        e->stride = (std::max(16, static_cast<int>(expect * 1.5) + 16) + 3) & ~3;
    }
    for (int attempt = 0; attempt < 5; ++attempt) {
        const size_t slices = (un + 31) / 32;
        EDGE_ALLOC(e, grow(e->rows, e->cap_rows, slices * static_cast<size_t>(e->stride) * 32));
        SearchArgs a{static_cast<int>(n), static_cast<int>(n_centers), e->stride, row, e->pq, d_x, d_y, d_z,
                     e->cell_start, d_owner, d_ok, e->rows, e->counts, e->d_status};
        k_edge_search<PERIODIC><<<blocks_for(n, kSearchThreads), kSearchThreads, 0, s>>>(g, a);
        ++e->launches;
        EDGE_CUDA(e, cub::DeviceScan::ExclusiveSum(e->temp, scan_bytes, e->counts, e->offsets, static_cast<int>(n), s));
        k_edge_total<<<1, 1, 0, s>>>(static_cast<int>(n), e->offsets, e->counts, e->d_status);
        ++e->launches;
        EDGE_CUDA(e, cudaGetLastError());
        // the one synchronisation of a build that does not overflow: edge count, bounds flag, row overflow
        EDGE_CUDA(e, cudaMemcpyAsync(e->h_status, e->d_status, sizeof(EdgeStatus), cudaMemcpyDeviceToHost, s));
        EDGE_CUDA(e, cudaStreamSynchronize(s));
        if (e->h_status->out_of_bounds)
            return efail(e, DSMD_ERR_OUT_OF_DOMAIN, "an atom lies outside the given box (or has a NaN position)");
        if (e->h_status->need_stride <= static_cast<unsigned>(e->stride)) return DSMD_OK;
        e->stride = (static_cast<int>(e->h_status->need_stride * 1.2) + 8 + 3) & ~3;
        EDGE_CUDA(e, cudaMemsetAsync(e->d_status, 0, sizeof(EdgeStatus), s));
    }
    return efail(e, DSMD_ERR_CAPACITY, "edge rows kept overflowing");
}

}  // namespace

extern "C" {

int dsmd_edges_create(int device, dsmd_edges** out) {
    if (!out) return DSMD_ERR_INVALID;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) return DSMD_ERR_CUDA;
    dsmd_edges* e = new dsmd_edges();
    e->device = device;
    *out = e;
    EDGE_CUDA(e, cudaSetDevice(device));
    EDGE_CUDA(e, cudaMalloc(&e->d_status, sizeof(EdgeStatus)));
    EDGE_CUDA(e, cudaMallocHost(&e->h_status, sizeof(EdgeStatus)));
    EDGE_CUDA(e, cudaMalloc(&e->bounds, sizeof(double) * 6));
    return DSMD_OK;
}

void dsmd_edges_destroy(dsmd_edges* e) {
    if (!e) return;
    cudaSetDevice(e->device);
    for (int k = 0; k < 2; ++k) { cudaFree(e->key[k]); cudaFree(e->val[k]); }
    cudaFree(e->pq); cudaFree(e->wraps); cudaFree(e->cell_start); cudaFree(e->rows); cudaFree(e->counts);
    cudaFree(e->offsets); cudaFree(e->temp); cudaFree(e->edges); cudaFree(e->shift); cudaFree(e->c_src);
    cudaFree(e->c_dst); cudaFree(e->c_shift); cudaFree(e->c_vec); cudaFree(e->bounds); cudaFree(e->d_status);
    cudaFree(e->img_counts); cudaFree(e->img_offsets); cudaFree(e->img_masks); cudaFree(e->virial_partials);
    if (e->h_virial) cudaFreeHost(e->h_virial);
    cudaFree(e->ext_type); cudaFree(e->ext_owner);
    for (int k = 0; k < 6; ++k) cudaFree(e->ext[k]);
    cudaFreeHost(e->h_status);
    delete e;
}

const char* dsmd_edges_last_error(const dsmd_edges* e) { return e ? e->error.c_str() : "null edge builder"; }

int dsmd_edges_build(dsmd_edges* e, const double* d_x, const double* d_y, const double* d_z, int64_t n, double cutoff,
                     const double* lo, const double* hi, int64_t n_centers, const int32_t* d_owner,
                     const double* d_shift_x, const double* d_shift_y, const double* d_shift_z,
                     const unsigned char* d_receiver_ok, int row, int64_t* n_edges, void* stream) {
    if (!e || !n_edges) return DSMD_ERR_INVALID;
    *n_edges = 0;
    e->n_edges = 0;
    e->have_shift = false;
    if (!(cutoff > 0.0)) return efail(e, DSMD_ERR_INVALID, "cutoff must be positive");
    if (n < 0 || n >= std::numeric_limits<int32_t>::max() / 2) return efail(e, DSMD_ERR_INVALID, "atom count out of range");
    const bool images = d_owner != nullptr;
    if (images && (n_centers < 0 || n_centers > n || !d_shift_x || !d_shift_y || !d_shift_z))
        return efail(e, DSMD_ERR_INVALID, "invalid periodic image description");
    if (!images) n_centers = n;
    if (d_receiver_ok && row != 0 && row != 1) return efail(e, DSMD_ERR_INVALID, "invalid prune description");
    if (n <= 1) return DSMD_OK;
    if (!d_x || !d_y || !d_z) return DSMD_ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    EDGE_CUDA(e, cudaSetDevice(e->device));

    double box_lo[3], box_hi[3];
    if (lo && hi) {
        for (int a = 0; a < 3; ++a) { box_lo[a] = lo[a]; box_hi[a] = hi[a]; }
    } else {   // bounding box on the device: one extra synchronisation
        const double* axes[3] = {d_x, d_y, d_z};
        size_t need = 0;
        cub::DeviceReduce::Min(nullptr, need, d_x, e->bounds, static_cast<int>(n), s);
        EDGE_ALLOC(e, grow(e->temp, e->cap_temp, need));
        for (int a = 0; a < 3; ++a) {
            EDGE_CUDA(e, cub::DeviceReduce::Min(e->temp, need, axes[a], e->bounds + a, static_cast<int>(n), s));
            EDGE_CUDA(e, cub::DeviceReduce::Max(e->temp, need, axes[a], e->bounds + 3 + a, static_cast<int>(n), s));
        }
        double h[6];
        EDGE_CUDA(e, cudaMemcpyAsync(h, e->bounds, sizeof(h), cudaMemcpyDeviceToHost, s));
        EDGE_CUDA(e, cudaStreamSynchronize(s));
        for (int a = 0; a < 3; ++a) { box_lo[a] = h[a]; box_hi[a] = h[3 + a]; }
    }
    for (int a = 0; a < 3; ++a)
        if (!(box_lo[a] <= box_hi[a]) || !std::isfinite(box_lo[a]) || !std::isfinite(box_hi[a]))
            return efail(e, DSMD_ERR_OUT_OF_DOMAIN, "invalid box or a non-finite position");

    Grid g{};
    { const int rc = edge_grid(e, g, box_lo, box_hi, false, cutoff, n); if (rc) return rc; }
    double volume = 1.0;
    for (int a = 0; a < 3; ++a) volume *= 1.0 / g.inv_len[a];
    { const int rc = edge_search<false>(e, g, d_x, d_y, d_z, n, n_centers, d_owner, d_receiver_ok, row,
                                        static_cast<double>(n) / volume, s); if (rc) return rc; }
    const int64_t E = e->h_status->edges;
    e->n_edges = E;
    *n_edges = E;
    if (E == 0) return DSMD_OK;
    EDGE_ALLOC(e, grow(e->edges, e->cap_edges, 2 * static_cast<size_t>(E)));
    if (images) EDGE_ALLOC(e, grow(e->shift, e->cap_shift, 3 * static_cast<size_t>(E)));
    k_edge_fill<<<blocks_for(n, kThreads), kThreads, 0, s>>>(static_cast<int>(n), E, e->stride, e->pq, e->rows, e->counts,
                                                            e->offsets, static_cast<int>(n_centers), d_owner, d_shift_x,
                                                            d_shift_y, d_shift_z, e->edges, images ? e->shift : nullptr);
    ++e->launches;
    EDGE_CUDA(e, cudaGetLastError());
    e->have_shift = images;
    return DSMD_OK;
}

int dsmd_edges_result(const dsmd_edges* e, const int64_t** d_edge_index, const double** d_edge_shift, int64_t* n_edges) {
    if (!e) return DSMD_ERR_INVALID;
    if (d_edge_index) *d_edge_index = reinterpret_cast<const int64_t*>(e->edges);
    if (d_edge_shift) *d_edge_shift = e->have_shift ? e->shift : nullptr;
    if (n_edges) *n_edges = e->n_edges;
    return DSMD_OK;
}

int dsmd_edges_build_periodic(dsmd_edges* e, const double* d_x, const double* d_y, const double* d_z, int64_t n,
                              const double box[3], double cutoff, int64_t* n_edges, void* stream) {
    if (!e || !n_edges || !box) return DSMD_ERR_INVALID;
    *n_edges = 0;
    e->n_edges = 0;
    if (!(cutoff > 0.0)) return efail(e, DSMD_ERR_INVALID, "cutoff must be positive");
    if (n < 0 || n >= std::numeric_limits<int32_t>::max() / 2) return efail(e, DSMD_ERR_INVALID, "atom count out of range");
    for (int a = 0; a < 3; ++a)
        if (!(box[a] > 2.0 * cutoff)) return efail(e, DSMD_ERR_BOX_TOO_SMALL, "box must be longer than two cutoffs");
    if (n <= 1) return DSMD_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    EDGE_CUDA(e, cudaSetDevice(e->device));
    Grid g{};
    const double zero[3] = {0.0, 0.0, 0.0};
    { const int rc = edge_grid(e, g, zero, box, true, cutoff, n); if (rc) return rc; }
    const double volume = box[0] * box[1] * box[2];
    { const int rc = edge_search<true>(e, g, d_x, d_y, d_z, n, n, nullptr, nullptr, 1, static_cast<double>(n) / volume, s);
      if (rc) return rc; }
    const int64_t E = e->h_status->edges;
    e->n_edges = E;
    *n_edges = E;
    if (E == 0) return DSMD_OK;
    EDGE_ALLOC(e, grow(e->c_src, e->cap_csrc, static_cast<size_t>(E)));
    EDGE_ALLOC(e, grow(e->c_dst, e->cap_cdst, static_cast<size_t>(E)));
    EDGE_ALLOC(e, grow(e->c_shift, e->cap_cshift, 3 * static_cast<size_t>(E)));
    EDGE_ALLOC(e, grow(e->c_vec, e->cap_cvec, 3 * static_cast<size_t>(E)));
    {
        k_edge_fill_compact<<<blocks_for(n, kThreads), kThreads, 0, s>>>(g, static_cast<int>(n), e->stride, e->pq, e->wraps,
                                                                         e->rows, e->counts, e->offsets, e->c_src, e->c_dst,
                                                                         e->c_shift, e->c_vec);
    }
    ++e->launches;
    EDGE_CUDA(e, cudaGetLastError());
    return DSMD_OK;
}

int dsmd_images_build(dsmd_edges* e, const double* d_x, const double* d_y, const double* d_z, const int32_t* d_type,
                      int64_t n, const double box[3], const double origin[3], const double region_lo[3],
                      const double region_hi[3], const int shells[3], int64_t* n_all, void* stream) {
    if (!e || !n_all || !box || !origin || !region_lo || !region_hi || !shells) return DSMD_ERR_INVALID;
    *n_all = 0;
    e->n_ext = 0;
    if (n < 0 || n >= std::numeric_limits<int32_t>::max() / 2) return efail(e, DSMD_ERR_INVALID, "atom count out of range");
    if (n == 0) return DSMD_OK;
    if (!d_x || !d_y || !d_z) return DSMD_ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    EDGE_CUDA(e, cudaSetDevice(e->device));
    ImageLattice lattice;
    for (int a = 0; a < 3; ++a) {
        if (shells[a] < 0 || shells[a] > 8) return efail(e, DSMD_ERR_INVALID, "image shells must be in 0 .. 8");
        if (shells[a] > 0 && !(box[a] > 0.0)) return efail(e, DSMD_ERR_INVALID, "box length must be positive on an image axis");
        lattice.period[a] = box[a];
        lattice.from[a] = origin[a];
        lattice.keep_lo[a] = region_lo[a];
        lattice.keep_hi[a] = region_hi[a];
        lattice.reach[a] = shells[a];
    }
    const size_t un = static_cast<size_t>(n);
    EDGE_ALLOC(e, grow(e->img_counts, e->cap_img_counts, un));
    EDGE_ALLOC(e, grow(e->img_offsets, e->cap_img_offsets, un));
    EDGE_ALLOC(e, grow(e->img_masks, e->cap_img_masks, un));
    size_t scan_bytes = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, scan_bytes, e->img_counts, e->img_offsets, static_cast<int>(n), s);
    EDGE_ALLOC(e, grow(e->temp, e->cap_temp, scan_bytes));
    k_image_masks<<<blocks_for(n, kThreads), kThreads, 0, s>>>(lattice, static_cast<int>(n), d_x, d_y, d_z, e->img_masks,
                                                              e->img_counts);
    EDGE_CUDA(e, cub::DeviceScan::ExclusiveSum(e->temp, scan_bytes, e->img_counts, e->img_offsets, static_cast<int>(n), s));
    // the image count comes to the host: the one synchronisation (MLIPStep::prepare does the same, src/MLIPStep.cu:254-255)
    long long last[2] = {0, 0};
    EDGE_CUDA(e, cudaMemcpyAsync(&last[0], e->img_offsets + (n - 1), sizeof(long long), cudaMemcpyDeviceToHost, s));
    EDGE_CUDA(e, cudaMemcpyAsync(&last[1], e->img_counts + (n - 1), sizeof(long long), cudaMemcpyDeviceToHost, s));
    EDGE_CUDA(e, cudaStreamSynchronize(s));
    const int64_t n_images = last[0] + last[1];
    const int64_t total = n + n_images;
    if (total >= std::numeric_limits<int32_t>::max() / 2) return efail(e, DSMD_ERR_CAPACITY, "too many image atoms");
    for (int k = 0; k < 6; ++k) EDGE_ALLOC(e, grow(e->ext[k], e->cap_ext[k], static_cast<size_t>(total)));
    EDGE_ALLOC(e, grow(e->ext_type, e->cap_ext_type, static_cast<size_t>(total)));
    EDGE_ALLOC(e, grow(e->ext_owner, e->cap_ext_owner, static_cast<size_t>(total)));
    k_image_fill<<<blocks_for(total, kThreads), kThreads, 0, s>>>(lattice, static_cast<int>(n), n_images, d_x, d_y, d_z, d_type,
                                                                 e->img_masks, e->img_offsets, e->ext[0], e->ext[1], e->ext[2],
                                                                 e->ext_type, e->ext_owner, e->ext[3], e->ext[4], e->ext[5]);
    e->launches += 2;
    EDGE_CUDA(e, cudaGetLastError());
    e->n_ext = total;
    e->n_img_src = n;
    *n_all = total;
    return DSMD_OK;
}

int dsmd_images_fold_forces(dsmd_edges* e, const double* d_fx, const double* d_fy, const double* d_fz, int64_t n_out,
                            int with_images, double* d_tx, double* d_ty, double* d_tz, void* stream) {
    if (!e || !d_fx || !d_fy || !d_fz || !d_tx || !d_ty || !d_tz) return DSMD_ERR_INVALID;
    if (e->n_img_src <= 0) return efail(e, DSMD_ERR_STATE, "no image atoms built");
    if (n_out < 0 || n_out > e->n_img_src) n_out = e->n_img_src;
    if (n_out == 0) return DSMD_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    k_image_fold<<<blocks_for(n_out, kThreads), kThreads, 0, s>>>(static_cast<int>(n_out), static_cast<int>(e->n_img_src),
                                                                 with_images, d_fx, d_fy, d_fz, e->img_offsets, e->img_counts,
                                                                 d_tx, d_ty, d_tz);
    ++e->launches;
    EDGE_CUDA(e, cudaGetLastError());
    return DSMD_OK;
}

int dsmd_virial_from_forces(dsmd_edges* e, const double* d_x, const double* d_y, const double* d_z, const double* d_fx,
                            const double* d_fy, const double* d_fz, int64_t n, double out[4], void* stream) {
    if (!e || !out || n < 0 || (n > 0 && (!d_x || !d_y || !d_z || !d_fx || !d_fy || !d_fz))) return DSMD_ERR_INVALID;
    out[0] = out[1] = out[2] = out[3] = 0.0;
    if (n == 0) return DSMD_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    EDGE_CUDA(e, cudaSetDevice(e->device));
    constexpr int kVirialBlocks = 592;   // 4 per SM of a B200: a fixed grid keeps the order of the sum the same for every n
    if (!e->virial_partials) {
        EDGE_CUDA(e, cudaMalloc(&e->virial_partials, sizeof(double) * (3 * kVirialBlocks + 4)));
        EDGE_CUDA(e, cudaMallocHost(&e->h_virial, sizeof(double) * 4));
    }
    const int blocks = static_cast<int>(std::min<int64_t>(kVirialBlocks, (n + kThreads - 1) / kThreads));
    k_virial_partials<<<blocks, kThreads, 0, s>>>(n, d_x, d_y, d_z, d_fx, d_fy, d_fz, e->virial_partials);
    k_virial_total<<<1, 32, 0, s>>>(blocks, e->virial_partials, e->virial_partials + 3 * kVirialBlocks);
    e->launches += 2;
    EDGE_CUDA(e, cudaGetLastError());
    EDGE_CUDA(e, cudaMemcpyAsync(e->h_virial, e->virial_partials + 3 * kVirialBlocks, sizeof(double) * 4,
                                 cudaMemcpyDeviceToHost, s));
    EDGE_CUDA(e, cudaStreamSynchronize(s));
    for (int k = 0; k < 4; ++k) out[k] = e->h_virial[k];
    return DSMD_OK;
}

int dsmd_images_result(const dsmd_edges* e, const double** d_x, const double** d_y, const double** d_z,
                       const int32_t** d_type, const int32_t** d_owner, const double** d_shift_x, const double** d_shift_y,
                       const double** d_shift_z, int64_t* n_all) {
    if (!e) return DSMD_ERR_INVALID;
    if (d_x) *d_x = e->ext[0];
    if (d_y) *d_y = e->ext[1];
    if (d_z) *d_z = e->ext[2];
    if (d_type) *d_type = e->ext_type;
    if (d_owner) *d_owner = e->ext_owner;
    if (d_shift_x) *d_shift_x = e->ext[3];
    if (d_shift_y) *d_shift_y = e->ext[4];
    if (d_shift_z) *d_shift_z = e->ext[5];
    if (n_all) *n_all = e->n_ext;
    return DSMD_OK;
}

int dsmd_mark_receivers(dsmd_edges* e, const double* d_x, const double* d_y, const double* d_z, int64_t n,
                        const double lo[3], const double hi[3], double reach, unsigned char* d_ok, void* stream) {
    if (!e || !lo || !hi || n < 0 || (n > 0 && (!d_x || !d_y || !d_z || !d_ok))) return DSMD_ERR_INVALID;
    if (n == 0) return DSMD_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    k_mark_receivers<<<blocks_for(n, kThreads), kThreads, 0, s>>>(static_cast<int>(n), d_x, d_y, d_z, lo[0], lo[1], lo[2],
                                                                 hi[0], hi[1], hi[2], reach * reach, d_ok);
    ++e->launches;
    EDGE_CUDA(e, cudaGetLastError());
    return DSMD_OK;
}

int dsmd_edges_result_compact(const dsmd_edges* e, const int32_t** d_src, const int32_t** d_dst, const int8_t** d_shift,
                              const float** d_vec, int64_t* n_edges) {
    if (!e) return DSMD_ERR_INVALID;
    if (d_src) *d_src = e->c_src;
    if (d_dst) *d_dst = e->c_dst;
    if (d_shift) *d_shift = reinterpret_cast<const int8_t*>(e->c_shift);
    if (d_vec) *d_vec = e->c_vec;
    if (n_edges) *n_edges = e->n_edges;
    return DSMD_OK;
}

}  // extern "C"
