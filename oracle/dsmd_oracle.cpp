// CPU oracle for the short-range nonbonded path. TEST INFRASTRUCTURE ONLY: nothing under the shipped package links,
// imports or calls this file; only the test-suite, the smoke check and the benchmark's cpu_baseline leg do.
//
// It restates, in plain fp64 C++ with no vector intrinsics and FMA contraction switched off, what the reference computes
// on this path. Each function names the reference lines it follows (paths relative to the reference tree):
//
//   pair set            src/neighbor_list_cpu.cpp:220-859   (SpatialVerletList::build: r^2 < (rc+skin)^2, owned centre,
//                                                           ghost-ghost pairs never listed, one entry per pair)
//   minimum image       include/md_types.h:55-91            (all periodic axes for an owned partner, only the unsplit axes
//                                                           for a ghost, which already carries its image shift)
//   LJ pair             src/force_calculator_cpu.cpp:81-98  (c6/c12 form, optional CHARMM switch on r^2)
//   LJ coefficients     src/force_calculator_cpu.cpp:468-485 (c6 = 4 eps sig^6, c12 = c6 sig^6)
//   real-space Ewald    src/force_calculator_cpu.cpp:41-79, 2165-2199 (linear table in r^2, spacing 0.04, first node 1e-4;
//                                                           erfc table for ordinary pairs, erf table for excluded ones)
//   alpha               src/pme_reciprocal_engine.cpp:17-24 (bisection of erfc(alpha rc) = 1e-5)
//   pair bookkeeping    src/force_calculator_cpu.cpp:1760-1891 (r^2 < rc^2 and r^2 >= 1e-10; force on owned atoms only;
//                                                           energy/virial by the owned-partner-or-smaller-global-id rule)
//   cubic Ewald table   include/ewald_real_table.h:31-122   (float-bit indexed piecewise cubics; what the device evaluates)
//   radius-graph edges  src/EdgeBuilder.cu:116-192          (ordered pairs, strict <, no minimum image, images, pruning)
//   periodic images     src/MLIPStep.cu:31-52,73-103        (wrap from lo, shells, fixed emission order)
//   image force fold    src/MLIPStep.cu:108-148             (forces of images added to their atoms in slot order; r.F sums)
//   receiver marking    src/MLIPStep.cu:150-161
//   ghost selection     src/md_system.cpp:855-891           (geometric rule only: every periodic image of an atom that
//                                                           lies within the halo width of the brick, edges and corners
//                                                           included; the library that does it in the reference is not
//                                                           in its tree)
//   velocity Verlet     src/integrator_kernels.cu:14-102
//
// Parity status: pinned against the reference's own CPU code compiled in this repository's oracle/_ref build (pair sets
// bit-exact, forces to 1e-12) and against committed fixtures produced by it. The reference ships no golden vector of its
// own for this path.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

struct Cells {
    int n[3];
    double lo[3], inv[3];
    std::vector<int> start, order;
    int coord(double v, int a) const {
        int c = static_cast<int>(std::floor((v - lo[a]) * inv[a]));
        return std::min(std::max(c, 0), n[a] - 1);
    }
};

// Bins points into a grid over [lo, hi] whose cells are at least `width` wide on every axis.
void bin_points(long n, const double* x, const double* y, const double* z, const double lo[3], const double hi[3],
                double width, Cells& g) {
    const double* p[3] = {x, y, z};
    long cells = 1;
    for (int a = 0; a < 3; ++a) {
        const double ext = std::max(hi[a] - lo[a], width);
        g.n[a] = std::max(1, std::min(256, static_cast<int>(std::floor(ext / width))));
        g.lo[a] = lo[a];
        g.inv[a] = g.n[a] / ext;
        cells *= g.n[a];
    }
    std::vector<int> cell(n);
    g.start.assign(cells + 1, 0);
    for (long i = 0; i < n; ++i) {
        const int c = g.coord(p[0][i], 0) + g.n[0] * (g.coord(p[1][i], 1) + g.n[1] * g.coord(p[2][i], 2));
        cell[i] = c;
        ++g.start[c + 1];
    }
    for (long c = 0; c < cells; ++c) g.start[c + 1] += g.start[c];
    g.order.resize(n);
    std::vector<int> cur(g.start.begin(), g.start.end() - 1);
    for (long i = 0; i < n; ++i) g.order[cur[cell[i]]++] = static_cast<int>(i);
}

inline double min_image(double d, double L) { return d - L * std::nearbyint(d / L); }

struct BoxRule {
    double L[3];
    bool wrap_owned[3];   // minimum image applied when the partner is owned (or there is no subdomain)
    bool wrap_ghost[3];   // minimum image applied when the partner is a ghost
};

BoxRule make_rule(const double L[3], const int periodic[3], const int split[3]) {
    BoxRule r;
    const bool sub = split[0] || split[1] || split[2];
    for (int a = 0; a < 3; ++a) {
        r.L[a] = L[a];
        r.wrap_owned[a] = periodic[a] != 0;
        r.wrap_ghost[a] = periodic[a] != 0 && (!sub || !split[a]);
    }
    return r;
}

inline void displacement(const BoxRule& r, bool partner_owned, double& dx, double& dy, double& dz) {
    const bool* w = partner_owned ? r.wrap_owned : r.wrap_ghost;
    if (w[0]) dx = min_image(dx, r.L[0]);
    if (w[1]) dy = min_image(dy, r.L[1]);
    if (w[2]) dz = min_image(dz, r.L[2]);
}

bool excluded_pair(const std::uint64_t* keys, long n_keys, int ga, int gb) {
    if (n_keys == 0) return false;
    const std::uint64_t lo = static_cast<std::uint64_t>(std::min(ga, gb)), hi = static_cast<std::uint64_t>(std::max(ga, gb));
    const std::uint64_t key = (lo << 32) | hi;
    return std::binary_search(keys, keys + n_keys, key);
}

}  // namespace

extern "C" {

int dsmd_oracle_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// ---- pair set -----------------------------------------------------------------------------------------------------
// Every pair (i owned, j) with r^2 < R^2, once: owned-owned pairs with i < j, owned-ghost pairs from the owned side.
// Positions of owned atoms must lie within one box length of the primary cell. Returns the pair count and writes at
// most `capacity` pairs, ordered by (i, j).
long dsmd_oracle_pairs(long n_total, long n_local, const double* x, const double* y, const double* z, const double L[3],
                       const int periodic[3], const int split[3], double R, int* out_i, int* out_j, long capacity) {
    const BoxRule rule = make_rule(L, periodic, split);
    const double R2 = R * R;
    // Bin wrapped copies so a periodic neighbour is found through wrapped cell indices.
    std::vector<double> wx(n_total), wy(n_total), wz(n_total);
    double lo[3] = {1e300, 1e300, 1e300}, hi[3] = {-1e300, -1e300, -1e300};
    const double* src[3] = {x, y, z};
    double* dst[3] = {wx.data(), wy.data(), wz.data()};
    for (int a = 0; a < 3; ++a) {
        for (long i = 0; i < n_total; ++i) {
            double v = src[a][i];
            if (rule.wrap_ghost[a]) v -= L[a] * std::floor(v / L[a]);   // axis resolved by minimum image for everyone
            dst[a][i] = v;
            lo[a] = std::min(lo[a], v);
            hi[a] = std::max(hi[a], v);
        }
        if (rule.wrap_ghost[a]) { lo[a] = 0.0; hi[a] = L[a]; }
    }
    Cells g;
    bin_points(n_total, wx.data(), wy.data(), wz.data(), lo, hi, R, g);
    std::vector<std::vector<int>> rows(n_local);
#pragma omp parallel for schedule(dynamic, 64)
    for (long i = 0; i < n_local; ++i) {
        const int ci[3] = {g.coord(wx[i], 0), g.coord(wy[i], 1), g.coord(wz[i], 2)};
        std::vector<int>& row = rows[i];
        int seen[27];
        int n_seen = 0;
        for (int dz = -1; dz <= 1; ++dz) for (int dy = -1; dy <= 1; ++dy) for (int dx = -1; dx <= 1; ++dx) {
            int c[3] = {ci[0] + dx, ci[1] + dy, ci[2] + dz};
            bool ok = true;
            for (int a = 0; a < 3; ++a) {
                if (c[a] < 0 || c[a] >= g.n[a]) {
                    if (rule.wrap_ghost[a]) c[a] = (c[a] + g.n[a]) % g.n[a]; else ok = false;
                }
            }
            if (!ok) continue;
            const int cell = c[0] + g.n[0] * (c[1] + g.n[1] * c[2]);
            bool dup = false;
            for (int k = 0; k < n_seen; ++k) dup = dup || seen[k] == cell;
            if (dup) continue;
            seen[n_seen++] = cell;
            for (int q = g.start[cell]; q < g.start[cell + 1]; ++q) {
                const int j = g.order[q];
                if (j == i) continue;
                const bool j_owned = j < n_local;
                if (j_owned && j < i) continue;
                double ddx = x[i] - x[j], ddy = y[i] - y[j], ddz = z[i] - z[j];
                displacement(rule, j_owned, ddx, ddy, ddz);
                if (ddx * ddx + ddy * ddy + ddz * ddz < R2) row.push_back(j);
            }
        }
        std::sort(row.begin(), row.end());
    }
    long count = 0;
    for (long i = 0; i < n_local; ++i) {
        for (int j : rows[i]) {
            if (count < capacity) { out_i[count] = static_cast<int>(i); out_j[count] = j; }
            ++count;
        }
    }
    return count;
}

// ---- Ewald helpers ------------------------------------------------------------------------------------------------

double dsmd_oracle_ewald_alpha(double cutoff) {
    double lo = 1e-4, hi = 10.0 / cutoff;
    for (int it = 0; it < 100; ++it) {
        const double mid = 0.5 * (lo + hi);
        if (std::erfc(mid * cutoff) > 1e-5) lo = mid; else hi = mid;
    }
    return 0.5 * (lo + hi);
}

// ---- forces -------------------------------------------------------------------------------------------------------
// Evaluates the listed pairs. c6/c12: [ntypes*ntypes]. ewald_mode: 0 = the reference CPU's linear table, 1 = exact erfc.
// exclusion keys: sorted (min gid << 32 | max gid). scalars = {PE, W, Wxx, Wyy, Wzz, pairs inside rc}.
int dsmd_oracle_forces(long n_total, long n_local, const double* x, const double* y, const double* z, const double* charge,
                       const int* type, const int* gid, const double L[3], const int periodic[3], const int split[3],
                       long n_pairs, const int* pair_i, const int* pair_j, int ntypes, const double* c6,
                       const double* c12, double rc, double switch_distance, int do_lj, int do_coulomb, double alpha,
                       int ewald_mode, long n_keys, const std::uint64_t* keys, double* fx, double* fy, double* fz,
                       double* scalars) {
    (void)n_total;
    const BoxRule rule = make_rule(L, periodic, split);
    const double rc2 = rc * rc;
    const bool switching = do_lj && switch_distance > 0.0;
    const double rs2 = switching ? switch_distance * switch_distance : 0.0;
    const double inv_denom = switching ? 1.0 / ((rc2 - rs2) * (rc2 - rs2) * (rc2 - rs2)) : 0.0;
    const double kc = 332.0636;
    const double two_a_sqrtpi = 1.1283791670955126 * alpha;

    // The reference CPU tables: nodes at r2_min + k * spacing, energy and force factor interleaved.
    const double t_min = 1e-4, t_h = 0.04;
    std::vector<double> tab, tab_x;
    if (do_coulomb && ewald_mode == 0) {
        const int n = static_cast<int>(std::ceil((rc2 - t_min) / t_h)) + 3;
        tab.resize(2 * n);
        tab_x.resize(2 * n);
        for (int k = 0; k < n; ++k) {
            const double r2 = t_min + k * t_h, r = std::sqrt(r2), zed = alpha * r, ex = std::exp(-zed * zed);
            tab[2 * k] = std::erfc(zed) / r;
            tab[2 * k + 1] = std::erfc(zed) / (r2 * r) + two_a_sqrtpi * ex / r2;
            tab_x[2 * k] = -std::erf(zed) / r;
            tab_x[2 * k + 1] = -(std::erf(zed) / (r2 * r) - two_a_sqrtpi * ex / r2);
        }
    }

    for (long i = 0; i < n_local; ++i) fx[i] = fy[i] = fz[i] = 0.0;
    double pe = 0.0, w = 0.0, wd[3] = {0.0, 0.0, 0.0};
    long inside = 0;
    for (long p = 0; p < n_pairs; ++p) {
        const int i = pair_i[p], j = pair_j[p];
        const bool j_owned = j < n_local;
        double dx = x[i] - x[j], dy = y[i] - y[j], dz = z[i] - z[j];
        displacement(rule, j_owned, dx, dy, dz);
        const double r2 = dx * dx + dy * dy + dz * dz;
        if (r2 >= rc2 || r2 < 1e-10) continue;
        ++inside;
        const int gi = gid ? gid[i] : i, gj = gid ? gid[j] : j;
        const bool excl = excluded_pair(keys, n_keys, gi, gj);
        const bool owner = j_owned || gi < gj;
        double fmag = 0.0, e = 0.0;
        if (do_lj && !excl) {
            const int t = (type ? type[i] : 0) * ntypes + (type ? type[j] : 0);
            const double r2inv = 1.0 / r2, r6inv = r2inv * r2inv * r2inv;
            const double att = c6[t] * r6inv, rep = c12[t] * r6inv * r6inv;
            double f = r2inv * (12.0 * rep - 6.0 * att), u = rep - att;
            if (switching && r2 > rs2) {
                const double a = rc2 - r2, b = rc2 + 2.0 * r2 - 3.0 * rs2;
                const double sw = a * a * b * inv_denom;
                f = sw * f + 12.0 * u * a * (r2 - rs2) * inv_denom;
                u *= sw;
            }
            fmag += f;
            e += u;
        }
        if (do_coulomb) {
            const double qq = kc * charge[i] * charge[j];
            double ef, ff;
            if (ewald_mode == 0) {
                double idx_f = (r2 - t_min) * (1.0 / t_h);
                if (idx_f < 0.0) idx_f = 0.0;
                const int idx = static_cast<int>(idx_f);
                const double frac = idx_f - idx;
                const double* node = (excl ? tab_x.data() : tab.data()) + 2 * idx;
                ef = node[0] + frac * (node[2] - node[0]);
                ff = node[1] + frac * (node[3] - node[1]);
            } else {
                const double r = std::sqrt(r2), zed = alpha * r, ex = std::exp(-zed * zed);
                if (excl) {
                    ef = -std::erf(zed) / r;
                    ff = -(std::erf(zed) / (r2 * r) - two_a_sqrtpi * ex / r2);
                } else {
                    ef = std::erfc(zed) / r;
                    ff = std::erfc(zed) / (r2 * r) + two_a_sqrtpi * ex / r2;
                }
            }
            fmag += qq * ff;
            e += qq * ef;
        }
        fx[i] += fmag * dx; fy[i] += fmag * dy; fz[i] += fmag * dz;
        if (j_owned) { fx[j] -= fmag * dx; fy[j] -= fmag * dy; fz[j] -= fmag * dz; }
        if (owner) {
            pe += e;
            w += r2 * fmag;
            wd[0] += fmag * dx * dx; wd[1] += fmag * dy * dy; wd[2] += fmag * dz * dz;
        }
    }
    scalars[0] = pe; scalars[1] = w; scalars[2] = wd[0]; scalars[3] = wd[1]; scalars[4] = wd[2];
    scalars[5] = static_cast<double>(inside);
    return 0;
}

// ---- the float-bit indexed cubic Ewald table (what the device kernel evaluates) -------------------------------------
// Intervals: 32 per octave of r^2 starting at r^2 = 0.5; four coefficients per interval, fitted through the four
// Chebyshev nodes of the interval. Returns the interval count for cutoff_sq (0 coefficients written when coef == null).
int dsmd_oracle_cubic_table(double alpha, double cutoff_sq, float* force_coef, float* energy_coef) {
    const int bits = 5, e0 = -1, max_oct = 16;
    const int top = static_cast<int>(std::ceil(std::log2(std::max(cutoff_sq, 1.0))));
    const int octaves = std::min(std::max(top - e0, 1), max_oct);
    const int intervals = octaves << bits;
    if (!force_coef || !energy_coef) return intervals;
    const double pi = 3.14159265358979323846;
    const double pref = 2.0 * alpha / std::sqrt(pi);
    double nodes[4];
    for (int k = 0; k < 4; ++k) nodes[k] = 0.5 - 0.5 * std::cos((2.0 * k + 1.0) * pi / 8.0);
    for (int iv = 0; iv < intervals; ++iv) {
        const double base = std::ldexp(1.0, e0 + iv / (1 << bits));
        const double begin = base * (1.0 + static_cast<double>(iv % (1 << bits)) / (1 << bits));
        const double width = base / (1 << bits);
        for (int which = 0; which < 2; ++which) {
            long double m[4][5];
            for (int row = 0; row < 4; ++row) {
                const double r2 = begin + nodes[row] * width, r = std::sqrt(r2);
                const double ev = std::erfc(alpha * r) / r;
                const double fv = (ev + pref * std::exp(-alpha * alpha * r2)) / r2;
                long double pw = 1.0L;
                for (int col = 0; col < 4; ++col) { m[row][col] = pw; pw *= nodes[row]; }
                m[row][4] = which == 0 ? fv : ev;
            }
            for (int col = 0; col < 4; ++col) {          // Gauss-Jordan with partial pivoting
                int piv = col;
                for (int row = col + 1; row < 4; ++row)
                    if (std::fabs(static_cast<double>(m[row][col])) > std::fabs(static_cast<double>(m[piv][col]))) piv = row;
                for (int k = 0; k < 5; ++k) std::swap(m[col][k], m[piv][k]);
                for (int row = 0; row < 4; ++row) {
                    if (row == col) continue;
                    const long double f = m[row][col] / m[col][col];
                    for (int k = col; k < 5; ++k) m[row][k] -= f * m[col][k];
                }
            }
            float* out = (which == 0 ? force_coef : energy_coef) + 4 * iv;
            for (int col = 0; col < 4; ++col) out[col] = static_cast<float>(static_cast<double>(m[col][4] / m[col][col]));
        }
    }
    return intervals;
}

// Float evaluation of one table with the device's arithmetic. Returns 0 when r2 is outside the table.
int dsmd_oracle_cubic_eval(const float* coef, int intervals, float r2, float* value) {
    std::uint32_t b;
    std::memcpy(&b, &r2, 4);
    const std::uint32_t shifted = b - (static_cast<std::uint32_t>(127 - 1) << 23);
    const std::uint32_t index = shifted >> (23 - 5);
    if (index >= static_cast<std::uint32_t>(intervals)) return 0;
    const std::uint32_t fb = 0x3F800000u | ((shifted << 5) & 0x007FFFFFu);
    float t;
    std::memcpy(&t, &fb, 4);
    t -= 1.0f;
    const float* c = coef + 4 * index;
    *value = ((c[3] * t + c[2]) * t + c[1]) * t + c[0];
    return 1;
}

// ---- radius-graph edges ---------------------------------------------------------------------------------------------
// All ordered pairs (i, j), i != j, |r_j - r_i| < cutoff, no minimum image. With owner != null the atoms from n_centers on
// are copies: they are never centres, row 1 holds owner[j] and shift = shift_xyz[j]. With ok != null an edge is kept only
// when its receiver (row 0: the centre, row 1: the neighbour's node) has ok != 0. Ordered by (i, found atom j).
long dsmd_oracle_edges(long n, const double* x, const double* y, const double* z, double cutoff, long n_centers,
                       const int* owner, const double* shift_x, const double* shift_y, const double* shift_z,
                       const unsigned char* ok, int row, long long* out_i, long long* out_j, double* out_shift,
                       long capacity) {
    if (n <= 1) return 0;
    double lo[3] = {1e300, 1e300, 1e300}, hi[3] = {-1e300, -1e300, -1e300};
    const double* p[3] = {x, y, z};
    for (int a = 0; a < 3; ++a)
        for (long i = 0; i < n; ++i) { lo[a] = std::min(lo[a], p[a][i]); hi[a] = std::max(hi[a], p[a][i]); }
    Cells g;
    bin_points(n, x, y, z, lo, hi, cutoff, g);
    const double c2 = cutoff * cutoff;
    std::vector<std::vector<int>> rows(n_centers);
#pragma omp parallel for schedule(dynamic, 64)
    for (long i = 0; i < n_centers; ++i) {
        if (ok && row == 0 && !ok[i]) continue;
        const int ci[3] = {g.coord(x[i], 0), g.coord(y[i], 1), g.coord(z[i], 2)};
        for (int cz = std::max(ci[2] - 1, 0); cz <= std::min(ci[2] + 1, g.n[2] - 1); ++cz)
            for (int cy = std::max(ci[1] - 1, 0); cy <= std::min(ci[1] + 1, g.n[1] - 1); ++cy)
                for (int cx = std::max(ci[0] - 1, 0); cx <= std::min(ci[0] + 1, g.n[0] - 1); ++cx) {
                    const int cell = cx + g.n[0] * (cy + g.n[1] * cz);
                    for (int q = g.start[cell]; q < g.start[cell + 1]; ++q) {
                        const int j = g.order[q];
                        if (j == i) continue;
                        const double dx = x[j] - x[i], dy = y[j] - y[i], dz = z[j] - z[i];
                        if (!(dx * dx + dy * dy + dz * dz < c2)) continue;
                        if (ok && row == 1 && !ok[owner ? owner[j] : j]) continue;
                        rows[i].push_back(j);
                    }
                }
        std::sort(rows[i].begin(), rows[i].end());
    }
    long count = 0;
    for (long i = 0; i < n_centers; ++i) {
        for (int j : rows[i]) {
            if (count < capacity) {
                out_i[count] = i;
                out_j[count] = owner ? owner[j] : j;
                if (out_shift) {
                    out_shift[3 * count] = owner ? shift_x[j] : 0.0;
                    out_shift[3 * count + 1] = owner ? shift_y[j] : 0.0;
                    out_shift[3 * count + 2] = owner ? shift_z[j] : 0.0;
                }
            }
            ++count;
        }
    }
    return count;
}

// Periodic images of n atoms for the axes with shells > 0: positions are wrapped from origin first; image (sx, sy, sz) != 0
// is kept when it lies inside [region_lo, region_hi] on every image axis; emission order sx, sy, sz ascending per atom,
// atoms in index order. Output arrays hold the n wrapped atoms followed by the images. Returns the total atom count.
long dsmd_oracle_images(long n, const double* x, const double* y, const double* z, const double box[3],
                        const double origin[3], const double region_lo[3], const double region_hi[3], const int shells[3],
                        double* ex, double* ey, double* ez, int* eowner, double* esx, double* esy, double* esz,
                        long capacity) {
    auto wrap = [&](double v, int a) { return shells[a] > 0 ? v - box[a] * std::floor((v - origin[a]) / box[a]) : v; };
    long total = n;
    for (long i = 0; i < n; ++i) {
        const double px = wrap(x[i], 0), py = wrap(y[i], 1), pz = wrap(z[i], 2);
        if (i < capacity) {
            ex[i] = px; ey[i] = py; ez[i] = pz;
            eowner[i] = static_cast<int>(i);
            esx[i] = esy[i] = esz[i] = 0.0;
        }
        for (int sx = -shells[0]; sx <= shells[0]; ++sx) {
            const double qx = px + sx * box[0];
            if (shells[0] > 0 && (qx < region_lo[0] || qx > region_hi[0])) continue;
            for (int sy = -shells[1]; sy <= shells[1]; ++sy) {
                const double qy = py + sy * box[1];
                if (shells[1] > 0 && (qy < region_lo[1] || qy > region_hi[1])) continue;
                for (int sz = -shells[2]; sz <= shells[2]; ++sz) {
                    if (sx == 0 && sy == 0 && sz == 0) continue;
                    const double qz = pz + sz * box[2];
                    if (shells[2] > 0 && (qz < region_lo[2] || qz > region_hi[2])) continue;
                    if (total < capacity) {
                        ex[total] = qx; ey[total] = qy; ez[total] = qz;
                        eowner[total] = static_cast<int>(i);
                        esx[total] = qx - px; esy[total] = qy - py; esz[total] = qz - pz;
                    }
                    ++total;
                }
            }
        }
    }
    return total;
}

// Forces of image atoms folded back onto the atoms they copy (src/MLIPStep.cu:108-124): target[i] += f[i] + the forces on
// the slots n + first[i] .. n + first[i] + count[i] - 1, added in that order, for i < n_out. count == null: f[i] alone.
void dsmd_oracle_fold_image_forces(long n_out, long n, const double* fx, const double* fy, const double* fz,
                                   const long* first, const long* count, double* tx, double* ty, double* tz) {
    for (long i = 0; i < n_out; ++i) {
        double ax = fx[i], ay = fy[i], az = fz[i];
        if (count)
            for (long k = 0; k < count[i]; ++k) {
                ax += fx[n + first[i] + k];
                ay += fy[n + first[i] + k];
                az += fz[n + first[i] + k];
            }
        tx[i] += ax;
        ty[i] += ay;
        tz[i] += az;
    }
}

// out = {sum r.F, sum x Fx, sum y Fy, sum z Fz} over n atoms (src/MLIPStep.cu:126-148), long double accumulators so that
// the comparison is against the exact sum rather than against one summation order.
void dsmd_oracle_virial_from_forces(long n, const double* x, const double* y, const double* z, const double* fx,
                                    const double* fy, const double* fz, double out[4]) {
    long double s[3] = {0.0L, 0.0L, 0.0L};
    for (long p = 0; p < n; ++p) {
        s[0] += static_cast<long double>(x[p]) * fx[p];
        s[1] += static_cast<long double>(y[p]) * fy[p];
        s[2] += static_cast<long double>(z[p]) * fz[p];
    }
    out[0] = static_cast<double>(s[0] + s[1] + s[2]);
    out[1] = static_cast<double>(s[0]);
    out[2] = static_cast<double>(s[1]);
    out[3] = static_cast<double>(s[2]);
}

// ok[i] = atom i lies within `reach` (Euclidean distance to the box [lo, hi]) of the box.
void dsmd_oracle_mark_receivers(long n, const double* x, const double* y, const double* z, const double lo[3],
                                const double hi[3], double reach, unsigned char* ok) {
    const double* p[3] = {x, y, z};
    for (long i = 0; i < n; ++i) {
        double d2 = 0.0;
        for (int a = 0; a < 3; ++a) {
            const double d = std::fmax(std::fmax(lo[a] - p[a][i], p[a][i] - hi[a]), 0.0);
            d2 += d * d;
        }
        ok[i] = d2 <= reach * reach ? 1 : 0;
    }
}

// ---- ghost selection ------------------------------------------------------------------------------------------------
// Brick grid dims[3] over the periodic box [0, L); brick `coords`. A ghost is a periodic image (shift s[a] in {-1, 0, 1}
// box lengths, non-zero only on split periodic axes) of an atom, lying inside [lo - h, hi + h) on every split axis (on an
// unsplit axis every atom qualifies and no shift is applied), and not itself an owned atom of the brick. Positions must be
// wrapped into [0, L). Writes (source atom index, image shift per axis), ordered by (source, sx, sy, sz).
long dsmd_oracle_ghosts(long n, const double* x, const double* y, const double* z, const double L[3], const int periodic[3],
                        const int dims[3], const int coords[3], double h, int* out_src, int* out_image, long capacity) {
    double lo[3], hi[3];
    bool split[3];
    for (int a = 0; a < 3; ++a) {
        split[a] = dims[a] > 1;
        lo[a] = L[a] * coords[a] / dims[a];
        hi[a] = L[a] * (coords[a] + 1) / dims[a];
    }
    const double* p[3] = {x, y, z};
    long count = 0;
    for (long i = 0; i < n; ++i) {
        int s_lo[3], s_hi[3];
        for (int a = 0; a < 3; ++a) {
            const bool images = split[a] && periodic[a];
            s_lo[a] = images ? -1 : 0;
            s_hi[a] = images ? 1 : 0;
        }
        for (int sx = s_lo[0]; sx <= s_hi[0]; ++sx) for (int sy = s_lo[1]; sy <= s_hi[1]; ++sy)
            for (int sz = s_lo[2]; sz <= s_hi[2]; ++sz) {
                const int s[3] = {sx, sy, sz};
                bool inside_halo = true, inside_brick = true;
                for (int a = 0; a < 3; ++a) {
                    if (!split[a]) continue;
                    const double q = p[a][i] + s[a] * L[a];
                    if (!(q >= lo[a] - h && q < hi[a] + h)) inside_halo = false;
                    if (!(q >= lo[a] && q < hi[a])) inside_brick = false;
                }
                if (!inside_halo) continue;
                if (inside_brick && sx == 0 && sy == 0 && sz == 0) continue;   // the owned atom itself
                if (count < capacity) {
                    out_src[count] = static_cast<int>(i);
                    out_image[3 * count] = sx; out_image[3 * count + 1] = sy; out_image[3 * count + 2] = sz;
                }
                ++count;
            }
    }
    return count;
}

// ---- integrator -------------------------------------------------------------------------------------------------------
// The two halves of velocity Verlet: v += 0.5 dt f / m * force_to_accel; (first half only) x += dt v.
void dsmd_oracle_vv_half(long n, double dt, double force_to_accel, int first_half, double* x, double* y, double* z,
                         double* vx, double* vy, double* vz, const double* fx, const double* fy, const double* fz,
                         const double* mass) {
    for (long i = 0; i < n; ++i) {
        const double s = 0.5 * dt * force_to_accel / mass[i];
        vx[i] += s * fx[i]; vy[i] += s * fy[i]; vz[i] += s * fz[i];
        if (first_half) { x[i] += dt * vx[i]; y[i] += dt * vy[i]; z[i] += dt * vz[i]; }
    }
}

// ---- distance constraints -----------------------------------------------------------------------------------------------
// SHAKE (positions) and RATTLE (velocities) as the reference's CPU solver does them (src/constraint_solver.cpp:15-146):
// Gauss-Seidel sweeps over the constraint list until every constraint holds to the tolerance; a constraint already inside
// the tolerance is left alone in a sweep. Minimum image per periodic axis by one box length (|d| > L / 2).
namespace {
inline void min_image(double d[3], const double L[3], const int periodic[3]) {
    for (int a = 0; a < 3; ++a)
        if (periodic[a]) {
            if (d[a] > 0.5 * L[a]) d[a] -= L[a];
            else if (d[a] < -0.5 * L[a]) d[a] += L[a];
        }
}
}  // namespace

// SHAKE: moves the atoms of every constraint (i, j, distance) along the bond vector the pair had BEFORE the drift
// (pre_x, pre_y, pre_z) until |r_ij|^2 is within `tolerance` (relative) of distance^2; the velocities take the
// displacement over dt. Returns 1 when converged within max_iterations sweeps.
int dsmd_oracle_shake(long n_constraints, const long* atom1, const long* atom2, const double* distance, double* x, double* y,
                      double* z, double* vx, double* vy, double* vz, const double* mass, const double* pre_x,
                      const double* pre_y, const double* pre_z, const double L[3], const int periodic[3], double dt,
                      int max_iterations, double tolerance) {
    if (n_constraints == 0) return 1;
    const double inv_dt = 1.0 / dt;
    for (int sweep = 0; sweep < max_iterations; ++sweep) {
        double worst = 0.0;
        for (long c = 0; c < n_constraints; ++c) {
            const long i = atom1[c], j = atom2[c];
            const double target2 = distance[c] * distance[c];
            double d[3] = {x[i] - x[j], y[i] - y[j], z[i] - z[j]};
            min_image(d, L, periodic);
            const double excess = (d[0] * d[0] + d[1] * d[1] + d[2] * d[2]) - target2;
            const double relative = std::fabs(excess) / target2;
            worst = std::max(worst, relative);
            if (relative < tolerance) continue;
            double o[3] = {pre_x[i] - pre_x[j], pre_y[i] - pre_y[j], pre_z[i] - pre_z[j]};
            min_image(o, L, periodic);
            const double along = o[0] * d[0] + o[1] * d[1] + o[2] * d[2];
            if (std::fabs(along) < 1e-12) continue;   // degenerate geometry: try again in the next sweep
            const double wi = 1.0 / mass[i], wj = 1.0 / mass[j];
            const double g = excess / (2.0 * (wi + wj) * along);
            const double cx = g * o[0], cy = g * o[1], cz = g * o[2];
            x[i] -= cx * wi; y[i] -= cy * wi; z[i] -= cz * wi;
            x[j] += cx * wj; y[j] += cy * wj; z[j] += cz * wj;
            vx[i] -= cx * wi * inv_dt; vy[i] -= cy * wi * inv_dt; vz[i] -= cz * wi * inv_dt;
            vx[j] += cx * wj * inv_dt; vy[j] += cy * wj * inv_dt; vz[j] += cz * wj * inv_dt;
        }
        if (worst < tolerance) return 1;
    }
    return 0;
}

// RATTLE: removes the relative velocity along every constrained bond (|r_ij . v_ij| below `tolerance`, absolute).
// virial_diag (may be null): diagonal of the constraint virial, -2 / (force_to_accel dt) * sum over corrections of
// k r_a^2, counted for a pair when the atom with the lower global id is owned (index < n_local).
int dsmd_oracle_rattle(long n_constraints, const long* atom1, const long* atom2, const double* x, const double* y,
                       const double* z, double* vx, double* vy, double* vz, const double* mass, const int* gid, long n_local,
                       const double L[3], const int periodic[3], double dt, double force_to_accel, int max_iterations,
                       double tolerance, double* virial_diag) {
    double w[3] = {0.0, 0.0, 0.0};
    int converged = n_constraints == 0 ? 1 : 0;
    const double prefactor = -2.0 / (force_to_accel * dt);
    for (int sweep = 0; sweep < max_iterations && !converged; ++sweep) {
        double worst = 0.0;
        for (long c = 0; c < n_constraints; ++c) {
            const long i = atom1[c], j = atom2[c];
            double d[3] = {x[i] - x[j], y[i] - y[j], z[i] - z[j]};
            min_image(d, L, periodic);
            const double r2 = d[0] * d[0] + d[1] * d[1] + d[2] * d[2];
            if (r2 < 1e-20) continue;
            const double along = d[0] * (vx[i] - vx[j]) + d[1] * (vy[i] - vy[j]) + d[2] * (vz[i] - vz[j]);
            worst = std::max(worst, std::fabs(along));
            if (std::fabs(along) < tolerance) continue;
            const double wi = 1.0 / mass[i], wj = 1.0 / mass[j];
            const double k = along / ((wi + wj) * r2);
            vx[i] -= k * wi * d[0]; vy[i] -= k * wi * d[1]; vz[i] -= k * wi * d[2];
            vx[j] += k * wj * d[0]; vy[j] += k * wj * d[1]; vz[j] += k * wj * d[2];
            const long lower = (gid ? gid[i] < gid[j] : i < j) ? i : j;
            if (lower < n_local)
                for (int a = 0; a < 3; ++a) w[a] += prefactor * k * d[a] * d[a];
        }
        if (worst < tolerance) converged = 1;
    }
    if (virial_diag)
        for (int a = 0; a < 3; ++a) virial_diag[a] = w[a];
    return converged;
}

// ---- bonded terms and scaled special pairs ------------------------------------------------------------------------------
// Restates ForceCalculatorCPU::compute_bond_forces / compute_angle_forces / compute_torsion_forces /
// compute_special_pair_forces (src/force_calculator_cpu.cpp:2437-2895), with the ownership rule of the reference's GPU
// kernels (src/force_calculator_cuda.cu:2703-3170): a term is evaluated when at least one of its atoms is owned
// (index < n_local), forces go to owned atoms only, energy and virial are counted where the atom with the lowest global
// id is owned. Minimum image per displacement on the periodic axes (one wrap, include/md_types.h:57-70).
//
//   bonds      U = k/2 (r - r0)^2                                 (k, r0)
//   angles     U = k/2 (theta - theta0)^2, theta at atom 2        (k, theta0 in radians)
//   torsions   n > 0: U = k (1 + cos(n phi - phi0));  n = 0: U = k (phi - phi0)^2 with the difference wrapped to
//              (-pi, pi]  (dihedrals and impropers alike)         (k, phi0 in radians, n)
//   specials   scaled 12-6 LJ (4 eps ((s/r)^12 - (s/r)^6) lj_scale) + plain Coulomb 332.0636 qi qj / r coulomb_scale
//
// Forces are ADDED to fx, fy, fz. out = {PE, W, Wxx, Wyy, Wzz}: bonds and specials contribute to W and the diagonal,
// angles and torsions to the diagonal only (their trace is zero).
namespace {
inline bool owns_term(const long* atoms, int count, const int* gid, long n_local) {
    long lowest = atoms[0];
    for (int k = 1; k < count; ++k)
        if ((gid ? gid[atoms[k]] < gid[lowest] : atoms[k] < lowest)) lowest = atoms[k];
    return lowest < n_local;
}
inline bool any_local(const long* atoms, int count, long n_local) {
    for (int k = 0; k < count; ++k)
        if (atoms[k] < n_local) return true;
    return false;
}
inline void add_force(double* fx, double* fy, double* fz, long i, long n_local, double x, double y, double z) {
    if (i < n_local) { fx[i] += x; fy[i] += y; fz[i] += z; }
}
}  // namespace

void dsmd_oracle_bonded(long n_local, const double* x, const double* y, const double* z, const int* gid, const double L[3],
                        const int periodic[3],
                        long n_bonds, const long* bond_atoms, const double* bond_k, const double* bond_r0,
                        long n_angles, const long* angle_atoms, const double* angle_k, const double* angle_theta0,
                        long n_torsions, const long* torsion_atoms, const double* torsion_k, const double* torsion_phi0,
                        const int* torsion_n,
                        long n_specials, const long* special_atoms, const double* special_sigma,
                        const double* special_epsilon, const double* special_lj_scale, const double* special_coulomb_scale,
                        const double* charge, double* fx, double* fy, double* fz, double out[5]) {
    double pe = 0.0, w = 0.0, wd[3] = {0.0, 0.0, 0.0};
    for (long b = 0; b < n_bonds; ++b) {
        const long* a = bond_atoms + 2 * b;
        if (!any_local(a, 2, n_local)) continue;
        double d[3] = {x[a[0]] - x[a[1]], y[a[0]] - y[a[1]], z[a[0]] - z[a[1]]};
        min_image(d, L, periodic);
        const double r = std::sqrt(d[0] * d[0] + d[1] * d[1] + d[2] * d[2]);
        if (r < 1e-10) continue;
        const double dr = r - bond_r0[b];
        const double fm = -bond_k[b] * dr / r;
        add_force(fx, fy, fz, a[0], n_local, fm * d[0], fm * d[1], fm * d[2]);
        add_force(fx, fy, fz, a[1], n_local, -fm * d[0], -fm * d[1], -fm * d[2]);
        if (owns_term(a, 2, gid, n_local)) {
            pe += 0.5 * bond_k[b] * dr * dr;
            w += fm * (d[0] * d[0] + d[1] * d[1] + d[2] * d[2]);
            for (int c = 0; c < 3; ++c) wd[c] += fm * d[c] * d[c];
        }
    }
    for (long t = 0; t < n_angles; ++t) {
        const long* a = angle_atoms + 3 * t;
        if (!any_local(a, 3, n_local)) continue;
        double u[3] = {x[a[0]] - x[a[1]], y[a[0]] - y[a[1]], z[a[0]] - z[a[1]]};
        double v[3] = {x[a[2]] - x[a[1]], y[a[2]] - y[a[1]], z[a[2]] - z[a[1]]};
        min_image(u, L, periodic);
        min_image(v, L, periodic);
        const double ru = std::sqrt(u[0] * u[0] + u[1] * u[1] + u[2] * u[2]);
        const double rv = std::sqrt(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]);
        if (ru < 1e-10 || rv < 1e-10) continue;
        double c = (u[0] * v[0] + u[1] * v[1] + u[2] * v[2]) / (ru * rv);
        c = std::min(1.0, std::max(-1.0, c));
        const double dtheta = std::acos(c) - angle_theta0[t];
        const bool owner = owns_term(a, 3, gid, n_local);
        if (owner) pe += 0.5 * angle_k[t] * dtheta * dtheta;
        if (std::fabs(dtheta) < 1e-10) continue;
        const double sine = std::sqrt(1.0 - c * c);
        if (sine < 1e-10) continue;
        const double fc = angle_k[t] * dtheta / sine;
        double fi[3], fk[3];
        for (int q = 0; q < 3; ++q) {
            fi[q] = fc * (v[q] / (ru * rv) - u[q] * c / (ru * ru));
            fk[q] = fc * (u[q] / (ru * rv) - v[q] * c / (rv * rv));
        }
        add_force(fx, fy, fz, a[0], n_local, fi[0], fi[1], fi[2]);
        add_force(fx, fy, fz, a[2], n_local, fk[0], fk[1], fk[2]);
        add_force(fx, fy, fz, a[1], n_local, -(fi[0] + fk[0]), -(fi[1] + fk[1]), -(fi[2] + fk[2]));
        if (owner)
            for (int q = 0; q < 3; ++q) wd[q] += u[q] * fi[q] + v[q] * fk[q];
    }
    for (long t = 0; t < n_torsions; ++t) {
        const long* a = torsion_atoms + 4 * t;
        if (!any_local(a, 4, n_local)) continue;
        double ij[3] = {x[a[0]] - x[a[1]], y[a[0]] - y[a[1]], z[a[0]] - z[a[1]]};
        double jk[3] = {x[a[1]] - x[a[2]], y[a[1]] - y[a[2]], z[a[1]] - z[a[2]]};
        double kl[3] = {x[a[2]] - x[a[3]], y[a[2]] - y[a[3]], z[a[2]] - z[a[3]]};
        min_image(ij, L, periodic);
        min_image(jk, L, periodic);
        min_image(kl, L, periodic);
        const double n1[3] = {ij[1] * jk[2] - ij[2] * jk[1], ij[2] * jk[0] - ij[0] * jk[2], ij[0] * jk[1] - ij[1] * jk[0]};
        const double n2[3] = {jk[1] * kl[2] - jk[2] * kl[1], jk[2] * kl[0] - jk[0] * kl[2], jk[0] * kl[1] - jk[1] * kl[0]};
        const double n1sq = n1[0] * n1[0] + n1[1] * n1[1] + n1[2] * n1[2];
        const double n2sq = n2[0] * n2[0] + n2[1] * n2[1] + n2[2] * n2[2];
        const double jksq = jk[0] * jk[0] + jk[1] * jk[1] + jk[2] * jk[2];
        if (n1sq < 1e-20 || n2sq < 1e-20 || jksq < 1e-20) continue;
        const double jkm = std::sqrt(jksq);
        const double cosine = n1[0] * n2[0] + n1[1] * n2[1] + n1[2] * n2[2];
        const double sine = (n1[1] * n2[2] - n1[2] * n2[1]) * jk[0] + (n1[2] * n2[0] - n1[0] * n2[2]) * jk[1] +
                            (n1[0] * n2[1] - n1[1] * n2[0]) * jk[2];
        const double phi = std::atan2(sine, cosine * jkm);
        const bool owner = owns_term(a, 4, gid, n_local);
        double slope;
        if (torsion_n[t] == 0) {
            const double dphi = std::remainder(phi - torsion_phi0[t], 2.0 * M_PI);
            if (owner) pe += torsion_k[t] * dphi * dphi;
            slope = 2.0 * torsion_k[t] * dphi;
        } else {
            const double dphi = torsion_n[t] * phi - torsion_phi0[t];
            if (owner) pe += torsion_k[t] * (1.0 + std::cos(dphi));
            slope = -torsion_k[t] * torsion_n[t] * std::sin(dphi);
        }
        const double si = -slope * jkm / n1sq, sl = slope * jkm / n2sq;
        const double pp = -(ij[0] * jk[0] + ij[1] * jk[1] + ij[2] * jk[2]) / jksq;
        const double qq = -(kl[0] * jk[0] + kl[1] * jk[1] + kl[2] * jk[2]) / jksq;
        double fi[3], fj[3], fk[3], fl[3];
        for (int q = 0; q < 3; ++q) {
            fi[q] = si * n1[q];
            fl[q] = sl * n2[q];
            fj[q] = (pp - 1.0) * fi[q] - qq * fl[q];
            fk[q] = -pp * fi[q] + (qq - 1.0) * fl[q];
        }
        add_force(fx, fy, fz, a[0], n_local, fi[0], fi[1], fi[2]);
        add_force(fx, fy, fz, a[1], n_local, fj[0], fj[1], fj[2]);
        add_force(fx, fy, fz, a[2], n_local, fk[0], fk[1], fk[2]);
        add_force(fx, fy, fz, a[3], n_local, fl[0], fl[1], fl[2]);
        if (owner)
            for (int q = 0; q < 3; ++q) wd[q] += ij[q] * fi[q] - jk[q] * fk[q] - (jk[q] + kl[q]) * fl[q];
    }
    for (long s = 0; s < n_specials; ++s) {
        const long* a = special_atoms + 2 * s;
        if (!any_local(a, 2, n_local)) continue;
        double d[3] = {x[a[0]] - x[a[1]], y[a[0]] - y[a[1]], z[a[0]] - z[a[1]]};
        min_image(d, L, periodic);
        const double r2 = d[0] * d[0] + d[1] * d[1] + d[2] * d[2];
        if (r2 < 1e-10) continue;
        double fm = 0.0, u = 0.0;
        if (special_epsilon[s] != 0.0) {
            const double r2inv = 1.0 / r2, sig2 = special_sigma[s] * special_sigma[s];
            const double att = sig2 * sig2 * sig2 * r2inv * r2inv * r2inv, rep = att * att;
            fm += 4.0 * special_epsilon[s] * r2inv * (12.0 * rep - 6.0 * att) * special_lj_scale[s];
            u += 4.0 * special_epsilon[s] * (rep - att) * special_lj_scale[s];
        }
        if (charge && charge[a[0]] != 0.0 && charge[a[1]] != 0.0) {
            const double r = std::sqrt(r2);
            const double qq = 332.0636 * charge[a[0]] * charge[a[1]] * special_coulomb_scale[s];
            fm += qq / (r2 * r);
            u += qq / r;
        }
        const bool owner = owns_term(a, 2, gid, n_local);
        if (owner) pe += u;
        if (fm == 0.0) continue;
        add_force(fx, fy, fz, a[0], n_local, fm * d[0], fm * d[1], fm * d[2]);
        add_force(fx, fy, fz, a[1], n_local, -fm * d[0], -fm * d[1], -fm * d[2]);
        if (owner) {
            w += r2 * fm;
            for (int c = 0; c < 3; ++c) wd[c] += fm * d[c] * d[c];
        }
    }
    out[0] = pe; out[1] = w; out[2] = wd[0]; out[3] = wd[1]; out[4] = wd[2];
}

}  // extern "C"
