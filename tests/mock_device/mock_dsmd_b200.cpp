// Test double of libdsmd_b200.so for the CPU tests of the MD driver: the entry points the driver calls, with the same
// meaning, computed on the host in double precision by an all-pairs loop (Lennard-Jones with plain truncation, periodic
// minimum image). Test infrastructure only: it exists so that the driver's host logic (step order, rebuild policy,
// output, thermostat, restart files) can run where there is no GPU; it is never built into or loaded by the package.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "dsmd_b200.h"

struct dsmd_ctx {
    std::string error;
    double box[3] = {0, 0, 0};
    int periodic[3] = {1, 1, 1};
    int ntypes = 0;
    std::vector<double> eps, sig;
    double cutoff = 0, skin = 0;
    int64_t n = 0;
    std::vector<double> r[11];          // x y z vx vy vz fx fy fz mass charge
    std::vector<int32_t> type, gid;
    std::vector<double> xref, yref, zref;
    bool list_valid = false;
    double scalars[6] = {0, 0, 0, 0, 0, 0};
    int64_t launches = 0;
};

namespace {

int fail(dsmd_ctx* c, int code, const char* what) {
    if (c) c->error = what;
    return code;
}

void forces(dsmd_ctx* c, bool energy) {
    const int64_t n = c->n;
    for (int f = 6; f < 9; ++f) std::fill(c->r[f].begin(), c->r[f].end(), 0.0);
    double pe = 0.0, w = 0.0, wd[3] = {0, 0, 0}, pairs = 0.0;
    const double rc2 = c->cutoff * c->cutoff;
    for (int64_t i = 0; i < n; ++i)
        for (int64_t j = i + 1; j < n; ++j) {
            double d[3];
            for (int a = 0; a < 3; ++a) {
                d[a] = c->r[a][i] - c->r[a][j];
                if (c->periodic[a]) d[a] -= c->box[a] * std::rint(d[a] / c->box[a]);
            }
            const double r2 = d[0] * d[0] + d[1] * d[1] + d[2] * d[2];
            if (!(r2 < rc2) || r2 < 1e-10) continue;
            const size_t t = static_cast<size_t>(c->type[i]) * c->ntypes + c->type[j];
            const double s2 = c->sig[t] * c->sig[t], s6 = s2 * s2 * s2;
            const double c6 = 4.0 * c->eps[t] * s6, c12 = c6 * s6;
            const double ir2 = 1.0 / r2, ir6 = ir2 * ir2 * ir2;
            const double fr = ir2 * (12.0 * c12 * ir6 * ir6 - 6.0 * c6 * ir6);
            for (int a = 0; a < 3; ++a) {
                c->r[6 + a][i] += fr * d[a];
                c->r[6 + a][j] -= fr * d[a];
                wd[a] += fr * d[a] * d[a];
            }
            pe += c12 * ir6 * ir6 - c6 * ir6;
            w += fr * r2;
            pairs += 1.0;
        }
    if (energy) {
        c->scalars[0] = pe; c->scalars[1] = w; c->scalars[2] = wd[0]; c->scalars[3] = wd[1]; c->scalars[4] = wd[2];
        c->scalars[5] = pairs;
    }
    ++c->launches;
}

double max_disp2(const dsmd_ctx* c) {
    double m = 0.0;
    for (int64_t i = 0; i < c->n; ++i) {
        const double dx = c->r[0][i] - c->xref[i], dy = c->r[1][i] - c->yref[i], dz = c->r[2][i] - c->zref[i];
        m = std::max(m, dx * dx + dy * dy + dz * dz);
    }
    return m;
}

}  // namespace

extern "C" {

int dsmd_create(int, int64_t capacity, dsmd_ctx** out) {
    if (!out || capacity <= 0) return DSMD_ERR_INVALID;
    *out = new dsmd_ctx();
    return DSMD_OK;
}
void dsmd_destroy(dsmd_ctx* c) { delete c; }
const char* dsmd_last_error(const dsmd_ctx* c) { return c ? c->error.c_str() : "no context"; }

int dsmd_set_box(dsmd_ctx* c, const double box[3], const int periodic[3], const double*, const double*, double) {
    if (!c || !box || !periodic) return DSMD_ERR_INVALID;
    for (int a = 0; a < 3; ++a) {
        if (!(box[a] > 0.0)) return fail(c, DSMD_ERR_INVALID, "box lengths must be positive");
        c->box[a] = box[a];
        c->periodic[a] = periodic[a];
    }
    return DSMD_OK;
}

int dsmd_set_pair_params(dsmd_ctx* c, int ntypes, const double* eps, const double* sig, double cutoff, double skin,
                         double switch_distance) {
    if (!c || ntypes <= 0 || !eps || !sig) return DSMD_ERR_INVALID;
    if (switch_distance > 0.0) return fail(c, DSMD_ERR_INVALID, "the test double has no switching function");
    c->ntypes = ntypes;
    c->eps.assign(eps, eps + ntypes * ntypes);
    c->sig.assign(sig, sig + ntypes * ntypes);
    c->cutoff = cutoff;
    c->skin = skin;
    return DSMD_OK;
}

int dsmd_set_coulomb(dsmd_ctx* c, int enabled, double) {
    if (!c) return DSMD_ERR_INVALID;
    return enabled ? fail(c, DSMD_ERR_INVALID, "the test double has no electrostatics") : DSMD_OK;
}

int dsmd_set_exclusions(dsmd_ctx* c, int64_t, int64_t n_pairs, const int32_t*, const int32_t*) {
    return n_pairs ? fail(c, DSMD_ERR_INVALID, "the test double has no exclusions") : DSMD_OK;
}

int dsmd_set_constraints(dsmd_ctx* c, int64_t, int64_t n_constraints, const int32_t*, const int32_t*, const double*, double, int) {
    return n_constraints ? fail(c, DSMD_ERR_INVALID, "the test double has no constraints") : DSMD_OK;
}

int dsmd_set_bonded(dsmd_ctx* c, int64_t, int64_t n_bonds, const int32_t*, const double*, const double*, int64_t n_angles,
                    const int32_t*, const double*, const double*, int64_t n_torsions, const int32_t*, const double*,
                    const double*, const int32_t*, int64_t n_specials, const int32_t*, const double*, const double*,
                    const double*, const double*) {
    return (n_bonds || n_angles || n_torsions || n_specials) ? fail(c, DSMD_ERR_INVALID, "the test double has no bonded terms")
                                                             : DSMD_OK;
}

int dsmd_compute_bonded(dsmd_ctx*, void*) { return DSMD_OK; }

int dsmd_set_type_charges(dsmd_ctx*, int, const double*) { return DSMD_OK; }

int dsmd_read_bonded_scalars(dsmd_ctx*, double out[5], void*) {
    for (int k = 0; k < 5; ++k) out[k] = 0.0;
    return DSMD_OK;
}

int dsmd_upload(dsmd_ctx* c, int64_t n_owned, int64_t n_total, const double* x, const double* y, const double* z,
                const double* vx, const double* vy, const double* vz, const double* mass, const double* charge,
                const int32_t* type, const int32_t* gid, void*) {
    if (!c || n_owned != n_total || !x || !y || !z || !mass) return DSMD_ERR_INVALID;
    const size_t n = static_cast<size_t>(n_total);
    c->n = n_total;
    const double* src[11] = {x, y, z, vx, vy, vz, nullptr, nullptr, nullptr, mass, charge};
    for (int f = 0; f < 11; ++f) {
        c->r[f].assign(n, 0.0);
        if (src[f]) std::copy(src[f], src[f] + n, c->r[f].begin());
    }
    c->type.assign(n, 0);
    if (type) std::copy(type, type + n, c->type.begin());
    c->gid.resize(n);
    for (size_t i = 0; i < n; ++i) c->gid[i] = gid ? gid[i] : static_cast<int32_t>(i);
    c->list_valid = false;
    return DSMD_OK;
}

int dsmd_download(dsmd_ctx* c, int field, int64_t n, void* out, void*) {
    if (!c || !out || n > c->n) return DSMD_ERR_INVALID;
    if (field >= 0 && field < 11) std::memcpy(out, c->r[field].data(), sizeof(double) * n);
    else if (field == DSMD_TYPE) std::memcpy(out, c->type.data(), sizeof(int32_t) * n);
    else if (field == DSMD_GLOBAL_ID) std::memcpy(out, c->gid.data(), sizeof(int32_t) * n);
    else return DSMD_ERR_INVALID;
    return DSMD_OK;
}

int dsmd_build_neighbor_list(dsmd_ctx* c, void*) {
    if (!c || c->n == 0) return DSMD_ERR_STATE;
    for (int a = 0; a < 3; ++a)
        if (c->periodic[a] && c->box[a] < 2.0 * (c->cutoff + c->skin))
            return fail(c, DSMD_ERR_BOX_TOO_SMALL, "box shorter than twice the list radius");
    c->xref = c->r[0]; c->yref = c->r[1]; c->zref = c->r[2];
    c->list_valid = true;
    return DSMD_OK;
}

int dsmd_max_displacement_sq(dsmd_ctx* c, double* out, void*) {
    if (!c || !out || !c->list_valid) return DSMD_ERR_STATE;
    *out = max_disp2(c);
    return DSMD_OK;
}

int dsmd_compute_forces(dsmd_ctx* c, int phase, int want_energy, void*) {
    if (!c || phase != DSMD_PHASE_FULL) return DSMD_ERR_INVALID;
    if (!c->list_valid) return fail(c, DSMD_ERR_STATE, "no neighbour list");
    if (max_disp2(c) > c->skin * c->skin / 4.0 * 1.0000001) return fail(c, DSMD_ERR_STATE, "the skin was outrun: list too old");
    forces(c, want_energy != 0);
    return DSMD_OK;
}

int dsmd_read_scalars(dsmd_ctx* c, double out[6], void*) {
    if (!c || !out) return DSMD_ERR_INVALID;
    std::copy(c->scalars, c->scalars + 6, out);
    return DSMD_OK;
}

int dsmd_integrate(dsmd_ctx* c, int half, double dt, double f2a, void*) {
    if (!c || (half != 1 && half != 2)) return DSMD_ERR_INVALID;
    for (int64_t i = 0; i < c->n; ++i) {
        const double a = 0.5 * dt * f2a / c->r[9][i];
        for (int k = 0; k < 3; ++k) {
            c->r[3 + k][i] += a * c->r[6 + k][i];
            if (half == 1) c->r[k][i] += dt * c->r[3 + k][i];
        }
    }
    return DSMD_OK;
}

int dsmd_kinetic_energy(dsmd_ctx* c, double* out, void*) {
    if (!c || !out) return DSMD_ERR_INVALID;
    double sum = 0.0;
    for (int64_t i = 0; i < c->n; ++i)
        sum += 0.5 * c->r[9][i] * (c->r[3][i] * c->r[3][i] + c->r[4][i] * c->r[4][i] + c->r[5][i] * c->r[5][i]);
    *out = sum;
    return DSMD_OK;
}

int dsmd_scale_velocities(dsmd_ctx* c, double factor, void*) {
    if (!c || !std::isfinite(factor)) return DSMD_ERR_INVALID;
    for (int k = 3; k < 6; ++k)
        for (double& v : c->r[k]) v *= factor;
    return DSMD_OK;
}

int dsmd_run_nve(dsmd_ctx* c, int64_t n_steps, double dt, double f2a, double hi_frac, int every, int, int64_t* n_rebuilds,
                 double* worst_disp_sq, void*) {
    if (!c || n_steps < 0) return DSMD_ERR_INVALID;
    if (!c->list_valid) {
        dsmd_build_neighbor_list(c, nullptr);
        forces(c, false);
    }
    int64_t rebuilds = 0;
    double worst = 0.0;
    int since = 0;
    const double limit2 = hi_frac * c->skin * hi_frac * c->skin;
    for (int64_t s = 0; s < n_steps; ++s) {
        dsmd_integrate(c, 1, dt, f2a, nullptr);
        ++since;
        const double d2 = max_disp2(c);
        if ((every > 0 && since >= every) || d2 > limit2) {
            dsmd_build_neighbor_list(c, nullptr);
            ++rebuilds;
            since = 0;
        } else {
            worst = std::max(worst, d2);
        }
        forces(c, false);
        dsmd_integrate(c, 2, dt, f2a, nullptr);
    }
    if (n_rebuilds) *n_rebuilds = rebuilds;
    if (worst_disp_sq) *worst_disp_sq = worst;
    return DSMD_OK;
}

}  // extern "C"
