// Holonomic distance constraints of small rigid groups (rigid water and the like): SHAKE after the drift, RATTLE after
// the second velocity half. Included by dsmd_core.cu.
//
// What the reference does in shake_cluster_kernel / rattle_cluster_kernel (src/force_calculator_cuda.cu:6168-6333) and,
// on the host, ConstraintSolver (src/constraint_solver.cpp:15-146): every connected group of constraints (a "cluster":
// the three O-H, O-H, H-H constraints of a water molecule) is solved by ONE thread, sweeping its constraints in their
// given order until each |r_ij|^2 is within `tolerance` (relative) of its target (SHAKE: corrections along the bond
// vectors the pairs had before the drift; velocities take the displacement over dt), or until the relative velocity
// along every bond is below `tolerance` (RATTLE). A cluster converged is a cluster left alone, so the result is the one
// of sweeping all constraints of the system in order, as the host solver does.
//
// Atoms are re-sorted by cell at every list build, so clusters name their atoms by global id and go through a
// gid -> slot map that the sort refreshes. Clusters hold at most kClusterAtoms atoms and kClusterCons constraints.
#pragma once

namespace {

constexpr int kClusterAtoms = 4;
constexpr int kClusterCons = 6;

struct ClusterTable {
    int n_clusters;
    const int* atom_gid;            // [n_clusters * kClusterAtoms], -1: unused
    const unsigned char* con_a;     // [n_clusters * kClusterCons] atom of the cluster (0 .. kClusterAtoms - 1), 255: unused
    const unsigned char* con_b;
    const double* con_d2;           // squared target distance
    const int* slot_of_gid;         // [n_global]
    double box[3];
    int periodic[3];
};

__device__ __forceinline__ void half_box_image(double d[3], const ClusterTable& t) {
#pragma unroll
    for (int a = 0; a < 3; ++a)
        if (t.periodic[a]) {
            if (d[a] > 0.5 * t.box[a]) d[a] -= t.box[a];
            else if (d[a] < -0.5 * t.box[a]) d[a] += t.box[a];
        }
}

__global__ void k_slot_of_gid(int n, const int* __restrict__ gid, int n_global, int* __restrict__ slot_of) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= n) return;
    const int g = gid[s];
    if (g >= 0 && g < n_global) slot_of[g] = s;
}

// SHAKE: positions after the drift are moved back onto the constraints; pre = positions before the drift.
__global__ void k_shake(ClusterTable t, double* __restrict__ x, double* __restrict__ y, double* __restrict__ z,
                        double* __restrict__ vx, double* __restrict__ vy, double* __restrict__ vz,
                        const double* __restrict__ pre_x, const double* __restrict__ pre_y,
                        const double* __restrict__ pre_z, const double* __restrict__ mass, double inv_dt,
                        double tolerance, int max_iterations, unsigned* __restrict__ failed) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= t.n_clusters) return;
    int slot[kClusterAtoms];
    double p[kClusterAtoms][3], v[kClusterAtoms][3], q[kClusterAtoms][3], w[kClusterAtoms];
    int na = 0;
    for (int a = 0; a < kClusterAtoms; ++a) {
        const int g = t.atom_gid[k * kClusterAtoms + a];
        if (g < 0) break;
        const int s = t.slot_of_gid[g];
        slot[a] = s;
        p[a][0] = x[s]; p[a][1] = y[s]; p[a][2] = z[s];
        v[a][0] = vx[s]; v[a][1] = vy[s]; v[a][2] = vz[s];
        q[a][0] = pre_x[s]; q[a][1] = pre_y[s]; q[a][2] = pre_z[s];
        w[a] = 1.0 / mass[s];
        na = a + 1;
    }
    bool converged = false;
    for (int sweep = 0; sweep < max_iterations && !converged; ++sweep) {
        double worst = 0.0;
        for (int j = 0; j < kClusterCons; ++j) {
            const int a = t.con_a[k * kClusterCons + j], b = t.con_b[k * kClusterCons + j];
            if (a == 255) break;
            const double target2 = t.con_d2[k * kClusterCons + j];
            double d[3] = {p[a][0] - p[b][0], p[a][1] - p[b][1], p[a][2] - p[b][2]};
            half_box_image(d, t);
            const double excess = (d[0] * d[0] + d[1] * d[1] + d[2] * d[2]) - target2;
            const double relative = fabs(excess) / target2;
            worst = fmax(worst, relative);
            if (relative < tolerance) continue;
            double o[3] = {q[a][0] - q[b][0], q[a][1] - q[b][1], q[a][2] - q[b][2]};
            half_box_image(o, t);
            const double along = o[0] * d[0] + o[1] * d[1] + o[2] * d[2];
            if (fabs(along) < 1e-12) continue;   // degenerate geometry: the next sweep tries again
            const double gm = excess / (2.0 * (w[a] + w[b]) * along);
#pragma unroll
            for (int c = 0; c < 3; ++c) {
                const double corr = gm * o[c];
                p[a][c] -= corr * w[a];
                p[b][c] += corr * w[b];
                v[a][c] -= corr * w[a] * inv_dt;
                v[b][c] += corr * w[b] * inv_dt;
            }
        }
        converged = worst < tolerance;
    }
    for (int a = 0; a < na; ++a) {
        const int s = slot[a];
        x[s] = p[a][0]; y[s] = p[a][1]; z[s] = p[a][2];
        vx[s] = v[a][0]; vy[s] = v[a][1]; vz[s] = v[a][2];
    }
    if (!converged) atomicAdd(failed, 1u);
}

// RATTLE: the relative velocity along every constrained bond is removed. partials (may be null): per-block sums of the
// diagonal of the constraint virial, -2 / (force_to_accel dt) * sum over corrections of k r_a^2 (`prefactor`).
__global__ void k_rattle(ClusterTable t, const double* __restrict__ x, const double* __restrict__ y,
                         const double* __restrict__ z, double* __restrict__ vx, double* __restrict__ vy,
                         double* __restrict__ vz, const double* __restrict__ mass, double tolerance, int max_iterations,
                         double prefactor, double* __restrict__ partials, unsigned* __restrict__ failed) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    double wsum[3] = {0.0, 0.0, 0.0};
    if (k < t.n_clusters) {
        int slot[kClusterAtoms];
        double p[kClusterAtoms][3], v[kClusterAtoms][3], w[kClusterAtoms];
        int na = 0;
        for (int a = 0; a < kClusterAtoms; ++a) {
            const int g = t.atom_gid[k * kClusterAtoms + a];
            if (g < 0) break;
            const int s = t.slot_of_gid[g];
            slot[a] = s;
            p[a][0] = x[s]; p[a][1] = y[s]; p[a][2] = z[s];
            v[a][0] = vx[s]; v[a][1] = vy[s]; v[a][2] = vz[s];
            w[a] = 1.0 / mass[s];
            na = a + 1;
        }
        bool converged = false;
        for (int sweep = 0; sweep < max_iterations && !converged; ++sweep) {
            double worst = 0.0;
            for (int j = 0; j < kClusterCons; ++j) {
                const int a = t.con_a[k * kClusterCons + j], b = t.con_b[k * kClusterCons + j];
                if (a == 255) break;
                double d[3] = {p[a][0] - p[b][0], p[a][1] - p[b][1], p[a][2] - p[b][2]};
                half_box_image(d, t);
                const double r2 = d[0] * d[0] + d[1] * d[1] + d[2] * d[2];
                if (r2 < 1e-20) continue;
                const double along = d[0] * (v[a][0] - v[b][0]) + d[1] * (v[a][1] - v[b][1]) + d[2] * (v[a][2] - v[b][2]);
                worst = fmax(worst, fabs(along));
                if (fabs(along) < tolerance) continue;
                const double km = along / ((w[a] + w[b]) * r2);
#pragma unroll
                for (int c = 0; c < 3; ++c) {
                    v[a][c] -= km * w[a] * d[c];
                    v[b][c] += km * w[b] * d[c];
                    wsum[c] += prefactor * km * d[c] * d[c];
                }
            }
            converged = worst < tolerance;
        }
        for (int a = 0; a < na; ++a) {
            const int s = slot[a];
            vx[s] = v[a][0]; vy[s] = v[a][1]; vz[s] = v[a][2];
        }
        if (!converged) atomicAdd(failed, 1u);
    }
    if (partials) block_sum_to_partials<3>(wsum, partials);
}

}  // namespace
