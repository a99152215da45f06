// Test infrastructure, not product code.
//
// Drives the C++ adapters of include/dsmd/ (ForceCalculatorB200, VerletListB200, EdgeBuilder) the way the reference's
// driver drives its own classes: an MDSystem filled with particles, box, force-field tables, topology exclusions and
// force configuration is handed to ForceCalculator::compute_forces; results come back through download_from_device and
// the ForceCalculator getters. Compiled against the reference's own interface headers where they lie (no reference
// source file is compiled), linked with libdsmd_b200.so; the GPU tests call it through ctypes and compare with the oracle.

#include <cuda_runtime.h>

#define USE_CUDA 1
#include "reference_members.hpp"

#include "dsmd/edge_builder.hpp"
#include "dsmd/force_calculator_b200.hpp"

extern "C" {

// One force evaluation through the reference-shaped interface. eps / sig: [ntypes x ntypes]. Forces are returned by
// global id. out_scalars = {PE, virial, Wxx, Wyy, Wzz, KE, needs_rebuild before / after moving one atom by 0.6 skin,
// the two lagged displacement answers, PE after a rebuild through HaloBackendB200}.
int dsmd_adapter_forces(long n, const double* x, const double* y, const double* z, const double* vx, const double* vy,
                        const double* vz, const double* mass, const double* charge, const int* type, const double box[3],
                        int ntypes, const double* eps, const double* sig, double cutoff, double skin, int do_coulomb,
                        long n_excl, const int* ea, const int* eb, double* out_f, double* out_scalars, char* error,
                        int error_len) {
    try {
        MDSystem system;
        system.topology = std::make_unique<Topology>();
        system.force_manager = std::make_unique<ForceManager>();
        ParticleData& p = system.get_particles();
        p.reset_counts(static_cast<size_t>(n), 0);
        p.resize(static_cast<size_t>(n));
        p.reset_counts(static_cast<size_t>(n), 0);
        for (long i = 0; i < n; ++i) {
            p.x[i] = x[i]; p.y[i] = y[i]; p.z[i] = z[i];
            p.vx[i] = vx ? vx[i] : 0.0; p.vy[i] = vy ? vy[i] : 0.0; p.vz[i] = vz ? vz[i] : 0.0;
            p.mass[i] = mass ? mass[i] : 1.0;
            p.charge[i] = charge ? charge[i] : 0.0;
            p.type[i] = type ? type[i] : 0;
            p.global_id[i] = static_cast<int>(i);
        }
        SimulationBox& b = system.get_box();
        b.lx = box[0]; b.ly = box[1]; b.lz = box[2];
        b.xlo = b.xhi = b.ylo = b.yhi = b.zlo = b.zhi = 0.0;
        b.periodic_x = b.periodic_y = b.periodic_z = true;
        b.update_box_length();
        ForceFieldParams& ff = system.get_ff_params();
        ff.num_atom_types = ntypes;
        ff.epsilon.assign(ntypes, 0.0);
        ff.sigma.assign(ntypes, 0.0);
        ff.epsilon_mixed.assign(ntypes, std::vector<Real>(ntypes));
        ff.sigma_mixed.assign(ntypes, std::vector<Real>(ntypes));
        for (int i = 0; i < ntypes; ++i)
            for (int j = 0; j < ntypes; ++j) {
                ff.epsilon_mixed[i][j] = eps[i * ntypes + j];
                ff.sigma_mixed[i][j] = sig[i * ntypes + j];
            }
        Topology& t = system.get_topology();
        t.atom_name_ids.assign(static_cast<size_t>(n), 0);
        for (long k = 0; k < n_excl; ++k) {
            const std::uint64_t lo = static_cast<std::uint64_t>(std::min(ea[k], eb[k]));
            const std::uint64_t hi = static_cast<std::uint64_t>(std::max(ea[k], eb[k]));
            t.exclusion_keys.push_back((lo << 32) | hi);
        }
        ForceManager::ForceConfig& cfg = system.force_manager->config;
        cfg.enable_bonds = cfg.enable_angles = cfg.enable_dihedrals = false;
        cfg.enable_lennard_jones = true;
        cfg.enable_coulomb = do_coulomb != 0;
        system.set_physical_cutoff(cutoff);
        system.set_verlet_skin(skin);

        dsmd::ForceCalculatorB200 calc(0);
        ForceCalculator& base = calc;                       // the driver holds it through the abstract interface
        calc.set_verlet_skin(skin);
        base.initialize();
        base.set_nonbonded_kernel("list");
        base.set_mixed_precision(true);
        calc.set_energy_readback_needed(true);
        base.compute_forces(system);
        base.calculate_kinetic_energy(system);
        out_scalars[0] = base.get_potential_energy();
        out_scalars[1] = base.get_virial();
        Real diag[3];
        base.get_virial_diag(diag);
        out_scalars[2] = diag[0]; out_scalars[3] = diag[1]; out_scalars[4] = diag[2];
        out_scalars[5] = base.get_kinetic_energy();
        calc.download_from_device(system);
        for (long s = 0; s < n; ++s) {
            const int g = p.global_id[s];
            out_f[3 * g] = p.fx[s]; out_f[3 * g + 1] = p.fy[s]; out_f[3 * g + 2] = p.fz[s];
        }
        // NeighborList seam: no rebuild needed right after a build; needed once an atom has moved 0.6 skin
        dsmd::VerletListB200 list(cutoff, skin, &calc);
        NeighborList& nl = list;
        const bool before = nl.needs_rebuild(p, b, static_cast<size_t>(n));
        double moved = 0.0;
        cudaMemcpy(&moved, calc.get_device_x(), sizeof(double), cudaMemcpyDeviceToHost);
        moved += 0.6 * skin;
        cudaMemcpy(calc.get_device_x(), &moved, sizeof(double), cudaMemcpyHostToDevice);
        const bool after = nl.needs_rebuild(p, b, static_cast<size_t>(n));
        out_scalars[6] = (before ? 1.0 : 0.0) + (after ? 2.0 : 0.0);   // expected 2
        if (std::fabs(nl.search_cutoff() - (cutoff + skin)) > 1e-12) throw std::runtime_error("search_cutoff");
        // the lagged displacement query: nothing yet, then the value of the call before (the atom moved 0.6 skin above)
        const double lag0 = calc.compute_max_displacement_lagged(static_cast<size_t>(n), b);
        const double lag1 = calc.compute_max_displacement_lagged(static_cast<size_t>(n), b);
        out_scalars[7] = lag0;
        out_scalars[8] = lag1;
        moved -= 0.6 * skin;   // back where it was
        cudaMemcpy(calc.get_device_x(), &moved, sizeof(double), cudaMemcpyHostToDevice);
        // the storage provider an external halo library would be given: a view of the device arrays, a resize in place
        struct View { size_t count; Real *x, *y, *z, *vx, *vy, *vz, *fx, *fy, *fz, *mass, *charge; int *type, *global_id; };
        struct Resized { View view; bool reallocated; };
        const View view = calc.particle_info_view_as<View>(static_cast<size_t>(n));
        const Resized grown = calc.resize_particle_info_as<Resized, View>(static_cast<size_t>(n) + 10, static_cast<size_t>(n));
        if (view.x != calc.get_device_x() || grown.view.x != view.x || grown.reallocated || grown.view.count != static_cast<size_t>(n) + 10)
            throw std::runtime_error("particle_info_view / resize_particle_info");
        calc.resize_particle_info_as<Resized, View>(static_cast<size_t>(n), static_cast<size_t>(n));
        bool refused = false;
        try { calc.particle_info_view_as<View>(calc.capacity() + 1); } catch (const std::runtime_error&) { refused = true; }
        if (!refused) throw std::runtime_error("a view beyond the capacity must throw");
        // HaloBackend / CommBackend over the native domain code, one rank: a rebuild step rebuilds the list, the
        // reductions are the identity, the energy afterwards is the one from before
        {
            dsmd_domain* dom = nullptr;
            const int dims[3] = {1, 1, 1};
            if (dsmd_domain_create(calc.context(), 0, 1, dims, box, cutoff + skin, skin, nullptr, nullptr, &dom) != DSMD_OK)
                throw std::runtime_error("dsmd_domain_create");
            dsmd::HaloBackendB200 halo(dom);
            dsmd::CommBackendB200 comm(dom, false, calc.get_force_stream());
            HaloBackend& hb = halo;
            CommBackend& cb = comm;
            bool rebuild = true;
            cb.unify_rebuild_decision(rebuild);
            if (!rebuild || cb.is_distributed() || !cb.is_gpu_single_rank(true)) throw std::runtime_error("CommBackendB200 flags");
            if (cb.migrate_particles_if_needed(system, rebuild, &calc)) throw std::runtime_error("one rank never migrates");
            if (!hb.try_gpu_direct_halo(system, &calc, rebuild) || !rebuild) throw std::runtime_error("HaloBackendB200 rebuild");
            bool no = false;
            if (!hb.try_gpu_direct_halo(system, &calc, no) || no) throw std::runtime_error("HaloBackendB200 refresh");
            if (cb.sum_reduce(2.5) != 2.5 || cb.max_reduce(-1.0) != -1.0 || cb.sum_int(7) != 7 || !cb.all_true(true) || cb.all_true(false))
                throw std::runtime_error("CommBackendB200 reductions");
            base.compute_forces(system);
            out_scalars[9] = base.get_potential_energy();
            dsmd_domain_destroy(dom);
        }
        base.finalize();
    } catch (const std::exception& e) {
        if (error && error_len > 0) std::snprintf(error, static_cast<size_t>(error_len), "%s", e.what());
        return 1;
    }
    return 0;
}

// EdgeBuilder with the reference's class shape: host positions in, edge list out (first call sizes, second call copies).
long dsmd_adapter_edges(long n, const double* x, const double* y, const double* z, double cutoff, long long* out_index,
                        long capacity, char* error, int error_len) {
    double *d_x = nullptr, *d_y = nullptr, *d_z = nullptr;
    long count = -1;
    try {
        cudaMalloc(&d_x, sizeof(double) * n); cudaMalloc(&d_y, sizeof(double) * n); cudaMalloc(&d_z, sizeof(double) * n);
        cudaMemcpy(d_x, x, sizeof(double) * n, cudaMemcpyHostToDevice);
        cudaMemcpy(d_y, y, sizeof(double) * n, cudaMemcpyHostToDevice);
        cudaMemcpy(d_z, z, sizeof(double) * n, cudaMemcpyHostToDevice);
        EdgeBuilder builder;
        const int64_t e = builder.build(d_x, d_y, d_z, n, cutoff, nullptr);
        if (e != builder.edge_count()) throw std::runtime_error("edge_count");
        count = static_cast<long>(e);
        if (out_index && capacity >= 2 * e && e > 0)
            cudaMemcpy(out_index, builder.edge_index(), sizeof(int64_t) * 2 * e, cudaMemcpyDeviceToHost);
        bool threw = false;
        try { builder.build(d_x, d_y, d_z, n, -1.0, nullptr); } catch (const std::invalid_argument&) { threw = true; }
        if (!threw) throw std::runtime_error("a negative cutoff must throw std::invalid_argument");
    } catch (const std::exception& e) {
        if (error && error_len > 0) std::snprintf(error, static_cast<size_t>(error_len), "%s", e.what());
        count = -1;
    }
    cudaFree(d_x); cudaFree(d_y); cudaFree(d_z);
    return count;
}

}  // extern "C"
