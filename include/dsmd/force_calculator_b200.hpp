// C++ adapters with the reference's class shapes for the short-range nonbonded path, over the C ABI (dsmd_b200.h).
//
// Compiled INSIDE the reference tree (it includes the reference's own interface headers by name):
//   ForceCalculatorB200 : ForceCalculator          include/force_calculator.h:12-91, CUDA extras of
//                                                   include/force_calculator_cuda.h:38-183 that the driver calls on this path
//   VerletListB200      : NeighborList             include/neighbor_list.h:20-63 (in CUDA runs the driver only asks it for
//                                                   search_cutoff(): src/force_calculator_cuda.cu:4621)
//   HaloBackendB200     : HaloBackend              include/halo_backend.h:10-27
//   CommBackendB200     : CommBackend              include/comm_backend.h:12-38
// Errors of the C ABI become std::runtime_error, as the reference's CUDA macros end the run (src/force_calculator_cuda.cu:39-46)
// and main() catches exceptions (src/main.cpp:85-93). Reciprocal-space PME, bonded terms and constraints are not part of
// this library: a run that needs them keeps the reference's own calculator for those terms.
#ifndef DSMD_FORCE_CALCULATOR_B200_HPP
#define DSMD_FORCE_CALCULATOR_B200_HPP

#include <cmath>
#include <cstdint>
#include <functional>
#include <stdexcept>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "comm_backend.h"      // reference headers
#include "force_calculator.h"
#include "halo_backend.h"
#include "md_system.h"
#include "neighbor_list.h"

#include "../dsmd_b200.h"

namespace dsmd {

inline void check(dsmd_ctx* ctx, int rc, const char* what) {
    if (rc != DSMD_OK) throw std::runtime_error(std::string(what) + ": " + dsmd_last_error(ctx));
}

class ForceCalculatorB200 : public ForceCalculator {
public:
    explicit ForceCalculatorB200(int device = 0, size_t capacity = 0) : device_(device), capacity_(capacity) {}
    ~ForceCalculatorB200() override { finalize(); }

    void initialize() override {
        cudaSetDevice(device_);
        cudaStreamCreate(&force_stream_);
        int lo = 0, hi = 0;
        cudaDeviceGetStreamPriorityRange(&lo, &hi);
        cudaStreamCreateWithPriority(&halo_stream_, cudaStreamNonBlocking, hi);
        cudaEventCreateWithFlags(&halo_done_, cudaEventDisableTiming);
    }
    void finalize() override {
        if (ctx_) dsmd_destroy(ctx_);
        ctx_ = nullptr;
        if (force_stream_) cudaStreamDestroy(force_stream_);
        if (halo_stream_) cudaStreamDestroy(halo_stream_);
        if (halo_done_) cudaEventDestroy(halo_done_);
        force_stream_ = halo_stream_ = nullptr;
        halo_done_ = nullptr;
    }

    // ForceCalculatorCUDA::initial_upload_to_device (src/force_calculator_cuda.cu:4281): particles, box, LJ tables,
    // exclusion CSR.
    void initial_upload_to_device(MDSystem& system) {
        ParticleData& p = system.get_particles();
        const size_t n = p.size();
        if (!ctx_) {
            const size_t cap = capacity_ ? capacity_ : n + n / 2 + 1024;
            check(nullptr, dsmd_create(device_, static_cast<int64_t>(cap), &ctx_), "dsmd_create");
        }
        configure(system);
        check(ctx_, dsmd_upload(ctx_, static_cast<int64_t>(p.owned_count()), static_cast<int64_t>(n), p.x.data(), p.y.data(),
                                p.z.data(), p.vx.data(), p.vy.data(), p.vz.data(), p.mass.data(), p.charge.data(),
                                p.type.data(), p.global_id.data(), force_stream_), "dsmd_upload");
        cudaStreamSynchronize(force_stream_);
        nlist_dirty_ = true;
    }

    // ForceCalculatorCUDA::download_from_device: host ParticleData in the context's current atom order.
    void download_from_device(MDSystem& system) {
        ParticleData& p = system.get_particles();
        int64_t n_owned = 0, n_total = 0;
        dsmd_counts(ctx_, &n_owned, &n_total);
        p.reset_counts(static_cast<size_t>(n_owned), static_cast<size_t>(n_total - n_owned));
        p.resize(static_cast<size_t>(n_total));
        double* real[] = {p.x.data(), p.y.data(), p.z.data(), p.vx.data(), p.vy.data(), p.vz.data(), p.fx.data(),
                          p.fy.data(), p.fz.data(), p.mass.data(), p.charge.data()};
        for (int f = 0; f < 11; ++f) check(ctx_, dsmd_download(ctx_, f, n_total, real[f], force_stream_), "dsmd_download");
        check(ctx_, dsmd_download(ctx_, DSMD_TYPE, n_total, p.type.data(), force_stream_), "dsmd_download");
        check(ctx_, dsmd_download(ctx_, DSMD_GLOBAL_ID, n_total, p.global_id.data(), force_stream_), "dsmd_download");
    }

    void build_neighbor_list_on_device(MDSystem&) {
        check(ctx_, dsmd_build_neighbor_list(ctx_, force_stream_), "dsmd_build_neighbor_list");
        nlist_dirty_ = false;
    }
    void update_reference_positions_on_device(size_t) {}   // the list build takes the reference positions itself

    Real compute_max_displacement_on_device(size_t, const SimulationBox&) {
        check(ctx_, dsmd_pack_positions(ctx_, 0, owned(), force_stream_), "dsmd_pack_positions");
        double d2 = 0.0;
        check(ctx_, dsmd_max_displacement_sq(ctx_, &d2, force_stream_), "dsmd_max_displacement_sq");
        return d2;
    }

    // ForceCalculatorCUDA::compute_max_displacement_lagged (src/force_calculator_cuda.cu:6723-6764): the value of the
    // previous call (negative: none yet for the current reference positions); the host does not wait for this step.
    Real compute_max_displacement_lagged(size_t, const SimulationBox&) {
        check(ctx_, dsmd_pack_positions(ctx_, 0, owned(), force_stream_), "dsmd_pack_positions");
        double d2 = -1.0;
        check(ctx_, dsmd_max_displacement_sq_lagged(ctx_, &d2, force_stream_), "dsmd_max_displacement_sq_lagged");
        return d2;
    }

    // ParticleInfo::Provider (ForceCalculatorCUDA::particle_info_view / resize_particle_info,
    // src/force_calculator_cuda.cu:4143-4216) for an engine that brings its own halo library: the decomposition library's
    // view / result types are the engine's, so they are template parameters here; a View needs the members count, x, y, z,
    // vx, vy, vz, fx, fy, fz, mass, charge, type, global_id, a Result the members view and reallocated. The context's
    // arrays never move (they are allocated for the capacity given at creation), so nothing is ever reallocated; asking
    // for more than the capacity throws.
    template <class View>
    View particle_info_view_as(size_t count) {
        if (count > capacity()) throw std::runtime_error("particle_info_view: more atoms than the context's capacity");
        View v{};
        v.count = count;
        v.x = get_device_x(); v.y = get_device_y(); v.z = get_device_z();
        v.vx = get_device_vx(); v.vy = get_device_vy(); v.vz = get_device_vz();
        v.fx = get_device_fx(); v.fy = get_device_fy(); v.fz = get_device_fz();
        v.mass = get_device_mass(); v.charge = get_device_charge();
        v.type = get_device_type(); v.global_id = get_device_global_id();
        return v;
    }
    template <class Result, class View>
    Result resize_particle_info_as(size_t required, size_t preserve_count) {
        if (required > capacity()) throw std::runtime_error("resize_particle_info: more atoms than the context's capacity");
        int64_t n_owned = 0, n_total = 0;
        dsmd_counts(ctx_, &n_owned, &n_total);
        if (static_cast<int64_t>(required) != n_total)
            check(ctx_, dsmd_set_counts(ctx_, std::min<int64_t>(n_owned, static_cast<int64_t>(required)), static_cast<int64_t>(required)),
                  "dsmd_set_counts");
        (void)preserve_count;   // every atom below the new count is preserved: the arrays stay where they are
        Result r{};
        r.view = particle_info_view_as<View>(required);
        r.reallocated = false;
        return r;
    }
    size_t capacity() const {
        int64_t cap = 0;
        if (ctx_) dsmd_capacity(ctx_, &cap);
        return static_cast<size_t>(cap);
    }

    // ForceCalculator::compute_forces: device-resident state, FULL phase. Energy and virial are read back only when
    // asked for (set_energy_readback_needed), as the reference does.
    void compute_forces(MDSystem& system) override {
        if (!ctx_) initial_upload_to_device(system);
        if (nlist_dirty_) build_neighbor_list_on_device(system);
        else check(ctx_, dsmd_pack_positions(ctx_, 0, total(), force_stream_), "dsmd_pack_positions");
        check(ctx_, dsmd_compute_forces(ctx_, DSMD_PHASE_FULL, energy_needed_ ? 1 : 0, force_stream_), "dsmd_compute_forces");
        if (bonded_) check(ctx_, dsmd_compute_bonded(ctx_, force_stream_), "dsmd_compute_bonded");
        if (energy_needed_) read_scalars();
    }
    bool supports_overlapped_forces(MDSystem&) const { return true; }
    void begin_forces_interior(MDSystem&) {
        check(ctx_, dsmd_pack_positions(ctx_, 0, owned(), force_stream_), "dsmd_pack_positions");
        check(ctx_, dsmd_compute_forces(ctx_, DSMD_PHASE_INTERIOR, energy_needed_ ? 1 : 0, force_stream_), "interior");
    }
    void finish_forces_boundary(MDSystem&) {
        check(ctx_, dsmd_compute_forces(ctx_, DSMD_PHASE_BOUNDARY, energy_needed_ ? 1 : 0, force_stream_), "boundary");
        if (bonded_) check(ctx_, dsmd_compute_bonded(ctx_, force_stream_), "dsmd_compute_bonded");   // ghost positions are in
        if (energy_needed_) read_scalars();
    }
    void make_force_stream_wait_for_halo() {
        cudaEventRecord(halo_done_, halo_stream_);
        cudaStreamWaitEvent(force_stream_, halo_done_, 0);
    }

    void calculate_kinetic_energy(MDSystem&) override {
        double ke = 0.0;
        check(ctx_, dsmd_kinetic_energy(ctx_, &ke, force_stream_), "dsmd_kinetic_energy");
        last_kinetic_energy = ke;   // one rank's share; the caller reduces (CommBackend::sum_reduce)
    }
    void integrate_on_device(MDSystem&, Real dt, const std::string&) {
        check(ctx_, dsmd_integrate(ctx_, 1, dt, FORCE_TO_ACCEL, force_stream_), "dsmd_integrate");
    }
    void complete_velocity_update_on_device(MDSystem&, Real dt, const std::string&) {
        check(ctx_, dsmd_integrate(ctx_, 2, dt, FORCE_TO_ACCEL, force_stream_), "dsmd_integrate");
    }

    bool supports_virial_tensor() const override { return true; }
    void set_mixed_precision(bool) override {}     // one precision: fp32 pair math, fp64 state and sums
    void set_nonbonded_kernel(const std::string& kernel) override { nonbonded_kernel_ = kernel; }   // one kernel
    void set_energy_readback_needed(bool needed) { energy_needed_ = needed; }

    Real* get_device_x() { return field<Real>(DSMD_X); }
    Real* get_device_y() { return field<Real>(DSMD_Y); }
    Real* get_device_z() { return field<Real>(DSMD_Z); }
    Real* get_device_vx() { return field<Real>(DSMD_VX); }
    Real* get_device_vy() { return field<Real>(DSMD_VY); }
    Real* get_device_vz() { return field<Real>(DSMD_VZ); }
    Real* get_device_fx() { return field<Real>(DSMD_FX); }
    Real* get_device_fy() { return field<Real>(DSMD_FY); }
    Real* get_device_fz() { return field<Real>(DSMD_FZ); }
    Real* get_device_mass() { return field<Real>(DSMD_MASS); }
    Real* get_device_charge() { return field<Real>(DSMD_CHARGE); }
    int* get_device_type() { return field<int>(DSMD_TYPE); }
    int* get_device_global_id() { return field<int>(DSMD_GLOBAL_ID); }
    cudaStream_t get_force_stream() const { return force_stream_; }
    cudaStream_t get_halo_stream() const { return halo_stream_; }
    int get_device_id() const { return device_; }
    dsmd_ctx* context() { return ctx_; }
    bool nlist_dirty_ = true;

private:
    template <class T>
    T* field(int id) {
        void* p = nullptr;
        check(ctx_, dsmd_device_pointer(ctx_, id, &p), "dsmd_device_pointer");
        return static_cast<T*>(p);
    }
    int64_t owned() const { int64_t a = 0, b = 0; dsmd_counts(ctx_, &a, &b); return a; }
    int64_t total() const { int64_t a = 0, b = 0; dsmd_counts(ctx_, &a, &b); return b; }

    void configure(MDSystem& system) {
        const SimulationBox& b = system.get_box();
        ForceFieldParams& ff = system.get_ff_params();
        const double box[3] = {b.lx, b.ly, b.lz};
        const int periodic[3] = {b.periodic_x, b.periodic_y, b.periodic_z};
        const double lo[3] = {b.xlo, b.ylo, b.zlo}, hi[3] = {b.xhi, b.yhi, b.zhi};
        check(ctx_, dsmd_set_box(ctx_, box, periodic, lo, hi, system.get_halo_width()), "dsmd_set_box");
        const int nt = ff.num_atom_types;
        std::vector<double> eps(static_cast<size_t>(nt) * nt), sig(eps.size());
        for (int i = 0; i < nt; ++i)
            for (int j = 0; j < nt; ++j) {
                eps[static_cast<size_t>(i) * nt + j] = ff.epsilon_mixed[i][j];
                sig[static_cast<size_t>(i) * nt + j] = ff.sigma_mixed[i][j];
            }
        if (ff.mie_repulsive_exponent != 12 || ff.mie_attractive_exponent != 6)
            throw std::runtime_error("ForceCalculatorB200: only Mie(12,6) Lennard-Jones is supported");
        check(ctx_, dsmd_set_pair_params(ctx_, nt, eps.data(), sig.data(), system.get_physical_cutoff(), verlet_skin_,
                                         ff.lj_switch_distance), "dsmd_set_pair_params");
        const auto& cfg = system.get_force_manager().get_config();
        check(ctx_, dsmd_set_coulomb(ctx_, cfg.enable_coulomb ? 1 : 0, 0.0), "dsmd_set_coulomb");
        if (system.has_topology()) {
            const auto& keys = system.get_topology().get_exclusion_keys();
            std::vector<int32_t> a(keys.size()), c(keys.size());
            for (size_t k = 0; k < keys.size(); ++k) {
                a[k] = static_cast<int32_t>(keys[k] >> 32);
                c[k] = static_cast<int32_t>(keys[k] & 0xffffffffu);
            }
            check(ctx_, dsmd_set_exclusions(ctx_, system.get_topology().get_num_atoms(), static_cast<int64_t>(keys.size()),
                                            a.data(), c.data()), "dsmd_set_exclusions");
            upload_bonded_terms(system);
        }
    }
    // The bonded terms of the whole topology, by global atom id, each with the parameters of its type (what the
    // reference copies per rank from MDSystem::get_local_bonds() ... get_local_special_pairs(), include/md_system.h:162-166;
    // here every rank holds the whole table and evaluates the terms one of whose atoms it owns). Each kind follows its
    // switch in the force configuration; special pairs run with the pair forces (src/force_calculator_cpu.cpp:792-815).
    void upload_bonded_terms(MDSystem& system) {
        const Topology& t = system.get_topology();
        const auto& cfg = system.get_force_manager().get_config();
        const ForceFieldParams& ff = system.get_ff_params();
        std::vector<int32_t> ba, aa, ta, tn, sa;
        std::vector<double> bk, br, ak, at, tk, tp, ss, se, sl, sc;
        if (cfg.enable_bonds)
            for (const Bond& b : t.get_bonds()) {
                const BondType& p = t.get_bond_type(b.type);
                ba.insert(ba.end(), {b.atom1, b.atom2});
                bk.push_back(p.k); br.push_back(p.r0);
            }
        if (cfg.enable_angles)
            for (const Angle& a : t.get_angles()) {
                const AngleType& p = t.get_angle_type(a.type);
                aa.insert(aa.end(), {a.atom1, a.atom2, a.atom3});
                ak.push_back(p.k); at.push_back(p.theta0);
            }
        if (cfg.enable_dihedrals) {
            auto torsion = [&](const Dihedral& d) {
                const DihedralType& p = t.get_dihedral_type(d.type);
                ta.insert(ta.end(), {d.atom1, d.atom2, d.atom3, d.atom4});
                tk.push_back(p.k); tp.push_back(p.phi0); tn.push_back(p.n);
            };
            for (const Dihedral& d : t.get_dihedrals()) torsion(d);
            for (const Dihedral& d : t.get_impropers()) torsion(d);
        }
        if (cfg.enable_lennard_jones || cfg.enable_coulomb)
            for (const SpecialPair& p : t.get_special_pairs()) {
                const int ti = t.get_atom_type_id(p.atom1), tj = t.get_atom_type_id(p.atom2);
                sa.insert(sa.end(), {p.atom1, p.atom2});
                ss.push_back(p.sigma >= 0.0 ? p.sigma : ff.sigma_mixed[ti][tj]);
                se.push_back(!cfg.enable_lennard_jones ? 0.0 : (p.epsilon >= 0.0 ? p.epsilon : ff.epsilon_mixed[ti][tj]));
                sl.push_back(p.lj_scale);
                sc.push_back(cfg.enable_coulomb ? p.coulomb_scale : 0.0);
            }
        bonded_ = !bk.empty() || !ak.empty() || !tk.empty() || !ss.empty();
        check(ctx_, dsmd_set_bonded(ctx_, t.get_num_atoms(), static_cast<int64_t>(bk.size()), ba.data(), bk.data(), br.data(),
                                    static_cast<int64_t>(ak.size()), aa.data(), ak.data(), at.data(),
                                    static_cast<int64_t>(tk.size()), ta.data(), tk.data(), tp.data(), tn.data(),
                                    static_cast<int64_t>(ss.size()), sa.data(), ss.data(), se.data(), sl.data(), sc.data()),
              "dsmd_set_bonded");
    }
    void read_scalars() {
        double s[6];
        check(ctx_, dsmd_read_scalars(ctx_, s, force_stream_), "dsmd_read_scalars");
        last_potential_energy = s[0];        // this rank's share; MDSimulation reduces through CommBackend::sum_reduce
        last_virial = s[1];
        for (int a = 0; a < 3; ++a) last_virial_diag[a] = s[2 + a];
        if (bonded_) {
            double b[5];
            check(ctx_, dsmd_read_bonded_scalars(ctx_, b, force_stream_), "dsmd_read_bonded_scalars");
            last_potential_energy += b[0];
            last_virial += b[1];
            for (int a = 0; a < 3; ++a) last_virial_diag[a] += b[2 + a];
        }
    }

public:
    void set_verlet_skin(Real skin) { verlet_skin_ = skin; }

private:
    int device_ = 0;
    size_t capacity_ = 0;
    dsmd_ctx* ctx_ = nullptr;
    cudaStream_t force_stream_ = nullptr, halo_stream_ = nullptr;
    cudaEvent_t halo_done_ = nullptr;
    bool energy_needed_ = true;
    bool bonded_ = false;
    Real verlet_skin_ = 2.0;
};

// NeighborList seam: in CUDA runs the list lives inside the calculator; the host object answers search_cutoff() and
// forwards rebuild questions to it (include/neighbor_list.h:20-63).
class VerletListB200 : public NeighborList {
public:
    VerletListB200(Real cutoff, Real skin, ForceCalculatorB200* calc = nullptr) : cutoff_(cutoff), skin_(skin), calc_(calc) {}
    void build(const ParticleData&, const SimulationBox&, size_t) override { if (calc_) calc_->nlist_dirty_ = true; }
    void update(const ParticleData& p, const SimulationBox& b, size_t n) override { build(p, b, n); }
    bool needs_rebuild(const ParticleData&, const SimulationBox& box, size_t n) const override {
        if (!calc_) return true;
        const Real d2 = calc_->compute_max_displacement_on_device(n, box);
        return d2 > (0.5 * skin_) * (0.5 * skin_);
    }
    const int* get_neighbors() const override { return nullptr; }     // device-resident list: no host CSR
    const int* get_offsets() const override { return nullptr; }
    int num_pairs() const override { return 0; }
    void prune_active(const ParticleData&, const SimulationBox&, size_t) override {}
    const int* get_active_neighbors() const override { return nullptr; }
    const int* get_active_offsets() const override { return nullptr; }
    int num_active_edges() const override { return 0; }
    void set_nonbonded_kernel(const std::string&) override {}
    bool needs_active_prune(const ParticleData&, const SimulationBox&, size_t) const override { return false; }
    Real search_cutoff() const override { return cutoff_ + skin_; }
    NeighborListBackend kind() const override { return NeighborListBackend::CPU_SPATIAL_VERLET; }

private:
    Real cutoff_, skin_;
    ForceCalculatorB200* calc_;
};

// HaloBackend seam (include/halo_backend.h:10-27) over the native domain code (dsmd_domain_*): on a rebuild step the
// whole rebuild (migration, owned sort, ghost plan and records, list), otherwise the positions-only refresh. A callable
// given at construction replaces that (an engine that keeps its own transport).
class HaloBackendB200 : public HaloBackend {
public:
    using Exchange = std::function<bool(ForceCalculatorB200&, bool rebuild)>;   // returns: ghost layout changed
    explicit HaloBackendB200(dsmd_domain* domain) : domain_(domain) {}
    explicit HaloBackendB200(Exchange exchange) : exchange_(std::move(exchange)) {}
    bool try_gpu_direct_halo(MDSystem&, ForceCalculator* force_calc, bool& should_rebuild) override {
        auto* calc = dynamic_cast<ForceCalculatorB200*>(force_calc);
        if (!calc) return false;
        if (exchange_) {
            if (exchange_(*calc, should_rebuild)) should_rebuild = true;
            return true;
        }
        if (!domain_) return false;
        if (should_rebuild) {
            const int rc = dsmd_domain_rebuild(domain_, calc->get_force_stream());
            if (rc != DSMD_OK) throw std::runtime_error(std::string("dsmd_domain_rebuild: ") + dsmd_domain_last_error(domain_));
            calc->nlist_dirty_ = false;   // the rebuild ends with the list build
        } else {
            const int rc = dsmd_domain_refresh(domain_, calc->get_force_stream());
            if (rc != DSMD_OK) throw std::runtime_error(std::string("dsmd_domain_refresh: ") + dsmd_domain_last_error(domain_));
        }
        return true;
    }
    void on_post_halo(MDSystem&, ForceCalculator*, bool, bool) override {}
    const char* name() const override { return "b200-nccl"; }

private:
    dsmd_domain* domain_ = nullptr;
    Exchange exchange_;
};

// CommBackend seam (include/comm_backend.h:12-38) over the native domain code: scalar reductions are dsmd_domain_reduce
// (NCCL all-reduce of a few doubles); migration is part of the rebuild that HaloBackendB200 runs on the same step, so
// migrate_particles_if_needed only reports that ownership may change. Callables, when set, replace the reductions.
class CommBackendB200 : public CommBackend {
public:
    CommBackendB200() = default;
    CommBackendB200(dsmd_domain* domain, bool several_ranks, cudaStream_t stream = nullptr)
        : distributed(several_ranks), domain_(domain), stream_(stream) {}
    std::function<double(double)> max_fn, sum_fn;
    std::function<bool(MDSystem&, ForceCalculator*)> migrate_fn;
    bool distributed = false;

    bool is_distributed() const override { return distributed; }
    void unify_rebuild_decision(bool& should_rebuild) override { should_rebuild = reduce(should_rebuild ? 1.0 : 0.0, 1) > 0.5; }
    bool migrate_particles_if_needed(MDSystem& system, bool should_rebuild, ForceCalculator* calc) override {
        if (migrate_fn) return should_rebuild && migrate_fn(system, calc);
        return should_rebuild && distributed;
    }
    bool is_gpu_single_rank(bool using_cuda) const override { return using_cuda && !distributed; }
    Real max_reduce(Real v) const override { return reduce(v, 1); }
    Real sum_reduce(Real v) const override { return reduce(v, 0); }
    int sum_int(int v) const override { return static_cast<int>(std::lround(reduce(v, 0))); }
    bool all_true(bool v) const override { return reduce(v ? 0.0 : 1.0, 1) < 0.5; }
    void reduce_max_force_particle(Real f, size_t id, int, Real& gf, size_t& gid) const override {
        gf = reduce(f, 1);
        gid = id;   // single rank: the local particle; several ranks: the engine's MAXLOC reduction decides the owner
    }

private:
    double reduce(double v, int op) const {
        if (op == 1 && max_fn) return max_fn(v);
        if (op == 0 && sum_fn) return sum_fn(v);
        if (!domain_ || !distributed) return v;
        const int rc = dsmd_domain_reduce(domain_, &v, 1, op, stream_);
        if (rc != DSMD_OK) throw std::runtime_error(std::string("dsmd_domain_reduce: ") + dsmd_domain_last_error(domain_));
        return v;
    }
    dsmd_domain* domain_ = nullptr;
    cudaStream_t stream_ = nullptr;
};

}  // namespace dsmd

#endif  // DSMD_FORCE_CALCULATOR_B200_HPP
