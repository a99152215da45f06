/* dsmd_b200.h - C ABI of the B200 (sm_100a) short-range nonbonded path.
 *
 * One opaque context per GPU. Every entry point returns an int status (DSMD_OK = 0) and never exits or throws;
 * dsmd_last_error() gives the text of the last failure. All device work is queued on the caller's stream
 * (a cudaStream_t passed as void*); entry points that return a value to the host synchronise that stream once,
 * and say so. A context is used from one host thread at a time.
 *
 * The reference has no C plugin interface: its seams are C++ abstract classes (ForceCalculator, NeighborList,
 * HaloBackend, CommBackend, EdgeBuilder). Each entry point below names the reference member it stands behind;
 * include/dsmd/ *.hpp holds C++ adapters with the reference's own class shapes that call only this ABI.
 */
#ifndef DSMD_B200_H
#define DSMD_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct dsmd_ctx dsmd_ctx;

enum {
    DSMD_OK = 0,
    DSMD_ERR_INVALID = 1,        /* bad argument */
    DSMD_ERR_CUDA = 2,           /* a CUDA runtime call failed */
    DSMD_ERR_BOX_TOO_SMALL = 3,  /* a periodic axis is shorter than the cell grid needs (reference: "returns nulls",
                                    src/neighbor_list_kernels.cu:596-617) */
    DSMD_ERR_OUT_OF_DOMAIN = 4,  /* an atom lies outside the subdomain + halo on a non-wrapping axis, or is NaN
                                    (reference: EdgeBuilder throws, src/EdgeBuilder.cu:319-321) */
    DSMD_ERR_CAPACITY = 5,       /* more atoms than the context was created for */
    DSMD_ERR_STATE = 6,          /* call order: e.g. forces before a list exists */
    DSMD_ERR_TIMEOUT = 7         /* a bounded device-side wait ran out */
};

/* phases of a force evaluation (reference: ForceCalculatorCUDA::run_force_phase, src/force_calculator_cuda.cu:5260) */
enum { DSMD_PHASE_FULL = 0, DSMD_PHASE_INTERIOR = 1, DSMD_PHASE_BOUNDARY = 2 };

/* per-atom device arrays (reference: ForceCalculatorCUDA::get_device_*, include/force_calculator_cuda.h:142-183) */
enum {
    DSMD_X = 0, DSMD_Y, DSMD_Z, DSMD_VX, DSMD_VY, DSMD_VZ, DSMD_FX, DSMD_FY, DSMD_FZ, DSMD_MASS, DSMD_CHARGE,
    DSMD_TYPE, DSMD_GLOBAL_ID, DSMD_FIELD_COUNT
};

/* -- life cycle ---------------------------------------------------------------------------------------------------- */

/* ForceCalculatorCUDA::initialize / finalize (include/force_calculator_cuda.h:38-40). capacity = most atoms
 * (owned + ghost) the context will ever hold. Allocates the particle arrays; list storage is sized at the first build. */
int dsmd_create(int device, int64_t capacity, dsmd_ctx** out);
void dsmd_destroy(dsmd_ctx* ctx);
const char* dsmd_last_error(const dsmd_ctx* ctx);

/* -- set-up --------------------------------------------------------------------------------------------------------- */

/* SimulationBox (include/md_types.h:29-37): orthorhombic box lengths, periodic flags and this rank's subdomain
 * [lo, hi]. lo[a] == hi[a] means the whole box length on that axis. An axis whose subdomain is narrower than the box is
 * "split": its ghosts arrive image-shifted through the halo exchange and the axis does not wrap; halo = how far ghosts
 * may sit outside [lo, hi] on a split axis. */
int dsmd_set_box(dsmd_ctx* ctx, const double box[3], const int periodic[3], const double lo[3], const double hi[3],
                 double halo);

/* ForceFieldParams mixing tables + cutoff_distance / verlet_skin / lj_switch_distance
 * (include/md_types.h:98-136, src/force_calculator_cuda.cu:4337-4377). eps, sig: full [ntypes x ntypes] matrices.
 * switch_distance <= 0: plain truncation. */
int dsmd_set_pair_params(dsmd_ctx* ctx, int ntypes, const double* eps, const double* sig, double cutoff, double skin,
                         double switch_distance);

/* Real-space Ewald on/off (force_calculation.type "PME"); alpha <= 0 derives it from erfc(alpha rc) = 1e-5 as
 * src/force_calculator_cuda.cu:6821-6828 does. Builds the float-bit indexed cubic table (include/ewald_real_table.h). */
int dsmd_set_coulomb(dsmd_ctx* ctx, int enabled, double alpha);
int dsmd_get_ewald_alpha(const dsmd_ctx* ctx, double* alpha);

/* Exclusion pairs by global id (Topology::get_exclusion_keys -> exclusion CSR upload,
 * src/force_calculator_cuda.cu:4379-4423). n_global = atoms in the whole system. */
int dsmd_set_exclusions(dsmd_ctx* ctx, int64_t n_global, int64_t n_pairs, const int32_t* a, const int32_t* b);

/* Distance constraints by global id (Topology constraints -> ConstraintSolver, src/constraint_solver.cpp:15-146; device
 * kernels shake_cluster_kernel / rattle_cluster_kernel, src/force_calculator_cuda.cu:6168-6333). Connected constraints
 * form a group solved by one thread (at most 4 atoms and 6 constraints per group: rigid water has 3 and 3). Once set,
 * dsmd_integrate applies SHAKE after the drift of half 1 and RATTLE after half 2, and so does dsmd_run_nve.
 * tolerance <= 0 / max_iterations <= 0 keep the reference's defaults (1e-8, 500). n_constraints = 0 removes them.
 * Single-rank systems only (a group's atoms must all be owned). */
int dsmd_set_constraints(dsmd_ctx* ctx, int64_t n_global, int64_t n_constraints, const int32_t* a, const int32_t* b,
                         const double* distance, double tolerance, int max_iterations);

/* Groups whose sweeps did not converge since the last list build (ConstraintSolver::apply_shake / apply_rattle return
 * false then). Synchronises `stream`. */
int dsmd_constraint_failures(dsmd_ctx* ctx, int64_t* failed_groups, void* stream);

/* RATTLE alone, with the diagonal of the constraint virial (ForceCalculatorCUDA::apply_rattle_on_device): velocities are
 * projected; device_virial_diag (3 device doubles, may be NULL) receives -2 / (force_to_accel dt) * sum k r_a^2. */
int dsmd_rattle(dsmd_ctx* ctx, double dt, double force_to_accel, double* device_virial_diag, void* stream);

/* -- particle storage ----------------------------------------------------------------------------------------------- */

/* ForceCalculatorCUDA::initial_upload_to_device (src/force_calculator_cuda.cu:4281): host arrays, owned atoms first
 * then ghosts. vx..vz, charge, type, gid may be NULL (zeros / 0 / 0..n-1). Asynchronous on `stream` for pinned memory. */
int dsmd_upload(dsmd_ctx* ctx, int64_t n_owned, int64_t n_total, const double* x, const double* y, const double* z,
                const double* vx, const double* vy, const double* vz, const double* mass, const double* charge,
                const int32_t* type, const int32_t* gid, void* stream);

/* Positions only, in the context's current atom order (the order of DSMD_GLOBAL_ID). */
int dsmd_upload_positions(dsmd_ctx* ctx, const double* x, const double* y, const double* z, void* stream);

/* ForceCalculatorCUDA::download_from_device: copies one field of the first n atoms to host memory in the context's
 * current atom order; doubles for every field but DSMD_TYPE / DSMD_GLOBAL_ID (int32). Synchronises `stream`. */
int dsmd_download(dsmd_ctx* ctx, int field, int64_t n, void* host_out, void* stream);

/* get_device_x() ... get_device_global_id(): the device array itself. The context sorts its atoms by cell at every
 * list build (owned atoms stay in [0, n_owned), ghosts behind them), so positions in these arrays change then;
 * DSMD_GLOBAL_ID identifies the atoms. */
int dsmd_device_pointer(dsmd_ctx* ctx, int field, void** out);
int dsmd_counts(const dsmd_ctx* ctx, int64_t* n_owned, int64_t* n_total);

/* ParticleInfo::Provider::resize_particle_info (src/force_calculator_cuda.cu:4143-4216): sets the owned / total counts
 * after the caller wrote atoms into the device arrays itself (halo exchange, migration). */
int dsmd_set_counts(dsmd_ctx* ctx, int64_t n_owned, int64_t n_total);

/* -- neighbour list -------------------------------------------------------------------------------------------------- */

/* ForceCalculatorCUDA::build_neighbor_list_on_device (src/force_calculator_cuda.cu:4604) = launch_cuda_tile_list_build
 * (src/neighbor_list_kernels.cu:554) + build_tile_lists_on_device (:4817): bins the atoms into cells, sorts them by
 * cell (owned and ghost segments separately), reorders every particle array, converts positions to the fixed-point
 * layout and builds the per-atom Verlet list with skin. Takes the current positions as the displacement reference
 * (update_reference_positions_on_device). Synchronises `stream` once to read the build status. */
int dsmd_build_neighbor_list(dsmd_ctx* ctx, void* stream);

/* The same, split for the multi-GPU rebuild step: sort only the owned atoms (before the halo plan is made), so that
 * their slots stay fixed when the ghosts arrive. */
int dsmd_sort_owned(dsmd_ctx* ctx, void* stream);

/* The owned-atom sort of a rebuild step that follows a migration (MDSystem::migrate_particles_on_device,
 * src/md_system.cpp:1495-1509): the n_outside owned atoms that lie outside the brick [lo, hi) on a split axis have been
 * sent to their new owners and are removed (they sort behind every cell and fall off the end; the owned count shrinks by
 * n_outside), arrivals that were appended behind the owned atoms are sorted in. Does not synchronise: the status of
 * this sort is read together with that of the dsmd_build_neighbor_list call that must follow. */
int dsmd_sort_owned_in_brick(dsmd_ctx* ctx, const double lo[3], const double hi[3], const int split[3], int64_t n_outside,
                             void* stream);

/* After a build: ghost_slot[k] = the slot, in the sorted arrays, of the k-th ghost as it was handed in (device int32
 * array of n_total - n_owned entries). The halo refresh unpacks through it. */
int dsmd_ghost_slots(dsmd_ctx* ctx, const int32_t** device_ghost_slot);

/* List statistics of the last build. pairs_listed counts directed entries (each owned-owned pair twice). */
int dsmd_list_stats(dsmd_ctx* ctx, int64_t* directed_entries, int64_t* interior_entries, int32_t* row_stride,
                    int32_t* cells, int32_t* rechecked_fp64);

/* Writes the list as directed (i, j) slot pairs into device int32 arrays of `capacity` entries each (test and parity
 * hook; the reference's counterpart is NeighborList::get_neighbors / get_offsets, include/neighbor_list.h:37-39).
 * flags[k] bit 0 = excluded pair. Returns the count in *n_pairs. Synchronises. */
int dsmd_list_export(dsmd_ctx* ctx, int32_t* device_i, int32_t* device_j, uint8_t* device_flags, int64_t capacity,
                     int64_t* n_pairs, void* stream);

/* -- per-step work ---------------------------------------------------------------------------------------------------- */

/* nlist_pack_slots_kernel (src/force_calculator_cuda.cu:1168) fused with compute_max_displacement_kernel (:6637):
 * converts the current double positions of atoms [first, first + count) to the fixed-point layout the pair kernel
 * reads and folds max |r - r_ref|^2 of the owned ones into the displacement word. */
int dsmd_pack_positions(dsmd_ctx* ctx, int64_t first, int64_t count, void* stream);

/* compute_max_displacement_on_device (:6689): max displacement^2 since the last build as of the last pack.
 * Synchronises `stream`. */
int dsmd_max_displacement_sq(dsmd_ctx* ctx, double* out, void* stream);

/* compute_max_displacement_lagged (src/force_calculator_cuda.cu:6723-6764): queues the read-back of the current value and
 * returns the one queued by the PREVIOUS call, so the host never waits for the step in flight; negative when there is
 * none yet, or when the list has been rebuilt since (the reference positions that value was measured against are gone). */
int dsmd_max_displacement_sq_lagged(dsmd_ctx* ctx, double* out, void* stream);

/* The device word behind it: the bit pattern of that non-negative double, 8 bytes. Bit patterns of non-negative doubles
 * order like the values, so ranks can take a MAX over it as a 64-bit integer (CommBackend::unify_rebuild_decision,
 * src/comm_backend.cpp:85) without a host round trip. Reset to zero by every list build. */
int dsmd_displacement_word(dsmd_ctx* ctx, void** device_word);

/* ForceCalculator::compute_forces / begin_forces_interior / finish_forces_boundary (include/force_calculator.h:24,
 * include/force_calculator_cuda.h:160-170): LJ (+ real-space Ewald) over the list. FULL and INTERIOR overwrite the
 * force arrays of the owned atoms (the reference clears, then adds); BOUNDARY adds the ghost-partner part.
 * want_energy != 0 also accumulates potential energy and virial (scalar + diagonal) in fp64. */
int dsmd_compute_forces(dsmd_ctx* ctx, int phase, int want_energy, void* stream);

/* get_potential_energy / get_virial / get_virial_diag (include/force_calculator.h:41-68): this rank's sums of the last
 * evaluation with want_energy (an owned-ghost pair counts half on each rank). out = {PE, W, Wxx, Wyy, Wzz, pairs}:
 * pairs = how many pairs were inside the cutoff (the count of ForceCalculator::get_lj_pair_counts, summed).
 * Synchronises `stream`. */
int dsmd_read_scalars(dsmd_ctx* ctx, double out[6], void* stream);

/* Optional: declares that every atom's charge is a function of its type (rigid water models, ions, united-atom and
 * coarse-grained force fields) and gives that function. The pair kernel then takes a partner's charge from a table in
 * shared memory, indexed by the type that arrives with the partner's position, instead of gathering it from the per-atom
 * array. ntypes must equal dsmd_set_pair_params'; atoms already uploaded are checked against the table
 * (DSMD_ERR_INVALID on a mismatch), atoms that arrive later (ghosts, migrated atoms) are the caller's word. The per-atom
 * charges stay in place for everything else (special pairs, downloads). Null or ntypes <= 0 switches back. No counterpart
 * in the reference, whose kernels read per-atom charges (src/force_calculator_cuda.cu:1604-1860). */
int dsmd_set_type_charges(dsmd_ctx* ctx, int ntypes, const double* charge_of_type);

/* Bonded terms and scaled special (1-4) pairs (compute_bond_forces_kernel, compute_angle_forces_kernel,
 * compute_dihedral_forces_kernel, compute_improper_forces_kernel, compute_special_pair_forces_kernel,
 * src/force_calculator_cuda.cu:2703-3170; MDSystem::LocalBond ... LocalSpecialPair, include/md_system.h:22-42). Atoms are
 * named by global id (< n_global); every term carries its own parameters:
 *   bonds     U = k/2 (r - r0)^2;   angles   U = k/2 (theta - theta0)^2 (radians, vertex = the second atom);
 *   torsions  (proper dihedrals and impropers alike) n > 0: U = k (1 + cos(n phi - phi0)); n = 0: U = k (phi - phi0)^2 with
 *             the difference wrapped to (-pi, pi];
 *   specials  4 eps ((sigma/r)^12 - (sigma/r)^6) lj_scale + 332.0636 qi qj / r coulomb_scale (charges from the context).
 * Replaces any earlier set; all counts zero clears. On several ranks give every rank the whole table: a term is evaluated
 * where one of its atoms is owned, forces go to owned atoms only, energy and virial where the lowest global id is owned
 * (the reference's rule). */
int dsmd_set_bonded(dsmd_ctx* ctx, int64_t n_global, int64_t n_bonds, const int32_t* bond_atoms, const double* bond_k,
                    const double* bond_r0, int64_t n_angles, const int32_t* angle_atoms, const double* angle_k,
                    const double* angle_theta0, int64_t n_torsions, const int32_t* torsion_atoms, const double* torsion_k,
                    const double* torsion_phi0, const int32_t* torsion_n, int64_t n_specials, const int32_t* special_atoms,
                    const double* special_sigma, const double* special_epsilon, const double* special_lj_scale,
                    const double* special_coulomb_scale);

/* ADDS the forces of the bonded terms to the force arrays of the owned atoms (call after dsmd_compute_forces of the FULL
 * or BOUNDARY phase, when ghost positions are current) and leaves their energy and virial for dsmd_read_bonded_scalars.
 * Forces are summed per atom in a fixed order (bitwise reproducible). Needs a list build since the last change of the
 * atom set (terms find their atoms through the sorted arrays). dsmd_run_nve calls it every step. */
int dsmd_compute_bonded(dsmd_ctx* ctx, void* stream);

/* out = {PE, W, Wxx, Wyy, Wzz} of the last dsmd_compute_bonded on this rank (bonds and specials contribute to W and the
 * diagonal, angles and torsions to the diagonal only: their trace is zero). Synchronises `stream`. DSMD_ERR_STATE when
 * a term had an owned atom whose partner was not on this rank (halo narrower than the term is long). */
int dsmd_read_bonded_scalars(dsmd_ctx* ctx, double out[5], void* stream);

/* Velocity Verlet halves (launch_vv_step1_kernel / launch_vv_step2_kernel, src/integrator_kernels.cu:149-208):
 * half 1: v += dt/2 f/m c; x += dt v (and packs positions, see dsmd_pack_positions); half 2: v += dt/2 f/m c;
 * half 3: half 2 of the previous step and half 1 of this one in one pass (v += dt f/m c; x += dt v; pack), for loops in
 * which nobody reads the velocities between two steps (dsmd_run_nve and dsmd_domain_run use it after their first step
 * and end on a plain half 2); not available with constraints, where RATTLE sits between the two. */
int dsmd_integrate(dsmd_ctx* ctx, int half, double dt, double force_to_accel, void* stream);

/* calculate_kinetic_energy (include/force_calculator.h:70): sum 1/2 m v^2 over owned atoms, raw units. Synchronises. */
int dsmd_kinetic_energy(dsmd_ctx* ctx, double* out, void* stream);

/* Thermostat of the velocity-scaling kind (launch_nose_hoover_thermostat_kernel, src/thermostat_kernels.cu:68-76,
 * 131-141): multiplies the velocities of the owned atoms by `factor` (which the host computes from the kinetic energy,
 * src/thermostat.cpp:78-95). */
int dsmd_scale_velocities(dsmd_ctx* ctx, double factor, void* stream);

/* The MD loop of MDSimulation::single_step (src/md_simulation.cpp:899-941) restricted to this path: n_steps of
 * integrate-1 + pack, rebuild decision (max displacement > (hi_frac skin)^2, or every `every` steps when every > 0;
 * lagged != 0 uses the previous step's read-back, extrapolated, as the reference does on several ranks), list rebuild,
 * forces, integrate-2. Single-rank systems only (no ghosts). Returns the number of rebuilds and the largest
 * displacement that was ever in effect when forces were evaluated (to check the skin was never outrun). */
int dsmd_run_nve(dsmd_ctx* ctx, int64_t n_steps, double dt, double force_to_accel, double hi_frac, int every, int lagged,
                 int64_t* n_rebuilds, double* worst_disp_sq, void* stream);

/* One force evaluation with host buffers, as a force-provider plugin is called: uploads positions (context order),
 * packs, evaluates, downloads forces (and the six scalars of dsmd_read_scalars when out6 != NULL). Rebuilds the list first when rebuild != 0.
 * Without rebuild and without out6, on a single-rank system tall enough to cut into at least four slabs of cell layers,
 * the call runs as a pipeline over two internal copy streams: slabs of the sorted atoms are uploaded, evaluated and
 * downloaded side by side (the same forces, bit for bit); pinned host buffers are what makes the copies overlap.
 * Synchronises. */
int dsmd_forces_host(dsmd_ctx* ctx, const double* x, const double* y, const double* z, int rebuild, double* fx,
                     double* fy, double* fz, double* out6, void* stream);

/* Kernel launches issued by this context so far (benchmark bookkeeping). */
int64_t dsmd_launch_count(const dsmd_ctx* ctx);

/* Queues a kernel of independent fp32 FMA chains on every SM and returns its flop count; the caller times it to get the
 * fp32 CUDA-core peak of this device (the compute-roofline denominator of the pair kernel). No reference counterpart. */
int dsmd_fma_probe(dsmd_ctx* ctx, int iters, double* flops, void* stream);

/* -- halo (ghost atoms) ----------------------------------------------------------------------------------------------- */

/* The data-plane half of MDSystem::exchange_halo_on_device (src/md_system.cpp:1448-1463); the transport between the
 * two calls is the caller's (NCCL send/recv).
 * pack: gathers positions of the owned atoms listed in device_send_index[0..count) into device_out as 3 doubles per
 * atom, adding device_image[3 * k + a] box lengths on axis a (the periodic image the receiving neighbour sees; NULL = no
 * shift). One launch serves every neighbour: the caller lays the send list out neighbour after neighbour. */
int dsmd_halo_pack(dsmd_ctx* ctx, const int32_t* device_send_index, const int8_t* device_image, int64_t count,
                   double* device_out, void* stream);
/* unpack: writes `count` received positions (3 doubles each) to the ghosts first_ghost .. first_ghost + count of the
 * hand-in order, i.e. to slots ghost_slot[first_ghost + k], in both the double arrays and the fixed-point layout. */
int dsmd_halo_unpack(dsmd_ctx* ctx, const double* device_in, int64_t first_ghost, int64_t count, void* stream);
/* Selects the owned atoms within [lo, hi) (a neighbour's brick grown by the halo, already shifted into this rank's
 * frame) into device_send_index; *count returns how many. Synchronises. */
int dsmd_halo_select(dsmd_ctx* ctx, const double lo[3], const double hi[3], int32_t* device_send_index, int64_t capacity,
                     int64_t* count, void* stream);
/* Full records for a plan (re)build: packs {x, y, z, vx, vy, vz, mass, charge} (+shift) as 8 doubles and
 * {type, gid} as 2 int32 per listed atom; append writes such records behind the current atoms as new ghosts. */
int dsmd_halo_pack_records(dsmd_ctx* ctx, const int32_t* device_send_index, int64_t count, const double shift[3],
                           double* device_real_out, int32_t* device_int_out, void* stream);
int dsmd_halo_append_records(dsmd_ctx* ctx, const double* device_real_in, const int32_t* device_int_in, int64_t count,
                             void* stream);

/* The same records as one run of nine doubles per atom - x y z vx vy vz mass charge and, in the ninth, the two int32 words
 * type (low) and global id (high) - so that one message per neighbour rank carries every field. */
int dsmd_halo_append_packed(dsmd_ctx* ctx, const double* device_records, int64_t count, void* stream);

/* The capacity the context was created with (ParticleInfo::Provider sizing, src/force_calculator_cuda.cu:4143-4216). */
int dsmd_capacity(const dsmd_ctx* ctx, int64_t* capacity);

/* -- several GPUs: bricks, migration, ghost plan, MD loop --------------------------------------------------------------- */

typedef struct dsmd_domain dsmd_domain;

/* The 128-byte NCCL unique id that rank 0 creates and hands to the other ranks by whatever channel the engine has (the
 * reference broadcasts it over MPI: src/force_calculator_cuda.cu:7524-7530). nccl_library_path may be NULL (the loader's
 * search path is used). */
int dsmd_nccl_unique_id(const char* nccl_library_path, char out[128]);

/* One rank's view of a dims[0] x dims[1] x dims[2] brick grid over the periodic box (rank = (cx * dims[1] + cy) * dims[2] + cz;
 * the context's box must have been set to this rank's brick, see dsmd_set_box). halo_width = how far ghosts are taken from
 * neighbouring bricks (cutoff + skin); skin = the Verlet skin of the rebuild vote. With world > 1 an NCCL communicator is
 * created (collective over the ranks). What the reference gets from dsdecompx::Decomp (src/md_system.cpp:853-993). */
int dsmd_domain_create(dsmd_ctx* ctx, int rank, int world, const int dims[3], const double box[3], double halo_width,
                       double skin, const char* nccl_library_path, const char unique_id[128], dsmd_domain** out);
void dsmd_domain_destroy(dsmd_domain* dom);
const char* dsmd_domain_last_error(const dsmd_domain* dom);

/* The rebuild step (MDSimulation::handle_neighbor_phase on a rebuild, src/md_simulation.cpp:1316-1401): send the atoms that
 * left the brick to their new owners (MDSystem::migrate_particles_on_device; only leavers and arrivals move), sort the
 * owned atoms, select and exchange the ghosts' full records (exchange_halo_on_device(rebuild = true)), build the list.
 * One message per neighbour RANK and way (at most 7 ranks on a 2 x 2 x 2 grid), no allocation. Collective; synchronises
 * `stream` four times (leaver counts, ghost counts, list status, agreement on the status), each wait bounded by the wait
 * limit. Every rank returns the same status: lost atoms, missing room and a failed list build are decided from values
 * that all ranks exchange. */
int dsmd_domain_rebuild(dsmd_domain* dom, void* stream);

/* Host waits of the domain (message sizes, votes) poll against this limit and return DSMD_ERR_TIMEOUT when it runs out
 * (default 120 s, or the environment's DSMD_WAIT_LIMIT_S). After a time-out the run cannot go on: call dsmd_domain_abort,
 * which aborts the communicators so that kernels still waiting for the missing rank are released (the reference's
 * behaviour on a failed rank: exception -> MPI_Abort, src/main.cpp:85-93). */
int dsmd_domain_set_wait_limit(dsmd_domain* dom, double seconds);
int dsmd_domain_abort(dsmd_domain* dom);

/* Positions-only ghost refresh (begin + end_halo_exchange_on_device, src/md_system.cpp:1465-1493): pack, grouped
 * ncclSend / ncclRecv with the neighbour directions, unpack, on the domain's side stream; `stream` then waits for it. */
int dsmd_domain_refresh(dsmd_domain* dom, void* stream);

/* dsmd_forces_host on several ranks: this rank's owned atoms' positions in (host buffers, the context's order), then
 * either the rebuild step (with_rebuild != 0: migration, ghosts, list; the owned set and its order may change, ask
 * dsmd_counts / DSMD_GLOBAL_ID afterwards) and a full pass, or pack, ghost refresh beside the interior pass and the
 * boundary pass; the owned atoms' forces out. buffer_atoms = how many atoms each host buffer holds (a rebuild may bring
 * atoms in: DSMD_ERR_CAPACITY when they do not fit). Collective; waits with the domain's deadline. */
int dsmd_domain_forces_host(dsmd_domain* dom, const double* x, const double* y, const double* z, int with_rebuild,
                            double* fx, double* fy, double* fz, int64_t buffer_atoms, void* stream);

/* n_steps MD steps (MDSimulation::single_step, src/md_simulation.cpp:899-941, restricted to this path): first
 * velocity-Verlet half + pack, rebuild vote (8-byte MAX all-reduce on a communicator and stream of its own, read one step
 * late and extrapolated), then either a rebuild + full force pass, or the ghost refresh on the side stream overlapped
 * with the interior force pass followed by the boundary pass; second half. Collective. Returns DSMD_ERR_TIMEOUT when a
 * vote does not arrive within the wait limit. */
int dsmd_domain_run(dsmd_domain* dom, int64_t n_steps, double dt, double force_to_accel, double hi_frac, void* stream);

/* MDSystem::reverse_halo_on_device (src/md_system.cpp:1511-1518): the forces this rank holds on its ghost atoms travel back
 * along the ghost plan and are added to the forces of the owners (one message per neighbour rank and way). The force
 * arrays are the context's (DSMD_FX ...). Queued on `stream`; collective. */
int dsmd_domain_reverse_forces(dsmd_domain* dom, void* stream);

/* MDSystem::exchange_field_on_device (src/md_system.cpp:1520-1545; contract include/MLIPHaloTransport.h:16-37): a
 * row-major device array [rows, width] of float (element_bytes 4) or double (8), rows = owned atoms then ghosts in the
 * context's current order. reverse == 0: the rows of the ghosts are overwritten with the rows of their owners;
 * reverse != 0: the rows of the ghosts are added to the rows of their owners. Queued on `stream`; collective. */
int dsmd_domain_exchange_field(dsmd_domain* dom, void* device_data, int64_t rows, int64_t width, int element_bytes,
                               int reverse, void* stream);

/* CommBackend::max_reduce / sum_reduce / sum_reduce3 (include/comm_backend.h:24-33): n host doubles (n <= 16) combined
 * over the ranks in place, op 0 = sum, 1 = max; every rank gets the result. Collective; synchronises `stream` (bounded). */
int dsmd_domain_reduce(dsmd_domain* dom, double* values, int n, int op, void* stream);

/* The distinct neighbour ranks of this brick and how many messages one exchange of the current ghost plan posts. */
int dsmd_domain_peers(const dsmd_domain* dom, int32_t* n_peers, int32_t peers[26], int32_t n_messages_per_exchange[1]);

/* Per-phase device times of dsmd_domain_run, accumulated while enabled (profiling mode synchronises every step, so the
 * totals are not a benchmark): phase_ms = {integrate 1 + pack, vote, refresh issue + interior forces (or nothing),
 * boundary forces incl. the wait for the refresh (or the full pass), integrate 2, rebuild, and the wall time of the
 * rebuild's four parts: migration, sort of the owned atoms, ghost plan, list build}. Returns the sums so far. */
int dsmd_domain_profile(dsmd_domain* dom, int enable, double phase_ms[10], int64_t* steps);

int dsmd_domain_stats(const dsmd_domain* dom, int64_t* rebuilds, int64_t* migrated_atoms, int64_t* ghosts,
                      int64_t* positions_sent_per_step, double* worst_disp_sq, int64_t* launches);

/* -- radius graph ------------------------------------------------------------------------------------------------------ */

typedef struct dsmd_edges dsmd_edges;

/* EdgeBuilder (include/EdgeBuilder.cuh:12-84). */
int dsmd_edges_create(int device, dsmd_edges** out);
void dsmd_edges_destroy(dsmd_edges* eb);
const char* dsmd_edges_last_error(const dsmd_edges* eb);

/* EdgeBuilder::build (include/EdgeBuilder.cuh:52-55): every ordered pair (i, j), i != j, |r_j - r_i| < cutoff over the n
 * atoms given (no minimum image). lo / hi: optional host box containing every atom. n_centers < n with owner / shift
 * arrays = EdgeBuilder::Images; receiver_ok / row = EdgeBuilder::Prune (NULL keeps every edge).
 * Results stay valid until the next build: edge_index int64 [2 * E] (row 0 = i, row 1 = j), edge_shift double [E * 3]
 * (written only with images). *n_edges returns E after the single synchronisation of `stream`. */
int dsmd_edges_build(dsmd_edges* eb, const double* d_x, const double* d_y, const double* d_z, int64_t n, double cutoff,
                     const double* lo, const double* hi, int64_t n_centers, const int32_t* d_owner,
                     const double* d_shift_x, const double* d_shift_y, const double* d_shift_z,
                     const unsigned char* d_receiver_ok, int row, int64_t* n_edges, void* stream);
int dsmd_edges_result(const dsmd_edges* eb, const int64_t** d_edge_index, const double** d_edge_shift, int64_t* n_edges);

/* Periodic image atoms for the axes a model sees as periodic but the MD does not decompose (MLIPStep::prepare,
 * src/MLIPStep.cu:31-103, 214-260): positions are wrapped from `origin` on the axes with shells > 0, and every image
 * (sx, sy, sz) != 0, |s_a| <= shells[a], that lies inside [region_lo, region_hi] on every image axis is appended behind
 * the n wrapped atoms (images of atom i are consecutive, in the order sx, sy, sz ascending). Results (valid until the next
 * call): positions, types, the atom each entry copies and its offset from it - the arrays EdgeBuilder::Images wants.
 * *n_all returns n + images after the single synchronisation of `stream`. */
int dsmd_images_build(dsmd_edges* eb, const double* d_x, const double* d_y, const double* d_z, const int32_t* d_type,
                      int64_t n, const double box[3], const double origin[3], const double region_lo[3],
                      const double region_hi[3], const int shells[3], int64_t* n_all, void* stream);
int dsmd_images_result(const dsmd_edges* eb, const double** d_x, const double** d_y, const double** d_z,
                       const int32_t** d_type, const int32_t** d_owner, const double** d_shift_x, const double** d_shift_y,
                       const double** d_shift_z, int64_t* n_all);

/* MLIPStep::add_forces (src/MLIPStep.cu:108-124, 373-381): target[i] += f[i] + the forces on the images of atom i (in the
 * order the images were created), for the first n_out of the atoms the last dsmd_images_build was given (n_out < 0: all
 * of them). d_f*: the model's forces on all n_all atoms of that build; with_images == 0 adds f[i] alone (the images were
 * used as edge shifts, not as atoms). Queued on `stream`. */
int dsmd_images_fold_forces(dsmd_edges* eb, const double* d_fx, const double* d_fy, const double* d_fz, int64_t n_out,
                            int with_images, double* d_target_x, double* d_target_y, double* d_target_z, void* stream);

/* MLIPStep::virial / virial_diag (src/MLIPStep.cu:126-148, 383-432): out = {sum r.F, sum x Fx, sum y Fy, sum z Fz} over the
 * n atoms given (owned, ghosts and images alike), summed in a fixed order. Synchronises `stream`. */
int dsmd_virial_from_forces(dsmd_edges* eb, const double* d_x, const double* d_y, const double* d_z, const double* d_fx,
                            const double* d_fy, const double* d_fz, int64_t n, double out[4], void* stream);

/* Receiver mask (mark_receivers_kernel, src/MLIPStep.cu:150-161): d_ok[i] = 1 when atom i lies within `reach` (Euclidean
 * distance) of the box [lo, hi]; a NaN position gives 0. The mask EdgeBuilder::Prune wants. */
int dsmd_mark_receivers(dsmd_edges* eb, const double* d_x, const double* d_y, const double* d_z, int64_t n,
                        const double lo[3], const double hi[3], double reach, unsigned char* d_ok, void* stream);

/* Compact periodic radius graph (no image atoms): n atoms in an orthorhombic periodic box; directed edges as
 * int32 src / dst, int8 lattice shift [E * 3] (dst image = pos[dst] + shift * box, in the coordinates as given, which
 * need not be wrapped into the box; shifts beyond +-127 do not fit) and fp32 edge vectors [E * 3]. Edges are grouped by
 * src, centres in cell order and the neighbours of a centre in the order of the search, as in the interface form (the
 * same order for the same input).
 * No counterpart in the reference, which feeds images as explicit atoms. */
int dsmd_edges_build_periodic(dsmd_edges* eb, const double* d_x, const double* d_y, const double* d_z, int64_t n,
                              const double box[3], double cutoff, int64_t* n_edges, void* stream);
int dsmd_edges_result_compact(const dsmd_edges* eb, const int32_t** d_src, const int32_t** d_dst,
                              const int8_t** d_shift, const float** d_vec, int64_t* n_edges);

/* -- without device allocation ------------------------------------------------------------------------------------------ */

/* Largest atom count dsmd_kinetic_energy_noalloc accepts: its scratch array (one double per 256 atoms, 512 KiB) is
 * compiled into the library for this size. */
#define DSMD_NOALLOC_MAX_ATOMS 16777216

/* No counterpart in the reference. The kinetic-energy sum of dsmd_kinetic_energy (sum of m v^2 / 2 over n atoms, raw
 * units), for callers that must not allocate device memory: a plugin called from inside an engine's step loop, where the
 * engine's pools already own the device memory and a cudaMalloc would either fail or stall every stream of the step by
 * synchronising the device. The caller passes device arrays and a device double for the result; the per-block partial
 * sums live in a fixed array inside the library image, which every GPU that loads the library holds (512 KiB) until the
 * process exits. Neither this call nor anything it calls allocates or frees memory.
 *   - n > DSMD_NOALLOC_MAX_ATOMS is refused with DSMD_ERR_CAPACITY and a message in *error (error may be NULL).
 *   - The first call on a device looks up the array's device address (once per device, with that device current); make
 *     that first call before any stream capture begins.
 *   - All calls on a device share the one array, which keeps what the last call wrote. Each call overwrites every
 *     entry it later reads, so nothing needs clearing between calls; but two calls whose kernels overlap on the GPU
 *     (different streams, no ordering between them) race on it and give wrong sums. Order them on one stream or with events.
 * Queued on `stream`; the result is in *d_out when the stream reaches that point. Uses the current device. */
int dsmd_kinetic_energy_noalloc(const double* d_vx, const double* d_vy, const double* d_vz, const double* d_mass,
                                int64_t n, double* d_out, void* stream, const char** error);

#ifdef __cplusplus
}
#endif
#endif /* DSMD_B200_H */
