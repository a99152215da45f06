/* C ABI of the host-side input layer (libdsmd_input.so): the reference's run description, coordinate, topology /
 * parameter and restart files, read into plain arrays that feed the device path of dsmd_b200.h. No CUDA here.
 *
 * What each entry point replaces in the reference (sjseo00/DeepScaleMD):
 *   dsmd_input_config_*   MDSimulation::parse_simulation_config          src/md_simulation.cpp:2753-3100
 *                         read_dsmd_input_manifest                        src/md_simulation.cpp:280-303
 *   dsmd_input_system_*   MDSystem::load_standard_xyz                     src/md_system.cpp:562-671
 *                         Topology::load_topology / load_canonical        src/topology.cpp:335-881
 *                         MDSystem::setup_force_field_params              src/md_system.cpp:716-790
 *                         MDSystem::initialize_velocities                 src/md_system.cpp:205-275
 *   dsmd_input_restart_*  MDSimulation::read_restart_file / write_restart_file   src/md_restart.cpp:110-300
 *   dsmd_input_nose_hoover_scale   nose_hoover_scale                      src/thermostat.cpp:78-95
 *
 * Every function returns 0 on success and a non-zero code otherwise; the message of the last failure of the calling
 * thread is available from dsmd_input_last_error(). Pointers handed out stay valid until the object is destroyed.
 */
#ifndef DSMD_INPUT_H
#define DSMD_INPUT_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DSMD_INPUT_OK 0
#define DSMD_INPUT_ERR_INVALID 1   /* null pointer, bad argument */
#define DSMD_INPUT_ERR_FORMAT 2    /* file missing, unreadable or not in the expected format (see the message) */

typedef struct dsmd_input_config dsmd_input_config;
typedef struct dsmd_input_system dsmd_input_system;

const char* dsmd_input_last_error(void);

/* Run description (YAML subset). */
int dsmd_input_config_read(const char* path, dsmd_input_config** out);
void dsmd_input_config_destroy(dsmd_input_config* config);
/* The resolved configuration as one JSON object (typed keys, "unsupported": what this path does not run, "entries": every
 * key read, as text). */
int dsmd_input_config_json(const dsmd_input_config* config, const char** json);

/* Particle system: coordinates + topology (+ parameters) named by the configuration; recentred into the box; velocities
 * zero until dsmd_input_system_velocities or dsmd_input_system_apply_restart. */
int dsmd_input_system_load(const dsmd_input_config* config, dsmd_input_system** out);
/* The same from explicit file names (parameter_file NULL or "": topology_file is a legacy .top; topology_file NULL or "":
 * coordinates only). */
int dsmd_input_system_load_files(const char* coordinate_file, const char* topology_file, const char* parameter_file,
                                 const double box[3], dsmd_input_system** out);
void dsmd_input_system_destroy(dsmd_input_system* system);
int dsmd_input_system_counts(const dsmd_input_system* system, int64_t* atoms, int32_t* types, int64_t* exclusions,
                             int64_t* constraints, int32_t* explicit_pairs);
/* Field: 0 x, 1 y, 2 z, 3 vx, 4 vy, 5 vz, 6 mass, 7 charge (double[atoms]). */
int dsmd_input_system_real(const dsmd_input_system* system, int field, const double** data);
int dsmd_input_system_types(const dsmd_input_system* system, const int32_t** type);
/* epsilon and sigma: double[types * types], row-major, symmetric; Mie exponents (12, 6 for Lennard-Jones). */
int dsmd_input_system_pair_table(const dsmd_input_system* system, const double** epsilon, const double** sigma,
                                 int32_t* mie_n, int32_t* mie_m);
/* pairs: int32[2 * exclusions] (smaller id, larger id), sorted, unique: the form dsmd_set_exclusions takes. */
int dsmd_input_system_exclusions(const dsmd_input_system* system, const int32_t** pairs);
/* i, j: int32[constraints]; distance: double[constraints]. */
int dsmd_input_system_constraints(const dsmd_input_system* system, const int32_t** i, const int32_t** j,
                                  const double** distance);
/* The bonded terms of a dsMD_input system with the parameters of every term written out, in the form dsmd_set_bonded
 * takes (Topology::load_canonical, src/topology.cpp:601-665, 760-796: angles and phases converted to radians, a harmonic
 * improper = multiplicity 0, a special pair without a listed parameter id takes the pair matrix of its atom types).
 * counts = {bonds, angles, torsions (dihedrals + impropers), dihedrals among them (they come first), special pairs};
 * atoms = {bond, angle, torsion, special} atom ids (2, 3, 4, 2 per term); parameters = {bond k, r0, angle k, theta0,
 * torsion k, phi0, special sigma, epsilon, LJ scale, Coulomb scale}. Null entries are skipped. A legacy .top system gives
 * zero counts (its bonded sections are counted by dsmd_input_system_counts only). */
int dsmd_input_system_bonded(const dsmd_input_system* system, int64_t counts[5], const int32_t** atoms[4],
                             const double** parameters[10], const int32_t** torsion_multiplicity);
/* Maxwell-Boltzmann velocities at the temperature (K) from the seed (A/fs). */
int dsmd_input_system_velocities(dsmd_input_system* system, double temperature, uint64_t seed);

/* Restart files. read: positions and velocities of the system are replaced (atom counts must agree); step, box (3),
 * thermostat state xi (0 when the file holds none or another thermostat) are returned. */
int dsmd_input_restart_read(const char* path, dsmd_input_system* system, int64_t* step, double box[3], double* timestep,
                            char thermostat_name[64], double* xi);
int dsmd_input_restart_write(const char* path, int64_t step, double timestep, const double box[3], const int32_t periodic[3],
                             const char* thermostat_name, const double* thermostat_state, int32_t n_thermostat_state,
                             int64_t atoms, const double* x, const double* y, const double* z, const double* vx,
                             const double* vy, const double* vz);

/* One Nose-Hoover application: returns the velocity scale in *scale and advances *xi (kinetic energy of the whole system
 * in kcal/mol, tau and dt in fs). */
int dsmd_input_nose_hoover_scale(double kinetic_kcal, int64_t atoms, double target_temperature, double tau, double dt,
                                 double dof_fraction, double* xi, double* scale);

/* -- host logic of the multi-GPU domain code, without a GPU (what the CPU tests drive) -------------------------------------
 * The decomposition library of the reference is external (dsDecompX 1.0, CMakeLists.txt:99); these are the host-side
 * decisions of its replacement, dsmd_domain_* in dsmd_b200.h. */

/* Neighbour directions of `rank` in a dims[0] x dims[1] x dims[2] periodic brick grid, ordered by destination rank
 * (dir_dest), the distinct neighbour ranks (peers, ascending) and how many of each peer's directions point back here. */
int dsmd_host_brick_plan(const int32_t dims[3], int32_t rank, int32_t* n_dirs, int32_t dir_dest[26], int32_t* n_peers,
                         int32_t peers[26], int32_t from_count[26]);

/* The verdict every rank reaches from the counts all ranks publish before a migration or ghost exchange
 * (counts[r * 29 + 0] stays, [1 + k] atoms along direction k, [27] atoms lost, [28] room left): *code = 0 to go on,
 * 4 when a rank lost atoms, 5 when arrivals exceed a rank's room; *about_rank says whose counts decided;
 * messages[r] = point-to-point messages rank r posts for these counts. The sentence is in dsmd_input_last_error(). */
int dsmd_host_counts_verdict(const int32_t dims[3], const int32_t* counts, int64_t scratch_capacity, int32_t* code,
                             int32_t* about_rank, int32_t messages[64]);

/* The real-space Ewald table the pair kernel evaluates (the builder behind dsmd_set_coulomb; the reference's is
 * ewald_real_table_build, include/ewald_real_table.h:41-105): 8 floats per interval, the force cubic then the energy
 * cubic. Returns the number of intervals; writes nothing when capacity_intervals is smaller. */
int dsmd_host_ewald_table(double alpha, double cutoff_sq, float* out, int32_t capacity_intervals);

/* Seeded random placement with a minimum distance in a periodic cube of edge `box` (uniform draws, a point is kept only
 * when it lies min_dist or more from every point kept before it): the disordered-solid input of the radius-graph build.
 * xyz receives n interleaved points; *draws (may be null) the number of draws made. The random stream is counter based, so
 * a seed gives the same points everywhere. Fails when the density cannot be reached. */
int dsmd_host_dart_throw(int64_t n, double box, double min_dist, uint64_t seed, double* xyz, int64_t* draws);

/* The bounded host wait of the domain code against a stand-in that becomes ready (or fails) after a number of polls,
 * -1 = never: returns 0 ready, 7 (DSMD_ERR_TIMEOUT) when limit_s ran out, 2 when the stand-in failed. */
int dsmd_host_wait_probe(double limit_s, int64_t ready_after_polls, int64_t fail_after_polls);

#ifdef __cplusplus
}
#endif

#endif /* DSMD_INPUT_H */
