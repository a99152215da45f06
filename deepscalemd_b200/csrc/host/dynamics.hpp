// Host-side pieces of the MD driver around the device path: unit constants of the reference (LAMMPS "real" units),
// Maxwell-Boltzmann start velocities (src/md_system.cpp:205-275) and the Nose-Hoover velocity-scaling thermostat
// (src/thermostat.cpp:78-95).
#pragma once

#include <cstdint>
#include <vector>

namespace dsmd::host {

constexpr double kBoltzmann = 0.0019872041;                  // kcal / (mol K)   (include/md_types.h:13)
constexpr double kForceToAccel = 4.184e-4;                   // (kcal/mol/A) / (g/mol) -> A / fs^2   (include/md_types.h:15)
constexpr double kMvv2e = 48.88821291 * 48.88821291;         // (g/mol)(A/fs)^2 -> kcal/mol   (include/md_types.h:17)

// Every component Gaussian with variance kT/m, centre-of-mass motion removed, scaled to exactly T with 3N - 3 degrees of
// freedom. The reference seeds from std::random_device; here the seed is an input so that runs can be repeated.
void maxwell_boltzmann(const std::vector<double>& mass, double temperature, uint64_t seed, std::vector<double>& vx,
                       std::vector<double>& vy, std::vector<double>& vz);

// Kinetic energy in kcal/mol of velocities in A/fs.
double kinetic_energy_kcal(const std::vector<double>& mass, const std::vector<double>& vx, const std::vector<double>& vy,
                           const std::vector<double>& vz);

// Instantaneous temperature from a kinetic energy in kcal/mol (3N - constraints degrees of freedom, as the reference's
// printed T).
double temperature_of(double kinetic_kcal, int64_t atoms, int64_t constraints);

// One application of the Nose-Hoover thermostat: advances the friction variable xi by half a step from the current
// kinetic energy, returns the factor the velocities are multiplied by, and advances xi by the second half step from the
// scaled kinetic energy. kinetic_kcal is the whole system's; tau in fs; dof_fraction = (3N - constraints) / 3N.
double nose_hoover_scale(double kinetic_kcal, int64_t atoms, double target_temperature, double tau, double dt, double& xi,
                         double dof_fraction);

}  // namespace dsmd::host
