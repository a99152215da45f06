#include "dynamics.hpp"

#include <algorithm>
#include <cmath>
#include <random>

namespace dsmd::host {

void maxwell_boltzmann(const std::vector<double>& mass, double temperature, uint64_t seed, std::vector<double>& vx,
                       std::vector<double>& vy, std::vector<double>& vz) {
    const size_t n = mass.size();
    vx.assign(n, 0.0);
    vy.assign(n, 0.0);
    vz.assign(n, 0.0);
    if (n == 0) return;
    std::mt19937_64 gen(seed);
    std::normal_distribution<double> normal(0.0, 1.0);
    for (size_t i = 0; i < n; ++i) {
        const double sigma = std::sqrt(kBoltzmann * std::max(temperature, 0.0) / (mass[i] * kMvv2e));
        vx[i] = sigma * normal(gen);
        vy[i] = sigma * normal(gen);
        vz[i] = sigma * normal(gen);
    }
    double px = 0.0, py = 0.0, pz = 0.0, total_mass = 0.0;
    for (size_t i = 0; i < n; ++i) {
        px += mass[i] * vx[i];
        py += mass[i] * vy[i];
        pz += mass[i] * vz[i];
        total_mass += mass[i];
    }
    const double cx = px / total_mass, cy = py / total_mass, cz = pz / total_mass;
    for (size_t i = 0; i < n; ++i) {
        vx[i] -= cx;
        vy[i] -= cy;
        vz[i] -= cz;
    }
    const double current = kinetic_energy_kcal(mass, vx, vy, vz);
    const double dof = 3.0 * static_cast<double>(n) - 3.0;
    const double target = 0.5 * dof * kBoltzmann * temperature;
    const double scale = current > 0.0 ? std::sqrt(target / current) : 0.0;
    for (size_t i = 0; i < n; ++i) {
        vx[i] *= scale;
        vy[i] *= scale;
        vz[i] *= scale;
    }
}

double kinetic_energy_kcal(const std::vector<double>& mass, const std::vector<double>& vx, const std::vector<double>& vy,
                           const std::vector<double>& vz) {
    double sum = 0.0;
    for (size_t i = 0; i < mass.size(); ++i) sum += 0.5 * mass[i] * (vx[i] * vx[i] + vy[i] * vy[i] + vz[i] * vz[i]);
    return sum * kMvv2e;
}

double temperature_of(double kinetic_kcal, int64_t atoms, int64_t constraints) {
    const double dof = 3.0 * static_cast<double>(atoms) - static_cast<double>(constraints);
    return dof > 0.0 ? 2.0 * kinetic_kcal / (dof * kBoltzmann) : 0.0;
}

double nose_hoover_scale(double kinetic_kcal, int64_t atoms, double target_temperature, double tau, double dt, double& xi,
                         double dof_fraction) {
    if (atoms <= 0 || target_temperature <= 0.0 || tau <= 0.0) return 1.0;
    const double dof = 3.0 * static_cast<double>(atoms) * dof_fraction;
    const double target_twice_ke = dof * kBoltzmann * target_temperature;
    const double thermostat_mass = target_twice_ke * tau * tau;
    if (!(thermostat_mass > 0.0)) return 1.0;
    xi += 0.5 * dt * (2.0 * kinetic_kcal - target_twice_ke) / thermostat_mass;
    const double scale = std::exp(-xi * dt);
    xi += 0.5 * dt * (2.0 * kinetic_kcal * scale * scale - target_twice_ke) / thermostat_mass;
    return scale;
}

}  // namespace dsmd::host
