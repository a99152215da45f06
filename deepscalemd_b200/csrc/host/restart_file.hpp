// Restart files "DSMDRST1" (layout: src/md_restart.cpp:3-12 of the reference): little-endian binary,
//   char[8] "DSMDRST1"; int64 step, atom count; double timestep (fs), box lx ly lz (A); int32 periodic x y z;
//   string thermostat name, int32 count + double[count] thermostat state (Nose-Hoover: xi);
//   string barostat name,   int32 count + double[count] barostat state;
//   double x[N] y[N] z[N] vx[N] vy[N] vz[N] in global atom id order; char[8] "DSMDEND1".
// A string is an int32 length and that many chars.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

namespace dsmd::host {

struct RestartState {
    int64_t step = 0;
    double timestep = 0.0;
    double box[3] = {0.0, 0.0, 0.0};
    int32_t periodic[3] = {1, 1, 1};
    std::string thermostat = "none", barostat = "none";
    std::vector<double> thermostat_state, barostat_state;
    std::vector<double> x, y, z, vx, vy, vz;   // by global atom id
};

// Throws std::runtime_error on a missing file, a wrong magic, a damaged length or an early end.
RestartState read_restart(const std::string& path);

// Writes to "<path>.tmp" and renames, so that a reader never sees half a file. Returns false when the file could not be
// written (the previous file, if any, is left as it was).
bool write_restart(const std::string& path, const RestartState& state);

}  // namespace dsmd::host
