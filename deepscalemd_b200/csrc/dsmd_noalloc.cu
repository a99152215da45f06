// Kinetic-energy sum without any device allocation.
//
// dsmd_kinetic_energy() keeps its per-block partial sums in a buffer that the context allocates with cudaMalloc (and
// grows when the atom count grows). Some callers of this library must not allocate: an MD engine that calls a plugin from
// inside its step loop has usually handed every byte of device memory to its own pools already, and a cudaMalloc there
// can fail outright or, because it synchronises the whole device, stall the halo and force streams that the step keeps in
// flight. For them this file offers the same sum with the partials kept in a fixed array that is part of the library
// image: nothing is allocated or freed, by this code or by any library routine it calls.
//
// The array is a file-scope __device__ object, so every GPU that loads the library holds its own copy of it (512 KiB) until
// the process exits, whether or not this entry point is ever called. Its name is a host-side handle, not a device address:
// the host code below asks the runtime for the address (cudaGetSymbolAddress) once per device, with that device current,
// and hands that pointer to the kernels.

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/dsmd_b200.h"

namespace {

constexpr int kBlock = 256;
constexpr int64_t kMaxAtoms = DSMD_NOALLOC_MAX_ATOMS;
constexpr int kMaxBlocks = static_cast<int>((kMaxAtoms + kBlock - 1) / kBlock);
constexpr int kMaxDevices = 64;

// One partial sum per thread block of the first kernel. Shared by every call on this device; holds whatever the last
// call left there.
static __device__ __align__(256) double g_partials[kMaxBlocks];

double* g_partials_address[kMaxDevices] = {};   // per device: where g_partials lives there (nullptr = not asked yet)

__global__ void __launch_bounds__(kBlock)
k_kinetic_partials(int64_t n, const double* __restrict__ vx, const double* __restrict__ vy,
                   const double* __restrict__ vz, const double* __restrict__ mass, double* __restrict__ partials) {
    const int64_t s = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    double v = 0.0;
    if (s < n) v = 0.5 * mass[s] * (vx[s] * vx[s] + vy[s] * vy[s] + vz[s] * vz[s]);
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    __shared__ double warp_sum[kBlock / 32];
    if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        double sum = 0.0;
        for (int w = 0; w < kBlock / 32; ++w) sum += warp_sum[w];
        partials[blockIdx.x] = sum;
    }
}

__global__ void __launch_bounds__(kBlock)
k_kinetic_total(const double* __restrict__ partials, int n_blocks, double* __restrict__ out) {
    __shared__ double sh[kBlock];
    double sum = 0.0;
    for (int b = threadIdx.x; b < n_blocks; b += blockDim.x) sum += partials[b];
    sh[threadIdx.x] = sum;
    __syncthreads();
    for (int o = blockDim.x / 2; o > 0; o >>= 1) {
        if (threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) out[0] = sh[0];
}

}  // namespace

extern "C" int dsmd_kinetic_energy_noalloc(const double* d_vx, const double* d_vy, const double* d_vz,
                                           const double* d_mass, int64_t n, double* d_out, void* stream,
                                           const char** error) {
    const char* ignored;
    if (!error) error = &ignored;
    *error = "";
    if (!d_vx || !d_vy || !d_vz || !d_mass || !d_out || n < 0) {
        *error = "dsmd_kinetic_energy_noalloc: null array or negative atom count";
        return DSMD_ERR_INVALID;
    }
    if (n > kMaxAtoms) {
        *error = "dsmd_kinetic_energy_noalloc: more atoms than DSMD_NOALLOC_MAX_ATOMS, the size the built-in scratch "
                 "array was compiled for; use dsmd_kinetic_energy, which allocates, or split the sum";
        return DSMD_ERR_CAPACITY;
    }
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
        *error = "dsmd_kinetic_energy_noalloc: no current CUDA device (or device ordinal beyond 63)";
        return DSMD_ERR_CUDA;
    }
    // Set-up, once per device, with that device current: the device address of this device's copy of the array.
    if (!g_partials_address[device]) {
        double* address = nullptr;
        const cudaError_t rc = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_partials);
        if (rc != cudaSuccess || !address) {
            *error = "dsmd_kinetic_energy_noalloc: cudaGetSymbolAddress failed for the scratch array";
            return DSMD_ERR_CUDA;
        }
        g_partials_address[device] = address;
    }
    double* partials = g_partials_address[device];
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int n_blocks = static_cast<int>((n + kBlock - 1) / kBlock);
    // Nothing has to be cleared: the second kernel reads exactly the n_blocks partials the first one has just written
    // (for n == 0 it reads none and writes 0), so what an earlier call left in the array is never seen.
    if (n_blocks > 0) k_kinetic_partials<<<n_blocks, kBlock, 0, s>>>(n, d_vx, d_vy, d_vz, d_mass, partials);
    k_kinetic_total<<<1, kBlock, 0, s>>>(partials, n_blocks, d_out);
    if (cudaGetLastError() != cudaSuccess) {
        *error = "dsmd_kinetic_energy_noalloc: kernel launch failed";
        return DSMD_ERR_CUDA;
    }
    return DSMD_OK;
}
