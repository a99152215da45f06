// Spatial domain decomposition over the GPUs of one node, native: brick grid, atom migration, ghost (halo) plan, the
// per-step positions-only refresh overlapped with the interior force pass, the rebuild vote, the reverse force halo and
// the feature-field exchange of the MLIP path, and the MD step loop around them - one process per GPU, NCCL point-to-point
// between neighbour bricks (NVLink / NVSwitch underneath).
//
// What the reference gets from its external decomposition library through MDSystem::migrate_particles_on_device,
// exchange_halo_on_device(rebuild), begin/end_halo_exchange_on_device, reverse_halo_on_device, exchange_field_on_device
// (src/md_system.cpp:1448-1545) and from CommBackend::unify_rebuild_decision (src/comm_backend.cpp:76-92). Conventions:
// owned atoms first, ghosts behind them; a ghost is every periodic image of a neighbour's atom within the halo width of
// this brick on the split axes (edges and corners included), already image-shifted; an axis with one brick gets no
// ghosts (the wrapping fixed-point coordinates resolve it).
//
// Messages. The up to 26 neighbour directions of a brick reach at most 7 distinct ranks on a 2 x 2 x 2 grid (1 on
// 2 x 1 x 1): directions are ordered by destination rank, so everything bound for one rank is one contiguous run and
// travels as ONE ncclSend - full records as nine doubles per atom at a rebuild, three doubles per ghost at the per-step
// refresh. The refresh runs on a high-priority side stream while the main stream computes the interior forces. The
// rebuild vote (an 8-byte MAX all-reduce, read by the host one step late) has a communicator and a stream of its own, so
// it never sits between the refresh and the force kernels. No allocation happens after dsmd_domain_create: every scratch
// array is sized there from the context's capacity. A rebuild synchronises the host three times (leaver counts, ghost
// counts, list status); every host wait polls against a deadline and returns DSMD_ERR_TIMEOUT instead of blocking for ever.
// Failures are decided collectively: every rank's lost-atom bin and failure flag travel with the counts, so all ranks
// leave a rebuild with the same status and nobody waits for a rank that has gone.
//
// Built on the public C ABI of the context (dsmd_b200.h) plus a few kernels of its own; NCCL is bound at run time
// (dlopen), so the library loads on machines without it as long as only one rank is used.

#include <cub/cub.cuh>
#include <dlfcn.h>
#include <nccl.h>
#include <thrust/iterator/counting_iterator.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../../include/dsmd_b200.h"
#include "host/brick_plan.hpp"
#include "host/deadline.hpp"

namespace {

constexpr int kThreads = 256;
using dsmd::host::kBinLost;
using dsmd::host::kBinRoom;
using dsmd::host::kBins;
using dsmd::host::kMaxDirs;
using dsmd::host::RankDirs;
constexpr int kRecord = 9;              // doubles per full record: x y z vx vy vz mass charge (type | gid << 32)
constexpr unsigned char kFlagLost = 255;

inline unsigned blocks_for(int64_t n, int threads) { return static_cast<unsigned>((n + threads - 1) / threads); }

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommSplit)(ncclComm_t, int, int, ncclComm_t*, ncclConfig_t*) = nullptr;   // optional (NCCL >= 2.18)
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi g_nccl;

bool load_nccl(const char* path, std::string& error) {
    if (g_nccl.handle) return true;
    const char* names[] = {path, "libnccl.so.2", "libnccl.so"};
    for (const char* name : names) {
        if (!name || !*name) continue;
        g_nccl.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
        if (g_nccl.handle) break;
    }
    if (!g_nccl.handle) {
        error = "cannot load the NCCL library (libnccl.so.2)";
        return false;
    }
#define DSMD_NCCL_SYM(field, symbol)                                                         \
    g_nccl.field = reinterpret_cast<decltype(g_nccl.field)>(dlsym(g_nccl.handle, symbol));   \
    if (!g_nccl.field) { error = std::string("NCCL symbol missing: ") + symbol; return false; }
    DSMD_NCCL_SYM(GetUniqueId, "ncclGetUniqueId")
    DSMD_NCCL_SYM(CommInitRank, "ncclCommInitRank")
    DSMD_NCCL_SYM(CommDestroy, "ncclCommDestroy")
    DSMD_NCCL_SYM(CommAbort, "ncclCommAbort")
    DSMD_NCCL_SYM(GroupStart, "ncclGroupStart")
    DSMD_NCCL_SYM(GroupEnd, "ncclGroupEnd")
    DSMD_NCCL_SYM(Send, "ncclSend")
    DSMD_NCCL_SYM(Recv, "ncclRecv")
    DSMD_NCCL_SYM(AllReduce, "ncclAllReduce")
    DSMD_NCCL_SYM(AllGather, "ncclAllGather")
    DSMD_NCCL_SYM(GetErrorString, "ncclGetErrorString")
#undef DSMD_NCCL_SYM
    g_nccl.CommSplit = reinterpret_cast<decltype(g_nccl.CommSplit)>(dlsym(g_nccl.handle, "ncclCommSplit"));
    return true;
}

struct DirTable {   // by value to the kernels
    int n;
    int e[kMaxDirs][3];
    int image[kMaxDirs][3];
    double lo[3], hi[3];      // this rank's brick
    double box[3];
    double halo;
    int split[3];
};

// Adds one to bin `bin` (or nothing when bin < 0) through a per-block histogram in shared memory: one global atomic per
// non-empty bin and block instead of one per atom (all atoms of a brick but a few hit the same "stays" bin). Holds a
// block-wide barrier: call it exactly once, from code that every thread of the block executes (never from one side of a
// branch, nor after an early return of some threads: a warp whose lanes reach two different barrier instructions hangs).
__device__ __forceinline__ void block_histogram_add(int* hist, int bin, int* __restrict__ counts) {
    if (bin >= 0) atomicAdd(&hist[bin], 1);
    __syncthreads();
    if (threadIdx.x < kBins && hist[threadIdx.x] > 0) atomicAdd(&counts[threadIdx.x], hist[threadIdx.x]);
}

// flag[i] = 0: stays; 1 + d: leaves along direction d; 255: lost (moved further than one brick, or not finite).
__global__ void k_classify_leave(DirTable t, int n_owned, const double* __restrict__ x, const double* __restrict__ y,
                                 const double* __restrict__ z, unsigned char* __restrict__ flag,
                                 int* __restrict__ counts, int room) {
    __shared__ int hist[kBins];
    if (threadIdx.x < kBins) hist[threadIdx.x] = 0;
    __syncthreads();
    if (blockIdx.x == 0 && threadIdx.x == 0) hist[kBinRoom] = room;   // published with the counts: every rank can check every rank
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    int bin = -1;   // threads past the end take part in the block's barrier below, with nothing to add
    if (i < n_owned) {
        const double p[3] = {x[i], y[i], z[i]};
        int e[3] = {0, 0, 0};
        bool lost = false;
        for (int a = 0; a < 3; ++a) {
            if (!t.split[a]) continue;
            const double w = t.hi[a] - t.lo[a];
            if (!(p[a] >= t.lo[a] - w && p[a] < t.hi[a] + w)) lost = true;
            e[a] = p[a] < t.lo[a] ? -1 : (p[a] >= t.hi[a] ? 1 : 0);
        }
        int k = 0;
        if (!lost && (e[0] || e[1] || e[2])) {
            k = -1;
            for (int d = 0; d < t.n; ++d)
                if (t.e[d][0] == e[0] && t.e[d][1] == e[1] && t.e[d][2] == e[2]) k = d + 1;
            if (k < 0) lost = true;
        }
        flag[i] = lost ? kFlagLost : static_cast<unsigned char>(k);
        bin = lost ? kBinLost : k;
    }
    block_histogram_add(hist, bin, counts);   // the one barrier of this kernel: every thread of the block reaches it
}

// (direction, atom) of the leavers selected into `index`, for the sort that groups them by direction.
__global__ void k_leaver_keys(int count, const int* __restrict__ index, const unsigned char* __restrict__ flag,
                              unsigned* __restrict__ key) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= count) return;
    const unsigned f = flag[index[k]];
    key[k] = f == kFlagLost ? 31u : f - 1u;
}

// Which neighbour directions need atom i as a ghost (bit d).
__device__ __forceinline__ unsigned halo_mask(const DirTable& t, double px, double py, double pz) {
    const double p[3] = {px, py, pz};
    int near_lo[3], near_hi[3];
    for (int a = 0; a < 3; ++a) {
        near_lo[a] = t.split[a] && p[a] < t.lo[a] + t.halo;
        near_hi[a] = t.split[a] && p[a] >= t.hi[a] - t.halo;
    }
    unsigned mask = 0;
    for (int d = 0; d < t.n; ++d) {
        bool in = true;
        for (int a = 0; a < 3; ++a) {
            if (t.e[d][a] > 0) in = in && near_hi[a];
            else if (t.e[d][a] < 0) in = in && near_lo[a];
        }
        if (in) mask |= 1u << d;
    }
    return mask;
}

__global__ void k_halo_count(DirTable t, int n_owned, const double* __restrict__ x, const double* __restrict__ y,
                             const double* __restrict__ z, int* __restrict__ cnt) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_owned) return;
    cnt[i] = __popc(halo_mask(t, x[i], y[i], z[i]));
}

__global__ void k_halo_expand(DirTable t, int n_owned, const double* __restrict__ x, const double* __restrict__ y,
                              const double* __restrict__ z, const int* __restrict__ off, unsigned* __restrict__ key,
                              int* __restrict__ val, int* __restrict__ counts, int capacity, int room) {
    __shared__ int hist[kBins];
    if (threadIdx.x < kBins) hist[threadIdx.x] = 0;
    __syncthreads();
    if (blockIdx.x == 0 && threadIdx.x == 0) hist[kBinRoom] = room;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_owned) {
        unsigned mask = halo_mask(t, x[i], y[i], z[i]);
        int o = off[i];
        while (mask) {
            const int d = __ffs(mask) - 1;
            mask &= mask - 1;
            if (o < capacity) {
                key[o] = static_cast<unsigned>(d);
                val[o] = i;
            }
            ++o;
            atomicAdd(&hist[1 + d], 1);
        }
    }
    block_histogram_add(hist, -1, counts);
}

struct Fields {
    const double *x, *y, *z, *vx, *vy, *vz, *mass, *charge;
    const int *type, *gid;
};

// Full records of the listed atoms, shifted by the image of the direction each entry travels.
__global__ void k_pack_records(DirTable t, int count, const int* __restrict__ index, const unsigned* __restrict__ key,
                               Fields f, double* __restrict__ out) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= count) return;
    const int s = index[k];
    const int d = static_cast<int>(key[k]);
    double sx = 0.0, sy = 0.0, sz = 0.0;
    if (d >= 0 && d < t.n) {
        sx = t.image[d][0] * t.box[0];
        sy = t.image[d][1] * t.box[1];
        sz = t.image[d][2] * t.box[2];
    }
    double* o = out + kRecord * static_cast<size_t>(k);
    o[0] = f.x[s] + sx; o[1] = f.y[s] + sy; o[2] = f.z[s] + sz;
    o[3] = f.vx[s]; o[4] = f.vy[s]; o[5] = f.vz[s];
    o[6] = f.mass[s]; o[7] = f.charge[s];
    const long long words = (static_cast<long long>(f.gid[s]) << 32) | static_cast<long long>(static_cast<unsigned>(f.type[s]));
    o[8] = __longlong_as_double(words);
}

__global__ void k_send_images(DirTable t, int count, const unsigned* __restrict__ key, signed char* __restrict__ image) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= count) return;
    const int d = static_cast<int>(key[k]);
    image[3 * k] = static_cast<signed char>(t.image[d][0]);
    image[3 * k + 1] = static_cast<signed char>(t.image[d][1]);
    image[3 * k + 2] = static_cast<signed char>(t.image[d][2]);
}

// ---- rows of a field along the ghost plan (forces are the width-3 case with three separate arrays) -------------------

// out[k][w] = data[row(k)][w], row(k) = index[k] (owned atoms of the send list) or the slot of ghost k.
template <class T>
__global__ void k_rows_gather(int count, int width, const int* __restrict__ index, const T* __restrict__ data,
                              T* __restrict__ out) {
    const long long t = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (t >= static_cast<long long>(count) * width) return;
    const int k = static_cast<int>(t / width), w = static_cast<int>(t % width);
    out[t] = data[static_cast<size_t>(index[k]) * width + w];
}

template <class T>
__global__ void k_rows_scatter(int count, int width, const int* __restrict__ index, const T* __restrict__ in,
                               T* __restrict__ data, int add) {
    const long long t = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (t >= static_cast<long long>(count) * width) return;
    const int k = static_cast<int>(t / width), w = static_cast<int>(t % width);
    T* dst = data + static_cast<size_t>(index[k]) * width + w;
    if (add) atomicAdd(dst, in[t]);   // an owned atom can be the ghost of several neighbours
    else *dst = in[t];
}

__global__ void k_force_gather(int count, const int* __restrict__ slot, const double* __restrict__ fx,
                               const double* __restrict__ fy, const double* __restrict__ fz, double* __restrict__ out) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= count) return;
    const int s = slot[k];
    out[3 * k] = fx[s];
    out[3 * k + 1] = fy[s];
    out[3 * k + 2] = fz[s];
}

__global__ void k_force_add(int count, const int* __restrict__ index, const double* __restrict__ in,
                            double* __restrict__ fx, double* __restrict__ fy, double* __restrict__ fz) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= count) return;
    const int s = index[k];
    atomicAdd(&fx[s], in[3 * k]);
    atomicAdd(&fy[s], in[3 * k + 1]);
    atomicAdd(&fz[s], in[3 * k + 2]);
}

}  // namespace

struct dsmd_domain {
    dsmd_ctx* ctx = nullptr;
    int rank = 0, world = 1;
    int dims[3] = {1, 1, 1}, coords[3] = {0, 0, 0};
    DirTable table{};
    RankDirs mine;
    dsmd::host::PeerPlan plan;   // the distinct neighbour ranks and the runs of directions that belong to each
    double skin = 0.0;
    double wait_limit_s = 120.0;
    ncclComm_t comm = nullptr, vote_comm = nullptr;
    cudaStream_t side = nullptr, vote_stream = nullptr;
    cudaEvent_t ev_main = nullptr, ev_side = nullptr, ev_disp = nullptr, ev_vote[2] = {nullptr, nullptr};
    std::string error;
    int64_t capacity = 0;
    std::vector<RankDirs> all_dirs;   // every rank's directions: any rank can work out who receives what
    int* d_verdict = nullptr;      // two ints: this rank's status of a rebuild, the MAX over the ranks
    int* h_verdict = nullptr;      // pinned

    // scratch (device), sized once from the context's capacity
    unsigned char* flag = nullptr;
    unsigned* key[2] = {nullptr, nullptr};
    int* val[2] = {nullptr, nullptr};
    size_t pair_capacity = 0;
    int* cnt = nullptr;
    int* off = nullptr;
    void* temp = nullptr;
    size_t temp_bytes = 0;
    int* d_counts = nullptr;                // [kBins] this rank, then [world * kBins] gathered
    int* h_counts = nullptr;                // pinned, same layout
    int* d_selected = nullptr;              // one int: leavers selected
    double* send_rec = nullptr;
    double* recv_rec = nullptr;
    // the plan of the per-step refresh
    int* send_index = nullptr;
    signed char* send_image = nullptr;
    double* send_pos = nullptr;
    double* recv_pos = nullptr;
    int send_to[kMaxDirs] = {}, recv_from[kMaxDirs] = {};   // atoms per peer
    int64_t n_send = 0, n_ghost = 0;
    // field exchange buffers (grown on demand: the width is the model's)
    void* field_send = nullptr;
    void* field_recv = nullptr;
    size_t field_bytes = 0;
    // rebuild vote
    unsigned long long* vote_word = nullptr;    // device
    unsigned long long* h_vote[2] = {nullptr, nullptr};
    int vote_pending = -1;
    double d_prev = 0.0, d_prev2 = 0.0;
    // statistics
    int64_t rebuilds = 0, migrated = 0, launches = 0;
    double worst_disp_sq = 0.0;
    // optional per-phase timing (profiling mode: synchronises every step)
    bool profile = false;
    cudaEvent_t ev_phase[8] = {};
    double phase_ms[8] = {};   // integrate1, vote, refresh issue + interior, boundary wait + boundary, integrate2, rebuild
    double rebuild_ms[4] = {}; // wall time of migrate, sort owned, ghost plan, list build (profiling mode)
    int64_t phase_steps = 0;
};

namespace {

int dfail(dsmd_domain* d, int code, const std::string& what) {
    d->error = what;
    return code;
}

#define DOM_CUDA(d, call)                                                             \
    do {                                                                              \
        cudaError_t err_ = (call);                                                    \
        if (err_ != cudaSuccess) {                                                    \
            (d)->error = std::string(#call) + ": " + cudaGetErrorString(err_);        \
            return DSMD_ERR_CUDA;                                                     \
        }                                                                             \
    } while (0)

#define DOM_NCCL(d, call)                                                             \
    do {                                                                              \
        ncclResult_t res_ = (call);                                                   \
        if (res_ != ncclSuccess) {                                                    \
            (d)->error = std::string(#call) + ": " + g_nccl.GetErrorString(res_);     \
            return DSMD_ERR_CUDA;                                                     \
        }                                                                             \
    } while (0)

#define DOM_CTX(d, call)                                                              \
    do {                                                                              \
        const int rc_ = (call);                                                       \
        if (rc_ != DSMD_OK) {                                                         \
            (d)->error = std::string(#call) + ": " + dsmd_last_error((d)->ctx);       \
            return rc_;                                                               \
        }                                                                             \
    } while (0)

// Host waits: poll against the domain's deadline; a wait that runs out is an error status, not a hang.
int wait_stream(dsmd_domain* d, cudaStream_t s, const char* what) {
    cudaError_t last = cudaSuccess;
    const dsmd::host::WaitResult r = dsmd::host::poll_until(
        [&]() {
            last = cudaStreamQuery(s);
            return last == cudaSuccess ? 1 : (last == cudaErrorNotReady ? 0 : -1);
        },
        d->wait_limit_s);
    if (r == dsmd::host::WaitResult::kReady) return DSMD_OK;
    if (r == dsmd::host::WaitResult::kFailed) return dfail(d, DSMD_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(last));
    return dfail(d, DSMD_ERR_TIMEOUT, std::string(what) + ": no answer from the GPU or a neighbour rank within the wait limit");
}

int wait_event(dsmd_domain* d, cudaEvent_t ev, const char* what) {
    cudaError_t last = cudaSuccess;
    const dsmd::host::WaitResult r = dsmd::host::poll_until(
        [&]() {
            last = cudaEventQuery(ev);
            return last == cudaSuccess ? 1 : (last == cudaErrorNotReady ? 0 : -1);
        },
        d->wait_limit_s);
    if (r == dsmd::host::WaitResult::kReady) return DSMD_OK;
    if (r == dsmd::host::WaitResult::kFailed) return dfail(d, DSMD_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(last));
    return dfail(d, DSMD_ERR_TIMEOUT, std::string(what) + ": no answer from the GPU or a neighbour rank within the wait limit");
}

struct MutableForces {
    double *fx, *fy, *fz;
};

Fields fields_of(dsmd_ctx* ctx) {
    Fields f{};
    void* p = nullptr;
    const int ids[8] = {DSMD_X, DSMD_Y, DSMD_Z, DSMD_VX, DSMD_VY, DSMD_VZ, DSMD_MASS, DSMD_CHARGE};
    const double** dst[8] = {&f.x, &f.y, &f.z, &f.vx, &f.vy, &f.vz, &f.mass, &f.charge};
    for (int k = 0; k < 8; ++k) { dsmd_device_pointer(ctx, ids[k], &p); *dst[k] = static_cast<const double*>(p); }
    dsmd_device_pointer(ctx, DSMD_TYPE, &p); f.type = static_cast<const int*>(p);
    dsmd_device_pointer(ctx, DSMD_GLOBAL_ID, &p); f.gid = static_cast<const int*>(p);
    return f;
}

MutableForces forces_of(dsmd_ctx* ctx) {
    MutableForces f{};
    void* p = nullptr;
    dsmd_device_pointer(ctx, DSMD_FX, &p); f.fx = static_cast<double*>(p);
    dsmd_device_pointer(ctx, DSMD_FY, &p); f.fy = static_cast<double*>(p);
    dsmd_device_pointer(ctx, DSMD_FZ, &p); f.fz = static_cast<double*>(p);
    return f;
}

// Sorts `n` (key, val) pairs by key (stable), result in key[1] / val[1].
int sort_pairs(dsmd_domain* d, int64_t n, int bits, cudaStream_t s) {
    size_t need = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, need, d->key[0], d->key[1], d->val[0], d->val[1], static_cast<int>(n), 0, bits, s);
    if (need > d->temp_bytes) return dfail(d, DSMD_ERR_CAPACITY, "sort scratch smaller than this sort needs");
    DOM_CUDA(d, cub::DeviceRadixSort::SortPairs(d->temp, need, d->key[0], d->key[1], d->val[0], d->val[1], static_cast<int>(n),
                                                0, bits, s));
    return DSMD_OK;
}

// Every rank's counts to every rank; h_counts[r * kBins + k] afterwards. One host synchronisation (with deadline).
int gather_counts(dsmd_domain* d, cudaStream_t s) {
    if (d->world > 1) {
        DOM_NCCL(d, g_nccl.AllGather(d->d_counts, d->d_counts + kBins, kBins, ncclInt32, d->comm, s));
        DOM_CUDA(d, cudaMemcpyAsync(d->h_counts, d->d_counts + kBins, sizeof(int) * kBins * d->world, cudaMemcpyDeviceToHost, s));
    } else {
        DOM_CUDA(d, cudaMemcpyAsync(d->h_counts, d->d_counts, sizeof(int) * kBins, cudaMemcpyDeviceToHost, s));
    }
    return wait_stream(d, s, "exchange of the message sizes");
}

// The same decision on every rank, from what every rank published.
int collective_status(dsmd_domain* d, const char* what) {
    const dsmd::host::CountsVerdict v = dsmd::host::counts_verdict(d->all_dirs, d->h_counts, d->capacity, what);
    return v.code == 0 ? DSMD_OK : dfail(d, v.code, v.text);
}

void per_peer_counts(const dsmd_domain* d, int* send_to, int* recv_from, int64_t& n_send, int64_t& n_recv) {
    long long s = 0, r = 0;
    dsmd::host::per_peer_counts(d->plan, d->h_counts, d->rank, send_to, recv_from, s, r);
    n_send = s;
    n_recv = r;
}

// One message per peer and way: `width` doubles per atom.
int exchange(dsmd_domain* d, const double* send, const int* send_to, double* recv, const int* recv_from, int width,
             cudaStream_t s) {
    if (d->world == 1) return DSMD_OK;
    DOM_NCCL(d, g_nccl.GroupStart());
    size_t so = 0, ro = 0;
    for (int p = 0; p < d->plan.n_peers; ++p) {
        if (recv_from[p] > 0)
            DOM_NCCL(d, g_nccl.Recv(recv + width * ro, static_cast<size_t>(width) * recv_from[p], ncclFloat64, d->plan.peer[p], d->comm, s));
        if (send_to[p] > 0)
            DOM_NCCL(d, g_nccl.Send(send + width * so, static_cast<size_t>(width) * send_to[p], ncclFloat64, d->plan.peer[p], d->comm, s));
        so += send_to[p];
        ro += recv_from[p];
    }
    DOM_NCCL(d, g_nccl.GroupEnd());
    return DSMD_OK;
}

// Atoms that left the brick go to their new owners, arrivals are appended behind the owned atoms (unsorted: the owned
// sort that follows removes the leavers, which stay where they are, and sorts the arrivals in). Returns the leaver count.
int migrate(dsmd_domain* d, cudaStream_t s, int64_t& n_leave_out) {
    n_leave_out = 0;
    int64_t n_owned = 0, n_total = 0;
    dsmd_counts(d->ctx, &n_owned, &n_total);
    DOM_CTX(d, dsmd_set_counts(d->ctx, n_owned, n_owned));   // the old ghosts are gone
    const int n = static_cast<int>(n_owned);
    DOM_CUDA(d, cudaMemsetAsync(d->d_counts, 0, sizeof(int) * kBins, s));
    Fields f = fields_of(d->ctx);
    k_classify_leave<<<blocks_for(n, kThreads), kThreads, 0, s>>>(d->table, n, f.x, f.y, f.z, d->flag, d->d_counts,
                                                                 static_cast<int>(d->capacity - n_owned));
    ++d->launches;
    // the leavers' indices, in index order (deterministic), for the few that there are
    size_t need = 0;
    thrust::counting_iterator<int> iota(0);
    cub::DeviceSelect::Flagged(nullptr, need, iota, d->flag, d->val[0], d->d_selected, n, s);
    if (need > d->temp_bytes) return dfail(d, DSMD_ERR_CAPACITY, "selection scratch too small");
    DOM_CUDA(d, cub::DeviceSelect::Flagged(d->temp, need, iota, d->flag, d->val[0], d->d_selected, n, s));
    { const int rc = gather_counts(d, s); if (rc) return rc; }
    { const int rc = collective_status(d, "migrating atoms"); if (rc) return rc; }
    int send_to[kMaxDirs], recv_from[kMaxDirs];
    int64_t n_leave = 0, n_arrive = 0;
    per_peer_counts(d, send_to, recv_from, n_leave, n_arrive);
    if (n_leave > 0) {
        k_leaver_keys<<<blocks_for(n_leave, kThreads), kThreads, 0, s>>>(static_cast<int>(n_leave), d->val[0], d->flag, d->key[0]);
        { const int rc = sort_pairs(d, n_leave, 5, s); if (rc) return rc; }
        k_pack_records<<<blocks_for(n_leave, kThreads), kThreads, 0, s>>>(d->table, static_cast<int>(n_leave), d->val[1], d->key[1],
                                                                        f, d->send_rec);
        d->launches += 2;
    }
    { const int rc = exchange(d, d->send_rec, send_to, d->recv_rec, recv_from, kRecord, s); if (rc) return rc; }
    DOM_CTX(d, dsmd_halo_append_packed(d->ctx, d->recv_rec, n_arrive, s));
    DOM_CTX(d, dsmd_set_counts(d->ctx, n_owned + n_arrive, n_owned + n_arrive));
    d->migrated += n_leave;
    n_leave_out = n_leave;
    return DSMD_OK;
}

int build_halo(dsmd_domain* d, cudaStream_t s) {
    int64_t n_owned = 0, n_total = 0;
    dsmd_counts(d->ctx, &n_owned, &n_total);
    const int n = static_cast<int>(n_owned);
    d->n_send = d->n_ghost = 0;
    std::fill(d->send_to, d->send_to + kMaxDirs, 0);
    std::fill(d->recv_from, d->recv_from + kMaxDirs, 0);
    if (d->world == 1 || d->table.n == 0) return DSMD_OK;
    Fields f = fields_of(d->ctx);
    k_halo_count<<<blocks_for(n, kThreads), kThreads, 0, s>>>(d->table, n, f.x, f.y, f.z, d->cnt);
    ++d->launches;
    size_t need = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, need, d->cnt, d->off, n, s);
    if (need > d->temp_bytes) return dfail(d, DSMD_ERR_CAPACITY, "scan scratch too small");
    DOM_CUDA(d, cub::DeviceScan::ExclusiveSum(d->temp, need, d->cnt, d->off, n, s));
    DOM_CUDA(d, cudaMemsetAsync(d->d_counts, 0, sizeof(int) * kBins, s));
    k_halo_expand<<<blocks_for(n, kThreads), kThreads, 0, s>>>(d->table, n, f.x, f.y, f.z, d->off, d->key[0], d->val[0],
                                                              d->d_counts, static_cast<int>(d->pair_capacity),
                                                              static_cast<int>(d->capacity - n_owned));
    ++d->launches;
    { const int rc = gather_counts(d, s); if (rc) return rc; }
    { const int rc = collective_status(d, "ghost atoms"); if (rc) return rc; }
    int64_t n_send = 0, n_recv = 0;
    per_peer_counts(d, d->send_to, d->recv_from, n_send, n_recv);
    { const int rc = sort_pairs(d, n_send, 5, s); if (rc) return rc; }
    if (n_send > 0) {
        k_pack_records<<<blocks_for(n_send, kThreads), kThreads, 0, s>>>(d->table, static_cast<int>(n_send), d->val[1],
                                                                        d->key[1], f, d->send_rec);
        k_send_images<<<blocks_for(n_send, kThreads), kThreads, 0, s>>>(d->table, static_cast<int>(n_send), d->key[1],
                                                                       d->send_image);
        d->launches += 2;
        DOM_CUDA(d, cudaMemcpyAsync(d->send_index, d->val[1], sizeof(int) * n_send, cudaMemcpyDeviceToDevice, s));
    }
    { const int rc = exchange(d, d->send_rec, d->send_to, d->recv_rec, d->recv_from, kRecord, s); if (rc) return rc; }
    DOM_CTX(d, dsmd_halo_append_packed(d->ctx, d->recv_rec, n_recv, s));
    d->n_send = n_send;
    d->n_ghost = n_recv;
    return DSMD_OK;
}

int rebuild(dsmd_domain* d, cudaStream_t s) {
    auto now = [&]() {
        if (d->profile) cudaStreamSynchronize(s);
        return std::chrono::steady_clock::now();
    };
    auto lap = [&](int k, std::chrono::steady_clock::time_point& t0) {
        if (!d->profile) return;
        const auto t1 = now();
        d->rebuild_ms[k] += std::chrono::duration<double, std::milli>(t1 - t0).count();
        t0 = t1;
    };
    auto t0 = now();
    int64_t n_leave = 0;
    if (d->world > 1) { const int rc = migrate(d, s, n_leave); if (rc) return rc; }
    lap(0, t0);
    if (d->world > 1) DOM_CTX(d, dsmd_sort_owned_in_brick(d->ctx, d->table.lo, d->table.hi, d->table.split, n_leave, s));
    else DOM_CTX(d, dsmd_sort_owned(d->ctx, s));
    lap(1, t0);
    { const int rc = build_halo(d, s); if (rc) return rc; }
    lap(2, t0);
    // The list build reads the status words of the sort and of the build with one synchronisation. Its verdict is taken
    // together (MAX over the ranks' status codes), so that a rank whose atoms went bad does not leave the others waiting
    // for its next message.
    int verdict = dsmd_build_neighbor_list(d->ctx, s);
    if (verdict != DSMD_OK) d->error = std::string("dsmd_build_neighbor_list: ") + dsmd_last_error(d->ctx);
    if (d->world > 1) {
        d->h_verdict[0] = verdict;
        DOM_CUDA(d, cudaMemcpyAsync(d->d_verdict, d->h_verdict, sizeof(int), cudaMemcpyHostToDevice, s));
        DOM_NCCL(d, g_nccl.AllReduce(d->d_verdict, d->d_verdict + 1, 1, ncclInt32, ncclMax, d->comm, s));
        DOM_CUDA(d, cudaMemcpyAsync(d->h_verdict + 1, d->d_verdict + 1, sizeof(int), cudaMemcpyDeviceToHost, s));
        { const int rc = wait_stream(d, s, "agreement on the list build"); if (rc) return rc; }
        if (verdict == DSMD_OK && d->h_verdict[1] != DSMD_OK) {
            verdict = d->h_verdict[1];
            d->error = "another rank's list build failed with status " + std::to_string(verdict);
        }
    }
    if (verdict != DSMD_OK) return verdict;
    lap(3, t0);
    ++d->rebuilds;
    d->vote_pending = -1;
    d->d_prev = d->d_prev2 = 0.0;
    return DSMD_OK;
}

// Positions-only refresh on the side stream: after `ev_main` (the pack of the owned atoms), before `ev_side`.
int refresh(dsmd_domain* d, cudaStream_t main_stream) {
    DOM_CUDA(d, cudaEventRecord(d->ev_main, main_stream));
    DOM_CUDA(d, cudaStreamWaitEvent(d->side, d->ev_main, 0));
    DOM_CTX(d, dsmd_halo_pack(d->ctx, d->send_index, reinterpret_cast<const int8_t*>(d->send_image), d->n_send, d->send_pos,
                              d->side));
    { const int rc = exchange(d, d->send_pos, d->send_to, d->recv_pos, d->recv_from, 3, d->side); if (rc) return rc; }
    DOM_CTX(d, dsmd_halo_unpack(d->ctx, d->recv_pos, 0, d->n_ghost, d->side));
    DOM_CUDA(d, cudaEventRecord(d->ev_side, d->side));
    return DSMD_OK;
}

int grow_field_buffers(dsmd_domain* d, size_t bytes) {
    if (bytes <= d->field_bytes) return DSMD_OK;
    const size_t grown = std::max(bytes, d->field_bytes + d->field_bytes / 2);
    if (d->field_send) cudaFree(d->field_send);
    if (d->field_recv) cudaFree(d->field_recv);
    d->field_send = d->field_recv = nullptr;
    d->field_bytes = 0;
    DOM_CUDA(d, cudaMalloc(&d->field_send, grown));
    DOM_CUDA(d, cudaMalloc(&d->field_recv, grown));
    d->field_bytes = grown;
    return DSMD_OK;
}

// Bytes between peers along the ghost plan. forward: what this rank sends per peer is send_to, receives recv_from;
// reverse: the other way round.
int exchange_bytes(dsmd_domain* d, const char* send, char* recv, size_t bytes_per_atom, bool reverse, cudaStream_t s) {
    const int* out_n = reverse ? d->recv_from : d->send_to;
    const int* in_n = reverse ? d->send_to : d->recv_from;
    DOM_NCCL(d, g_nccl.GroupStart());
    size_t so = 0, ro = 0;
    for (int p = 0; p < d->plan.n_peers; ++p) {
        if (in_n[p] > 0) DOM_NCCL(d, g_nccl.Recv(recv + bytes_per_atom * ro, bytes_per_atom * in_n[p], ncclUint8, d->plan.peer[p], d->comm, s));
        if (out_n[p] > 0) DOM_NCCL(d, g_nccl.Send(send + bytes_per_atom * so, bytes_per_atom * out_n[p], ncclUint8, d->plan.peer[p], d->comm, s));
        so += out_n[p];
        ro += in_n[p];
    }
    DOM_NCCL(d, g_nccl.GroupEnd());
    return DSMD_OK;
}

template <class T>
int exchange_field_typed(dsmd_domain* d, T* data, int width, bool reverse, cudaStream_t s) {
    const int32_t* ghost_slot = nullptr;
    DOM_CTX(d, dsmd_ghost_slots(d->ctx, &ghost_slot));
    const int64_t n_out = reverse ? d->n_ghost : d->n_send, n_in = reverse ? d->n_send : d->n_ghost;
    const size_t row = sizeof(T) * static_cast<size_t>(width);
    { const int rc = grow_field_buffers(d, row * static_cast<size_t>(std::max(n_out, n_in)) + 16); if (rc) return rc; }
    T* out = static_cast<T*>(d->field_send);
    T* in = static_cast<T*>(d->field_recv);
    const int* from_rows = reverse ? ghost_slot : d->send_index;
    const int* to_rows = reverse ? d->send_index : ghost_slot;
    if (n_out > 0) {
        k_rows_gather<T><<<blocks_for(n_out * width, kThreads), kThreads, 0, s>>>(static_cast<int>(n_out), width, from_rows, data, out);
        ++d->launches;
    }
    { const int rc = exchange_bytes(d, reinterpret_cast<const char*>(out), reinterpret_cast<char*>(in), row, reverse, s); if (rc) return rc; }
    if (n_in > 0) {
        k_rows_scatter<T><<<blocks_for(n_in * width, kThreads), kThreads, 0, s>>>(static_cast<int>(n_in), width, to_rows, in, data,
                                                                                 reverse ? 1 : 0);
        ++d->launches;
    }
    DOM_CUDA(d, cudaGetLastError());
    return DSMD_OK;
}

}  // namespace

extern "C" {

int dsmd_nccl_unique_id(const char* nccl_library_path, char out[128]) {
    std::string error;
    if (!out || !load_nccl(nccl_library_path, error)) return DSMD_ERR_INVALID;
    ncclUniqueId id;
    if (g_nccl.GetUniqueId(&id) != ncclSuccess) return DSMD_ERR_CUDA;
    static_assert(sizeof(id) == 128, "ncclUniqueId is 128 bytes");
    std::memcpy(out, &id, 128);
    return DSMD_OK;
}

int dsmd_domain_create(dsmd_ctx* ctx, int rank, int world, const int dims[3], const double box[3], double halo_width,
                       double skin, const char* nccl_library_path, const char unique_id[128], dsmd_domain** out) {
    if (!ctx || !out || !dims || !box || rank < 0 || world < 1 || rank >= world) return DSMD_ERR_INVALID;
    if (dims[0] * dims[1] * dims[2] != world) return DSMD_ERR_INVALID;
    dsmd_domain* d = new dsmd_domain();
    *out = d;
    d->ctx = ctx;
    d->rank = rank;
    d->world = world;
    d->skin = skin;
    if (const char* limit = std::getenv("DSMD_WAIT_LIMIT_S")) {
        const double v = std::atof(limit);
        if (v > 0.0) d->wait_limit_s = v;
    }
    for (int a = 0; a < 3; ++a) d->dims[a] = dims[a];
    dsmd::host::coords_of(dims, rank, d->coords);
    DirTable& t = d->table;
    t.halo = halo_width;
    for (int a = 0; a < 3; ++a) {
        t.box[a] = box[a];
        t.split[a] = dims[a] > 1;
        t.lo[a] = box[a] * d->coords[a] / dims[a];
        t.hi[a] = box[a] * (d->coords[a] + 1) / dims[a];
        if (t.split[a] && box[a] / dims[a] < halo_width)
            return dfail(d, DSMD_ERR_BOX_TOO_SMALL, "a brick is narrower than the halo width");
    }
    d->all_dirs.resize(world);
    for (int r = 0; r < world; ++r) d->all_dirs[r] = dsmd::host::dirs_of(dims, r);
    d->mine = d->all_dirs[rank];
    t.n = d->mine.n;
    for (int k = 0; k < t.n; ++k)
        for (int a = 0; a < 3; ++a) { t.e[k][a] = d->mine.e[k][a]; t.image[k][a] = d->mine.image[k][a]; }
    d->plan = dsmd::host::peer_plan(d->all_dirs, rank);
    DOM_CTX(d, dsmd_capacity(ctx, &d->capacity));
    const size_t cap = static_cast<size_t>(d->capacity);
    // scratch, once: nothing is allocated after this call
    d->pair_capacity = 2 * cap + 1024;   // an atom is needed by at most 7 directions, and only atoms near a face by any
    DOM_CUDA(d, cudaMalloc(&d->flag, cap + 16));
    for (int k = 0; k < 2; ++k) {
        DOM_CUDA(d, cudaMalloc(&d->key[k], sizeof(unsigned) * d->pair_capacity));
        DOM_CUDA(d, cudaMalloc(&d->val[k], sizeof(int) * d->pair_capacity));
    }
    DOM_CUDA(d, cudaMalloc(&d->cnt, sizeof(int) * (cap + 1)));
    DOM_CUDA(d, cudaMalloc(&d->off, sizeof(int) * (cap + 1)));
    {
        size_t a = 0, b = 0, c2 = 0;
        thrust::counting_iterator<int> iota(0);
        cub::DeviceRadixSort::SortPairs(nullptr, a, d->key[0], d->key[1], d->val[0], d->val[1], static_cast<int>(d->pair_capacity), 0, 5);
        cub::DeviceScan::ExclusiveSum(nullptr, b, d->cnt, d->off, static_cast<int>(cap));
        cub::DeviceSelect::Flagged(nullptr, c2, iota, d->flag, d->val[0], d->d_selected, static_cast<int>(cap));
        d->temp_bytes = std::max(a, std::max(b, c2)) + 256;
        DOM_CUDA(d, cudaMalloc(&d->temp, d->temp_bytes));
    }
    DOM_CUDA(d, cudaMalloc(&d->d_counts, sizeof(int) * kBins * (world + 1)));
    DOM_CUDA(d, cudaMallocHost(&d->h_counts, sizeof(int) * kBins * (world + 1)));
    DOM_CUDA(d, cudaMalloc(&d->d_selected, sizeof(int) * 4));
    DOM_CUDA(d, cudaMalloc(&d->d_verdict, sizeof(int) * 2));
    DOM_CUDA(d, cudaMallocHost(&d->h_verdict, sizeof(int) * 2));
    DOM_CUDA(d, cudaMalloc(&d->send_rec, sizeof(double) * kRecord * (cap + 16)));
    DOM_CUDA(d, cudaMalloc(&d->recv_rec, sizeof(double) * kRecord * (cap + 16)));
    DOM_CUDA(d, cudaMalloc(&d->send_index, sizeof(int) * (cap + 16)));
    DOM_CUDA(d, cudaMalloc(&d->send_image, 3 * (cap + 16)));
    DOM_CUDA(d, cudaMalloc(&d->send_pos, sizeof(double) * 3 * (cap + 16)));
    DOM_CUDA(d, cudaMalloc(&d->recv_pos, sizeof(double) * 3 * (cap + 16)));
    DOM_CUDA(d, cudaMalloc(&d->vote_word, sizeof(unsigned long long) * 2));
    DOM_CUDA(d, cudaMemset(d->vote_word, 0, sizeof(unsigned long long) * 2));
    for (int k = 0; k < 2; ++k) {
        DOM_CUDA(d, cudaMallocHost(&d->h_vote[k], sizeof(unsigned long long)));
        *d->h_vote[k] = 0ull;
        DOM_CUDA(d, cudaEventCreateWithFlags(&d->ev_vote[k], cudaEventDisableTiming));
    }
    int lo_prio = 0, hi_prio = 0;
    DOM_CUDA(d, cudaDeviceGetStreamPriorityRange(&lo_prio, &hi_prio));
    DOM_CUDA(d, cudaStreamCreateWithPriority(&d->side, cudaStreamNonBlocking, hi_prio));
    DOM_CUDA(d, cudaStreamCreateWithPriority(&d->vote_stream, cudaStreamNonBlocking, lo_prio));
    DOM_CUDA(d, cudaEventCreateWithFlags(&d->ev_main, cudaEventDisableTiming));
    DOM_CUDA(d, cudaEventCreateWithFlags(&d->ev_side, cudaEventDisableTiming));
    DOM_CUDA(d, cudaEventCreateWithFlags(&d->ev_disp, cudaEventDisableTiming));
    if (world > 1) {
        if (!unique_id) return dfail(d, DSMD_ERR_INVALID, "several ranks need the NCCL unique id of rank 0");
        if (!load_nccl(nccl_library_path, d->error)) return DSMD_ERR_INVALID;
        ncclUniqueId id;
        std::memcpy(&id, unique_id, 128);
        DOM_NCCL(d, g_nccl.CommInitRank(&d->comm, world, id, rank));
        // the vote's own communicator: its all-reduce then never queues between the refresh messages and the force kernels
        if (g_nccl.CommSplit && g_nccl.CommSplit(d->comm, 0, rank, &d->vote_comm, nullptr) != ncclSuccess) d->vote_comm = nullptr;
        // Connections to the peers are made on first use: use each of them once now (one double either way, and the
        // vote's all-reduce), so that no step of a run pays for it.
        double* scratch = d->send_pos;
        DOM_NCCL(d, g_nccl.GroupStart());
        for (int p = 0; p < d->plan.n_peers; ++p) {
            DOM_NCCL(d, g_nccl.Recv(d->recv_pos + p, 1, ncclFloat64, d->plan.peer[p], d->comm, d->side));
            DOM_NCCL(d, g_nccl.Send(scratch + p, 1, ncclFloat64, d->plan.peer[p], d->comm, d->side));
        }
        DOM_NCCL(d, g_nccl.GroupEnd());
        DOM_NCCL(d, g_nccl.AllGather(d->d_counts, d->d_counts + kBins, kBins, ncclInt32, d->comm, d->side));
        { const int rc = wait_stream(d, d->side, "first contact with the neighbour ranks"); if (rc) return rc; }
        DOM_NCCL(d, g_nccl.AllReduce(d->vote_word, d->vote_word + 1, 1, ncclUint64, ncclMax,
                                     d->vote_comm ? d->vote_comm : d->comm, d->vote_stream));
        { const int rc = wait_stream(d, d->vote_stream, "first all-reduce of the rebuild vote"); if (rc) return rc; }
    }
    return DSMD_OK;
}

void dsmd_domain_destroy(dsmd_domain* d) {
    if (!d) return;
    if (d->vote_comm) g_nccl.CommDestroy(d->vote_comm);
    if (d->comm) g_nccl.CommDestroy(d->comm);
    for (int k = 0; k < 2; ++k) {
        cudaFree(d->key[k]); cudaFree(d->val[k]);
        cudaFreeHost(d->h_vote[k]);
        if (d->ev_vote[k]) cudaEventDestroy(d->ev_vote[k]);
    }
    cudaFree(d->flag); cudaFree(d->cnt); cudaFree(d->off); cudaFree(d->temp); cudaFree(d->d_counts); cudaFreeHost(d->h_counts);
    cudaFree(d->d_selected); cudaFree(d->d_verdict); cudaFreeHost(d->h_verdict); cudaFree(d->send_rec); cudaFree(d->recv_rec); cudaFree(d->send_index); cudaFree(d->send_image);
    cudaFree(d->send_pos); cudaFree(d->recv_pos); cudaFree(d->vote_word); cudaFree(d->field_send); cudaFree(d->field_recv);
    if (d->side) cudaStreamDestroy(d->side);
    if (d->vote_stream) cudaStreamDestroy(d->vote_stream);
    if (d->ev_main) cudaEventDestroy(d->ev_main);
    if (d->ev_side) cudaEventDestroy(d->ev_side);
    if (d->ev_disp) cudaEventDestroy(d->ev_disp);
    for (auto& ev : d->ev_phase)
        if (ev) cudaEventDestroy(ev);
    delete d;
}

const char* dsmd_domain_last_error(const dsmd_domain* d) { return d ? d->error.c_str() : "null domain"; }

int dsmd_domain_set_wait_limit(dsmd_domain* d, double seconds) {
    if (!d || !(seconds > 0.0)) return DSMD_ERR_INVALID;
    d->wait_limit_s = seconds;
    return DSMD_OK;
}

int dsmd_domain_abort(dsmd_domain* d) {
    if (!d) return DSMD_ERR_INVALID;
    // after DSMD_ERR_TIMEOUT: the communicators may hold kernels that wait for a rank that is gone; abort releases them
    if (d->vote_comm) { g_nccl.CommAbort(d->vote_comm); d->vote_comm = nullptr; }
    if (d->comm) { g_nccl.CommAbort(d->comm); d->comm = nullptr; }
    return DSMD_OK;
}

int dsmd_domain_rebuild(dsmd_domain* d, void* stream) {
    if (!d) return DSMD_ERR_INVALID;
    return rebuild(d, static_cast<cudaStream_t>(stream));
}

int dsmd_domain_refresh(dsmd_domain* d, void* stream) {
    if (!d) return DSMD_ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (d->world == 1) return DSMD_OK;
    { const int rc = refresh(d, s); if (rc) return rc; }
    DOM_CUDA(d, cudaStreamWaitEvent(s, d->ev_side, 0));
    return DSMD_OK;
}

int dsmd_domain_forces_host(dsmd_domain* d, const double* x, const double* y, const double* z, int with_rebuild, double* fx,
                            double* fy, double* fz, int64_t buffer_atoms, void* stream) {
    if (!d || !x || !y || !z || !fx || !fy || !fz || buffer_atoms < 0) return DSMD_ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    {   // the owned atoms, in the context's order
        int64_t n_owned = 0, n_total = 0;
        dsmd_counts(d->ctx, &n_owned, &n_total);
        if (n_owned > buffer_atoms) return dfail(d, DSMD_ERR_CAPACITY, "the host buffers are shorter than the owned atoms");
        const double* src[3] = {x, y, z};
        const int ids[3] = {DSMD_X, DSMD_Y, DSMD_Z};
        for (int a = 0; a < 3; ++a) {
            void* dst = nullptr;
            DOM_CTX(d, dsmd_device_pointer(d->ctx, ids[a], &dst));
            DOM_CUDA(d, cudaMemcpyAsync(dst, src[a], sizeof(double) * n_owned, cudaMemcpyHostToDevice, s));
        }
    }
    if (with_rebuild) {
        { const int rc = rebuild(d, s); if (rc) return rc; }
        DOM_CTX(d, dsmd_compute_forces(d->ctx, DSMD_PHASE_FULL, 0, s));
    } else {
        int64_t n_owned = 0, n_total = 0;
        dsmd_counts(d->ctx, &n_owned, &n_total);
        DOM_CTX(d, dsmd_pack_positions(d->ctx, 0, n_owned, s));
        if (d->world > 1) {
            // the ghost refresh on the side stream beside the interior pass, then the boundary pass
            { const int rc = refresh(d, s); if (rc) return rc; }
            DOM_CTX(d, dsmd_compute_forces(d->ctx, DSMD_PHASE_INTERIOR, 0, s));
            DOM_CUDA(d, cudaStreamWaitEvent(s, d->ev_side, 0));
            DOM_CTX(d, dsmd_compute_forces(d->ctx, DSMD_PHASE_BOUNDARY, 0, s));
        } else {
            DOM_CTX(d, dsmd_compute_forces(d->ctx, DSMD_PHASE_FULL, 0, s));
        }
    }
    int64_t n_owned = 0, n_total = 0;
    dsmd_counts(d->ctx, &n_owned, &n_total);
    if (n_owned > buffer_atoms)   // a rebuild brought more atoms in than the buffers hold
        return dfail(d, DSMD_ERR_CAPACITY, "the host buffers are shorter than the owned atoms after the rebuild");
    const MutableForces f = forces_of(d->ctx);
    const double* src[3] = {f.fx, f.fy, f.fz};
    double* dst[3] = {fx, fy, fz};
    for (int a = 0; a < 3; ++a)
        DOM_CUDA(d, cudaMemcpyAsync(dst[a], src[a], sizeof(double) * n_owned, cudaMemcpyDeviceToHost, s));
    return wait_stream(d, s, "host-buffer force call");
}

int dsmd_domain_reverse_forces(dsmd_domain* d, void* stream) {
    if (!d) return DSMD_ERR_INVALID;
    if (d->world == 1 || d->plan.n_peers == 0) return DSMD_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int32_t* ghost_slot = nullptr;
    DOM_CTX(d, dsmd_ghost_slots(d->ctx, &ghost_slot));
    MutableForces f = forces_of(d->ctx);
    // the forces on this rank's ghosts go back the way the ghosts came; what comes back is added to the owners
    if (d->n_ghost > 0) {
        k_force_gather<<<blocks_for(d->n_ghost, kThreads), kThreads, 0, s>>>(static_cast<int>(d->n_ghost), ghost_slot, f.fx, f.fy,
                                                                           f.fz, d->recv_pos);
        ++d->launches;
    }
    { const int rc = exchange(d, d->recv_pos, d->recv_from, d->send_pos, d->send_to, 3, s); if (rc) return rc; }
    if (d->n_send > 0) {
        k_force_add<<<blocks_for(d->n_send, kThreads), kThreads, 0, s>>>(static_cast<int>(d->n_send), d->send_index, d->send_pos,
                                                                       f.fx, f.fy, f.fz);
        ++d->launches;
    }
    DOM_CUDA(d, cudaGetLastError());
    return DSMD_OK;
}

int dsmd_domain_exchange_field(dsmd_domain* d, void* device_data, int64_t rows, int64_t width, int element_bytes, int reverse,
                               void* stream) {
    if (!d || !device_data || width <= 0 || width > (1 << 20)) return DSMD_ERR_INVALID;
    int64_t n_owned = 0, n_total = 0;
    dsmd_counts(d->ctx, &n_owned, &n_total);
    if (rows != n_total)
        return dfail(d, DSMD_ERR_INVALID, "the field has " + std::to_string(rows) + " rows, the halo has " + std::to_string(n_owned) +
                                              " owned + " + std::to_string(n_total - n_owned) + " ghost atoms");
    if (element_bytes != 4 && element_bytes != 8) return dfail(d, DSMD_ERR_INVALID, "field elements must be 4 or 8 bytes wide");
    if (d->world == 1 || d->plan.n_peers == 0) return DSMD_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (element_bytes == 4) return exchange_field_typed<float>(d, static_cast<float*>(device_data), static_cast<int>(width), reverse != 0, s);
    return exchange_field_typed<double>(d, static_cast<double*>(device_data), static_cast<int>(width), reverse != 0, s);
}

int dsmd_domain_reduce(dsmd_domain* d, double* values, int n, int op, void* stream) {
    if (!d || !values || n < 1 || n > 16 || (op != 0 && op != 1)) return DSMD_ERR_INVALID;
    if (d->world == 1) return DSMD_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    double* scratch = d->send_pos;   // idle between exchanges; ordered on the caller's stream like them
    DOM_CUDA(d, cudaMemcpyAsync(scratch, values, sizeof(double) * n, cudaMemcpyHostToDevice, s));
    DOM_NCCL(d, g_nccl.AllReduce(scratch, scratch + 16, n, ncclFloat64, op == 0 ? ncclSum : ncclMax, d->comm, s));
    DOM_CUDA(d, cudaMemcpyAsync(values, scratch + 16, sizeof(double) * n, cudaMemcpyDeviceToHost, s));
    return wait_stream(d, s, "reduction over the ranks");
}

int dsmd_domain_run(dsmd_domain* d, int64_t n_steps, double dt, double force_to_accel, double hi_frac, void* stream) {
    if (!d || n_steps < 0) return DSMD_ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const double limit2 = (hi_frac * d->skin) * (hi_frac * d->skin);
    void* word = nullptr;
    DOM_CTX(d, dsmd_displacement_word(d->ctx, &word));
    auto bits_to_double = [](unsigned long long b) { double v; std::memcpy(&v, &b, sizeof(v)); return v; };
    auto mark = [&](int k) { if (d->profile) cudaEventRecord(d->ev_phase[k], s); };
    for (int64_t step = 0; step < n_steps; ++step) {
        mark(0);
        // v += dt/2 a, x += dt v, pack owned, displacement; after the first step of the call the kick is a whole dt: the
        // second half of the previous step (left out below) and this first half use the same forces
        DOM_CTX(d, dsmd_integrate(d->ctx, step > 0 ? 3 : 1, dt, force_to_accel, s));
        mark(1);
        // The vote: all ranks take the MAX of their displacement words; the host reads the result of the PREVIOUS step (its
        // copy finished long ago) and extrapolates by its last growth (src/md_simulation.cpp:1232-1245). The word is copied
        // aside and reduced on the vote's own stream and communicator: nothing on the main or side stream waits for it.
        const int slot = static_cast<int>(step & 1);
        if (d->vote_pending >= 0) {
            { const int rc = wait_event(d, d->ev_vote[d->vote_pending], "rebuild vote of the previous step"); if (rc) return rc; }
            d->d_prev2 = d->d_prev;
            d->d_prev = std::sqrt(bits_to_double(*d->h_vote[d->vote_pending]));
            d->worst_disp_sq = std::max(d->worst_disp_sq, d->d_prev * d->d_prev);
        }
        if (d->world > 1) {
            DOM_CUDA(d, cudaEventRecord(d->ev_disp, s));
            DOM_CUDA(d, cudaStreamWaitEvent(d->vote_stream, d->ev_disp, 0));
            DOM_CUDA(d, cudaMemcpyAsync(d->vote_word, word, sizeof(unsigned long long), cudaMemcpyDeviceToDevice, d->vote_stream));
            DOM_NCCL(d, g_nccl.AllReduce(d->vote_word, d->vote_word + 1, 1, ncclUint64, ncclMax,
                                         d->vote_comm ? d->vote_comm : d->comm, d->vote_stream));
            DOM_CUDA(d, cudaMemcpyAsync(d->h_vote[slot], d->vote_word + 1, sizeof(unsigned long long), cudaMemcpyDeviceToHost,
                                        d->vote_stream));
            DOM_CUDA(d, cudaEventRecord(d->ev_vote[slot], d->vote_stream));
        } else {
            DOM_CUDA(d, cudaMemcpyAsync(d->h_vote[slot], word, sizeof(unsigned long long), cudaMemcpyDeviceToHost, s));
            DOM_CUDA(d, cudaEventRecord(d->ev_vote[slot], s));
        }
        d->vote_pending = slot;
        const double predicted = d->d_prev + 1.5 * std::max(d->d_prev - d->d_prev2, 0.0);
        mark(2);
        bool rebuilt = false;
        if (predicted * predicted > limit2) {
            if (d->world > 1 && !d->vote_comm) {
                // one communicator for everything: the vote in flight must finish before the rebuild's messages are queued
                DOM_CUDA(d, cudaStreamWaitEvent(s, d->ev_vote[slot], 0));
            }
            { const int rc = rebuild(d, s); if (rc) return rc; }
            rebuilt = true;
            mark(3);
            DOM_CTX(d, dsmd_compute_forces(d->ctx, DSMD_PHASE_FULL, 0, s));
            mark(4);
        } else if (d->world == 1) {
            mark(3);
            DOM_CTX(d, dsmd_compute_forces(d->ctx, DSMD_PHASE_FULL, 0, s));
            mark(4);
        } else {
            if (!d->vote_comm) DOM_CUDA(d, cudaStreamWaitEvent(d->side, d->ev_vote[slot], 0));
            { const int rc = refresh(d, s); if (rc) return rc; }
            DOM_CTX(d, dsmd_compute_forces(d->ctx, DSMD_PHASE_INTERIOR, 0, s));
            mark(3);
            DOM_CUDA(d, cudaStreamWaitEvent(s, d->ev_side, 0));
            DOM_CTX(d, dsmd_compute_forces(d->ctx, DSMD_PHASE_BOUNDARY, 0, s));
            mark(4);
        }
        // bonded terms (none set: returns at once): ghost positions are current after the boundary pass; a term is
        // evaluated on every rank that owns one of its atoms, forces go to owned atoms only
        DOM_CTX(d, dsmd_compute_bonded(d->ctx, s));
        if (step + 1 == n_steps) DOM_CTX(d, dsmd_integrate(d->ctx, 2, dt, force_to_accel, s));
        mark(5);
        if (d->profile) {
            { const int rc = wait_stream(d, s, "profiled step"); if (rc) return rc; }
            float ms = 0.f;
            for (int k = 0; k < 5; ++k) {
                cudaEventElapsedTime(&ms, d->ev_phase[k], d->ev_phase[k + 1]);
                d->phase_ms[(rebuilt && k == 2) ? 5 : k] += ms;
            }
            ++d->phase_steps;
        }
    }
    return DSMD_OK;
}

int dsmd_domain_profile(dsmd_domain* d, int enable, double phase_ms[10], int64_t* steps) {
    if (!d) return DSMD_ERR_INVALID;
    if (enable && !d->ev_phase[0])
        for (int k = 0; k < 8; ++k) DOM_CUDA(d, cudaEventCreate(&d->ev_phase[k]));
    if (phase_ms) {
        for (int k = 0; k < 6; ++k) phase_ms[k] = d->phase_ms[k];
        for (int k = 0; k < 4; ++k) phase_ms[6 + k] = d->rebuild_ms[k];
    }
    if (steps) *steps = d->phase_steps;
    d->profile = enable != 0;
    return DSMD_OK;
}

int dsmd_domain_stats(const dsmd_domain* d, int64_t* rebuilds, int64_t* migrated, int64_t* ghosts, int64_t* sent_per_step,
                      double* worst_disp_sq, int64_t* launches) {
    if (!d) return DSMD_ERR_INVALID;
    if (rebuilds) *rebuilds = d->rebuilds;
    if (migrated) *migrated = d->migrated;
    if (ghosts) *ghosts = d->n_ghost;
    if (sent_per_step) *sent_per_step = d->n_send;
    if (worst_disp_sq) *worst_disp_sq = d->worst_disp_sq;
    if (launches) *launches = d->launches;
    return DSMD_OK;
}

int dsmd_domain_peers(const dsmd_domain* d, int32_t* n_peers, int32_t peers[26], int32_t n_messages_per_exchange[1]) {
    if (!d || !n_peers) return DSMD_ERR_INVALID;
    *n_peers = d->plan.n_peers;
    if (peers)
        for (int p = 0; p < d->plan.n_peers; ++p) peers[p] = d->plan.peer[p];
    if (n_messages_per_exchange) {
        int m = 0;
        for (int p = 0; p < d->plan.n_peers; ++p) m += (d->send_to[p] > 0) + (d->recv_from[p] > 0);
        n_messages_per_exchange[0] = m;
    }
    return DSMD_OK;
}

}  // extern "C"
