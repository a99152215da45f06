// Spatial domain decomposition over the GPUs of one node, native: brick grid, atom migration, ghost (halo) plan, the
// per-step positions-only refresh overlapped with the interior force pass, the rebuild vote, and the MD step loop around
// them - one process per GPU, NCCL point-to-point between neighbour bricks (NVLink / NVSwitch underneath).
//
// What the reference gets from its external decomposition library through MDSystem::migrate_particles_on_device,
// exchange_halo_on_device(rebuild), begin/end_halo_exchange_on_device (src/md_system.cpp:1448-1509) and from
// CommBackend::unify_rebuild_decision (src/comm_backend.cpp:76-92). Conventions: owned atoms first, ghosts behind them; a
// ghost is every periodic image of a neighbour's atom within the halo width of this brick on the split axes (edges and
// corners included), already image-shifted; an axis with one brick gets no ghosts (the wrapping fixed-point coordinates
// resolve it). Data path per step: one pack kernel -> grouped ncclSend/ncclRecv with the (at most 26) neighbour
// directions -> one unpack kernel, on a high-priority side stream while the main stream computes the interior forces.
// No collective on the data path; an 8-byte MAX all-reduce carries the rebuild vote, an all-gather of the per-direction
// counts sizes the messages at a rebuild.
//
// Built on the public C ABI of the context (dsmd_b200.h) plus a few kernels of its own; NCCL is bound at run time
// (dlopen), so the library loads on machines without it as long as only one rank is used.

#include <cub/cub.cuh>
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/dsmd_b200.h"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxDirs = 26;

inline unsigned blocks_for(int64_t n, int threads) { return static_cast<unsigned>((n + threads - 1) / threads); }

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
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
    DSMD_NCCL_SYM(GroupStart, "ncclGroupStart")
    DSMD_NCCL_SYM(GroupEnd, "ncclGroupEnd")
    DSMD_NCCL_SYM(Send, "ncclSend")
    DSMD_NCCL_SYM(Recv, "ncclRecv")
    DSMD_NCCL_SYM(AllReduce, "ncclAllReduce")
    DSMD_NCCL_SYM(AllGather, "ncclAllGather")
    DSMD_NCCL_SYM(GetErrorString, "ncclGetErrorString")
#undef DSMD_NCCL_SYM
    return true;
}

struct DirTable {
    int n;                    // directions in use
    int e[kMaxDirs][3];       // the way the data travels
    int image[kMaxDirs][3];   // box lengths added to the sender's coordinates
    double lo[3], hi[3];      // this rank's brick
    double box[3];
    double halo;
    int split[3];
};

// key 0 = stays; key 1 + d = leaves along direction d; key n + 1 = lost (moved further than one brick, or not finite).
// Adds one to bin `bin` (or nothing when bin < 0) through a per-block histogram in shared memory: one global atomic per
// non-empty bin and block instead of one per atom (all atoms of a brick but a few hit the same "stays" bin). Holds a
// block-wide barrier: call it exactly once, from code that every thread of the block executes (never from one side of a
// branch, nor after an early return of some threads: a warp whose lanes reach two different barrier instructions hangs).
__device__ __forceinline__ void block_histogram_add(int* hist, int bin, int* __restrict__ counts) {
    if (bin >= 0) atomicAdd(&hist[bin], 1);
    __syncthreads();
    if (threadIdx.x < kMaxDirs + 2 && hist[threadIdx.x] > 0) atomicAdd(&counts[threadIdx.x], hist[threadIdx.x]);
}

__global__ void k_classify_leave(DirTable t, int n_owned, const double* __restrict__ x, const double* __restrict__ y,
                                 const double* __restrict__ z, unsigned* __restrict__ key, int* __restrict__ val,
                                 int* __restrict__ counts) {
    __shared__ int hist[kMaxDirs + 2];
    if (threadIdx.x < kMaxDirs + 2) hist[threadIdx.x] = 0;
    __syncthreads();
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
        unsigned k = 0;
        if (lost) {
            k = static_cast<unsigned>(t.n + 1);
        } else if (e[0] || e[1] || e[2]) {
            k = static_cast<unsigned>(t.n + 1);
            for (int d = 0; d < t.n; ++d)
                if (t.e[d][0] == e[0] && t.e[d][1] == e[1] && t.e[d][2] == e[2]) k = static_cast<unsigned>(d + 1);
        }
        key[i] = k;
        val[i] = i;
        bin = static_cast<int>(k);
    }
    block_histogram_add(hist, bin, counts);   // the one barrier of this kernel: every thread of the block reaches it
}

// How many neighbour directions need atom i as a ghost, and which (bit d).
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
                              int* __restrict__ val, int* __restrict__ counts, int capacity) {
    __shared__ int hist[kMaxDirs + 2];
    if (threadIdx.x < kMaxDirs + 2) hist[threadIdx.x] = 0;
    __syncthreads();
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
            atomicAdd(&hist[d], 1);
        }
    }
    block_histogram_add(hist, -1, counts);
}

struct Fields {
    const double *x, *y, *z, *vx, *vy, *vz, *mass, *charge;
    const int *type, *gid;
};

// Full records {x, y, z, vx, vy, vz, mass, charge} + {type, gid} of the listed atoms, shifted by the image of the
// direction each entry travels (key_offset: 1 for migration keys, 0 for halo keys; entries with no direction get no shift).
__global__ void k_pack_records(DirTable t, int count, const int* __restrict__ index, const unsigned* __restrict__ key,
                               int key_offset, Fields f, double* __restrict__ real_out, int* __restrict__ int_out) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= count) return;
    const int s = index[k];
    const int d = static_cast<int>(key[k]) - key_offset;
    double sx = 0.0, sy = 0.0, sz = 0.0;
    if (d >= 0 && d < t.n) {
        sx = t.image[d][0] * t.box[0];
        sy = t.image[d][1] * t.box[1];
        sz = t.image[d][2] * t.box[2];
    }
    double* o = real_out + 8 * static_cast<size_t>(k);
    o[0] = f.x[s] + sx; o[1] = f.y[s] + sy; o[2] = f.z[s] + sz;
    o[3] = f.vx[s]; o[4] = f.vy[s]; o[5] = f.vz[s];
    o[6] = f.mass[s]; o[7] = f.charge[s];
    int_out[2 * k] = f.type[s];
    int_out[2 * k + 1] = f.gid[s];
}

__global__ void k_send_images(DirTable t, int count, const unsigned* __restrict__ key, signed char* __restrict__ image) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= count) return;
    const int d = static_cast<int>(key[k]);
    image[3 * k] = static_cast<signed char>(t.image[d][0]);
    image[3 * k + 1] = static_cast<signed char>(t.image[d][1]);
    image[3 * k + 2] = static_cast<signed char>(t.image[d][2]);
}

template <class T>
bool grow(T*& ptr, size_t& capacity, size_t needed) {
    if (needed <= capacity) return true;
    const size_t grown = std::max(needed, capacity + capacity / 2);
    if (ptr) cudaFree(ptr);
    ptr = nullptr;
    capacity = 0;
    if (cudaMalloc(&ptr, grown * sizeof(T)) != cudaSuccess) return false;
    capacity = grown;
    return true;
}

}  // namespace

struct dsmd_domain {
    dsmd_ctx* ctx = nullptr;
    int rank = 0, world = 1;
    int dims[3] = {1, 1, 1}, coords[3] = {0, 0, 0};
    DirTable table{};
    int dest[kMaxDirs], src[kMaxDirs];
    double skin = 0.0;
    ncclComm_t comm = nullptr;
    cudaStream_t side = nullptr;
    cudaEvent_t ev_main = nullptr, ev_side = nullptr, ev_vote[2] = {nullptr, nullptr};
    std::string error;

    // scratch (device)
    unsigned* key[2] = {nullptr, nullptr};  size_t cap_key[2] = {0, 0};
    int* val[2] = {nullptr, nullptr};       size_t cap_val[2] = {0, 0};
    int* cnt = nullptr;                     size_t cap_cnt = 0;
    int* off = nullptr;                     size_t cap_off = 0;
    void* temp = nullptr;                   size_t cap_temp = 0;   // bytes (as unsigned char)
    int* d_counts = nullptr;                // [kMaxDirs + 2] this rank, then [world * (kMaxDirs + 2)] gathered
    int* h_counts = nullptr;                // pinned, same layout
    double* send_real = nullptr;            size_t cap_send_real = 0;
    int* send_int = nullptr;                size_t cap_send_int = 0;
    double* recv_real = nullptr;            size_t cap_recv_real = 0;
    int* recv_int = nullptr;                size_t cap_recv_int = 0;
    double* stay_real = nullptr;            size_t cap_stay_real = 0;
    int* stay_int = nullptr;                size_t cap_stay_int = 0;
    // the plan of the per-step refresh
    int* send_index = nullptr;              size_t cap_send_index = 0;
    signed char* send_image = nullptr;      size_t cap_send_image = 0;
    double* send_pos = nullptr;             size_t cap_send_pos = 0;
    double* recv_pos = nullptr;             size_t cap_recv_pos = 0;
    int send_counts[kMaxDirs] = {}, recv_counts[kMaxDirs] = {};
    int64_t n_send = 0, n_ghost = 0;
    // rebuild vote
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

#define DOM_ALLOC(d, ok)                                                              \
    do {                                                                              \
        if (!(ok)) return dfail(d, DSMD_ERR_CUDA, "device allocation failed");        \
    } while (0)

int rank_of(const dsmd_domain* d, const int c[3]) { return (c[0] * d->dims[1] + c[1]) * d->dims[2] + c[2]; }

// Neighbour of brick `coords` along e with periodic wrap; image = box lengths the receiver adds.
int neighbour(const dsmd_domain* d, const int e[3], int image[3]) {
    int c[3];
    for (int a = 0; a < 3; ++a) {
        int v = d->coords[a] + e[a];
        image[a] = 0;
        if (v < 0) { v += d->dims[a]; image[a] = 1; }
        else if (v >= d->dims[a]) { v -= d->dims[a]; image[a] = -1; }
        c[a] = v;
    }
    return rank_of(d, c);
}

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

// Sorts `n` (key, val) pairs by key (stable), result in key[1] / val[1].
int sort_pairs(dsmd_domain* d, int64_t n, int bits, cudaStream_t s) {
    size_t need = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, need, d->key[0], d->key[1], d->val[0], d->val[1], static_cast<int>(n), 0, bits, s);
    unsigned char* t = static_cast<unsigned char*>(d->temp);
    DOM_ALLOC(d, grow(t, d->cap_temp, need));
    d->temp = t;
    DOM_CUDA(d, cub::DeviceRadixSort::SortPairs(d->temp, need, d->key[0], d->key[1], d->val[0], d->val[1], static_cast<int>(n),
                                                0, bits, s));
    return DSMD_OK;
}

// Every rank's per-key counts to every rank; h_counts[r * stride + k] afterwards. One host synchronisation.
int gather_counts(dsmd_domain* d, cudaStream_t s) {
    const int stride = kMaxDirs + 2;
    if (d->world > 1) {
        DOM_NCCL(d, g_nccl.AllGather(d->d_counts, d->d_counts + stride, stride, ncclInt32, d->comm, s));
        DOM_CUDA(d, cudaMemcpyAsync(d->h_counts, d->d_counts + stride, sizeof(int) * stride * d->world, cudaMemcpyDeviceToHost, s));
    } else {
        DOM_CUDA(d, cudaMemcpyAsync(d->h_counts, d->d_counts, sizeof(int) * stride, cudaMemcpyDeviceToHost, s));
    }
    DOM_CUDA(d, cudaStreamSynchronize(s));
    return DSMD_OK;
}

// Exchanges records: the entries of send_real / send_int are grouped by direction (send_n[dir]); what arrives is laid
// out direction after direction in recv_real / recv_int (recv_n[dir]).
int exchange_records(dsmd_domain* d, const int* send_n, const int* recv_n, cudaStream_t s) {
    if (d->world == 1) return DSMD_OK;
    DOM_NCCL(d, g_nccl.GroupStart());
    size_t so = 0, ro = 0;
    for (int k = 0; k < d->table.n; ++k) {
        if (recv_n[k] > 0) {
            DOM_NCCL(d, g_nccl.Recv(d->recv_real + 8 * ro, 8 * static_cast<size_t>(recv_n[k]), ncclFloat64, d->src[k], d->comm, s));
            DOM_NCCL(d, g_nccl.Recv(d->recv_int + 2 * ro, 2 * static_cast<size_t>(recv_n[k]), ncclInt32, d->src[k], d->comm, s));
        }
        if (send_n[k] > 0) {
            DOM_NCCL(d, g_nccl.Send(d->send_real + 8 * so, 8 * static_cast<size_t>(send_n[k]), ncclFloat64, d->dest[k], d->comm, s));
            DOM_NCCL(d, g_nccl.Send(d->send_int + 2 * so, 2 * static_cast<size_t>(send_n[k]), ncclInt32, d->dest[k], d->comm, s));
        }
        so += send_n[k];
        ro += recv_n[k];
    }
    DOM_NCCL(d, g_nccl.GroupEnd());
    return DSMD_OK;
}

int migrate(dsmd_domain* d, cudaStream_t s) {
    const int stride = kMaxDirs + 2;
    int64_t n_owned = 0, n_total = 0;
    dsmd_counts(d->ctx, &n_owned, &n_total);
    const int n = static_cast<int>(n_owned);
    for (int k = 0; k < 2; ++k) {
        DOM_ALLOC(d, grow(d->key[k], d->cap_key[k], static_cast<size_t>(n) + 1));
        DOM_ALLOC(d, grow(d->val[k], d->cap_val[k], static_cast<size_t>(n) + 1));
    }
    DOM_CUDA(d, cudaMemsetAsync(d->d_counts, 0, sizeof(int) * stride, s));
    Fields f = fields_of(d->ctx);
    k_classify_leave<<<blocks_for(n, kThreads), kThreads, 0, s>>>(d->table, n, f.x, f.y, f.z, d->key[0], d->val[0], d->d_counts);
    ++d->launches;
    { const int rc = sort_pairs(d, n, 5, s); if (rc) return rc; }
    { const int rc = gather_counts(d, s); if (rc) return rc; }
    const int* mine = d->h_counts + static_cast<size_t>(d->rank) * stride * (d->world > 1 ? 1 : 0);
    if (mine[d->table.n + 1] > 0)
        return dfail(d, DSMD_ERR_OUT_OF_DOMAIN, "atoms moved further than one brick between list builds (or are not finite)");
    const int n_stay = mine[0];
    int send_n[kMaxDirs] = {}, recv_n[kMaxDirs] = {};
    int n_leave = 0, n_arrive = 0;
    for (int k = 0; k < d->table.n; ++k) {
        send_n[k] = mine[1 + k];
        recv_n[k] = d->world > 1 ? d->h_counts[static_cast<size_t>(d->src[k]) * stride + 1 + k] : 0;
        n_leave += send_n[k];
        n_arrive += recv_n[k];
    }
    // records of the stayers and of the leavers (sorted order: stayers first, then direction after direction)
    DOM_ALLOC(d, grow(d->stay_real, d->cap_stay_real, 8 * static_cast<size_t>(n_stay) + 8));
    DOM_ALLOC(d, grow(d->stay_int, d->cap_stay_int, 2 * static_cast<size_t>(n_stay) + 2));
    DOM_ALLOC(d, grow(d->send_real, d->cap_send_real, 8 * static_cast<size_t>(n_leave) + 8));
    DOM_ALLOC(d, grow(d->send_int, d->cap_send_int, 2 * static_cast<size_t>(n_leave) + 2));
    DOM_ALLOC(d, grow(d->recv_real, d->cap_recv_real, 8 * static_cast<size_t>(n_arrive) + 8));
    DOM_ALLOC(d, grow(d->recv_int, d->cap_recv_int, 2 * static_cast<size_t>(n_arrive) + 2));
    if (n_stay > 0) {
        k_pack_records<<<blocks_for(n_stay, kThreads), kThreads, 0, s>>>(d->table, n_stay, d->val[1], d->key[1], 1, f,
                                                                        d->stay_real, d->stay_int);
        ++d->launches;
    }
    if (n_leave > 0) {
        k_pack_records<<<blocks_for(n_leave, kThreads), kThreads, 0, s>>>(d->table, n_leave, d->val[1] + n_stay,
                                                                         d->key[1] + n_stay, 1, f, d->send_real, d->send_int);
        ++d->launches;
    }
    { const int rc = exchange_records(d, send_n, recv_n, s); if (rc) return rc; }
    DOM_CTX(d, dsmd_set_counts(d->ctx, 0, 0));
    DOM_CTX(d, dsmd_halo_append_records(d->ctx, d->stay_real, d->stay_int, n_stay, s));
    DOM_CTX(d, dsmd_halo_append_records(d->ctx, d->recv_real, d->recv_int, n_arrive, s));
    DOM_CTX(d, dsmd_set_counts(d->ctx, n_stay + n_arrive, n_stay + n_arrive));
    d->migrated += n_leave;
    return DSMD_OK;
}

int build_halo(dsmd_domain* d, cudaStream_t s) {
    const int stride = kMaxDirs + 2;
    int64_t n_owned = 0, n_total = 0;
    dsmd_counts(d->ctx, &n_owned, &n_total);
    const int n = static_cast<int>(n_owned);
    d->n_send = d->n_ghost = 0;
    std::fill(d->send_counts, d->send_counts + kMaxDirs, 0);
    std::fill(d->recv_counts, d->recv_counts + kMaxDirs, 0);
    if (d->world == 1 || d->table.n == 0) return DSMD_OK;
    Fields f = fields_of(d->ctx);
    DOM_ALLOC(d, grow(d->cnt, d->cap_cnt, static_cast<size_t>(n) + 1));
    DOM_ALLOC(d, grow(d->off, d->cap_off, static_cast<size_t>(n) + 1));
    k_halo_count<<<blocks_for(n, kThreads), kThreads, 0, s>>>(d->table, n, f.x, f.y, f.z, d->cnt);
    ++d->launches;
    size_t need = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, need, d->cnt, d->off, n, s);
    unsigned char* t = static_cast<unsigned char*>(d->temp);
    DOM_ALLOC(d, grow(t, d->cap_temp, need));
    d->temp = t;
    DOM_CUDA(d, cub::DeviceScan::ExclusiveSum(d->temp, need, d->cnt, d->off, n, s));
    // An atom is needed by at most 7 directions, and only atoms near a face by any: 2 n entries cover every sane brick;
    // the exact total comes back with the counts and is checked.
    const size_t capacity = 2 * static_cast<size_t>(n) + 1024;
    for (int k = 0; k < 2; ++k) {
        DOM_ALLOC(d, grow(d->key[k], d->cap_key[k], capacity));
        DOM_ALLOC(d, grow(d->val[k], d->cap_val[k], capacity));
    }
    DOM_CUDA(d, cudaMemsetAsync(d->d_counts, 0, sizeof(int) * stride, s));
    k_halo_expand<<<blocks_for(n, kThreads), kThreads, 0, s>>>(d->table, n, f.x, f.y, f.z, d->off, d->key[0], d->val[0],
                                                              d->d_counts, static_cast<int>(capacity));
    ++d->launches;
    { const int rc = gather_counts(d, s); if (rc) return rc; }
    const int* mine = d->h_counts + static_cast<size_t>(d->rank) * stride;
    int64_t n_send = 0, n_recv = 0;
    for (int k = 0; k < d->table.n; ++k) {
        d->send_counts[k] = mine[k];
        d->recv_counts[k] = d->h_counts[static_cast<size_t>(d->src[k]) * stride + k];
        n_send += d->send_counts[k];
        n_recv += d->recv_counts[k];
    }
    if (static_cast<size_t>(n_send) > capacity)
        return dfail(d, DSMD_ERR_CAPACITY, "halo wider than the brick: more ghost sends than twice the owned atoms");
    { const int rc = sort_pairs(d, n_send, 5, s); if (rc) return rc; }
    DOM_ALLOC(d, grow(d->send_real, d->cap_send_real, 8 * static_cast<size_t>(n_send) + 8));
    DOM_ALLOC(d, grow(d->send_int, d->cap_send_int, 2 * static_cast<size_t>(n_send) + 2));
    DOM_ALLOC(d, grow(d->recv_real, d->cap_recv_real, 8 * static_cast<size_t>(n_recv) + 8));
    DOM_ALLOC(d, grow(d->recv_int, d->cap_recv_int, 2 * static_cast<size_t>(n_recv) + 2));
    DOM_ALLOC(d, grow(d->send_index, d->cap_send_index, static_cast<size_t>(n_send) + 1));
    DOM_ALLOC(d, grow(d->send_image, d->cap_send_image, 3 * static_cast<size_t>(n_send) + 3));
    DOM_ALLOC(d, grow(d->send_pos, d->cap_send_pos, 3 * static_cast<size_t>(n_send) + 3));
    DOM_ALLOC(d, grow(d->recv_pos, d->cap_recv_pos, 3 * static_cast<size_t>(n_recv) + 3));
    if (n_send > 0) {
        k_pack_records<<<blocks_for(n_send, kThreads), kThreads, 0, s>>>(d->table, static_cast<int>(n_send), d->val[1],
                                                                        d->key[1], 0, f, d->send_real, d->send_int);
        k_send_images<<<blocks_for(n_send, kThreads), kThreads, 0, s>>>(d->table, static_cast<int>(n_send), d->key[1],
                                                                       d->send_image);
        d->launches += 2;
        DOM_CUDA(d, cudaMemcpyAsync(d->send_index, d->val[1], sizeof(int) * n_send, cudaMemcpyDeviceToDevice, s));
    }
    { const int rc = exchange_records(d, d->send_counts, d->recv_counts, s); if (rc) return rc; }
    DOM_CTX(d, dsmd_halo_append_records(d->ctx, d->recv_real, d->recv_int, n_recv, s));
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
    if (d->world > 1) { const int rc = migrate(d, s); if (rc) return rc; }
    lap(0, t0);
    DOM_CTX(d, dsmd_sort_owned(d->ctx, s));
    lap(1, t0);
    { const int rc = build_halo(d, s); if (rc) return rc; }
    lap(2, t0);
    DOM_CTX(d, dsmd_build_neighbor_list(d->ctx, s));
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
    DOM_NCCL(d, g_nccl.GroupStart());
    size_t so = 0, ro = 0;
    for (int k = 0; k < d->table.n; ++k) {
        if (d->recv_counts[k] > 0)
            DOM_NCCL(d, g_nccl.Recv(d->recv_pos + 3 * ro, 3 * static_cast<size_t>(d->recv_counts[k]), ncclFloat64, d->src[k],
                                    d->comm, d->side));
        if (d->send_counts[k] > 0)
            DOM_NCCL(d, g_nccl.Send(d->send_pos + 3 * so, 3 * static_cast<size_t>(d->send_counts[k]), ncclFloat64, d->dest[k],
                                    d->comm, d->side));
        so += d->send_counts[k];
        ro += d->recv_counts[k];
    }
    DOM_NCCL(d, g_nccl.GroupEnd());
    DOM_CTX(d, dsmd_halo_unpack(d->ctx, d->recv_pos, 0, d->n_ghost, d->side));
    DOM_CUDA(d, cudaEventRecord(d->ev_side, d->side));
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
    for (int a = 0; a < 3; ++a) d->dims[a] = dims[a];
    d->coords[0] = rank / (dims[1] * dims[2]);
    d->coords[1] = (rank / dims[2]) % dims[1];
    d->coords[2] = rank % dims[2];
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
    t.n = 0;
    for (int ex = -1; ex <= 1; ++ex)
        for (int ey = -1; ey <= 1; ++ey)
            for (int ez = -1; ez <= 1; ++ez) {
                const int e[3] = {ex, ey, ez};
                if (!ex && !ey && !ez) continue;
                bool ok = true;
                for (int a = 0; a < 3; ++a) ok = ok && (e[a] == 0 || t.split[a]);
                if (!ok) continue;
                const int k = t.n++;
                int image[3], back[3] = {-ex, -ey, -ez}, unused[3];
                d->dest[k] = neighbour(d, e, image);
                d->src[k] = neighbour(d, back, unused);
                for (int a = 0; a < 3; ++a) { t.e[k][a] = e[a]; t.image[k][a] = image[a]; }
            }
    const int stride = kMaxDirs + 2;
    DOM_CUDA(d, cudaMalloc(&d->d_counts, sizeof(int) * stride * (world + 1)));
    DOM_CUDA(d, cudaMallocHost(&d->h_counts, sizeof(int) * stride * (world + 1)));
    for (int k = 0; k < 2; ++k) {
        DOM_CUDA(d, cudaMallocHost(&d->h_vote[k], sizeof(unsigned long long)));
        *d->h_vote[k] = 0ull;
        DOM_CUDA(d, cudaEventCreateWithFlags(&d->ev_vote[k], cudaEventDisableTiming));
    }
    int lo_prio = 0, hi_prio = 0;
    DOM_CUDA(d, cudaDeviceGetStreamPriorityRange(&lo_prio, &hi_prio));
    DOM_CUDA(d, cudaStreamCreateWithPriority(&d->side, cudaStreamNonBlocking, hi_prio));
    DOM_CUDA(d, cudaEventCreateWithFlags(&d->ev_main, cudaEventDisableTiming));
    DOM_CUDA(d, cudaEventCreateWithFlags(&d->ev_side, cudaEventDisableTiming));
    if (world > 1) {
        if (!unique_id) return dfail(d, DSMD_ERR_INVALID, "several ranks need the NCCL unique id of rank 0");
        if (!load_nccl(nccl_library_path, d->error)) return DSMD_ERR_INVALID;
        ncclUniqueId id;
        std::memcpy(&id, unique_id, 128);
        DOM_NCCL(d, g_nccl.CommInitRank(&d->comm, world, id, rank));
    }
    return DSMD_OK;
}

void dsmd_domain_destroy(dsmd_domain* d) {
    if (!d) return;
    if (d->comm) g_nccl.CommDestroy(d->comm);
    for (int k = 0; k < 2; ++k) {
        cudaFree(d->key[k]); cudaFree(d->val[k]);
        cudaFreeHost(d->h_vote[k]);
        if (d->ev_vote[k]) cudaEventDestroy(d->ev_vote[k]);
    }
    cudaFree(d->cnt); cudaFree(d->off); cudaFree(d->temp); cudaFree(d->d_counts); cudaFreeHost(d->h_counts);
    cudaFree(d->send_real); cudaFree(d->send_int); cudaFree(d->recv_real); cudaFree(d->recv_int);
    cudaFree(d->stay_real); cudaFree(d->stay_int); cudaFree(d->send_index); cudaFree(d->send_image);
    cudaFree(d->send_pos); cudaFree(d->recv_pos);
    if (d->side) cudaStreamDestroy(d->side);
    if (d->ev_main) cudaEventDestroy(d->ev_main);
    if (d->ev_side) cudaEventDestroy(d->ev_side);
    delete d;
}

const char* dsmd_domain_last_error(const dsmd_domain* d) { return d ? d->error.c_str() : "null domain"; }

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
        DOM_CTX(d, dsmd_integrate(d->ctx, 1, dt, force_to_accel, s));   // v += dt/2 a, x += dt v, pack owned, displacement
        mark(1);
        // The vote: all ranks take the MAX of their displacement words; the host reads the result of the PREVIOUS step (its
        // copy finished long ago) and extrapolates by its last growth (src/md_simulation.cpp:1232-1245). The all-reduce
        // is issued on the main stream, before the refresh goes to the side stream: every call on the communicator is
        // then ordered by the streams themselves (main -> ev_main -> side -> ev_side -> main).
        if (d->world > 1) DOM_NCCL(d, g_nccl.AllReduce(word, word, 1, ncclUint64, ncclMax, d->comm, s));
        cudaStream_t vote_stream = s;
        if (d->vote_pending >= 0) {
            DOM_CUDA(d, cudaEventSynchronize(d->ev_vote[d->vote_pending]));
            d->d_prev2 = d->d_prev;
            d->d_prev = std::sqrt(bits_to_double(*d->h_vote[d->vote_pending]));
            d->worst_disp_sq = std::max(d->worst_disp_sq, d->d_prev * d->d_prev);
        }
        const int slot = static_cast<int>(step & 1);
        DOM_CUDA(d, cudaMemcpyAsync(d->h_vote[slot], word, sizeof(unsigned long long), cudaMemcpyDeviceToHost, vote_stream));
        DOM_CUDA(d, cudaEventRecord(d->ev_vote[slot], vote_stream));
        d->vote_pending = slot;
        const double predicted = d->d_prev + 1.5 * std::max(d->d_prev - d->d_prev2, 0.0);
        mark(2);
        bool rebuilt = false;
        if (predicted * predicted > limit2) {
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
            { const int rc = refresh(d, s); if (rc) return rc; }
            DOM_CTX(d, dsmd_compute_forces(d->ctx, DSMD_PHASE_INTERIOR, 0, s));
            mark(3);
            DOM_CUDA(d, cudaStreamWaitEvent(s, d->ev_side, 0));
            DOM_CTX(d, dsmd_compute_forces(d->ctx, DSMD_PHASE_BOUNDARY, 0, s));
            mark(4);
        }
        DOM_CTX(d, dsmd_integrate(d->ctx, 2, dt, force_to_accel, s));
        mark(5);
        if (d->profile) {
            DOM_CUDA(d, cudaStreamSynchronize(s));
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

}  // extern "C"
