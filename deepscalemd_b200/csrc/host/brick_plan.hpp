// Host-side bookkeeping of the brick decomposition: who the neighbours of a rank are, how the per-direction counts that
// the ranks publish turn into one message per neighbour rank, and the verdict every rank reaches from those counts.
// Plain C++ (no CUDA): used by the domain code and, through test hooks, by the CPU tests.
#pragma once

#include <algorithm>
#include <string>
#include <vector>

namespace dsmd::host {

constexpr int kMaxDirs = 26;
constexpr int kBins = kMaxDirs + 3;     // what a rank publishes: stays, per direction, lost atoms, room for more atoms
constexpr int kBinLost = kMaxDirs + 1;
constexpr int kBinRoom = kMaxDirs + 2;

// The neighbour directions of one rank of a dims[0] x dims[1] x dims[2] periodic brick grid, ordered by destination
// rank, so that everything bound for one rank is one contiguous run of directions.
struct RankDirs {
    int n = 0;
    int e[kMaxDirs][3];       // the way the data travels
    int image[kMaxDirs][3];   // box lengths added to the sender's coordinates
    int dest[kMaxDirs];
};

inline void coords_of(const int dims[3], int rank, int out[3]) {
    out[0] = rank / (dims[1] * dims[2]);
    out[1] = (rank / dims[2]) % dims[1];
    out[2] = rank % dims[2];
}

inline RankDirs dirs_of(const int dims[3], int rank) {
    int at[3];
    coords_of(dims, rank, at);
    struct One { int e[3], image[3], dest; };
    std::vector<One> all;
    for (int ex = -1; ex <= 1; ++ex)
        for (int ey = -1; ey <= 1; ++ey)
            for (int ez = -1; ez <= 1; ++ez) {
                const int e[3] = {ex, ey, ez};
                if (!ex && !ey && !ez) continue;
                bool usable = true;
                for (int a = 0; a < 3; ++a) usable = usable && (e[a] == 0 || dims[a] > 1);
                if (!usable) continue;
                One one{};
                int c[3];
                for (int a = 0; a < 3; ++a) {
                    int v = at[a] + e[a];
                    one.e[a] = e[a];
                    one.image[a] = 0;
                    if (v < 0) { v += dims[a]; one.image[a] = 1; }
                    else if (v >= dims[a]) { v -= dims[a]; one.image[a] = -1; }
                    c[a] = v;
                }
                one.dest = (c[0] * dims[1] + c[1]) * dims[2] + c[2];
                all.push_back(one);
            }
    std::stable_sort(all.begin(), all.end(), [](const One& a, const One& b) { return a.dest < b.dest; });
    RankDirs out;
    out.n = static_cast<int>(all.size());
    for (int k = 0; k < out.n; ++k) {
        for (int a = 0; a < 3; ++a) { out.e[k][a] = all[k].e[a]; out.image[k][a] = all[k].image[a]; }
        out.dest[k] = all[k].dest;
    }
    return out;
}

// The distinct ranks a rank exchanges with (ascending), the run of its own directions that goes to each, and the run of
// each peer's directions that points back at it.
struct PeerPlan {
    int n_peers = 0;
    int peer[kMaxDirs];
    int dir_first[kMaxDirs + 1];
    int from_first[kMaxDirs], from_last[kMaxDirs];
};

inline PeerPlan peer_plan(const std::vector<RankDirs>& all, int rank) {
    PeerPlan plan;
    const RankDirs& mine = all[rank];
    for (int k = 0; k < mine.n; ++k) {
        if (plan.n_peers == 0 || plan.peer[plan.n_peers - 1] != mine.dest[k]) {
            plan.peer[plan.n_peers] = mine.dest[k];
            plan.dir_first[plan.n_peers] = k;
            ++plan.n_peers;
        }
    }
    plan.dir_first[plan.n_peers] = mine.n;
    for (int p = 0; p < plan.n_peers; ++p) {
        const RankDirs& theirs = all[plan.peer[p]];
        int first = theirs.n, last = theirs.n;
        for (int k = 0; k < theirs.n; ++k)
            if (theirs.dest[k] == rank) { if (first == theirs.n) first = k; last = k + 1; }
        plan.from_first[p] = first;
        plan.from_last[p] = last;
    }
    return plan;
}

// counts[r * kBins + 1 + k] = atoms rank r sends along its k-th direction. Per peer of `rank`: atoms sent and received.
inline void per_peer_counts(const PeerPlan& plan, const int* counts, int rank, int* send_to, int* recv_from, long long& n_send,
                            long long& n_recv) {
    const int* own = counts + static_cast<size_t>(rank) * kBins;
    n_send = n_recv = 0;
    for (int p = 0; p < plan.n_peers; ++p) {
        int s = 0, r = 0;
        for (int k = plan.dir_first[p]; k < plan.dir_first[p + 1]; ++k) s += own[1 + k];
        const int* theirs = counts + static_cast<size_t>(plan.peer[p]) * kBins;
        for (int k = plan.from_first[p]; k < plan.from_last[p]; ++k) r += theirs[1 + k];
        send_to[p] = s;
        recv_from[p] = r;
        n_send += s;
        n_recv += r;
    }
}

// The verdict every rank reaches from the same gathered counts (so all ranks leave an exchange with the same status):
// 0 = go on; otherwise the status code, the rank it is about and a sentence. Codes are the C ABI's (4 = atoms lost,
// 5 = no room).
struct CountsVerdict {
    int code = 0;
    int rank = -1;
    std::string text;
};

inline CountsVerdict counts_verdict(const std::vector<RankDirs>& all, const int* counts, long long scratch_capacity,
                                    const char* what) {
    const int world = static_cast<int>(all.size());
    CountsVerdict v;
    for (int r = 0; r < world; ++r) {
        const int* c = counts + static_cast<size_t>(r) * kBins;
        if (c[kBinLost] > 0) {
            v.code = 4;
            v.rank = r;
            v.text = "rank " + std::to_string(r) + ": " + std::to_string(c[kBinLost]) +
                     " atoms moved further than one brick between list builds (or are not finite)";
            return v;
        }
        long long arriving = 0, leaving = 0;
        for (int q = 0; q < world; ++q) {
            if (q == r) continue;
            const int* cq = counts + static_cast<size_t>(q) * kBins;
            for (int k = 0; k < all[q].n; ++k)
                if (all[q].dest[k] == r) arriving += cq[1 + k];
        }
        for (int k = 0; k < kMaxDirs; ++k) leaving += c[1 + k];
        if (arriving > c[kBinRoom]) {
            v.code = 5;
            v.rank = r;
            v.text = "rank " + std::to_string(r) + ": " + std::to_string(arriving) + " " + what + " arrive, the context has room for " +
                     std::to_string(c[kBinRoom]);
            return v;
        }
        if (leaving > scratch_capacity) {
            v.code = 5;
            v.rank = r;
            v.text = "rank " + std::to_string(r) + ": more " + std::string(what) + " to send than the scratch holds";
            return v;
        }
    }
    return v;
}

}  // namespace dsmd::host
