// C++ adapter with the reference's EdgeBuilder class shape (include/EdgeBuilder.cuh:12-84) over the C ABI.
//
// Same public interface: build(d_x, d_y, d_z, n, cutoff, stream, lo, hi, images, prune) -> E, edge_index(), edge_shift(),
// edge_count(); same Images / Prune structs; same exceptions (std::invalid_argument for bad arguments, std::runtime_error
// for an atom outside the box or a CUDA failure). A translation unit of the reference that includes this header instead of
// "EdgeBuilder.cuh" (MLIPStep.cu does) compiles unchanged.
#ifndef DSMD_EDGE_BUILDER_HPP
#define DSMD_EDGE_BUILDER_HPP

#include <cstdint>
#include <stdexcept>
#include <string>

#include <cuda_runtime.h>

#include "../dsmd_b200.h"

class EdgeBuilder {
public:
    struct Images {
        int64_t n_centers = 0;
        const int32_t* d_owner = nullptr;
        const double* d_shift_x = nullptr;
        const double* d_shift_y = nullptr;
        const double* d_shift_z = nullptr;
    };
    struct Prune {
        const unsigned char* d_receiver_ok = nullptr;
        int row = 1;
    };

    EdgeBuilder() {
        int device = 0;
        cudaGetDevice(&device);
        if (dsmd_edges_create(device, &impl_) != DSMD_OK) throw std::runtime_error("EdgeBuilder: dsmd_edges_create failed");
    }
    ~EdgeBuilder() { dsmd_edges_destroy(impl_); }
    EdgeBuilder(const EdgeBuilder&) = delete;
    EdgeBuilder& operator=(const EdgeBuilder&) = delete;

    int64_t build(const double* d_x, const double* d_y, const double* d_z, int64_t n, double cutoff, cudaStream_t stream,
                  const double* lo = nullptr, const double* hi = nullptr, const Images* images = nullptr,
                  const Prune* prune = nullptr) {
        if (images && (images->n_centers < 0 || images->n_centers > n || !images->d_owner || !images->d_shift_x ||
                       !images->d_shift_y || !images->d_shift_z))
            throw std::invalid_argument("EdgeBuilder::build: invalid periodic image description");
        if (prune && (!prune->d_receiver_ok || (prune->row != 0 && prune->row != 1)))
            throw std::invalid_argument("EdgeBuilder::build: invalid prune description");
        int64_t n_edges = 0;
        const int rc = dsmd_edges_build(impl_, d_x, d_y, d_z, n, cutoff, lo, hi, images ? images->n_centers : n,
                                        images ? images->d_owner : nullptr, images ? images->d_shift_x : nullptr,
                                        images ? images->d_shift_y : nullptr, images ? images->d_shift_z : nullptr,
                                        prune ? prune->d_receiver_ok : nullptr, prune ? prune->row : 1, &n_edges,
                                        static_cast<void*>(stream));
        if (rc == DSMD_ERR_INVALID) throw std::invalid_argument(std::string("EdgeBuilder::build: ") + dsmd_edges_last_error(impl_));
        if (rc != DSMD_OK) throw std::runtime_error(std::string("EdgeBuilder::build: ") + dsmd_edges_last_error(impl_));
        return n_edges;
    }

    const int64_t* edge_index() const {
        const int64_t* p = nullptr;
        dsmd_edges_result(impl_, &p, nullptr, nullptr);
        return p;
    }
    const double* edge_shift() const {
        const double* p = nullptr;
        dsmd_edges_result(impl_, nullptr, &p, nullptr);
        return p;
    }
    int64_t edge_count() const {
        int64_t n = 0;
        dsmd_edges_result(impl_, nullptr, nullptr, &n);
        return n;
    }

private:
    dsmd_edges* impl_ = nullptr;
};

#endif  // DSMD_EDGE_BUILDER_HPP
