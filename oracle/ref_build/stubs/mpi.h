// Serial stand-in for <mpi.h>: test infrastructure only.
// Lets the reference's CPU neighbour-list and force sources compile as a one-rank build.
// Reductions copy send -> recv (honouring MPI_IN_PLACE); everything else is a no-op.
#ifndef DSMD_ORACLE_STUB_MPI_H
#define DSMD_ORACLE_STUB_MPI_H
#include <cstring>
#include <cstddef>

typedef int MPI_Comm;
typedef int MPI_Datatype;
typedef int MPI_Op;
typedef int MPI_Request;
struct MPI_Status { int unused; };

#define MPI_COMM_WORLD 1
#define MPI_COMM_NULL 0
#define MPI_DOUBLE 8
#define MPI_INT 4
#define MPI_FLOAT 5
#define MPI_CHAR 1
#define MPI_UNSIGNED_LONG_LONG 9
#define MPI_LONG_LONG 10
#define MPI_UINT64_T 11
#define MPI_INT64_T 12
#define MPI_BYTE 13
#define MPI_MAX 1
#define MPI_SUM 2
#define MPI_MIN 3
#define MPI_ROOT (-3)
#define MPI_PROC_NULL (-2)
#define MPI_IN_PLACE ((void*)1)
#define MPI_STATUS_IGNORE ((MPI_Status*)0)
#define MPI_REQUEST_NULL 0
#define MPI_SUCCESS 0

inline size_t dsmd_stub_mpi_size(MPI_Datatype t) {
    switch (t) {
        case MPI_DOUBLE: case MPI_UNSIGNED_LONG_LONG: case MPI_LONG_LONG: case MPI_UINT64_T: case MPI_INT64_T: return 8;
        case MPI_INT: case MPI_FLOAT: return 4;
        default: return 1;
    }
}
inline int MPI_Initialized(int* flag) { *flag = 0; return MPI_SUCCESS; }
inline int MPI_Comm_rank(MPI_Comm, int* r) { *r = 0; return MPI_SUCCESS; }
inline int MPI_Comm_size(MPI_Comm, int* s) { *s = 1; return MPI_SUCCESS; }
inline int MPI_Bcast(void*, int, MPI_Datatype, int, MPI_Comm) { return MPI_SUCCESS; }
inline int MPI_Wait(MPI_Request*, MPI_Status*) { return MPI_SUCCESS; }
inline int MPI_Barrier(MPI_Comm) { return MPI_SUCCESS; }
inline int MPI_Allreduce(const void* send, void* recv, int count, MPI_Datatype t, MPI_Op, MPI_Comm) {
    if (send != MPI_IN_PLACE && send != recv) std::memcpy(recv, send, dsmd_stub_mpi_size(t) * static_cast<size_t>(count));
    return MPI_SUCCESS;
}
inline int MPI_Reduce(const void* send, void* recv, int count, MPI_Datatype t, MPI_Op, int, MPI_Comm) {
    if (send != MPI_IN_PLACE && recv && send != recv) std::memcpy(recv, send, dsmd_stub_mpi_size(t) * static_cast<size_t>(count));
    return MPI_SUCCESS;
}
inline int MPI_Ireduce(const void* send, void* recv, int count, MPI_Datatype t, MPI_Op op, int root, MPI_Comm c,
                       MPI_Request* req) {
    if (req) *req = MPI_REQUEST_NULL;
    return MPI_Reduce(send, recv, count, t, op, root, c);
}
#endif
