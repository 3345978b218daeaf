// Minimal single-process stand-in for <mpi.h>: every MPI rank is a thread of
// one process.  Only what the reference's collectives and stand-alone phases call is provided
// (rank / size / type size, Isend / Irecv / Wait / Waitall, Reduce_local,
// Barrier, Wtime).  Small sends are eager (the payload is copied into the
// destination's mailbox), large non-blocking sends are copied once, by the
// receiver, straight from the sender's buffer; receives match on (source, tag)
// in arrival order.
// This exists so that the reference's own sources can be compiled unmodified
// and timed on a machine without an MPI installation.
#pragma once
#include <cstddef>
#include <cstdint>
#include <climits>
#include <cmath>
#include <cstdlib>
#include <cstring>   // the reference's older sources rely on their MPI header bringing these in

typedef int MPI_Comm;
typedef int MPI_Datatype;   // value = element size in bytes, except the tags below; >= 1000: derived type
typedef int MPI_Op;
typedef long MPI_Aint;
struct MPI_Status { int MPI_SOURCE, MPI_TAG, MPI_ERROR; };
struct ShimRequest;
typedef ShimRequest* MPI_Request;

#define MPI_COMM_WORLD 0
#define MPI_SUCCESS 0
#define MPI_ERR_NO_MEM 1
#define MPI_ERR_OTHER 2
#define MPI_ERR_COUNT 3
#define MPI_ERR_OP 4
#define MPI_ERR_ARG 5
#define MPI_CHAR 1
#define MPI_INT 4
#define MPI_DOUBLE 8
#define MPI_FLOAT 104      /* 4-byte float, told apart from MPI_INT */
#define MPI_SUM 0
#define MPI_MAX 1
#define MPI_MIN 2
#define MPI_IN_PLACE ((void*)-1)
#define MPI_DATATYPE_NULL 0
#define MPI_COMM_NULL (-1)
#define MPI_UNDEFINED (-32766)
#define MPI_STATUS_IGNORE ((MPI_Status*)0)
#define MPI_STATUSES_IGNORE ((MPI_Status*)0)

int MPI_Comm_rank(MPI_Comm, int*);
int MPI_Comm_size(MPI_Comm, int*);
int MPI_Type_size(MPI_Datatype, int*);
int MPI_Isend(const void*, int, MPI_Datatype, int, int, MPI_Comm, MPI_Request*);
int MPI_Irecv(void*, int, MPI_Datatype, int, int, MPI_Comm, MPI_Request*);
int MPI_Wait(MPI_Request*, MPI_Status*);
int MPI_Waitall(int, MPI_Request*, MPI_Status*);
int MPI_Reduce_local(const void*, void*, int, MPI_Datatype, MPI_Op);
int MPI_Barrier(MPI_Comm);
double MPI_Wtime();
// blocking forms (the stand-alone phase sources use them)
int MPI_Send(const void*, int, MPI_Datatype, int, int, MPI_Comm);
int MPI_Recv(void*, int, MPI_Datatype, int, int, MPI_Comm, MPI_Status*);
int MPI_Sendrecv(const void*, int, MPI_Datatype, int, int, void*, int, MPI_Datatype, int, int, MPI_Comm, MPI_Status*);
int MPI_Op_commutative(MPI_Op, int*);
int MPI_Comm_split(MPI_Comm, int, int, MPI_Comm*);
int MPI_Comm_free(MPI_Comm*);
// derived datatypes: lists of byte segments of a basic type (what the recursive-doubling reduce-scatter builds)
int MPI_Type_create_hindexed(int, const int*, const MPI_Aint*, MPI_Datatype, MPI_Datatype*);
int MPI_Type_commit(MPI_Datatype*);
int MPI_Type_free(MPI_Datatype*);
int MPI_Type_get_extent(MPI_Datatype, MPI_Aint*, MPI_Aint*);
int MPI_Type_get_true_extent(MPI_Datatype, MPI_Aint*, MPI_Aint*);
// in-place form only (what the reference's ring allreduce uses): every rank's block already sits at displs[rank]
int MPI_Allgatherv(const void*, int, MPI_Datatype, void*, const int*, const int*, MPI_Datatype, MPI_Comm);
// MPI_Reduce / MPI_Allreduce / MPI_Bcast are real (the SMP allreduce and the all-to-all-v use them); the rest of
// this block is only called by the reference's own test mains, which are compiled but never run: stubs that flag a failure.
int MPI_Init(int*, char***);
int MPI_Finalize();
int MPI_Abort(MPI_Comm, int);
int MPI_Allgather(const void*, int, MPI_Datatype, void*, int, MPI_Datatype, MPI_Comm);
int MPI_Allreduce(const void*, void*, int, MPI_Datatype, MPI_Op, MPI_Comm);
int MPI_Reduce(const void*, void*, int, MPI_Datatype, MPI_Op, int, MPI_Comm);
int MPI_Bcast(void*, int, MPI_Datatype, int, MPI_Comm);
int MPI_Gather(const void*, int, MPI_Datatype, void*, int, MPI_Datatype, int, MPI_Comm);
int MPI_Scatter(const void*, int, MPI_Datatype, void*, int, MPI_Datatype, int, MPI_Comm);
int MPI_Reduce_scatter(const void*, void*, const int*, MPI_Datatype, MPI_Op, MPI_Comm);
int MPI_Reduce_scatter_block(const void*, void*, int, MPI_Datatype, MPI_Op, MPI_Comm);
int MPI_Alltoallv(const void*, const int*, const int*, MPI_Datatype, void*, const int*, const int*, MPI_Datatype, MPI_Comm);

// shim control (not MPI): world size, per-thread rank, failure flag
void shim_init(int nprocs);
void shim_set_rank(int rank);
int shim_failed();
