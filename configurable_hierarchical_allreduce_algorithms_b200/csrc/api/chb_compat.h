/* Reference-compatible entry points.
 *
 * The reference exposes free functions over MPI types, e.g.
 *   int all_reduce_radix_batch(char* sendbuf, char* recvbuf, int count, MPI_Datatype datatype,
 *                              MPI_Op op, MPI_Comm comm, int k, int b);
 *   (testing/custom_implementations/work_dir/all_reduce/all_reduce_radix_batch.cpp:202-204,
 *    .../all_gather/all_gather_radix_batch_1_0.cpp:37,
 *    .../reduce_scatter/reduce_scatter_radix_batch.cpp:200-202,
 *    testing/main.cpp:13-31, testing/mpich_implementations/reduce_scatter/reduce_scatter.hpp:11-14).
 * The same names and argument orders are kept; MPI_Comm becomes a communicator
 * handle, MPI_Datatype / MPI_Op the CHB_* enums, buffers are device pointers
 * and the call is enqueued on the stream set with chb_set_stream (default
 * stream if never set).  Return value: 0 or a CHB_ERR_* code, like
 * MPI_SUCCESS / MPI_ERR_*.  CHB_IN_PLACE as sendbuf is honoured by
 * reduce-scatter and allreduce (input taken from recvbuf) and by the
 * allgathers (the rank's block already sits at its slot of recvbuf, as in
 * MPI); gather and the stand-alone phases answer CHB_ERR_ARG.  All ranks of
 * one call must pass buffers of the same kind (all inside the communicator's
 * peer-visible region or all outside it, all in place or none): the schedule
 * is chosen from the local pointers without cross-rank agreement, and ranks
 * that disagree would run different schedules and end in a wait that expires.
 * Counts are 64-bit where the reference's are
 * MPI_Aint and int where the reference's are int (values beyond 2^31 go
 * through chb_collective).
 */
#ifndef CHB_COMPAT_H_
#define CHB_COMPAT_H_
#include <cuda_runtime.h>
#include <stdint.h>

#include "chb.h"

#ifdef __cplusplus
extern "C" {
#endif

struct chb_comm;
typedef struct chb_comm* CHB_Comm;
typedef int CHB_Datatype; /* CHB_F32 ... */
typedef int CHB_Op;       /* CHB_SUM ... */
#define CHB_IN_PLACE ((void*)-1)

enum { CHB_ALLREDUCE = 0, CHB_REDUCE_SCATTER = 1, CHB_ALLGATHER = 2, CHB_ALLTOALL = 3, CHB_GATHER = 4, CHB_PHASE = 5 };

void chb_set_stream(cudaStream_t s);

/* generic: one pointer per local rank, any algorithm name, fused scale.
 * algo: a schedule name ("radix_batch", "ring", "recursive_doubling", ...; chb_list_algorithms), optionally
 * followed by ":ll" (owners push flagged lines: one NVLink traversal per round, rounds overlap line by line) or
 * ":pull" (readers pull: the persistent interpreter with its tile scheduler); without a suffix allreduce,
 * reduce-scatter, allgather and all-to-all run as push programs up to CHB_LL_PROGRAM_MAX bytes (environment,
 * default 4 MiB) when their messages fit the inbox and as pull programs above.  The kernel-level names "ll",
 * "ll2", "nvls", "nvls1" and "bulk" select the hand-written kernels. */
int chb_collective(CHB_Comm c, int coll, const char* algo, int k, int b, int aux, int dtype, int op,
                   const void* const* in, void* const* out, int64_t count, float scale, int nctas,
                   cudaStream_t stream);
void chb_collective_cache_clear(CHB_Comm c);

/* hierarchical radix-k / group-b collectives */
int allgather_radix_batch(char* sendbuf, int sendcount, CHB_Datatype datatype, char* recvbuf, CHB_Comm comm, int k, int b);
int reduce_scatter_radix_batch(const void* sendbuf, void* recvbuf, int64_t recvcount, CHB_Datatype datatype, CHB_Op op,
                               CHB_Comm comm, int k, int b);
int all_reduce_radix_batch(char* sendbuf, char* recvbuf, int count, CHB_Datatype datatype, CHB_Op op, CHB_Comm comm, int k, int b);
int all_reduce_semi_radix_batch(char* sendbuf, char* recvbuf, int count, CHB_Datatype datatype, CHB_Op op, CHB_Comm comm, int k, int b);
/* earlier variants kept by the reference */
int reduce_scatter_radix_block(char* sendbuf, char* recvbuf, int count, CHB_Datatype datatype, CHB_Op op, CHB_Comm comm, int r, int b);
int allgather_k_brucks(char* sendbuf, int sendcount, CHB_Datatype datatype, char* recvbuf, CHB_Comm comm, int k);
int gather_k_nomial(char* sendbuf, int sendcount, CHB_Datatype datatype, char* recvbuf, CHB_Comm comm, int k, int root);

/* the phases of the hierarchical collectives as calls of their own, with the reference's buffer layouts
 * (c = count argument, T = ceil((P/b) / b) stages; see csrc/sched/gen_chiara.cc "stand-alone phases"):
 *   intra_gather_k_nomial             send c        recv b*c     at the group root (slot group % b)
 *   inter_allgather_linear            send b*c      recv T*b*c
 *   intra_allgather_k_brucks          send T*c      recv (P/b)*c
 *   intra_reduce_scatter_radix_batch  send P*c      recv T*b*c
 *   inter_reduce_linear               send T*b*c    recv b*c     at the lane roots
 *   intra_scatter_radix_batch         send b*c      recv c */
int intra_gather_k_nomial(char* sendbuf, int count, CHB_Datatype datatype, char* recvbuf, CHB_Comm comm, int k, int b);
int intra_allgather_k_brucks(char* sendbuf, int count, CHB_Datatype datatype, char* recvbuf, CHB_Comm comm, int k, int b);
int inter_allgather_linear(char* sendbuf, int sendcount, CHB_Datatype datatype, char* recvbuf, CHB_Comm comm, int b);
int intra_reduce_scatter_radix_batch(const void* sendbuf, void* recvbuf, int64_t recvcount, CHB_Datatype datatype, CHB_Op op,
                                     CHB_Comm comm, int k, int b);
int inter_reduce_linear(const void* sendbuf, void* recvbuf, int64_t recvcount, CHB_Datatype datatype, CHB_Op op,
                        CHB_Comm comm, int b);
int intra_scatter_radix_batch(char* sendbuf, int recvcount, CHB_Datatype datatype, char* recvbuf, CHB_Comm comm, int k, int b);

/* MPICH-style baselines */
int MPICH_Allreduce_recursive_doubling(const char* sendbuf, char* recvbuf, int count, CHB_Datatype datatype, CHB_Op op, CHB_Comm comm);
int MPICH_Allreduce_ring(const char* sendbuf, char* recvbuf, int count, CHB_Datatype datatype, CHB_Op op, CHB_Comm comm);
int MPICH_Allreduce_reduce_scatter_allgather(const char* sendbuf, char* recvbuf, int count, CHB_Datatype datatype, CHB_Op op, CHB_Comm comm);
int MPICH_Allreduce_recursive_multiplying(const char* sendbuf, char* recvbuf, int count, CHB_Datatype datatype, CHB_Op op, CHB_Comm comm, int k);
int MPICH_Allreduce_k_reduce_scatter_allgather(const char* sendbuf, char* recvbuf, int count, CHB_Datatype datatype, CHB_Op op,
                                               CHB_Comm comm, int k, int single_phase_recv);
int MPICH_Allreduce_recursive_exchange(const char* sendbuf, char* recvbuf, int count, CHB_Datatype datatype, CHB_Op op,
                                       CHB_Comm comm, int k, int single_phase_recv);
/* the reference fixes the node size at compile time (-DRANKS_PER_NODE); here it is an argument */
int MPICH_Allreduce_inter_reduce_exchange_bcast(const char* sendbuf, char* recvbuf, int count, CHB_Datatype datatype, CHB_Op op,
                                                CHB_Comm comm, int ranks_per_node);
int MPICH_reduce_scatter_rec_halving(const void* sendbuf, void* recvbuf, int64_t recvcount, CHB_Datatype datatype, CHB_Op op, CHB_Comm comm);
int MPICH_reduce_scatter_rec_doubling(const void* sendbuf, void* recvbuf, int64_t recvcount, CHB_Datatype datatype, CHB_Op op, CHB_Comm comm);
int MPICH_reduce_scatter_pairwise(const void* sendbuf, void* recvbuf, int64_t recvcount, CHB_Datatype datatype, CHB_Op op, CHB_Comm comm);
int MPICH_reduce_scatter_radix(const void* sendbuf, void* recvbuf, int64_t recvcount, CHB_Datatype datatype, CHB_Op op, CHB_Comm comm, int k);
int MPICH_reduce_scatter_k_nomial(const char* sendbuf, char* recvbuf, int count, CHB_Datatype datatype, CHB_Op op, CHB_Comm comm, int k);

/* all-to-all-v with the radix-r / batch-b store-and-forward routing.  The blocks must be packed
 * (sdispls / rdispls are the running sums of the counts) and sendtype == recvtype.  The ranks first
 * exchange their count rows on the device, which synchronises the calling thread with the stream. */
int tuna2_algorithm(int r, int b, char* sendbuf, int* sendcounts, int* sdispls, CHB_Datatype sendtype,
                    char* recvbuf, int* recvcounts, int* rdispls, CHB_Datatype recvtype, CHB_Comm comm);

#ifdef __cplusplus
}
#endif
#endif /* CHB_COMPAT_H_ */
