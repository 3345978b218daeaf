/* Process rendezvous for the ranks of one box, without MPI and without Python:
 * a POSIX shared-memory segment with one slot per rank, a generation-counting
 * barrier and an allgather of small blobs (cudaIpc handles, a library unique id,
 * timing results).  Every wait has a deadline; a rank that never arrives makes
 * the others return CHB_ERR_TIMEOUT instead of hanging.
 *
 * Plays the role of MPI_Init / MPI_Comm_rank / MPI_Allgather / MPI_Barrier in the
 * reference's drivers (testing/custom_implementations/work_dir/all_reduce/main.cpp:111-199)
 * for the native launcher. */
#ifndef CHB_BOOTSTRAP_H_
#define CHB_BOOTSTRAP_H_
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct chb_bootstrap chb_bootstrap;

#define CHB_BOOT_SLOT_BYTES 4096

/* name: "/something" (shm_open rules), the same on every rank and unique per job.
 * Rank 0 creates the segment, the others attach; all return once everybody has. */
int chb_bootstrap_create(const char* name, int rank, int world, int timeout_ms, chb_bootstrap** out);
int chb_bootstrap_rank(const chb_bootstrap* b);
int chb_bootstrap_world(const chb_bootstrap* b);
const char* chb_bootstrap_name(const chb_bootstrap* b);
/* all[r * bytes .. ) = rank r's `mine`; bytes <= CHB_BOOT_SLOT_BYTES. */
int chb_bootstrap_allgather(chb_bootstrap* b, const void* mine, void* all, size_t bytes);
int chb_bootstrap_barrier(chb_bootstrap* b);
/* File descriptors cross process boundaries as ancillary data of Unix datagrams (SCM_RIGHTS); every rank
 * listens on an abstract socket derived from the rendezvous name.  my_fd < 0: this rank has nothing to hand
 * out.  On return fds[r] is this process's duplicate of rank r's descriptor (-1 if r offered none; fds[rank]
 * is my_fd itself).  The caller closes what it receives.  Bounded by the rendezvous timeout. */
int chb_bootstrap_exchange_fds(chb_bootstrap* b, int my_fd, int* fds);
/* Tell the others to give up (their current or next wait returns CHB_ERR_OTHER at once). */
void chb_bootstrap_abort(chb_bootstrap* b);
void chb_bootstrap_destroy(chb_bootstrap* b);

#ifdef __cplusplus
}
#endif
#endif
